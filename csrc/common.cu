// Host-side pieces shared by all kernels: the device status word and tensor-map encoding through
// the driver entry point (resolved at run time, so the library links against cudart only).
#include "common.cuh"

#include <cudaTypedefs.h>
#include <cstdio>
#include <mutex>

namespace ttcd {

static PFN_cuTensorMapEncodeTiled_v12000 get_encode() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
    }
  });
  return fn;
}

// What the last failed tensor-map encode was asked for (per thread), for the error message of the binding.
static thread_local char g_tmap_error[320] = "";

int make_tmap_bf16_3d(CUtensorMap* map, const void* base, uint64_t inner, uint64_t rows, uint64_t batch,
                      uint64_t row_stride_elems, uint64_t batch_stride_elems, uint32_t box_inner,
                      uint32_t box_rows) {
  auto encode = get_encode();
  if (encode == nullptr) return TTCD_ERR_TMAP;
  // The encode is a driver call and wants a current context.  A thread whose first CUDA work is one of these
  // launches (an autograd worker running a GEMM as the first node of a backward pass) has made no runtime call yet
  // that would have bound the primary context to it: bind it once per thread.
  static thread_local bool context_bound = false;
  if (!context_bound) {
    cudaFree(nullptr);
    context_bound = true;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (row_stride_elems % 8) != 0) return TTCD_ERR_ARG;
  if (batch > 1 && (batch_stride_elems % 8) != 0) return TTCD_ERR_ARG;
  cuuint64_t dims[3] = {inner, rows, batch == 0 ? 1 : batch};
  cuuint64_t bstride = batch > 1 ? batch_stride_elems : rows * row_stride_elems;
  if (bstride == 0) bstride = 8;
  cuuint64_t strides[2] = {row_stride_elems * sizeof(bf16), bstride * sizeof(bf16)};
  cuuint32_t box[3] = {box_inner, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    std::snprintf(g_tmap_error, sizeof(g_tmap_error),
                  "cuTensorMapEncodeTiled -> %d: base %p dims {%llu, %llu, %llu} strides(bytes) {%llu, %llu} box {%u, %u, 1}",
                  static_cast<int>(r), base, static_cast<unsigned long long>(dims[0]), static_cast<unsigned long long>(dims[1]),
                  static_cast<unsigned long long>(dims[2]), static_cast<unsigned long long>(strides[0]),
                  static_cast<unsigned long long>(strides[1]), box_inner, box_rows);
  return r == CUDA_SUCCESS ? TTCD_OK : TTCD_ERR_TMAP;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace ttcd

// Copies the description of this thread's last failed tensor-map encode into buf (empty string if none).
TTCD_EXPORT int ttcd_last_tmap_error(char* buf, int size) {
  if (buf == nullptr || size <= 0) return TTCD_ERR_ARG;
  std::snprintf(buf, static_cast<size_t>(size), "%s", ttcd::g_tmap_error);
  return TTCD_OK;
}

