// Peer-memory communication layer for one process per GPU on an NVLink/NVSwitch node.
//
// Host side: symmetric buffers are plain cudaMalloc allocations whose CUDA IPC handles are exchanged
// through the existing torch.distributed group; every rank then holds a device pointer to each
// peer's buffer.  Device side: kernels issue ordinary loads/stores (and red.add) on those pointers,
// which travel over NVLink; no TMA multicast is used anywhere.
//
// Kernels:
//   comm_barrier            : all-to-all flag barrier (release stores to every peer, bounded acquire spin)
//   rs_cast_scale_norm      : gradient reduce-scatter fused with the bf16->fp32 cast, the 1/world scale
//                             and the squared-norm partial: each rank pulls its shard from every peer
//   adamw_push              : AdamW on the local fp32 shard fused with the parameter all-gather: the new
//                             bf16 values are stored straight into every peer's flat parameter buffer
//   peer_add / peer_copy    : accumulate / copy a peer's buffer into a local one (halo exchange, TP)
//
// Every wait is bounded (TTCD_PEER_WAIT_NS); on expiry the kernel records an error code in the status
// word and returns, leaving the context usable.  The reference has no counterpart: its only transport
// is NCCL through torch.distributed (flame/models/parallelize_fla.py:436-497).
#include "common.cuh"

#include <algorithm>
#include <cstring>

#ifndef TTCD_PEER_WAIT_NS
#define TTCD_PEER_WAIT_NS 10000000000ull  // 10 s: peers may legitimately be a whole kernel behind
#endif

namespace ttcd {

constexpr int MAX_RANKS = 16;

struct PeerPtrs {
  void* p[MAX_RANKS];
};

__device__ __forceinline__ void st_release_sys(int* addr, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// flags.p[r] -> rank r's flag array int[world * slots]; slot `slot`, entry [slot * world + writer].
// Rank `rank` publishes `epoch` to every peer and waits until every peer has published >= epoch to it.
// A wait that runs out records 500 + the absent rank in the status word and, when `fail` is given, stores 1.0f
// there: kernels later in the step read that word and leave their outputs untouched (see adamw_push).
__global__ void comm_barrier_kernel(PeerPtrs flags, int rank, int world, int slot, int epoch, uint64_t wait_ns,
                                    float* fail) {
  const int r = threadIdx.x;
  if (r >= world) return;
  __threadfence_system();  // make this GPU's earlier writes visible before the flag
  st_release_sys(static_cast<int*>(flags.p[r]) + slot * world + rank, epoch);
  const int* mine = static_cast<const int*>(flags.p[rank]) + slot * world + r;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t it = 0;; ++it) {
    if (ld_acquire_sys(mine) >= epoch) break;
    if ((it & 0x3f) == 0x3f) {
      if (globaltimer_ns() - t0 > wait_ns) {
        atomicCAS(&g_status, 0, 500 + r);
        if (fail != nullptr) *fail = 1.f;
        break;
      }
      __nanosleep(200);
    }
  }
}

__device__ __forceinline__ void add8(float (&acc)[8], uint4 raw) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = unpack_bf16(w[i]);
    acc[2 * i] += t.x;
    acc[2 * i + 1] += t.y;
  }
}

// out[i] = scale * sum_r grads.p[r][offset + i]   (bf16 in, fp32 out), norm_sq += sum(out^2)
__global__ void __launch_bounds__(256) rs_cast_scale_norm_kernel(PeerPtrs grads, int world, int64_t offset, int64_t n,
                                                                 float scale, float* __restrict__ out,
                                                                 float* __restrict__ norm_sq) {
  __shared__ float red[8];
  float ss = 0.f;
  const int64_t nvec = n / 8;
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec;
       v += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < world; ++r)
      add8(acc, *reinterpret_cast<const uint4*>(static_cast<const bf16*>(grads.p[r]) + offset + v * 8));
    float4 lo, hi;
    lo.x = acc[0] * scale; lo.y = acc[1] * scale; lo.z = acc[2] * scale; lo.w = acc[3] * scale;
    hi.x = acc[4] * scale; hi.y = acc[5] * scale; hi.z = acc[6] * scale; hi.w = acc[7] * scale;
    ss += lo.x * lo.x + lo.y * lo.y + lo.z * lo.z + lo.w * lo.w + hi.x * hi.x + hi.y * hi.y + hi.z * hi.z + hi.w * hi.w;
    *reinterpret_cast<float4*>(out + v * 8) = lo;
    *reinterpret_cast<float4*>(out + v * 8 + 4) = hi;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 8) {
    float t = red[threadIdx.x];
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffu, t, o);
    if (threadIdx.x == 0 && norm_sq != nullptr) atomicAdd(norm_sq, t);
  }
}

// AdamW on the local fp32 shard; the updated bf16 values go to params.p[r] + offset for every rank r.
__global__ void __launch_bounds__(256) adamw_push_kernel(float* __restrict__ p, const float* __restrict__ g,
                                                         float* __restrict__ m, float* __restrict__ v, PeerPtrs params,
                                                         int world, int64_t offset, int64_t n, float lr, float beta1,
                                                         float beta2, float eps, float wd, float bc1, float bc2_sqrt,
                                                         const float* __restrict__ coef, const int* __restrict__ skip) {
  if (skip != nullptr && *skip != 0) return;
  const float c = coef != nullptr ? *coef : 1.f;
  const float step_size = lr / bc1;
  const int64_t nvec = n / 8;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float o[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int64_t base = i * 8 + h * 4;
      const float4 gv = *reinterpret_cast<const float4*>(g + base);
      float4 pv = *reinterpret_cast<float4*>(p + base);
      float4 mv = *reinterpret_cast<float4*>(m + base);
      float4 vv = *reinterpret_cast<float4*>(v + base);
      const float gs[4] = {gv.x * c, gv.y * c, gv.z * c, gv.w * c};
      float ps[4] = {pv.x, pv.y, pv.z, pv.w}, ms[4] = {mv.x, mv.y, mv.z, mv.w}, vs[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        ps[k] *= (1.f - lr * wd);
        ms[k] = beta1 * ms[k] + (1.f - beta1) * gs[k];
        vs[k] = beta2 * vs[k] + (1.f - beta2) * gs[k] * gs[k];
        ps[k] -= step_size * ms[k] / (sqrtf(vs[k]) / bc2_sqrt + eps);
        o[h * 4 + k] = ps[k];
      }
      *reinterpret_cast<float4*>(p + base) = make_float4(ps[0], ps[1], ps[2], ps[3]);
      *reinterpret_cast<float4*>(m + base) = make_float4(ms[0], ms[1], ms[2], ms[3]);
      *reinterpret_cast<float4*>(v + base) = make_float4(vs[0], vs[1], vs[2], vs[3]);
    }
    uint4 pk;
    pk.x = pack_bf16(o[0], o[1]); pk.y = pack_bf16(o[2], o[3]);
    pk.z = pack_bf16(o[4], o[5]); pk.w = pack_bf16(o[6], o[7]);
    for (int r = 0; r < world; ++r)
      *reinterpret_cast<uint4*>(static_cast<bf16*>(params.p[r]) + offset + i * 8) = pk;
  }
}

// params.p[r][offset + i] = bf16(src[i]) for every rank r: publishes an owner-computed fp32 tensor
__global__ void __launch_bounds__(256) push_cast_kernel(const float* __restrict__ src, PeerPtrs params, int world,
                                                        int64_t offset, int64_t n) {
  const int64_t nvec = n / 8;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const float4 a = *reinterpret_cast<const float4*>(src + i * 8);
    const float4 b = *reinterpret_cast<const float4*>(src + i * 8 + 4);
    uint4 pk;
    pk.x = pack_bf16(a.x, a.y); pk.y = pack_bf16(a.z, a.w);
    pk.z = pack_bf16(b.x, b.y); pk.w = pack_bf16(b.z, b.w);
    for (int r = 0; r < world; ++r)
      *reinterpret_cast<uint4*>(static_cast<bf16*>(params.p[r]) + offset + i * 8) = pk;
  }
}

// dst[i] (+)= src[i] over 16-byte vectors of bf16 (src is usually a peer pointer)
__global__ void __launch_bounds__(256) peer_add_kernel(bf16* __restrict__ dst, const bf16* __restrict__ src, int64_t n,
                                                       int accumulate) {
  const int64_t nvec = n / 8;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    uint4 s = *reinterpret_cast<const uint4*>(src + i * 8);
    if (accumulate) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      add8(acc, s);
      add8(acc, *reinterpret_cast<const uint4*>(dst + i * 8));
      s.x = pack_bf16(acc[0], acc[1]); s.y = pack_bf16(acc[2], acc[3]);
      s.z = pack_bf16(acc[4], acc[5]); s.w = pack_bf16(acc[6], acc[7]);
    }
    *reinterpret_cast<uint4*>(dst + i * 8) = s;
  }
}

// dst[i] = sum_r srcs.p[r][i] in fp32 (ordered: deterministic); used for small fp32 all-reduces over peer memory
__global__ void __launch_bounds__(256) peer_sum_f32_kernel(float* __restrict__ dst, PeerPtrs srcs, int world, int64_t n,
                                                           int first, int count) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < count; ++k) acc += static_cast<const float*>(srcs.p[(first + k) % world])[i];
    dst[i] = acc;
  }
}

static PeerPtrs make_ptrs(const long long* ptrs, int world) {
  PeerPtrs pp;
  for (int i = 0; i < MAX_RANKS; ++i) pp.p[i] = i < world ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
  return pp;
}
static unsigned grid_for(long long nvec) {
  return static_cast<unsigned>(std::max<long long>(1, std::min<long long>((nvec + 255) / 256, 148LL * 8)));
}

}  // namespace ttcd

TTCD_DEFINE_STATUS_READER(comm)
using namespace ttcd;

// ---- symmetric allocation + CUDA IPC -------------------------------------------------------------
TTCD_EXPORT int ttcd_symm_alloc(long long nbytes, long long* out_ptr) {
  void* p = nullptr;
  TTCD_CUDA_CHECK(cudaMalloc(&p, static_cast<size_t>(nbytes)));
  TTCD_CUDA_CHECK(cudaMemset(p, 0, static_cast<size_t>(nbytes)));
  *out_ptr = reinterpret_cast<long long>(p);
  return TTCD_OK;
}
TTCD_EXPORT int ttcd_symm_free(long long ptr) { return static_cast<int>(cudaFree(reinterpret_cast<void*>(ptr))); }
TTCD_EXPORT int ttcd_ipc_handle_size() { return static_cast<int>(sizeof(cudaIpcMemHandle_t)); }
TTCD_EXPORT int ttcd_ipc_get_handle(long long ptr, void* out_handle) {
  cudaIpcMemHandle_t h;
  TTCD_CUDA_CHECK(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(ptr)));
  memcpy(out_handle, &h, sizeof(h));
  return TTCD_OK;
}
TTCD_EXPORT int ttcd_ipc_open_handle(const void* handle, long long* out_ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  TTCD_CUDA_CHECK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *out_ptr = reinterpret_cast<long long>(p);
  return TTCD_OK;
}
TTCD_EXPORT int ttcd_ipc_close(long long ptr) {
  return static_cast<int>(cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr)));
}

// ---- kernels ---------------------------------------------------------------------------------------
TTCD_EXPORT int ttcd_comm_barrier(const long long* flag_ptrs, int rank, int world, int slot, int epoch,
                                  long long wait_ns, float* fail, void* stream_ptr) {
  if (world < 1 || world > MAX_RANKS) return TTCD_ERR_ARG;
  const uint64_t w = wait_ns > 0 ? static_cast<uint64_t>(wait_ns) : TTCD_PEER_WAIT_NS;
  comm_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_ptr)>>>(make_ptrs(flag_ptrs, world), rank, world,
                                                                           slot, epoch, w, fail);
  return static_cast<int>(cudaGetLastError());
}

TTCD_EXPORT int ttcd_rs_cast_scale_norm(const long long* grad_ptrs, int world, long long offset, long long n,
                                        float scale, float* out, float* norm_sq, void* stream_ptr) {
  if (world < 1 || world > MAX_RANKS || n % 8 != 0 || offset % 8 != 0) return TTCD_ERR_ARG;
  if (n == 0) return TTCD_OK;
  rs_cast_scale_norm_kernel<<<grid_for(n / 8), 256, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      make_ptrs(grad_ptrs, world), world, offset, n, scale, out, norm_sq);
  return static_cast<int>(cudaGetLastError());
}

TTCD_EXPORT int ttcd_adamw_push(float* p, const float* g, float* m, float* v, const long long* param_ptrs, int world,
                                long long offset, long long n, float lr, float beta1, float beta2, float eps, float wd,
                                float bc1, float bc2_sqrt, const float* coef, const int* skip, void* stream_ptr) {
  if (world < 1 || world > MAX_RANKS || n % 8 != 0 || offset % 8 != 0) return TTCD_ERR_ARG;
  if (n == 0) return TTCD_OK;
  adamw_push_kernel<<<grid_for(n / 8), 256, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      p, g, m, v, make_ptrs(param_ptrs, world), world, offset, n, lr, beta1, beta2, eps, wd, bc1, bc2_sqrt, coef, skip);
  return static_cast<int>(cudaGetLastError());
}

TTCD_EXPORT int ttcd_push_cast(const float* src, const long long* param_ptrs, int world, long long offset, long long n,
                               void* stream_ptr) {
  if (world < 1 || world > MAX_RANKS || n % 8 != 0 || offset % 8 != 0) return TTCD_ERR_ARG;
  if (n == 0) return TTCD_OK;
  push_cast_kernel<<<grid_for(n / 8), 256, 0, static_cast<cudaStream_t>(stream_ptr)>>>(src, make_ptrs(param_ptrs, world),
                                                                                     world, offset, n);
  return static_cast<int>(cudaGetLastError());
}

TTCD_EXPORT int ttcd_peer_add(void* dst, const void* src, long long n, int accumulate, void* stream_ptr) {
  if (n % 8 != 0) return TTCD_ERR_ARG;
  if (n == 0) return TTCD_OK;
  peer_add_kernel<<<grid_for(n / 8), 256, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      static_cast<bf16*>(dst), static_cast<const bf16*>(src), n, accumulate);
  return static_cast<int>(cudaGetLastError());
}

TTCD_EXPORT int ttcd_peer_sum_f32(float* dst, const long long* src_ptrs, int world, long long n, int first, int count,
                                  void* stream_ptr) {
  if (world < 1 || world > MAX_RANKS || count < 0 || count > world) return TTCD_ERR_ARG;
  if (n == 0) return TTCD_OK;
  peer_sum_f32_kernel<<<grid_for(n), 256, 0, static_cast<cudaStream_t>(stream_ptr)>>>(dst, make_ptrs(src_ptrs, world),
                                                                                    world, n, first, count);
  return static_cast<int>(cudaGetLastError());
}
