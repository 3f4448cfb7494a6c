// y[M, N] = alpha * x[M, K] @ w[N, K]^T for a handful of rows (M <= 16): the single-token decode step, where a
// 128-row tensor-core tile would be 1 % full and the op is bound by reading w once.  One warp per output column
// streams that row of w with 16-byte loads and keeps M fp32 accumulators; x (a few KB) is read through L1.  The
// reference's decode step (custom_models/ipttcd/modeling_ipttcdv9.py forward with a KV cache) runs nn.Linear on
// one row through the library; this is the equivalent for the row counts a decode step has.
#include "common.cuh"

namespace ttcd {

template <int M>
__global__ void __launch_bounds__(256) gemv_small_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                         bf16* __restrict__ y, int N, int K, int64_t ldx, int64_t ldw,
                                                         int64_t ldy, float alpha) {
  const int lane = threadIdx.x & 31;
  const int n = (blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5));
  if (n >= N) return;
  float acc[M];
#pragma unroll
  for (int m = 0; m < M; ++m) acc[m] = 0.f;
  const bf16* wr = w + static_cast<int64_t>(n) * ldw;
  for (int k = lane * 8; k < K; k += 256) {
    const uint4 wv = *reinterpret_cast<const uint4*>(wr + k);
    const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
    for (int m = 0; m < M; ++m) {
      const uint4 xv = *reinterpret_cast<const uint4*>(x + m * ldx + k);
      const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 a = unpack_bf16(ww[i]), b = unpack_bf16(xw[i]);
        acc[m] = fmaf(a.x, b.x, fmaf(a.y, b.y, acc[m]));
      }
    }
  }
#pragma unroll
  for (int m = 0; m < M; ++m) {
    float v = acc[m];
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    if (lane == 0) y[m * ldy + n] = __float2bfloat16(v * alpha);
  }
}

}  // namespace ttcd

// x: [M, K] bf16 rows ldx apart, w: [N, K] bf16 rows ldw apart, y: [M, N] bf16; 1 <= M <= 16, K a multiple of 8,
// x / w 16-byte aligned with ldx, ldw multiples of 8.
TTCD_EXPORT int ttcd_gemv_small(const void* x, const void* w, void* y, int M, int N, int K, long long ldx, long long ldw,
                                long long ldy, float alpha, void* stream_ptr) {
  using namespace ttcd;
  if (M < 1 || M > 16 || N < 1 || K < 8 || K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0) return TTCD_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(x) & 15u) || (reinterpret_cast<uintptr_t>(w) & 15u)) return TTCD_ERR_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  const unsigned blocks = static_cast<unsigned>((N + 7) / 8);
  const bf16* xp = static_cast<const bf16*>(x);
  const bf16* wp = static_cast<const bf16*>(w);
  bf16* yp = static_cast<bf16*>(y);
#define TTCD_GEMV_CASE(MM) \
  case MM: gemv_small_kernel<MM><<<blocks, 256, 0, stream>>>(xp, wp, yp, N, K, ldx, ldw, ldy, alpha); break;
  switch (M) {
    TTCD_GEMV_CASE(1) TTCD_GEMV_CASE(2) TTCD_GEMV_CASE(3) TTCD_GEMV_CASE(4) TTCD_GEMV_CASE(5) TTCD_GEMV_CASE(6)
    TTCD_GEMV_CASE(7) TTCD_GEMV_CASE(8) TTCD_GEMV_CASE(9) TTCD_GEMV_CASE(10) TTCD_GEMV_CASE(11) TTCD_GEMV_CASE(12)
    TTCD_GEMV_CASE(13) TTCD_GEMV_CASE(14) TTCD_GEMV_CASE(15) TTCD_GEMV_CASE(16)
    default: return TTCD_ERR_ARG;
  }
#undef TTCD_GEMV_CASE
  return static_cast<int>(cudaGetLastError());
}
