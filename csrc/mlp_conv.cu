// SwiGLU (forward/backward) and the depthwise causal convolution with per-chunk reset
// (forward/backward) for sm_100a.  The convolution covers both uses in the framework: the TTT
// teacher/student convs (K = 5, zero left context per ttt_chunk) and the sequence-level short
// conv (K = 4, chunk = whole sequence).  Replaces fla/modules/activations.py:402-486,
// profiling/fused_conv.py:15-48 and the cuDNN path of
// custom_models/ipttcd/modeling_ipttcdv9.py:203-211 (forward and backward).
#include "common.cuh"

#include <algorithm>

namespace ttcd {

__device__ __forceinline__ void load8(const bf16* p, float (&f)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = unpack_bf16(w[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(bf16* p, const float (&f)[8]) {
  uint4 raw;
  raw.x = pack_bf16(f[0], f[1]);
  raw.y = pack_bf16(f[2], f[3]);
  raw.z = pack_bf16(f[4], f[5]);
  raw.w = pack_bf16(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = raw;
}

// z = gate * sigmoid(gate) * up;  gate/up rows may be strided views of one packed buffer.
__global__ void __launch_bounds__(256) swiglu_fwd_kernel(const bf16* __restrict__ gate, const bf16* __restrict__ up,
                                                         bf16* __restrict__ z, int64_t rows, int d, int64_t ldg,
                                                         int64_t ldu, int64_t ldz) {
  const int vec_per_row = d / 8;
  const int64_t total = rows * vec_per_row;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / vec_per_row;
    const int c = static_cast<int>(i % vec_per_row) * 8;
    float g[8], u[8], o[8];
    load8(gate + r * ldg + c, g);
    load8(up + r * ldu + c, u);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = g[k] / (1.f + __expf(-g[k])) * u[k];
    store8(z + r * ldz + c, o);
  }
}

__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const bf16* __restrict__ dz, const bf16* __restrict__ gate,
                                                         const bf16* __restrict__ up, bf16* __restrict__ dgate,
                                                         bf16* __restrict__ dup, int64_t rows, int d, int64_t lddz,
                                                         int64_t ldg, int64_t ldu, int64_t lddg, int64_t lddu) {
  const int vec_per_row = d / 8;
  const int64_t total = rows * vec_per_row;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / vec_per_row;
    const int c = static_cast<int>(i % vec_per_row) * 8;
    float g[8], u[8], dzv[8], dg[8], du[8];
    load8(dz + r * lddz + c, dzv);
    load8(gate + r * ldg + c, g);
    load8(up + r * ldu + c, u);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float sg = 1.f / (1.f + __expf(-g[k]));
      const float silu = g[k] * sg;
      du[k] = dzv[k] * silu;
      dg[k] = dzv[k] * u[k] * (sg + silu * (1.f - sg));
    }
    store8(dgate + r * lddg + c, dg);
    store8(dup + r * lddu + c, du);
  }
}

// ------------------------------------------------------------------------------------------------
// Depthwise conv over the C axis of x[n][C][D] with zero context at every chunk start.
//   causal : y[c] = sum_j w[d][j] * x[c - (K-1) + j]
//   centred: y[c] = sum_j w[d][j] * x[c - K/2 + j]
// Thread = 8 channels x ROWS consecutive positions, sliding the K-row window through registers.
// ------------------------------------------------------------------------------------------------
constexpr int CONV_ROWS = 64;
constexpr int CONV_MAXK = 8;
constexpr int CONV_BATCH = 8;      // rows whose loads are issued together (memory-level parallelism per thread)

__device__ __forceinline__ void conv_unpack(const uint4& raw, float (&dst)[8]) {
  const float2 a = unpack_bf16(raw.x), b = unpack_bf16(raw.y), c = unpack_bf16(raw.z), d = unpack_bf16(raw.w);
  dst[0] = a.x; dst[1] = a.y; dst[2] = b.x; dst[3] = b.y; dst[4] = c.x; dst[5] = c.y; dst[6] = d.x; dst[7] = d.y;
}

// CONV_BATCH rows starting at ``row`` (rows outside [0, C) read as zero); the loads carry no dependence on one
// another, so they are all in flight before the first use.
__device__ __forceinline__ void conv_load_rows(const bf16* __restrict__ col, int row, int C, int D, uint4 (&raw)[CONV_BATCH]) {
#pragma unroll
  for (int i = 0; i < CONV_BATCH; ++i) {
    const int c = row + i;
    raw[i] = (c >= 0 && c < C) ? __ldg(reinterpret_cast<const uint4*>(col + static_cast<int64_t>(c) * D)) : make_uint4(0, 0, 0, 0);
  }
}

template <int K>
__device__ __forceinline__ void conv_preload(const bf16* __restrict__ col, int row, int C, int D, float (&win)[K][8]) {
#pragma unroll
  for (int j = 0; j < K - 1; ++j) {
    const int c = row + j;
    const uint4 raw = (c >= 0 && c < C) ? __ldg(reinterpret_cast<const uint4*>(col + static_cast<int64_t>(c) * D)) : make_uint4(0, 0, 0, 0);
    conv_unpack(raw, win[j]);
  }
}

template <int K>
__device__ __forceinline__ void conv_shift(float (&win)[K][8]) {
#pragma unroll
  for (int j = 0; j < K - 1; ++j)
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) win[j][ch] = win[j + 1][ch];
}

template <int K>
__global__ void __launch_bounds__(128) dwconv_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                         bf16* __restrict__ y, int C, int D, int left) {
  const int cv = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (cv >= D) return;
  const int c0 = blockIdx.y * CONV_ROWS;
  const int64_t base = static_cast<int64_t>(blockIdx.z) * C * D + cv;
  float wv[8][K];
#pragma unroll
  for (int ch = 0; ch < 8; ++ch)
#pragma unroll
    for (int j = 0; j < K; ++j) wv[ch][j] = __bfloat162float(w[(cv + ch) * K + j]);
  float win[K][8];
  conv_preload<K>(x + base, c0 - left, C, D, win);          // rows c0-left .. c0-left+K-2
  for (int r0 = 0; r0 < CONV_ROWS && c0 + r0 < C; r0 += CONV_BATCH) {
    uint4 raw[CONV_BATCH];
    conv_load_rows(x + base, c0 + r0 - left + K - 1, C, D, raw);
#pragma unroll
    for (int i = 0; i < CONV_BATCH; ++i) {
      const int c = c0 + r0 + i;
      conv_unpack(raw[i], win[K - 1]);
      float o[8];
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < K; ++j) acc += wv[ch][j] * win[j][ch];
        o[ch] = acc;
      }
      if (c < C) store8(y + base + static_cast<int64_t>(c) * D, o);
      conv_shift<K>(win);
    }
  }
}

// Backward: dx[c] = sum_j w[d][j] * dy[c + left - j];  dw[d][j] = sum_{n,c} dy[c] * x[c - left + j].
// dw partial sums go to dw_partial[blockIdx.z * gridDim.y + blockIdx.y][D][K].
template <int K>
__global__ void __launch_bounds__(128) dwconv_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                                         const bf16* __restrict__ w, bf16* __restrict__ dx,
                                                         float* __restrict__ dw_partial, int C, int D, int left) {
  const int cv = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (cv >= D) return;
  const int c0 = blockIdx.y * CONV_ROWS;
  const int64_t base = static_cast<int64_t>(blockIdx.z) * C * D + cv;
  // dx pass: window over dy rows c+left-(K-1) .. c+left
  {
    float wv[8][K];
#pragma unroll
    for (int ch = 0; ch < 8; ++ch)
#pragma unroll
      for (int j = 0; j < K; ++j) wv[ch][j] = __bfloat162float(w[(cv + ch) * K + j]);
    float win[K][8];
    conv_preload<K>(dy + base, c0 + left - (K - 1), C, D, win);
    for (int r0 = 0; r0 < CONV_ROWS && c0 + r0 < C; r0 += CONV_BATCH) {
      uint4 raw[CONV_BATCH];
      conv_load_rows(dy + base, c0 + r0 + left, C, D, raw);
#pragma unroll
      for (int i = 0; i < CONV_BATCH; ++i) {
        const int c = c0 + r0 + i;
        conv_unpack(raw[i], win[K - 1]);
        float o[8];
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          float acc = 0.f;
          // win[m] holds dy[c + left - (K-1) + m]; it pairs with tap j = K-1-m
#pragma unroll
          for (int m = 0; m < K; ++m) acc += wv[ch][K - 1 - m] * win[m][ch];
          o[ch] = acc;
        }
        if (c < C) store8(dx + base + static_cast<int64_t>(c) * D, o);
        conv_shift<K>(win);
      }
    }
  }
  // dw pass: for output position c, x window rows c-left .. c-left+K-1 (rows of dy past C read as zero: no term)
  if (dw_partial != nullptr) {
    float dwacc[8][K];
#pragma unroll
    for (int ch = 0; ch < 8; ++ch)
#pragma unroll
      for (int j = 0; j < K; ++j) dwacc[ch][j] = 0.f;
    float win[K][8];
    conv_preload<K>(x + base, c0 - left, C, D, win);
    for (int r0 = 0; r0 < CONV_ROWS && c0 + r0 < C; r0 += CONV_BATCH) {
      uint4 raw[CONV_BATCH], graw[CONV_BATCH];
      conv_load_rows(x + base, c0 + r0 - left + K - 1, C, D, raw);
      conv_load_rows(dy + base, c0 + r0, C, D, graw);
#pragma unroll
      for (int i = 0; i < CONV_BATCH; ++i) {
        conv_unpack(raw[i], win[K - 1]);
        float g[8];
        conv_unpack(graw[i], g);
#pragma unroll
        for (int ch = 0; ch < 8; ++ch)
#pragma unroll
          for (int j = 0; j < K; ++j) dwacc[ch][j] += g[ch] * win[j][ch];
        conv_shift<K>(win);
      }
    }
    float* out = dw_partial + (static_cast<int64_t>(blockIdx.z) * gridDim.y + blockIdx.y) * D * K;
#pragma unroll
    for (int ch = 0; ch < 8; ++ch)
#pragma unroll
      for (int j = 0; j < K; ++j) out[(cv + ch) * K + j] = dwacc[ch][j];
  }
}

}  // namespace ttcd

using namespace ttcd;

TTCD_EXPORT int ttcd_swiglu_fwd(const void* gate, const void* up, void* z, long long rows, int d, long long ldg,
                                long long ldu, long long ldz, void* stream_ptr) {
  if (d % 8 != 0 || ldg % 8 != 0 || ldu % 8 != 0 || ldz % 8 != 0 || rows <= 0) return TTCD_ERR_ARG;
  const long long total = rows * (d / 8);
  const unsigned grid = static_cast<unsigned>(std::min<long long>((total + 255) / 256, 148LL * 32));
  swiglu_fwd_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      static_cast<const bf16*>(gate), static_cast<const bf16*>(up), static_cast<bf16*>(z), rows, d, ldg, ldu, ldz);
  return static_cast<int>(cudaGetLastError());
}

TTCD_EXPORT int ttcd_swiglu_bwd(const void* dz, const void* gate, const void* up, void* dgate, void* dup,
                                long long rows, int d, long long lddz, long long ldg, long long ldu, long long lddg,
                                long long lddu, void* stream_ptr) {
  if (d % 8 != 0 || ldg % 8 != 0 || ldu % 8 != 0 || lddz % 8 != 0 || lddg % 8 != 0 || lddu % 8 != 0 || rows <= 0)
    return TTCD_ERR_ARG;
  const long long total = rows * (d / 8);
  const unsigned grid = static_cast<unsigned>(std::min<long long>((total + 255) / 256, 148LL * 32));
  swiglu_bwd_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      static_cast<const bf16*>(dz), static_cast<const bf16*>(gate), static_cast<const bf16*>(up),
      static_cast<bf16*>(dgate), static_cast<bf16*>(dup), rows, d, lddz, ldg, ldu, lddg, lddu);
  return static_cast<int>(cudaGetLastError());
}

static int conv_left(int K, int causal) { return causal ? K - 1 : K / 2; }

// x, y: [n_chunks][C][D] contiguous bf16; w: [D][K] bf16.  K in 2..8.
TTCD_EXPORT int ttcd_dwconv_fwd(const void* x, const void* w, void* y, long long n_chunks, int C, int D, int K,
                                int causal, void* stream_ptr) {
  if (D % 8 != 0 || K < 2 || K > CONV_MAXK || n_chunks <= 0 || n_chunks > 65535) return TTCD_ERR_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream_ptr);
  dim3 grid((D / 8 + 127) / 128, (C + CONV_ROWS - 1) / CONV_ROWS, static_cast<unsigned>(n_chunks));
  const int left = conv_left(K, causal);
#define LAUNCH(KK) dwconv_fwd_kernel<KK><<<grid, 128, 0, st>>>(static_cast<const bf16*>(x), static_cast<const bf16*>(w), static_cast<bf16*>(y), C, D, left)
  switch (K) {
    case 2: LAUNCH(2); break; case 3: LAUNCH(3); break; case 4: LAUNCH(4); break; case 5: LAUNCH(5); break;
    case 6: LAUNCH(6); break; case 7: LAUNCH(7); break; default: LAUNCH(8); break;
  }
#undef LAUNCH
  return static_cast<int>(cudaGetLastError());
}

// dw_partial: fp32 [n_chunks * ceil(C/64)][D][K] (summed by the caller) or null to skip dw.
TTCD_EXPORT int ttcd_dwconv_bwd(const void* dy, const void* x, const void* w, void* dx, float* dw_partial,
                                long long n_chunks, int C, int D, int K, int causal, void* stream_ptr) {
  if (D % 8 != 0 || K < 2 || K > CONV_MAXK || n_chunks <= 0 || n_chunks > 65535) return TTCD_ERR_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream_ptr);
  dim3 grid((D / 8 + 127) / 128, (C + CONV_ROWS - 1) / CONV_ROWS, static_cast<unsigned>(n_chunks));
  const int left = conv_left(K, causal);
#define LAUNCH(KK) dwconv_bwd_kernel<KK><<<grid, 128, 0, st>>>(static_cast<const bf16*>(dy), static_cast<const bf16*>(x), static_cast<const bf16*>(w), static_cast<bf16*>(dx), dw_partial, C, D, left)
  switch (K) {
    case 2: LAUNCH(2); break; case 3: LAUNCH(3); break; case 4: LAUNCH(4); break; case 5: LAUNCH(5); break;
    case 6: LAUNCH(6); break; case 7: LAUNCH(7); break; default: LAUNCH(8); break;
  }
#undef LAUNCH
  return static_cast<int>(cudaGetLastError());
}

TTCD_EXPORT int ttcd_dwconv_rows_per_block() { return CONV_ROWS; }
