// Row-wise cross-entropy with in-place gradient, LSE merge of two partial attention results, fused
// AdamW over flat shards (with device-side clip coefficient and skip flag, so no host sync) and the
// squared-norm reduction used for gradient clipping.  Replaces
// fla/modules/fused_linear_cross_entropy.py:33-190, profiling/lse_dual_attn.py:106-160 and
// torch._fused_adamw_ / clip_grad_norm_ on the reference's training path.
#include "common.cuh"

#include <algorithm>

namespace ttcd {

__device__ __forceinline__ float block_reduce(float v, float* scratch, bool is_max) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  v = is_max ? warp_max(v) : warp_sum(v);
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < warps ? scratch[lane] : (is_max ? -INFINITY : 0.f);
    t = is_max ? warp_max(t) : warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  const float out = scratch[32];
  __syncthreads();
  return out;
}

// One block per row of logits [rows][ld] (bf16).  With eps = label smoothing and zeta = the weight of lse^2:
//   loss_row[row] = lse - (1 - eps) logit[label] - eps mean(logits) + zeta lse^2      (0 when the label is ignored)
// and, when write_grad, the row is overwritten with its gradient times (*grad_scale):
//   softmax (1 + 2 zeta lse) - (1 - eps) onehot - eps / V
// l2_factor > 0 adds the l2-warp term on EVERY row (ignored ones too, as the reference's fused linear-CE does,
// fla/modules/fused_linear_cross_entropy.py:250-283): max logit * l2_factor * (*grad_scale) at the arg-max column
// (the lowest column on ties); the loss value is unchanged by it.
__global__ void __launch_bounds__(1024) ce_rows_kernel(bf16* __restrict__ logits, const int64_t* __restrict__ labels,
                                                       float* __restrict__ loss_row, float* __restrict__ lse_row,
                                                       const float* __restrict__ grad_scale, int V, int64_t ld,
                                                       int ignore_index, int write_grad, float eps, float zeta,
                                                       float l2_factor, const float2* __restrict__ lse_part, int n_parts) {
  __shared__ float scratch[33];
  const int64_t row = blockIdx.x;
  bf16* lr = logits + row * ld;
  const int64_t label = labels[row];
  const int nvec = V / 8;
  float m = -INFINITY, s = 0.f, sumx = 0.f;
  int arg = 0;
  // the producing GEMM left (max, sum) per column tile of this row: merge them instead of reading the row
  const bool have_parts = lse_part != nullptr;
  if (have_parts) {
    for (int i = threadIdx.x; i < n_parts; i += blockDim.x) {
      const float2 t = lse_part[row * n_parts + i];
      if (t.x > m) {
        s *= __expf(m - t.x);
        m = t.x;
      }
      if (t.x != -INFINITY) s += t.y * __expf(t.x - m);
    }
  }
  for (int i = threadIdx.x; i < (have_parts ? 0 : nvec); i += blockDim.x) {
    const uint4 raw = *reinterpret_cast<const uint4*>(lr + i * 8);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    float f[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 t = unpack_bf16(w[k]);
      f[2 * k] = t.x;
      f[2 * k + 1] = t.y;
    }
    float lm = f[0];
    int la = 0;
#pragma unroll
    for (int k = 1; k < 8; ++k)
      if (f[k] > lm) { lm = f[k]; la = k; }
    if (lm > m) {
      s *= __expf(m - lm);
      m = lm;
      arg = i * 8 + la;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      s += __expf(f[k] - m);
      sumx += f[k];
    }
  }
  for (int i = nvec * 8 + threadIdx.x; i < (have_parts ? 0 : V); i += blockDim.x) {
    const float f = __bfloat162float(lr[i]);
    if (f > m) {
      s *= __expf(m - f);
      m = f;
      arg = i;
    }
    s += __expf(f - m);
    sumx += f;
  }
  const float gm = block_reduce(m, scratch, true);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  const float gs = block_reduce(s, scratch, false);
  const float lse = gm + __logf(gs);
  float mean_x = 0.f;
  if (eps != 0.f) mean_x = block_reduce(sumx, scratch, false) / static_cast<float>(V);
  int arg_col = -1;
  if (l2_factor != 0.f && write_grad)         // column indices are below 2^24: exact as floats
    arg_col = -static_cast<int>(block_reduce(m == gm ? -static_cast<float>(arg) : -INFINITY, scratch, true));
  const bool valid = label != ignore_index && label >= 0 && label < V;
  if (threadIdx.x == 0) {
    loss_row[row] = valid ? lse - (1.f - eps) * __bfloat162float(lr[label]) - eps * mean_x + zeta * lse * lse : 0.f;
    if (lse_row != nullptr) lse_row[row] = lse;
  }
  if (!write_grad) return;
  const float gsc = *grad_scale;
  const float scale = valid ? gsc : 0.f;
  const float pw = 1.f + 2.f * zeta * lse, hot = 1.f - eps, flat = eps / static_cast<float>(V);
  const float warp_term = gm * l2_factor * gsc;
  __syncthreads();  // label logit read above before the row is overwritten
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    uint4 raw = *reinterpret_cast<const uint4*>(lr + i * 8);
    uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 t = unpack_bf16(w[k]);
      const int c = i * 8 + 2 * k;
      t.x = (__expf(t.x - lse) * pw - (c == label ? hot : 0.f) - flat) * scale + (c == arg_col ? warp_term : 0.f);
      t.y = (__expf(t.y - lse) * pw - (c + 1 == label ? hot : 0.f) - flat) * scale + (c + 1 == arg_col ? warp_term : 0.f);
      w[k] = pack_bf16(t.x, t.y);
    }
    raw.x = w[0]; raw.y = w[1]; raw.z = w[2]; raw.w = w[3];
    *reinterpret_cast<uint4*>(lr + i * 8) = raw;
  }
  for (int i = nvec * 8 + threadIdx.x; i < V; i += blockDim.x) {
    const float f = __bfloat162float(lr[i]);
    lr[i] = __float2bfloat16((__expf(f - lse) * pw - (i == label ? hot : 0.f) - flat) * scale + (i == arg_col ? warp_term : 0.f));
  }
}

// out = merge of two partial softmax results over disjoint key sets.
// o_*: [rows][H][D] bf16, lse_*: [B][H][T] fp32 with rows = B*T; one warp per (row, head).
__global__ void __launch_bounds__(256) lse_merge_kernel(const bf16* __restrict__ oa, const float* __restrict__ la,
                                                        const bf16* __restrict__ ob, const float* __restrict__ lb,
                                                        bf16* __restrict__ out, float* __restrict__ lse_out,
                                                        int64_t B, int T, int H, int D) {
  const int lane = threadIdx.x & 31;
  const int64_t item = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= B * T * H) return;
  const int h = static_cast<int>(item % H);
  const int64_t bt = item / H;
  const int64_t b = bt / T, t = bt % T;
  const int64_t li = (b * H + h) * T + t;
  const float a = la[li], c = lb[li];
  float m = fmaxf(a, c);
  if (m == -INFINITY) m = 0.f;
  const float wa = __expf(a - m), wb = __expf(c - m);
  const float inv = 1.f / fmaxf(wa + wb, 1e-38f);
  if (lane == 0 && lse_out != nullptr) lse_out[li] = m + __logf(fmaxf(wa + wb, 1e-38f));
  const int64_t base = item * D;
  for (int d = lane * 2; d < D; d += 64) {
    const float2 x = unpack_bf16(*reinterpret_cast<const uint32_t*>(oa + base + d));
    const float2 y = unpack_bf16(*reinterpret_cast<const uint32_t*>(ob + base + d));
    *reinterpret_cast<uint32_t*>(out + base + d) =
        pack_bf16((x.x * wa + y.x * wb) * inv, (x.y * wa + y.y * wb) * inv);
  }
}

// Fused AdamW on a flat fp32 master shard.  grad is bf16 or fp32.  coef (device scalar, may be
// null) multiplies the gradient (clip); skip (device int, may be null) != 0 leaves everything as is.
template <typename GradT>
__global__ void __launch_bounds__(256) adamw_kernel(float* __restrict__ p, const GradT* __restrict__ g,
                                                    float* __restrict__ m, float* __restrict__ v,
                                                    bf16* __restrict__ p_bf16, int64_t n, float lr, float beta1,
                                                    float beta2, float eps, float wd, float bc1, float bc2_sqrt,
                                                    const float* __restrict__ coef, const int* __restrict__ skip) {
  if (skip != nullptr && *skip != 0) return;
  const float c = coef != nullptr ? *coef : 1.f;
  const float step_size = lr / bc1;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float gi;
    if constexpr (sizeof(GradT) == 2) gi = __bfloat162float(g[i]) * c;
    else gi = g[i] * c;
    float pi = p[i] * (1.f - lr * wd);
    const float mi = beta1 * m[i] + (1.f - beta1) * gi;
    const float vi = beta2 * v[i] + (1.f - beta2) * gi * gi;
    pi -= step_size * mi / (sqrtf(vi) / bc2_sqrt + eps);
    p[i] = pi;
    m[i] = mi;
    v[i] = vi;
    if (p_bf16 != nullptr) p_bf16[i] = __float2bfloat16(pi);
  }
}

// out[0] += sum(x^2) (atomicAdd of per-block partials; zero `out` beforehand).
template <typename T>
__global__ void __launch_bounds__(256) sumsq_kernel(const T* __restrict__ x, int64_t n, float* __restrict__ out) {
  __shared__ float scratch[33];
  float acc = 0.f;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float f;
    if constexpr (sizeof(T) == 2) f = __bfloat162float(x[i]);
    else f = x[i];
    acc += f * f;
  }
  acc = block_reduce(acc, scratch, false);
  if (threadIdx.x == 0) atomicAdd(out, acc);
}

// y[i] = x[i] * scale (+ y[i] when accumulate): bucket cast/scale used by the gradient path.
template <typename TI, typename TO>
__global__ void __launch_bounds__(256) cast_scale_kernel(const TI* __restrict__ x, TO* __restrict__ y, int64_t n,
                                                         float scale, int accumulate) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float f;
    if constexpr (sizeof(TI) == 2) f = __bfloat162float(x[i]);
    else f = x[i];
    f *= scale;
    if constexpr (sizeof(TO) == 2) {
      if (accumulate) f += __bfloat162float(y[i]);
      y[i] = __float2bfloat16(f);
    } else {
      if (accumulate) f += y[i];
      y[i] = f;
    }
  }
}

}  // namespace ttcd

using namespace ttcd;

static unsigned flat_grid(long long n) {
  return static_cast<unsigned>(std::max<long long>(1, std::min<long long>((n + 255) / 256, 148LL * 16)));
}

// logits: [rows][ld] bf16 (modified in place when write_grad); labels: int64 [rows].
// lse_part (may be null): fp32 [rows][n_parts][2] left by ttcd_gemm_bf16_lse for these logits; the first pass over the
// row is then skipped (not with label smoothing or the l2-warp term, which need the row's mean / arg-max).
TTCD_EXPORT int ttcd_ce_rows(void* logits, const long long* labels, float* loss_row, float* lse_row,
                             const float* grad_scale, long long rows, int V, long long ld, int ignore_index,
                             int write_grad, float label_smoothing, float lse_square_scale, float l2_factor,
                             const float* lse_part, int n_parts, void* stream_ptr) {
  if (rows <= 0 || V <= 0 || ld % 8 != 0 || (write_grad && grad_scale == nullptr)) return TTCD_ERR_ARG;
  if (label_smoothing < 0.f || label_smoothing >= 1.f || V >= (1 << 24)) return TTCD_ERR_ARG;
  if (lse_part != nullptr && (n_parts <= 0 || label_smoothing != 0.f || l2_factor != 0.f)) return TTCD_ERR_ARG;
  ce_rows_kernel<<<static_cast<unsigned>(rows), 1024, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      static_cast<bf16*>(logits), reinterpret_cast<const int64_t*>(labels), loss_row, lse_row, grad_scale, V, ld,
      ignore_index, write_grad, label_smoothing, lse_square_scale, l2_factor, reinterpret_cast<const float2*>(lse_part),
      n_parts);
  return static_cast<int>(cudaGetLastError());
}

TTCD_EXPORT int ttcd_lse_merge(const void* oa, const float* la, const void* ob, const float* lb, void* out,
                               float* lse_out, long long B, int T, int H, int D, void* stream_ptr) {
  if (D % 2 != 0 || B <= 0) return TTCD_ERR_ARG;
  const long long items = B * T * H;
  lse_merge_kernel<<<static_cast<unsigned>((items + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      static_cast<const bf16*>(oa), la, static_cast<const bf16*>(ob), lb, static_cast<bf16*>(out), lse_out, B, T, H, D);
  return static_cast<int>(cudaGetLastError());
}

TTCD_EXPORT int ttcd_adamw(float* p, const void* g, int grad_is_bf16, float* m, float* v, void* p_bf16, long long n,
                           float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2_sqrt,
                           const float* coef, const int* skip, void* stream_ptr) {
  if (n <= 0) return TTCD_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream_ptr);
  if (grad_is_bf16)
    adamw_kernel<bf16><<<flat_grid(n), 256, 0, st>>>(p, static_cast<const bf16*>(g), m, v, static_cast<bf16*>(p_bf16), n,
                                                     lr, beta1, beta2, eps, wd, bc1, bc2_sqrt, coef, skip);
  else
    adamw_kernel<float><<<flat_grid(n), 256, 0, st>>>(p, static_cast<const float*>(g), m, v, static_cast<bf16*>(p_bf16),
                                                      n, lr, beta1, beta2, eps, wd, bc1, bc2_sqrt, coef, skip);
  return static_cast<int>(cudaGetLastError());
}

TTCD_EXPORT int ttcd_sumsq(const void* x, int is_bf16, long long n, float* out, void* stream_ptr) {
  if (n <= 0) return TTCD_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream_ptr);
  if (is_bf16) sumsq_kernel<bf16><<<flat_grid(n), 256, 0, st>>>(static_cast<const bf16*>(x), n, out);
  else sumsq_kernel<float><<<flat_grid(n), 256, 0, st>>>(static_cast<const float*>(x), n, out);
  return static_cast<int>(cudaGetLastError());
}

// kind: 0 bf16->fp32, 1 fp32->bf16, 2 fp32->fp32, 3 bf16->bf16
TTCD_EXPORT int ttcd_cast_scale(const void* x, void* y, long long n, float scale, int kind, int accumulate,
                                void* stream_ptr) {
  if (n <= 0) return TTCD_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream_ptr);
  const unsigned grid = flat_grid(n);
  switch (kind) {
    case 0: cast_scale_kernel<bf16, float><<<grid, 256, 0, st>>>(static_cast<const bf16*>(x), static_cast<float*>(y), n, scale, accumulate); break;
    case 1: cast_scale_kernel<float, bf16><<<grid, 256, 0, st>>>(static_cast<const float*>(x), static_cast<bf16*>(y), n, scale, accumulate); break;
    case 2: cast_scale_kernel<float, float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), static_cast<float*>(y), n, scale, accumulate); break;
    case 3: cast_scale_kernel<bf16, bf16><<<grid, 256, 0, st>>>(static_cast<const bf16*>(x), static_cast<bf16*>(y), n, scale, accumulate); break;
    default: return TTCD_ERR_ARG;
  }
  return static_cast<int>(cudaGetLastError());
}
