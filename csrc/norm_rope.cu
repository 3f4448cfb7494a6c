// Fused add+RMSNorm (forward/backward) and per-head q/k RMSNorm fused with NeoX rotary embedding
// (forward/backward) for sm_100a: 16-byte vector accesses, fp32 math on bf16 storage, one warp per
// row (or per head).  They replace the Triton kernels of the reference
// (fla/modules/layernorm.py:254-526, fla/modules/rotary.py:35-135).

#include "common.cuh"

#include <algorithm>

namespace ttcd {

struct alignas(16) Vec8 {
  uint4 raw;
  __device__ __forceinline__ void load(const bf16* p) { raw = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ void store(bf16* p) const { *reinterpret_cast<uint4*>(p) = raw; }
  __device__ __forceinline__ void to_float(float (&f)[8]) const {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 t = unpack_bf16(w[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
  __device__ __forceinline__ void from_float(const float (&f)[8]) {
    raw.x = pack_bf16(f[0], f[1]);
    raw.y = pack_bf16(f[2], f[3]);
    raw.z = pack_bf16(f[4], f[5]);
    raw.w = pack_bf16(f[6], f[7]);
  }
};

// ------------------------------------------------------------------------------------------------
// RMSNorm forward: s = x (+ res); y = s * rsqrt(mean(s^2) + eps) * w.  One warp per row.
// ------------------------------------------------------------------------------------------------
template <int CHUNKS>
__global__ void __launch_bounds__(256) rmsnorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ res,
                                                          const bf16* __restrict__ w, bf16* __restrict__ y,
                                                          bf16* __restrict__ sum_out, float* __restrict__ rstd_out,
                                                          int64_t rows, int D, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const bf16* xr = x + row * D;
  float v[CHUNKS][8];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int col = (c * 32 + lane) * 8;
    if (col < D) {
      Vec8 a;
      a.load(xr + col);
      a.to_float(v[c]);
      if (res != nullptr) {
        Vec8 b;
        float r[8];
        b.load(res + row * D + col);
        b.to_float(r);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[c][i] += r[i];
      }
      if (sum_out != nullptr) {
        Vec8 o;
        o.from_float(v[c]);
        o.store(sum_out + row * D + col);
        // statistics use the stored (rounded) residual so forward and backward see the same input
        o.to_float(v[c]);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += v[c][i] * v[c][i];
    }
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / D + eps);
  if (lane == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int col = (c * 32 + lane) * 8;
    if (col < D) {
      float wv[8];
      if (w != nullptr) {
        Vec8 ww;
        ww.load(w + col);
        ww.to_float(wv);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) wv[i] = 1.f;
      }
      float o[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = v[c][i] * rstd * wv[i];
      Vec8 ov;
      ov.from_float(o);
      ov.store(y + row * D + col);
    }
  }
}

// RMSNorm backward.  s: the (summed) pre-norm input saved by the forward.  dx = dnorm(dy) (+ dres).
// dw partial sums are written per block to dw_partial[gridDim.x][D].
template <int CHUNKS>
__global__ void __launch_bounds__(256, (CHUNKS <= 4 ? 2 : 1)) rmsnorm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ s,
                                                          const bf16* __restrict__ w, const float* __restrict__ rstd_in,
                                                          const bf16* __restrict__ dres, bf16* __restrict__ dx,
                                                          float* __restrict__ dw_partial, int64_t rows, int D) {
  extern __shared__ float red[];  // [warps][D]
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int warps = blockDim.x >> 5;
  float wv[CHUNKS][8];
  float dwacc[CHUNKS][8];
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int col = (c * 32 + lane) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) { dwacc[c][i] = 0.f; wv[c][i] = 1.f; }
    if (col < D && w != nullptr) {
      Vec8 ww;
      ww.load(w + col);
      ww.to_float(wv[c]);
    }
  }
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * warps + warp; row < rows;
       row += static_cast<int64_t>(gridDim.x) * warps) {
    const float rstd = rstd_in[row];
    float g[CHUNKS][8], xh[CHUNKS][8];
    float dot = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int col = (c * 32 + lane) * 8;
      if (col < D) {
        Vec8 a, b;
        a.load(dy + row * D + col);
        b.load(s + row * D + col);
        a.to_float(g[c]);
        b.to_float(xh[c]);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xh[c][i] *= rstd;
          dwacc[c][i] += g[c][i] * xh[c][i];
          g[c][i] *= wv[c][i];
          dot += g[c][i] * xh[c][i];
        }
      }
    }
    dot = warp_sum(dot) / D;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int col = (c * 32 + lane) * 8;
      if (col < D) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = rstd * (g[c][i] - xh[c][i] * dot);
        if (dres != nullptr) {
          Vec8 r;
          float rf[8];
          r.load(dres + row * D + col);
          r.to_float(rf);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += rf[i];
        }
        Vec8 ov;
        ov.from_float(o);
        ov.store(dx + row * D + col);
      }
    }
  }
  if (dw_partial == nullptr) return;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int col = (c * 32 + lane) * 8;
    if (col < D) {
#pragma unroll
      for (int i = 0; i < 8; ++i) red[warp * D + col + i] = dwacc[c][i];
    }
  }
  __syncthreads();
  for (int col = threadIdx.x; col < D; col += blockDim.x) {
    float acc = 0.f;
    for (int wi = 0; wi < warps; ++wi) acc += red[wi * D + col];
    dw_partial[static_cast<int64_t>(blockIdx.x) * D + col] = acc;
  }
}

// ------------------------------------------------------------------------------------------------
// Wide rows (D > 2048): the row no longer fits in a warp's registers, so each pass streams it (the second
// pass hits L1 / L2).  One warp per row, same math as the kernels above.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) rmsnorm_fwd_wide_kernel(const bf16* __restrict__ x, const bf16* __restrict__ res,
                                                               const bf16* __restrict__ w, bf16* __restrict__ y,
                                                               bf16* __restrict__ sum_out, float* __restrict__ rstd_out,
                                                               int64_t rows, int D, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  auto load_sum = [&](int col, float (&v)[8]) {
    Vec8 a;
    a.load(x + row * D + col);
    a.to_float(v);
    if (res != nullptr) {
      Vec8 b;
      float r[8];
      b.load(res + row * D + col);
      b.to_float(r);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] += r[i];
    }
    if (sum_out != nullptr) {      // statistics use the stored (rounded) residual, as the backward will
      Vec8 o;
      o.from_float(v);
      o.to_float(v);
    }
  };
  float ss = 0.f;
  for (int col = lane * 8; col < D; col += 256) {
    float v[8];
    load_sum(col, v);
    if (sum_out != nullptr) {
      Vec8 o;
      o.from_float(v);
      o.store(sum_out + row * D + col);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / D + eps);
  if (lane == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
  for (int col = lane * 8; col < D; col += 256) {
    float v[8], wv[8];
    load_sum(col, v);
    if (w != nullptr) {
      Vec8 ww;
      ww.load(w + col);
      ww.to_float(wv);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) wv[i] = 1.f;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = v[i] * rstd * wv[i];
    Vec8 ov;
    ov.from_float(v);
    ov.store(y + row * D + col);
  }
}

// dw partial sums accumulate in shared memory ([warps][D], each lane owns its columns) instead of registers.
__global__ void __launch_bounds__(128) rmsnorm_bwd_wide_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ s,
                                                               const bf16* __restrict__ w, const float* __restrict__ rstd_in,
                                                               const bf16* __restrict__ dres, bf16* __restrict__ dx,
                                                               float* __restrict__ dw_partial, int64_t rows, int D) {
  extern __shared__ float red[];  // [warps][D]
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int warps = blockDim.x >> 5;
  float* mine = red + static_cast<size_t>(warp) * D;
  for (int col = lane; col < D; col += 32) mine[col] = 0.f;
  __syncwarp();
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * warps + warp; row < rows;
       row += static_cast<int64_t>(gridDim.x) * warps) {
    const float rstd = rstd_in[row];
    float dot = 0.f;
    for (int col = lane * 8; col < D; col += 256) {
      Vec8 a, b;
      float g[8], xh[8], wv[8];
      a.load(dy + row * D + col);
      b.load(s + row * D + col);
      a.to_float(g);
      b.to_float(xh);
      if (w != nullptr) {
        Vec8 ww;
        ww.load(w + col);
        ww.to_float(wv);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        xh[i] *= rstd;
        mine[col + i] += g[i] * xh[i];
        dot += (w != nullptr ? g[i] * wv[i] : g[i]) * xh[i];
      }
    }
    dot = warp_sum(dot) / D;
    for (int col = lane * 8; col < D; col += 256) {
      Vec8 a, b;
      float g[8], xh[8], wv[8], o[8];
      a.load(dy + row * D + col);
      b.load(s + row * D + col);
      a.to_float(g);
      b.to_float(xh);
      if (w != nullptr) {
        Vec8 ww;
        ww.load(w + col);
        ww.to_float(wv);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = rstd * ((w != nullptr ? g[i] * wv[i] : g[i]) - xh[i] * rstd * dot);
      if (dres != nullptr) {
        Vec8 r;
        float rf[8];
        r.load(dres + row * D + col);
        r.to_float(rf);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] += rf[i];
      }
      Vec8 ov;
      ov.from_float(o);
      ov.store(dx + row * D + col);
    }
  }
  if (dw_partial == nullptr) return;
  __syncthreads();
  for (int col = threadIdx.x; col < D; col += blockDim.x) {
    float acc = 0.f;
    for (int wi = 0; wi < warps; ++wi) acc += red[static_cast<size_t>(wi) * D + col];
    dw_partial[static_cast<int64_t>(blockIdx.x) * D + col] = acc;
  }
}

// ------------------------------------------------------------------------------------------------
// Two-input RMSNorm of the fast-weight blocks: x = norm(r + a_T), t = norm(r + a_S) with one weight, and the
// updated residual r + a_T.  The residual is read once; both sums are stored for the backward.
// (The reference calls its norm twice with the same residual: custom_models/ipttcd/modeling_ipttcdv9.py:700-708.)
// ------------------------------------------------------------------------------------------------
template <int CHUNKS>
__global__ void __launch_bounds__(256) rmsnorm_dual_fwd_kernel(const bf16* __restrict__ a_t, const bf16* __restrict__ a_s,
                                                               const bf16* __restrict__ res, const bf16* __restrict__ w,
                                                               bf16* __restrict__ y_t, bf16* __restrict__ y_s,
                                                               bf16* __restrict__ sum_t, bf16* __restrict__ sum_s,
                                                               float* __restrict__ rstd_t, float* __restrict__ rstd_s,
                                                               int64_t rows, int D, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  float vt[CHUNKS][8], vs[CHUNKS][8];
  float sst = 0.f, sss = 0.f;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int col = (c * 32 + lane) * 8;
    if (col < D) {
      Vec8 a, b, r;
      float rf[8];
      a.load(a_t + row * D + col);
      b.load(a_s + row * D + col);
      r.load(res + row * D + col);
      a.to_float(vt[c]);
      b.to_float(vs[c]);
      r.to_float(rf);
#pragma unroll
      for (int i = 0; i < 8; ++i) { vt[c][i] += rf[i]; vs[c][i] += rf[i]; }
      Vec8 ot, os;
      ot.from_float(vt[c]);
      os.from_float(vs[c]);
      ot.store(sum_t + row * D + col);
      os.store(sum_s + row * D + col);
      ot.to_float(vt[c]);      // statistics use the stored (rounded) sums so forward and backward see the same input
      os.to_float(vs[c]);
#pragma unroll
      for (int i = 0; i < 8; ++i) { sst += vt[c][i] * vt[c][i]; sss += vs[c][i] * vs[c][i]; }
    }
  }
  sst = warp_sum(sst);
  sss = warp_sum(sss);
  const float rt = rsqrtf(sst / D + eps), rs = rsqrtf(sss / D + eps);
  if (lane == 0) { rstd_t[row] = rt; rstd_s[row] = rs; }
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int col = (c * 32 + lane) * 8;
    if (col < D) {
      float wv[8];
      Vec8 ww;
      ww.load(w + col);
      ww.to_float(wv);
      float ot[8], os[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) { ot[i] = vt[c][i] * rt * wv[i]; os[i] = vs[c][i] * rs * wv[i]; }
      Vec8 o1, o2;
      o1.from_float(ot);
      o2.from_float(os);
      o1.store(y_t + row * D + col);
      o2.store(y_s + row * D + col);
    }
  }
}

// Backward of the two-input norm: d_at = dnorm_T(dy_t) + dres, d_as = dnorm_S(dy_s), d_res = d_at + d_as, and one
// set of dw partial sums for both streams.  The two streams go through the registers one after the other.
template <int CHUNKS>
__global__ void __launch_bounds__(256) rmsnorm_dual_bwd_kernel(const bf16* __restrict__ dy_t, const bf16* __restrict__ dy_s,
                                                               const bf16* __restrict__ s_t, const bf16* __restrict__ s_s,
                                                               const bf16* __restrict__ w, const float* __restrict__ rstd_t,
                                                               const float* __restrict__ rstd_s, const bf16* __restrict__ dres,
                                                               bf16* __restrict__ d_at, bf16* __restrict__ d_as,
                                                               bf16* __restrict__ d_res, float* __restrict__ dw_partial,
                                                               int64_t rows, int D) {
  extern __shared__ float red[];  // [warps][D]
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int warps = blockDim.x >> 5;
  float dwacc[CHUNKS][8];
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
    for (int i = 0; i < 8; ++i) dwacc[c][i] = 0.f;
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * warps + warp; row < rows;
       row += static_cast<int64_t>(gridDim.x) * warps) {
    uint4 first[CHUNKS];          // d_at of this row, kept packed until d_res is formed
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
      const bf16* dy = pass == 0 ? dy_t : dy_s;
      const bf16* s = pass == 0 ? s_t : s_s;
      const float rstd = (pass == 0 ? rstd_t : rstd_s)[row];
      float g[CHUNKS][8], xh[CHUNKS][8];
      float dot = 0.f;
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c) {
        const int col = (c * 32 + lane) * 8;
        if (col < D) {
          Vec8 a, b, ww;
          float wv[8];
          a.load(dy + row * D + col);
          b.load(s + row * D + col);
          ww.load(w + col);
          a.to_float(g[c]);
          b.to_float(xh[c]);
          ww.to_float(wv);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            xh[c][i] *= rstd;
            dwacc[c][i] += g[c][i] * xh[c][i];
            g[c][i] *= wv[i];
            dot += g[c][i] * xh[c][i];
          }
        }
      }
      dot = warp_sum(dot) / D;
#pragma unroll
      for (int c = 0; c < CHUNKS; ++c) {
        const int col = (c * 32 + lane) * 8;
        if (col < D) {
          float o[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = rstd * (g[c][i] - xh[c][i] * dot);
          Vec8 ov;
          if (pass == 0) {
            if (dres != nullptr) {
              Vec8 r;
              float rf[8];
              r.load(dres + row * D + col);
              r.to_float(rf);
#pragma unroll
              for (int i = 0; i < 8; ++i) o[i] += rf[i];
            }
            ov.from_float(o);
            ov.store(d_at + row * D + col);
            first[c] = ov.raw;
          } else {
            ov.from_float(o);
            ov.store(d_as + row * D + col);
            Vec8 f;
            float ff[8];
            f.raw = first[c];
            f.to_float(ff);
            ov.to_float(o);           // the sum of the two stored (rounded) gradients
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] += ff[i];
            ov.from_float(o);
            ov.store(d_res + row * D + col);
          }
        }
      }
    }
  }
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int col = (c * 32 + lane) * 8;
    if (col < D) {
#pragma unroll
      for (int i = 0; i < 8; ++i) red[warp * D + col + i] = dwacc[c][i];
    }
  }
  __syncthreads();
  for (int col = threadIdx.x; col < D; col += blockDim.x) {
    float acc = 0.f;
    for (int wi = 0; wi < warps; ++wi) acc += red[wi * D + col];
    dw_partial[static_cast<int64_t>(blockIdx.x) * D + col] = acc;
  }
}


// ------------------------------------------------------------------------------------------------
// Per-head RMSNorm (optional) + NeoX rotary.  One warp per (token, head); q heads then k heads.
// Lane l handles the rotary pairs (l + 32 i, l + 32 i + half).
// ------------------------------------------------------------------------------------------------
struct QKRopeParams {
  const bf16* q_in; const bf16* k_in; int64_t ldq, ldk;     // pre-norm inputs (strided rows)
  bf16* q_out; bf16* k_out; int64_t ldqo, ldko;              // forward: outputs; backward: dx
  const bf16* dq; const bf16* dk; int64_t lddq, lddk;        // backward: incoming gradients
  const bf16* qw; const bf16* kw;                             // norm weights [D] or null
  const bf16* cos; const bf16* sin;                           // [max_pos, half] or null
  const int* positions;                                       // [rows] or null
  int64_t rows; int T; int pos_offset; int H, HK, D, half; float eps;
  float* dqw_partial; float* dkw_partial;                     // backward: [gridDim.x][D] or null
};

template <int MAXP>
__global__ void __launch_bounds__(256) qk_norm_rope_fwd_kernel(const QKRopeParams p) {
  const int lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  const int heads = p.H + p.HK;
  const int64_t total = p.rows * heads;
  for (int64_t item = static_cast<int64_t>(blockIdx.x) * warps + (threadIdx.x >> 5); item < total;
       item += static_cast<int64_t>(gridDim.x) * warps) {
    const int64_t row = item / heads;
    const int h = static_cast<int>(item % heads);
    const bool is_q = h < p.H;
    const int hh = is_q ? h : h - p.H;
    const bf16* in = (is_q ? p.q_in + row * p.ldq : p.k_in + row * p.ldk) + hh * p.D;
    bf16* out = (is_q ? p.q_out + row * p.ldqo : p.k_out + row * p.ldko) + hh * p.D;
    const bf16* w = is_q ? p.qw : p.kw;
    const int pos = p.positions != nullptr ? p.positions[row] : static_cast<int>(row % p.T) + p.pos_offset;
    float x1[MAXP], x2[MAXP];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAXP; ++i) {
      const int idx = lane + 32 * i;
      x1[i] = x2[i] = 0.f;
      if (idx < p.half) {
        x1[i] = __bfloat162float(in[idx]);
        x2[i] = __bfloat162float(in[idx + p.half]);
        ss += x1[i] * x1[i] + x2[i] * x2[i];
      }
    }
    float rstd = 1.f;
    if (w != nullptr) rstd = rsqrtf(warp_sum(ss) / p.D + p.eps);
#pragma unroll
    for (int i = 0; i < MAXP; ++i) {
      const int idx = lane + 32 * i;
      if (idx < p.half) {
        float y1 = x1[i] * rstd, y2 = x2[i] * rstd;
        if (w != nullptr) {
          y1 *= __bfloat162float(w[idx]);
          y2 *= __bfloat162float(w[idx + p.half]);
        }
        float c = 1.f, s = 0.f;
        if (p.cos != nullptr) {
          c = __bfloat162float(p.cos[static_cast<int64_t>(pos) * p.half + idx]);
          s = __bfloat162float(p.sin[static_cast<int64_t>(pos) * p.half + idx]);
        }
        out[idx] = __float2bfloat16(y1 * c - y2 * s);
        out[idx + p.half] = __float2bfloat16(y1 * s + y2 * c);
      }
    }
  }
}

template <int MAXP>
__global__ void __launch_bounds__(256) qk_norm_rope_bwd_kernel(const QKRopeParams p) {
  __shared__ float red[2][8][256];  // [q|k][warp][D <= 256]
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int warps = blockDim.x >> 5;
  const int heads = p.H + p.HK;
  const int64_t total = p.rows * heads;
  float dwq1[MAXP], dwq2[MAXP], dwk1[MAXP], dwk2[MAXP];
#pragma unroll
  for (int i = 0; i < MAXP; ++i) dwq1[i] = dwq2[i] = dwk1[i] = dwk2[i] = 0.f;

  for (int64_t item = static_cast<int64_t>(blockIdx.x) * warps + warp; item < total;
       item += static_cast<int64_t>(gridDim.x) * warps) {
    const int64_t row = item / heads;
    const int h = static_cast<int>(item % heads);
    const bool is_q = h < p.H;
    const int hh = is_q ? h : h - p.H;
    const bf16* in = (is_q ? p.q_in + row * p.ldq : p.k_in + row * p.ldk) + hh * p.D;
    const bf16* gin = (is_q ? p.dq + row * p.lddq : p.dk + row * p.lddk) + hh * p.D;
    bf16* out = (is_q ? p.q_out + row * p.ldqo : p.k_out + row * p.ldko) + hh * p.D;
    const bf16* w = is_q ? p.qw : p.kw;
    const int pos = p.positions != nullptr ? p.positions[row] : static_cast<int>(row % p.T) + p.pos_offset;
    float x1[MAXP], x2[MAXP], g1[MAXP], g2[MAXP];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAXP; ++i) {
      const int idx = lane + 32 * i;
      x1[i] = x2[i] = g1[i] = g2[i] = 0.f;
      if (idx < p.half) {
        x1[i] = __bfloat162float(in[idx]);
        x2[i] = __bfloat162float(in[idx + p.half]);
        ss += x1[i] * x1[i] + x2[i] * x2[i];
        const float d1 = __bfloat162float(gin[idx]);
        const float d2 = __bfloat162float(gin[idx + p.half]);
        float c = 1.f, s = 0.f;
        if (p.cos != nullptr) {
          c = __bfloat162float(p.cos[static_cast<int64_t>(pos) * p.half + idx]);
          s = __bfloat162float(p.sin[static_cast<int64_t>(pos) * p.half + idx]);
        }
        g1[i] = d1 * c + d2 * s;   // transpose of the rotation
        g2[i] = -d1 * s + d2 * c;
      }
    }
    if (w == nullptr) {
#pragma unroll
      for (int i = 0; i < MAXP; ++i) {
        const int idx = lane + 32 * i;
        if (idx < p.half) {
          out[idx] = __float2bfloat16(g1[i]);
          out[idx + p.half] = __float2bfloat16(g2[i]);
        }
      }
      continue;
    }
    const float rstd = rsqrtf(warp_sum(ss) / p.D + p.eps);
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < MAXP; ++i) {
      const int idx = lane + 32 * i;
      if (idx < p.half) {
        x1[i] *= rstd;
        x2[i] *= rstd;
        if (is_q) { dwq1[i] += g1[i] * x1[i]; dwq2[i] += g2[i] * x2[i]; }
        else      { dwk1[i] += g1[i] * x1[i]; dwk2[i] += g2[i] * x2[i]; }
        g1[i] *= __bfloat162float(w[idx]);
        g2[i] *= __bfloat162float(w[idx + p.half]);
        dot += g1[i] * x1[i] + g2[i] * x2[i];
      }
    }
    dot = warp_sum(dot) / p.D;
#pragma unroll
    for (int i = 0; i < MAXP; ++i) {
      const int idx = lane + 32 * i;
      if (idx < p.half) {
        out[idx] = __float2bfloat16(rstd * (g1[i] - x1[i] * dot));
        out[idx + p.half] = __float2bfloat16(rstd * (g2[i] - x2[i] * dot));
      }
    }
  }
  if (p.dqw_partial == nullptr) return;
#pragma unroll
  for (int i = 0; i < MAXP; ++i) {
    const int idx = lane + 32 * i;
    if (idx < p.half) {
      red[0][warp][idx] = dwq1[i];
      red[0][warp][idx + p.half] = dwq2[i];
      red[1][warp][idx] = dwk1[i];
      red[1][warp][idx + p.half] = dwk2[i];
    }
  }
  __syncthreads();
  for (int col = threadIdx.x; col < 2 * p.half; col += blockDim.x) {
    float aq = 0.f, ak = 0.f;
    for (int wi = 0; wi < warps; ++wi) { aq += red[0][wi][col]; ak += red[1][wi][col]; }
    p.dqw_partial[static_cast<int64_t>(blockIdx.x) * p.D + col] = aq;
    p.dkw_partial[static_cast<int64_t>(blockIdx.x) * p.D + col] = ak;
  }
}


// ------------------------------------------------------------------------------------------------
// Vectorised variants for the common layout (rotary over the whole head: 2 * half == D, half % 8 == 0):
// LPH lanes share one (token, head); lane l owns elements [8l, 8l+8) of each half, so every access is a
// 16-byte vector and a warp works on 32 / LPH heads at once.  Same math as the scalar kernels above.
// ------------------------------------------------------------------------------------------------
template <int LPH>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = LPH / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ void ld8(const bf16* p, float (&f)[8]) {
  Vec8 v;
  v.load(p);
  v.to_float(f);
}
__device__ __forceinline__ void st8(bf16* p, const float (&f)[8]) {
  Vec8 v;
  v.from_float(f);
  v.store(p);
}

template <int LPH>
__global__ void __launch_bounds__(256) qk_norm_rope_fwd_vec_kernel(const QKRopeParams p) {
  constexpr int GPW = 32 / LPH;                         // (token, head) items per warp
  const int lane = threadIdx.x & 31, sub = lane % LPH, grp = lane / LPH;
  const int warps = blockDim.x >> 5;
  const int heads = p.H + p.HK;
  const int64_t total = p.rows * heads;
  const int64_t step = static_cast<int64_t>(gridDim.x) * warps * GPW;
  for (int64_t base = (static_cast<int64_t>(blockIdx.x) * warps + (threadIdx.x >> 5)) * GPW; base < total; base += step) {
    const int64_t item = base + grp;
    const bool live = item < total;
    const int64_t row = live ? item / heads : 0;
    const int h = live ? static_cast<int>(item % heads) : 0;
    const bool is_q = h < p.H;
    const int hh = is_q ? h : h - p.H;
    const bf16* in = (is_q ? p.q_in + row * p.ldq : p.k_in + row * p.ldk) + hh * p.D + sub * 8;
    bf16* out = (is_q ? p.q_out + row * p.ldqo : p.k_out + row * p.ldko) + hh * p.D + sub * 8;
    const bf16* w = is_q ? p.qw : p.kw;
    const int pos = p.positions != nullptr ? p.positions[row] : static_cast<int>(row % p.T) + p.pos_offset;
    float x1[8], x2[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) x1[i] = x2[i] = 0.f;
    if (live) { ld8(in, x1); ld8(in + p.half, x2); }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += x1[i] * x1[i] + x2[i] * x2[i];
    float rstd = 1.f;
    if (w != nullptr) rstd = rsqrtf(group_sum<LPH>(ss) / p.D + p.eps);
    if (!live) continue;
    float w1[8], w2[8], c[8], sn[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { w1[i] = w2[i] = c[i] = 1.f; sn[i] = 0.f; }
    if (w != nullptr) { ld8(w + sub * 8, w1); ld8(w + p.half + sub * 8, w2); }
    if (p.cos != nullptr) {
      ld8(p.cos + static_cast<int64_t>(pos) * p.half + sub * 8, c);
      ld8(p.sin + static_cast<int64_t>(pos) * p.half + sub * 8, sn);
    }
    float o1[8], o2[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float y1 = x1[i] * rstd * w1[i], y2 = x2[i] * rstd * w2[i];
      o1[i] = y1 * c[i] - y2 * sn[i];
      o2[i] = y1 * sn[i] + y2 * c[i];
    }
    st8(out, o1);
    st8(out + p.half, o2);
  }
}

template <int LPH>
__global__ void __launch_bounds__(256) qk_norm_rope_bwd_vec_kernel(const QKRopeParams p) {
  __shared__ float red[2][256];                           // [q|k][D <= 256], shared atomics at the end
  constexpr int GPW = 32 / LPH;
  const int lane = threadIdx.x & 31, sub = lane % LPH, grp = lane / LPH;
  const int warps = blockDim.x >> 5;
  const int heads = p.H + p.HK;
  const int64_t total = p.rows * heads;
  const int64_t step = static_cast<int64_t>(gridDim.x) * warps * GPW;
  float dwq1[8], dwq2[8], dwk1[8], dwk2[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) dwq1[i] = dwq2[i] = dwk1[i] = dwk2[i] = 0.f;
  for (int i = threadIdx.x; i < 512; i += blockDim.x) (&red[0][0])[i] = 0.f;
  __syncthreads();

  for (int64_t base = (static_cast<int64_t>(blockIdx.x) * warps + (threadIdx.x >> 5)) * GPW; base < total; base += step) {
    const int64_t item = base + grp;
    const bool live = item < total;
    const int64_t row = live ? item / heads : 0;
    const int h = live ? static_cast<int>(item % heads) : 0;
    const bool is_q = h < p.H;
    const int hh = is_q ? h : h - p.H;
    const bf16* in = (is_q ? p.q_in + row * p.ldq : p.k_in + row * p.ldk) + hh * p.D + sub * 8;
    const bf16* gin = (is_q ? p.dq + row * p.lddq : p.dk + row * p.lddk) + hh * p.D + sub * 8;
    bf16* out = (is_q ? p.q_out + row * p.ldqo : p.k_out + row * p.ldko) + hh * p.D + sub * 8;
    const bf16* w = is_q ? p.qw : p.kw;
    const int pos = p.positions != nullptr ? p.positions[row] : static_cast<int>(row % p.T) + p.pos_offset;
    float x1[8], x2[8], d1[8], d2[8], c[8], sn[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { x1[i] = x2[i] = d1[i] = d2[i] = 0.f; c[i] = 1.f; sn[i] = 0.f; }
    if (live) {
      ld8(gin, d1); ld8(gin + p.half, d2);
      if (w != nullptr) { ld8(in, x1); ld8(in + p.half, x2); }
      if (p.cos != nullptr) {
        ld8(p.cos + static_cast<int64_t>(pos) * p.half + sub * 8, c);
        ld8(p.sin + static_cast<int64_t>(pos) * p.half + sub * 8, sn);
      }
    }
    float g1[8], g2[8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      g1[i] = d1[i] * c[i] + d2[i] * sn[i];               // transpose of the rotation
      g2[i] = -d1[i] * sn[i] + d2[i] * c[i];
      ss += x1[i] * x1[i] + x2[i] * x2[i];
    }
    if (w == nullptr) {
      if (live) { st8(out, g1); st8(out + p.half, g2); }
      continue;
    }
    const float rstd = rsqrtf(group_sum<LPH>(ss) / p.D + p.eps);
    float w1[8], w2[8];
    ld8(w + sub * 8, w1);
    ld8(w + p.half + sub * 8, w2);
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      x1[i] *= rstd;
      x2[i] *= rstd;
      if (live) {
        if (is_q) { dwq1[i] += g1[i] * x1[i]; dwq2[i] += g2[i] * x2[i]; }
        else      { dwk1[i] += g1[i] * x1[i]; dwk2[i] += g2[i] * x2[i]; }
      }
      g1[i] *= w1[i];
      g2[i] *= w2[i];
      dot += g1[i] * x1[i] + g2[i] * x2[i];
    }
    dot = group_sum<LPH>(dot) / p.D;
    if (!live) continue;
    float o1[8], o2[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      o1[i] = rstd * (g1[i] - x1[i] * dot);
      o2[i] = rstd * (g2[i] - x2[i] * dot);
    }
    st8(out, o1);
    st8(out + p.half, o2);
  }
  if (p.dqw_partial == nullptr) return;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    atomicAdd(&red[0][sub * 8 + i], dwq1[i]);
    atomicAdd(&red[0][p.half + sub * 8 + i], dwq2[i]);
    atomicAdd(&red[1][sub * 8 + i], dwk1[i]);
    atomicAdd(&red[1][p.half + sub * 8 + i], dwk2[i]);
  }
  __syncthreads();
  for (int col = threadIdx.x; col < p.D; col += blockDim.x) {
    p.dqw_partial[static_cast<int64_t>(blockIdx.x) * p.D + col] = red[0][col];
    p.dkw_partial[static_cast<int64_t>(blockIdx.x) * p.D + col] = red[1][col];
  }
}

}  // namespace ttcd

using namespace ttcd;

constexpr int RMSNORM_MAX_D = 16384;    // wide-row kernels: 4 warps x D floats of shared memory in the backward

// y = rmsnorm(x + res) * w.  res, w, sum_out, rstd may be null.  D % 8 == 0, D <= 16384 (rows wider than 2048 take
// the streaming kernels).
TTCD_EXPORT int ttcd_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* sum_out, float* rstd,
                                 long long rows, int D, float eps, void* stream_ptr) {
  if (D % 8 != 0 || D > RMSNORM_MAX_D || rows <= 0) return TTCD_ERR_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream_ptr);
  const int warps = 8;
  const unsigned grid = static_cast<unsigned>((rows + warps - 1) / warps);
  if (D > 2048) {
    rmsnorm_fwd_wide_kernel<<<grid, warps * 32, 0, st>>>(static_cast<const bf16*>(x), static_cast<const bf16*>(res),
                                                         static_cast<const bf16*>(w), static_cast<bf16*>(y),
                                                         static_cast<bf16*>(sum_out), rstd, rows, D, eps);
    return static_cast<int>(cudaGetLastError());
  }
  const int chunks = (D + 255) / 256;
#define LAUNCH(C)                                                                                          \
  rmsnorm_fwd_kernel<C><<<grid, warps * 32, 0, st>>>(static_cast<const bf16*>(x), static_cast<const bf16*>(res), \
                                                     static_cast<const bf16*>(w), static_cast<bf16*>(y),       \
                                                     static_cast<bf16*>(sum_out), rstd, rows, D, eps)
  switch (chunks) {
    case 1: LAUNCH(1); break;
    case 2: LAUNCH(2); break;
    case 3: LAUNCH(3); break;
    case 4: LAUNCH(4); break;
    case 5: case 6: LAUNCH(6); break;
    default: LAUNCH(8); break;
  }
#undef LAUNCH
  return static_cast<int>(cudaGetLastError());
}

// dx = rmsnorm_backward(dy; s, w, rstd) (+ dres).  dw_partial: [nblocks][D] fp32 or null.
TTCD_EXPORT int ttcd_rmsnorm_bwd(const void* dy, const void* s, const void* w, const float* rstd, const void* dres,
                                 void* dx, float* dw_partial, long long rows, int D, int nblocks, void* stream_ptr) {
  if (D % 8 != 0 || D > RMSNORM_MAX_D || rows <= 0 || nblocks <= 0) return TTCD_ERR_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream_ptr);
  if (D > 2048) {
    const size_t wide_smem = static_cast<size_t>(4) * D * sizeof(float);
    static bool configured = false;
    if (!configured) {
      TTCD_CUDA_CHECK(cudaFuncSetAttribute(rmsnorm_bwd_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           4 * RMSNORM_MAX_D * static_cast<int>(sizeof(float)) > 227 * 1024
                                               ? 227 * 1024 : 4 * RMSNORM_MAX_D * static_cast<int>(sizeof(float))));
      configured = true;
    }
    if (wide_smem > 227 * 1024) return TTCD_ERR_SIZE;
    rmsnorm_bwd_wide_kernel<<<nblocks, 128, wide_smem, st>>>(
        static_cast<const bf16*>(dy), static_cast<const bf16*>(s), static_cast<const bf16*>(w), rstd,
        static_cast<const bf16*>(dres), static_cast<bf16*>(dx), dw_partial, rows, D);
    return static_cast<int>(cudaGetLastError());
  }
  const int warps = 8;
  const size_t smem = static_cast<size_t>(warps) * D * sizeof(float);
  const int chunks = (D + 255) / 256;
#define LAUNCH(C)                                                                                           \
  rmsnorm_bwd_kernel<C><<<nblocks, warps * 32, smem, st>>>(                                                 \
      static_cast<const bf16*>(dy), static_cast<const bf16*>(s), static_cast<const bf16*>(w), rstd,          \
      static_cast<const bf16*>(dres), static_cast<bf16*>(dx), dw_partial, rows, D)
  if (smem > 48 * 1024) {
    if (chunks <= 6) cudaFuncSetAttribute(rmsnorm_bwd_kernel<6>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    else cudaFuncSetAttribute(rmsnorm_bwd_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
  }
  switch (chunks) {
    case 1: LAUNCH(1); break;
    case 2: LAUNCH(2); break;
    case 3: LAUNCH(3); break;
    case 4: LAUNCH(4); break;
    case 5: case 6: LAUNCH(6); break;
    default: LAUNCH(8); break;
  }
#undef LAUNCH
  return static_cast<int>(cudaGetLastError());
}

// Two-input norm of the fast-weight blocks (see rmsnorm_dual_fwd_kernel).  All tensors bf16 [rows][D] contiguous;
// rstd_* fp32 [rows].  D % 8 == 0, D <= 2048.
TTCD_EXPORT int ttcd_rmsnorm_dual_fwd(const void* a_t, const void* a_s, const void* res, const void* w, void* y_t, void* y_s,
                                      void* sum_t, void* sum_s, float* rstd_t, float* rstd_s, long long rows, int D,
                                      float eps, void* stream_ptr) {
  if (D % 8 != 0 || D > 2048 || rows <= 0 || w == nullptr) return TTCD_ERR_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream_ptr);
  const int warps = 8;
  const unsigned grid = static_cast<unsigned>((rows + warps - 1) / warps);
  const int chunks = (D + 255) / 256;
#define LAUNCH(C)                                                                                              \
  rmsnorm_dual_fwd_kernel<C><<<grid, warps * 32, 0, st>>>(                                                     \
      static_cast<const bf16*>(a_t), static_cast<const bf16*>(a_s), static_cast<const bf16*>(res),             \
      static_cast<const bf16*>(w), static_cast<bf16*>(y_t), static_cast<bf16*>(y_s), static_cast<bf16*>(sum_t), \
      static_cast<bf16*>(sum_s), rstd_t, rstd_s, rows, D, eps)
  switch (chunks) {
    case 1: LAUNCH(1); break;
    case 2: LAUNCH(2); break;
    case 3: LAUNCH(3); break;
    case 4: LAUNCH(4); break;
    case 5: case 6: LAUNCH(6); break;
    default: LAUNCH(8); break;
  }
#undef LAUNCH
  return static_cast<int>(cudaGetLastError());
}

// d_at, d_as, d_res of the two-input norm; dres (gradient of the updated residual) may be null.
// dw_partial: [nblocks][D] fp32 (both streams summed).
TTCD_EXPORT int ttcd_rmsnorm_dual_bwd(const void* dy_t, const void* dy_s, const void* s_t, const void* s_s, const void* w,
                                      const float* rstd_t, const float* rstd_s, const void* dres, void* d_at, void* d_as,
                                      void* d_res, float* dw_partial, long long rows, int D, int nblocks, void* stream_ptr) {
  if (D % 8 != 0 || D > 2048 || rows <= 0 || nblocks <= 0 || w == nullptr || dw_partial == nullptr) return TTCD_ERR_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream_ptr);
  const int warps = 8;
  const size_t smem = static_cast<size_t>(warps) * D * sizeof(float);
  const int chunks = (D + 255) / 256;
#define LAUNCH(C)                                                                                              \
  rmsnorm_dual_bwd_kernel<C><<<nblocks, warps * 32, smem, st>>>(                                               \
      static_cast<const bf16*>(dy_t), static_cast<const bf16*>(dy_s), static_cast<const bf16*>(s_t),           \
      static_cast<const bf16*>(s_s), static_cast<const bf16*>(w), rstd_t, rstd_s, static_cast<const bf16*>(dres), \
      static_cast<bf16*>(d_at), static_cast<bf16*>(d_as), static_cast<bf16*>(d_res), dw_partial, rows, D)
  if (smem > 48 * 1024) {
    if (chunks <= 6) cudaFuncSetAttribute(rmsnorm_dual_bwd_kernel<6>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    else cudaFuncSetAttribute(rmsnorm_dual_bwd_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
  }
  switch (chunks) {
    case 1: LAUNCH(1); break;
    case 2: LAUNCH(2); break;
    case 3: LAUNCH(3); break;
    case 4: LAUNCH(4); break;
    case 5: case 6: LAUNCH(6); break;
    default: LAUNCH(8); break;
  }
#undef LAUNCH
  return static_cast<int>(cudaGetLastError());
}

// The vectorised kernels need rotary over the whole head and 16-byte aligned rows / heads.
static bool qk_vec_ok(const QKRopeParams& p) {
  auto al = [](const void* q) { return q == nullptr || (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
  const int lph = p.half / 8;
  if (2 * p.half != p.D || p.half % 8 != 0 || (lph != 4 && lph != 8 && lph != 16)) return false;
  if ((p.qw == nullptr) != (p.kw == nullptr)) return false;      // group reductions must stay warp-uniform
  if ((p.ldq | p.ldk | p.ldqo | p.ldko) % 8 != 0) return false;
  if (p.dq != nullptr && (p.lddq | p.lddk) % 8 != 0) return false;
  return al(p.q_in) && al(p.k_in) && al(p.q_out) && al(p.k_out) && al(p.dq) && al(p.dk) && al(p.qw) && al(p.kw) &&
         al(p.cos) && al(p.sin);
}

static int qk_check(int D, int half) { return (D > 256 || half * 2 > D || half <= 0) ? TTCD_ERR_ARG : TTCD_OK; }

// Forward: q_out/k_out = rope(headnorm(q_in/k_in)).  Row strides in elements.
TTCD_EXPORT int ttcd_qk_norm_rope_fwd(const void* q_in, long long ldq, const void* k_in, long long ldk, void* q_out,
                                      long long ldqo, void* k_out, long long ldko, const void* qw, const void* kw,
                                      const void* cos, const void* sin, const int* positions, long long rows, int T,
                                      int pos_offset, int H, int HK, int D, int half, float eps, void* stream_ptr) {
  if (qk_check(D, half) != TTCD_OK || rows <= 0) return TTCD_ERR_ARG;
  QKRopeParams p{};
  p.q_in = static_cast<const bf16*>(q_in); p.k_in = static_cast<const bf16*>(k_in); p.ldq = ldq; p.ldk = ldk;
  p.q_out = static_cast<bf16*>(q_out); p.k_out = static_cast<bf16*>(k_out); p.ldqo = ldqo; p.ldko = ldko;
  p.qw = static_cast<const bf16*>(qw); p.kw = static_cast<const bf16*>(kw);
  p.cos = static_cast<const bf16*>(cos); p.sin = static_cast<const bf16*>(sin); p.positions = positions;
  p.rows = rows; p.T = T; p.pos_offset = pos_offset; p.H = H; p.HK = HK; p.D = D; p.half = half; p.eps = eps;
  cudaStream_t st = static_cast<cudaStream_t>(stream_ptr);
  const long long items = rows * (H + HK);
  const unsigned grid = static_cast<unsigned>(std::min<long long>((items + 7) / 8, 148LL * 16));
  if (qk_vec_ok(p)) {
    const int lph = half / 8;
    const unsigned vgrid = static_cast<unsigned>(std::min<long long>((items * lph / 32 + 7) / 8 + 1, 148LL * 16));
    if (lph == 4) qk_norm_rope_fwd_vec_kernel<4><<<vgrid, 256, 0, st>>>(p);
    else if (lph == 8) qk_norm_rope_fwd_vec_kernel<8><<<vgrid, 256, 0, st>>>(p);
    else qk_norm_rope_fwd_vec_kernel<16><<<vgrid, 256, 0, st>>>(p);
    return static_cast<int>(cudaGetLastError());
  }
  if (half <= 32) qk_norm_rope_fwd_kernel<1><<<grid, 256, 0, st>>>(p);
  else if (half <= 64) qk_norm_rope_fwd_kernel<2><<<grid, 256, 0, st>>>(p);
  else qk_norm_rope_fwd_kernel<4><<<grid, 256, 0, st>>>(p);
  return static_cast<int>(cudaGetLastError());
}

// Backward: dq_in/dk_in (written to q_out/k_out slots) from gradients w.r.t. the rotated outputs.
TTCD_EXPORT int ttcd_qk_norm_rope_bwd(const void* dq, long long lddq, const void* dk, long long lddk, const void* q_in,
                                      long long ldq, const void* k_in, long long ldk, void* dq_in, long long ldqo,
                                      void* dk_in, long long ldko, const void* qw, const void* kw, const void* cos,
                                      const void* sin, const int* positions, float* dqw_partial, float* dkw_partial,
                                      int nblocks, long long rows, int T, int pos_offset, int H, int HK, int D,
                                      int half, float eps, void* stream_ptr) {
  if (qk_check(D, half) != TTCD_OK || rows <= 0 || nblocks <= 0) return TTCD_ERR_ARG;
  QKRopeParams p{};
  p.q_in = static_cast<const bf16*>(q_in); p.k_in = static_cast<const bf16*>(k_in); p.ldq = ldq; p.ldk = ldk;
  p.q_out = static_cast<bf16*>(dq_in); p.k_out = static_cast<bf16*>(dk_in); p.ldqo = ldqo; p.ldko = ldko;
  p.dq = static_cast<const bf16*>(dq); p.dk = static_cast<const bf16*>(dk); p.lddq = lddq; p.lddk = lddk;
  p.qw = static_cast<const bf16*>(qw); p.kw = static_cast<const bf16*>(kw);
  p.cos = static_cast<const bf16*>(cos); p.sin = static_cast<const bf16*>(sin); p.positions = positions;
  p.rows = rows; p.T = T; p.pos_offset = pos_offset; p.H = H; p.HK = HK; p.D = D; p.half = half; p.eps = eps;
  p.dqw_partial = dqw_partial; p.dkw_partial = dkw_partial;
  cudaStream_t st = static_cast<cudaStream_t>(stream_ptr);
  if (qk_vec_ok(p)) {
    const int lph = half / 8;
    if (lph == 4) qk_norm_rope_bwd_vec_kernel<4><<<nblocks, 256, 0, st>>>(p);
    else if (lph == 8) qk_norm_rope_bwd_vec_kernel<8><<<nblocks, 256, 0, st>>>(p);
    else qk_norm_rope_bwd_vec_kernel<16><<<nblocks, 256, 0, st>>>(p);
    return static_cast<int>(cudaGetLastError());
  }
  if (half <= 32) qk_norm_rope_bwd_kernel<1><<<nblocks, 256, 0, st>>>(p);
  else if (half <= 64) qk_norm_rope_bwd_kernel<2><<<nblocks, 256, 0, st>>>(p);
  else qk_norm_rope_bwd_kernel<4><<<nblocks, 256, 0, st>>>(p);
  return static_cast<int>(cudaGetLastError());
}

// ------------------------------------------------------------------------------------------------
// RMSNorm backward that allocates nothing: the per-block weight-gradient partial sums go to an array
// in the library image instead of a caller-provided buffer, and a second small kernel folds them into
// dw[D].  Contract and limits: ttcd_no_alloc.h.
// ------------------------------------------------------------------------------------------------
#include "ttcd_no_alloc.h"

namespace ttcd {

static __device__ __align__(256) float g_rmsnorm_dw_scratch[TTCD_NO_ALLOC_MAX_BLOCKS * TTCD_NO_ALLOC_MAX_D];

__global__ void __launch_bounds__(256) rmsnorm_dw_fold_kernel(const float* __restrict__ partial, int nblocks, int D,
                                                              float* __restrict__ dw) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= D) return;
  float acc = 0.f;
  for (int b = 0; b < nblocks; ++b) acc += partial[static_cast<int64_t>(b) * D + col];   // fixed order: deterministic
  dw[col] = acc;
}

constexpr int kNoAllocMaxDevices = 64;
static float* g_scratch_addr[kNoAllocMaxDevices] = {};

// Device address of this device's copy of the array; looked up once per device.
static int no_alloc_scratch(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices) return TTCD_NO_ALLOC_ERR_DEVICE;
  if (g_scratch_addr[dev] == nullptr) {
    float* addr = nullptr;
    const cudaError_t rc = cudaGetSymbolAddress(reinterpret_cast<void**>(&addr), g_rmsnorm_dw_scratch);
    if (rc != cudaSuccess || addr == nullptr) {
      (void)cudaGetLastError();
      return TTCD_NO_ALLOC_ERR_DEVICE;
    }
    if (cudaFuncSetAttribute(rmsnorm_bwd_kernel<6>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(rmsnorm_bwd_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024) != cudaSuccess) {
      (void)cudaGetLastError();
      return TTCD_NO_ALLOC_ERR_DEVICE;
    }
    g_scratch_addr[dev] = addr;
  }
  *out = g_scratch_addr[dev];
  return TTCD_NO_ALLOC_OK;
}

}  // namespace ttcd

TTCD_EXPORT int ttcd_rmsnorm_bwd_no_alloc(const void* dy, const void* s, const void* w, const float* rstd,
                                          const void* dres, void* dx, float* dw, long long rows, int D,
                                          void* stream_ptr) {
  if (dy == nullptr || s == nullptr || rstd == nullptr || dx == nullptr || rows <= 0 || D <= 0 || D % 8 != 0 ||
      (w != nullptr && dw == nullptr))
    return TTCD_NO_ALLOC_ERR_SHAPE;
  if (D > TTCD_NO_ALLOC_MAX_D) return TTCD_NO_ALLOC_ERR_TOO_LARGE;
  float* scratch = nullptr;
  const int rc = no_alloc_scratch(&scratch);
  if (rc != TTCD_NO_ALLOC_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream_ptr);
  const int warps = 8;
  const long long want = (rows + warps - 1) / warps;
  const int nblocks = static_cast<int>(want < TTCD_NO_ALLOC_MAX_BLOCKS ? want : TTCD_NO_ALLOC_MAX_BLOCKS);
  const size_t smem = static_cast<size_t>(warps) * D * sizeof(float);
  float* partial = w != nullptr ? scratch : nullptr;
  const int chunks = (D + 255) / 256;
#define LAUNCH(C)                                                                                           \
  rmsnorm_bwd_kernel<C><<<nblocks, warps * 32, smem, st>>>(                                                 \
      static_cast<const bf16*>(dy), static_cast<const bf16*>(s), static_cast<const bf16*>(w), rstd,          \
      static_cast<const bf16*>(dres), static_cast<bf16*>(dx), partial, rows, D)
  switch (chunks) {
    case 1: LAUNCH(1); break;
    case 2: LAUNCH(2); break;
    case 3: LAUNCH(3); break;
    case 4: LAUNCH(4); break;
    case 5: case 6: LAUNCH(6); break;
    default: LAUNCH(8); break;
  }
#undef LAUNCH
  if (partial != nullptr) rmsnorm_dw_fold_kernel<<<(D + 255) / 256, 256, 0, st>>>(partial, nblocks, D, dw);
  return static_cast<int>(cudaGetLastError());
}
