// The chunk-local part of the (gated) delta rule, forward and backward, one CTA per (batch, head, 64-token chunk)
// (sm_100a; fp32 FMA work on 64 x 64 tiles in shared memory: the products of a chunk are 64 x 64 x D, the point of the
// kernels is to replace some forty element-wise / batched-GEMM / triangular-solve launches over fp32 [B,H,T,D]
// tensors by one pass that reads q, k, v once).
//
// With q, k the (optionally L2-normalised, q also scaled) rows of the chunk, beta the write strengths, G the running
// sum of the log decays g inside the chunk (G = 0 without a gate), dec_ij = e^{G_i - G_j} for i >= j:
//
//   L   = strict_lower(beta_i dec_ij k_i.k_j)          T = (I + L)^-1           (unit lower triangular)
//   w   = T (beta e^G k)      u = T (beta v)            the WY factors
//   kt  = e^{G_last - G} k    q_in = e^G q    qk = lower(dec_ij q_i.k_j)    gamma = e^{G_last}
//
// (the role of fwd_prepare_wy_repr / chunk_scaled_dot_kkt / solve_tril of fla/ops/delta_rule/wy_fast.py and
// fla/ops/gated_delta_rule/wy_fast.py; the chain over chunks that consumes w, u, kt, gamma is csrc/delta_chain.cu).
// The backward kernel takes the gradients of those six outputs, rebuilds L and T from q, k, beta, g (cheaper than
// keeping them) and writes dq, dk, dv, dbeta, dg:
//
//   d_kbg = T^T d_w    d_vb = T^T d_u    d_T = d_w (beta e^G k)^T + d_u (beta v)^T    d_L = -strict_lower(T^T d_T T^T)
//   M1 = d_L beta_i dec   M2 = d_qk dec   E = d_L L + M2 (q k^T)
//   dk = (M1 + M1^T) k + M2^T q + beta e^G d_kbg + e^{G_last-G} d_kt        dq = M2 k + e^G d_qin
//   dv = beta d_vb        dbeta_i = sum_j d_L dec (k k^T) + e^G d_kbg.k + d_vb.v
//   dG_i = sum_j E_ij - sum_j E_ji + d_kbg.(beta e^G k) + d_qin.(e^G q) - d_kt.(e^{G_last-G} k)
//   dG_last += sum_i d_kt.(e^{G_last-G} k) + d_gamma gamma;   dg = reverse running sum of dG
//
// followed by the backward of the row normalisation.  Nothing here waits on another CTA or on an asynchronous copy.
#include "common.cuh"

namespace ttcd {

constexpr int DP_C = 64;                  // rows of a chunk
constexpr int DP_LD = 68;                 // row stride (floats) of a 64 x 64 tile: 16-byte rows, rows 4 banks apart
constexpr int DP_TILE = DP_C * DP_LD;
constexpr int DP_THREADS = 256;
constexpr int DP_VEC = 12 * DP_C;         // per-row vectors
constexpr int DP_SMEM_FWD = (5 * DP_TILE + DP_VEC) * 4;
constexpr int DP_SMEM_BWD = (6 * DP_TILE + DP_VEC) * 4;

struct DeltaPrepParams {
  const void* q; const void* k; const void* v;      // [B, T, H, D | Dv], bf16 or fp32 (in_bf16)
  const float* beta; const float* g;                // [B, T, H]; g null: no gate
  int T, H, D, Dv, n;                               // n = chunks per sequence
  float scale; int l2norm; int in_bf16;
  float *w, *u, *kt, *q_in, *qk, *gamma;            // forward outputs, chunk layout [B*H, n, 64, *]
  const float *d_w, *d_u, *d_kt, *d_qin, *d_qk, *d_gamma;
  float *dq, *dk, *dv, *dbeta, *dg;                 // backward outputs, token layout [B, T, H, *] fp32
};

// ---- 64 x 64 x 64 products; thread (ty, tx) of the 16 x 16 grid owns rows ty + 16 a -----------------------------
// acc[a][b] += sum_d X[ty + 16 a][d] Y[tx + 16 b][d]     (X Y^T: the thread's columns are tx + 16 b)
__device__ __forceinline__ void mm_nt(float (&acc)[4][4], const float* X, const float* Y, int ty, int tx) {
#pragma unroll 2
  for (int d = 0; d < DP_C; d += 4) {
    float4 x[4], y[4];
#pragma unroll
    for (int a = 0; a < 4; ++a) x[a] = *reinterpret_cast<const float4*>(X + (ty + 16 * a) * DP_LD + d);
#pragma unroll
    for (int b = 0; b < 4; ++b) y[b] = *reinterpret_cast<const float4*>(Y + (tx + 16 * b) * DP_LD + d);
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b)
        acc[a][b] = fmaf(x[a].x, y[b].x, fmaf(x[a].y, y[b].y, fmaf(x[a].z, y[b].z, fmaf(x[a].w, y[b].w, acc[a][b]))));
  }
}
// acc[a][b] += sum_j M[ty + 16 a][j] X[j][4 tx + b]      (M X: the thread's columns are 4 tx + b)
__device__ __forceinline__ void mm_nn(float (&acc)[4][4], const float* M, const float* X, int ty, int tx) {
#pragma unroll 2
  for (int j = 0; j < DP_C; j += 4) {
    float4 m[4], x[4];
#pragma unroll
    for (int a = 0; a < 4; ++a) m[a] = *reinterpret_cast<const float4*>(M + (ty + 16 * a) * DP_LD + j);
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) x[jj] = *reinterpret_cast<const float4*>(X + (j + jj) * DP_LD + 4 * tx);
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      acc[a][0] = fmaf(m[a].x, x[0].x, fmaf(m[a].y, x[1].x, fmaf(m[a].z, x[2].x, fmaf(m[a].w, x[3].x, acc[a][0]))));
      acc[a][1] = fmaf(m[a].x, x[0].y, fmaf(m[a].y, x[1].y, fmaf(m[a].z, x[2].y, fmaf(m[a].w, x[3].y, acc[a][1]))));
      acc[a][2] = fmaf(m[a].x, x[0].z, fmaf(m[a].y, x[1].z, fmaf(m[a].z, x[2].z, fmaf(m[a].w, x[3].z, acc[a][2]))));
      acc[a][3] = fmaf(m[a].x, x[0].w, fmaf(m[a].y, x[1].w, fmaf(m[a].z, x[2].w, fmaf(m[a].w, x[3].w, acc[a][3]))));
    }
  }
}
__device__ __forceinline__ void zero(float (&acc)[4][4]) {
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
}
// sum over the 16 threads (tx) that share a row; every one of them gets the total
__device__ __forceinline__ float row_sum16(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 8);
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v;
}

// ---- tile loads: 64 rows x 64 columns -> shared memory, times a per-row factor ----------------------------------
// thread f = tid + 256 e handles row f / 16, columns 4 (f % 16) .. +3
__device__ __forceinline__ float4 load4(const void* base, int64_t elem, bool bf) {
  if (bf) {
    const uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const bf16*>(base) + elem);
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    return make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
  }
  return *reinterpret_cast<const float4*>(static_cast<const float*>(base) + elem);
}
// token layout [.., T, H, width]: row r of the chunk is token t0 + r (zero beyond `rows`)
__device__ __forceinline__ void load_tokens(float* dst, const void* src, bool bf, int64_t elem0, int64_t row_stride, int rows,
                                            const float* mul) {
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int f = threadIdx.x + DP_THREADS * e, r = f >> 4, c4 = (f & 15) * 4;
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < rows) x = load4(src, elem0 + r * row_stride + c4, bf);
    const float m = mul != nullptr ? mul[r] : 1.f;
    *reinterpret_cast<float4*>(dst + r * DP_LD + c4) = make_float4(x.x * m, x.y * m, x.z * m, x.w * m);
  }
}
// chunk layout [.., 64, width] fp32 (all 64 rows exist)
__device__ __forceinline__ void load_chunk(float* dst, const float* src, int width, const float* mul) {
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int f = threadIdx.x + DP_THREADS * e, r = f >> 4, c4 = (f & 15) * 4;
    const float4 x = *reinterpret_cast<const float4*>(src + static_cast<int64_t>(r) * width + c4);
    const float m = mul != nullptr ? mul[r] : 1.f;
    *reinterpret_cast<float4*>(dst + r * DP_LD + c4) = make_float4(x.x * m, x.y * m, x.z * m, x.w * m);
  }
}

// per-row vectors in shared memory
struct DeltaVec {
  float *beta, *G, *eg, *to_end, *rq, *rk, *v0, *v1, *v2, *v3, *v4, *v5;
  __device__ explicit DeltaVec(float* p)
      : beta(p), G(p + 64), eg(p + 128), to_end(p + 192), rq(p + 256), rk(p + 320), v0(p + 384), v1(p + 448),
        v2(p + 512), v3(p + 576), v4(p + 640), v5(p + 704) {}
};

struct ChunkCoord {
  int64_t tok0;        // index of the chunk's first token row in [B*T]
  int rows;            // valid token rows (the last chunk may be short)
  int h;
  int64_t chunk;       // index of the chunk in [B*H*n]
};

// beta, the running decay sums and the normalisation factors of the chunk's rows
__device__ __forceinline__ void chunk_rows(const DeltaPrepParams& p, const ChunkCoord& cc, const DeltaVec& vec) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid < DP_C) {
    const bool ok = tid < cc.rows;
    const int64_t at = (cc.tok0 + tid) * p.H + cc.h;
    vec.beta[tid] = ok ? p.beta[at] : 0.f;
    vec.v0[tid] = (ok && p.g != nullptr) ? p.g[at] : 0.f;
  }
  // row norms: warp w takes rows 8 w .. 8 w + 7
  for (int rr = 0; rr < 8; ++rr) {
    const int r = warp * 8 + rr;
    float sq = 0.f, sk = 0.f;
    if (p.l2norm && r < cc.rows) {
      const int64_t row = ((cc.tok0 + r) * p.H + cc.h) * p.D;
      for (int c4 = lane * 4; c4 < p.D; c4 += 128) {
        const float4 a = load4(p.q, row + c4, p.in_bf16), b = load4(p.k, row + c4, p.in_bf16);
        sq += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
        sk += b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      sq += __shfl_xor_sync(0xffffffffu, sq, o);
      sk += __shfl_xor_sync(0xffffffffu, sk, o);
    }
    if (lane == 0) {
      vec.rq[r] = p.l2norm ? p.scale / fmaxf(sqrtf(sq), 1e-6f) : p.scale;
      vec.rk[r] = p.l2norm ? 1.f / fmaxf(sqrtf(sk), 1e-6f) : 1.f;
    }
  }
  __syncthreads();
  if (tid < DP_C) {
    float s = 0.f;
    for (int j = 0; j <= tid; ++j) s += vec.v0[j];
    vec.G[tid] = s;
  }
  __syncthreads();
  if (tid < DP_C) {
    vec.eg[tid] = expf(vec.G[tid]);
    vec.to_end[tid] = expf(vec.G[DP_C - 1] - vec.G[tid]);
  }
  __syncthreads();
}

// A = k k^T and QK = q k^T over all D (thread-owned elements [ty + 16 a][tx + 16 b]); S0, S1: two scratch tiles
__device__ __forceinline__ void chunk_grams(const DeltaPrepParams& p, const ChunkCoord& cc, const DeltaVec& vec, float* S0,
                                            float* S1, float (&A)[4][4], float (&QK)[4][4], int ty, int tx) {
  zero(A);
  zero(QK);
  const int64_t row_stride = static_cast<int64_t>(p.H) * p.D;
  const int64_t elem0 = (cc.tok0 * p.H + cc.h) * p.D;
  for (int s = 0; s < p.D; s += DP_C) {
    load_tokens(S0, p.k, p.in_bf16, elem0 + s, row_stride, cc.rows, vec.rk);
    load_tokens(S1, p.q, p.in_bf16, elem0 + s, row_stride, cc.rows, vec.rq);
    __syncthreads();
    mm_nt(A, S0, S0, ty, tx);
    mm_nt(QK, S1, S0, ty, tx);
    __syncthreads();
  }
}

// T = (I + L)^-1 by forward substitution, column by column: column c belongs to the four lanes 4 c .. 4 c + 3 of one
// warp, which split the sum over earlier rows.  Writes T (Tm) and, if asked, its transpose (TTm).
__device__ __forceinline__ void chunk_inverse(const float* Lm, float* Tm, float* TTm) {
  const int c = threadIdx.x >> 2, part = threadIdx.x & 3;
  for (int i = 0; i < DP_C; ++i) {
    float s = 0.f;
    for (int j = c + part; j < i; j += 4) s = fmaf(Lm[i * DP_LD + j], Tm[j * DP_LD + c], s);
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    if (part == 0) {
      const float t = i == c ? 1.f : (i > c ? -s : 0.f);
      Tm[i * DP_LD + c] = t;
      if (TTm != nullptr) TTm[c * DP_LD + i] = t;
    }
    __syncwarp();
  }
}

__device__ __forceinline__ ChunkCoord chunk_coord(const DeltaPrepParams& p) {
  ChunkCoord cc;
  const int i = blockIdx.x, bh = blockIdx.y;
  const int b = bh / p.H;
  cc.h = bh % p.H;
  cc.tok0 = static_cast<int64_t>(b) * p.T + static_cast<int64_t>(i) * DP_C;
  cc.rows = min(DP_C, p.T - i * DP_C);
  cc.chunk = static_cast<int64_t>(bh) * p.n + i;
  return cc;
}

// =====================================================================================================
// forward
// =====================================================================================================
__global__ void __launch_bounds__(DP_THREADS, 2) delta_prep_fwd_kernel(const DeltaPrepParams p) {
  extern __shared__ __align__(16) float dp_smem[];
  float* Lm = dp_smem;                   // L, then T with the columns scaled for w
  float* Tm = Lm + DP_TILE;
  float* Tu = Tm + DP_TILE;              // T with the columns scaled for u
  float* S0 = Tu + DP_TILE;
  float* S1 = S0 + DP_TILE;
  const DeltaVec vec(dp_smem + 5 * DP_TILE);
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const ChunkCoord cc = chunk_coord(p);

  chunk_rows(p, cc, vec);
  float A[4][4], QK[4][4];
  chunk_grams(p, cc, vec, S0, S1, A, QK, ty, tx);
  // L (strictly lower) into shared memory, qk = lower(dec QK) into S1 for a coalesced copy out
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int i = ty + 16 * a, j = tx + 16 * b;
      const float dec = i >= j ? expf(vec.G[i] - vec.G[j]) : 0.f;
      Lm[i * DP_LD + j] = i > j ? vec.beta[i] * dec * A[a][b] : 0.f;
      S1[i * DP_LD + j] = dec * QK[a][b];
    }
  __syncthreads();
  {
    float* out = p.qk + cc.chunk * DP_C * DP_C;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int f = tid + DP_THREADS * e, r = f >> 4, c4 = (f & 15) * 4;
      *reinterpret_cast<float4*>(out + r * DP_C + c4) = *reinterpret_cast<const float4*>(S1 + r * DP_LD + c4);
    }
    if (tid == 0) p.gamma[cc.chunk] = vec.eg[DP_C - 1];
  }
  chunk_inverse(Lm, Tm, nullptr);
  __syncthreads();
  // fold the row factors of the right-hand sides into the columns of T:  w = (T diag(beta e^G)) k,  u = (T diag(beta)) v
#pragma unroll
  for (int e = 0; e < 16; ++e) {
    const int f = tid + DP_THREADS * e, i = f >> 6, j = f & 63;
    const float t = Tm[i * DP_LD + j];
    Lm[i * DP_LD + j] = t * vec.beta[j] * vec.eg[j];
    Tu[i * DP_LD + j] = t * vec.beta[j];
  }
  __syncthreads();
  const float* Tw = Lm;
  const int64_t row_stride = static_cast<int64_t>(p.H) * p.D;
  const int64_t elem0 = (cc.tok0 * p.H + cc.h) * p.D;
  for (int s = 0; s < p.D; s += DP_C) {
    load_tokens(S0, p.k, p.in_bf16, elem0 + s, row_stride, cc.rows, vec.rk);
    load_tokens(S1, p.q, p.in_bf16, elem0 + s, row_stride, cc.rows, vec.rq);
    __syncthreads();
    // kt = e^{G_last - G} k, q_in = e^G q (element-wise, in the loaders' layout)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int f = tid + DP_THREADS * e, r = f >> 4, c4 = (f & 15) * 4;
      const float4 kk = *reinterpret_cast<const float4*>(S0 + r * DP_LD + c4);
      const float4 qq = *reinterpret_cast<const float4*>(S1 + r * DP_LD + c4);
      const float te = vec.to_end[r], eg = vec.eg[r];
      const int64_t at = (cc.chunk * DP_C + r) * p.D + s + c4;
      *reinterpret_cast<float4*>(p.kt + at) = make_float4(kk.x * te, kk.y * te, kk.z * te, kk.w * te);
      *reinterpret_cast<float4*>(p.q_in + at) = make_float4(qq.x * eg, qq.y * eg, qq.z * eg, qq.w * eg);
    }
    float acc[4][4];
    zero(acc);
    mm_nn(acc, Tw, S0, ty, tx);
#pragma unroll
    for (int a = 0; a < 4; ++a)
      *reinterpret_cast<float4*>(p.w + (cc.chunk * DP_C + ty + 16 * a) * p.D + s + 4 * tx) =
          make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]);
    __syncthreads();
  }
  const int64_t vrow_stride = static_cast<int64_t>(p.H) * p.Dv;
  const int64_t velem0 = (cc.tok0 * p.H + cc.h) * p.Dv;
  for (int s = 0; s < p.Dv; s += DP_C) {
    load_tokens(S0, p.v, p.in_bf16, velem0 + s, vrow_stride, cc.rows, nullptr);
    __syncthreads();
    float acc[4][4];
    zero(acc);
    mm_nn(acc, Tu, S0, ty, tx);
#pragma unroll
    for (int a = 0; a < 4; ++a)
      *reinterpret_cast<float4*>(p.u + (cc.chunk * DP_C + ty + 16 * a) * p.Dv + s + 4 * tx) =
          make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]);
    __syncthreads();
  }
}

// =====================================================================================================
// backward
// =====================================================================================================
__global__ void __launch_bounds__(DP_THREADS, 2) delta_prep_bwd_kernel(const DeltaPrepParams p) {
  extern __shared__ __align__(16) float dp_smem[];
  float* t0 = dp_smem;                   // L -> d_T -> M1 + M1^T
  float* t1 = t0 + DP_TILE;              // T -> M2^T
  float* t2 = t1 + DP_TILE;              // T^T
  float* t3 = t2 + DP_TILE;              // T^T d_T -> M2
  float* S0 = t3 + DP_TILE;
  float* S1 = S0 + DP_TILE;
  const DeltaVec vec(dp_smem + 6 * DP_TILE);
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const ChunkCoord cc = chunk_coord(p);
  const int64_t row_stride = static_cast<int64_t>(p.H) * p.D, vrow_stride = static_cast<int64_t>(p.H) * p.Dv;
  const int64_t elem0 = (cc.tok0 * p.H + cc.h) * p.D, velem0 = (cc.tok0 * p.H + cc.h) * p.Dv;

  chunk_rows(p, cc, vec);
  float A[4][4], QK[4][4];
  chunk_grams(p, cc, vec, S0, S1, A, QK, ty, tx);
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int i = ty + 16 * a, j = tx + 16 * b;
      t0[i * DP_LD + j] = i > j ? vec.beta[i] * expf(vec.G[i] - vec.G[j]) * A[a][b] : 0.f;
    }
  if (tid < DP_C) { vec.v1[tid] = vec.beta[tid] * vec.eg[tid] * vec.rk[tid]; vec.v2[tid] = vec.beta[tid]; }
  __syncthreads();
  chunk_inverse(t0, t1, t2);
  __syncthreads();

  // ---- d_T = d_w (beta e^G k)^T + d_u (beta v)^T
  float acc[4][4];
  zero(acc);
  for (int s = 0; s < p.D; s += DP_C) {
    load_chunk(S0, p.d_w + cc.chunk * DP_C * p.D + s, p.D, nullptr);
    load_tokens(S1, p.k, p.in_bf16, elem0 + s, row_stride, cc.rows, vec.v1);
    __syncthreads();
    mm_nt(acc, S0, S1, ty, tx);
    __syncthreads();
  }
  for (int s = 0; s < p.Dv; s += DP_C) {
    load_chunk(S0, p.d_u + cc.chunk * DP_C * p.Dv + s, p.Dv, nullptr);
    load_tokens(S1, p.v, p.in_bf16, velem0 + s, vrow_stride, cc.rows, vec.v2);
    __syncthreads();
    mm_nt(acc, S0, S1, ty, tx);
    __syncthreads();
  }
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) t0[(ty + 16 * a) * DP_LD + tx + 16 * b] = acc[a][b];
  __syncthreads();
  // ---- d_L = -strict_lower(T^T d_T T^T)
  zero(acc);
  mm_nn(acc, t2, t0, ty, tx);                                   // X1 = T^T d_T   (columns 4 tx + b)
#pragma unroll
  for (int a = 0; a < 4; ++a)
    *reinterpret_cast<float4*>(t3 + (ty + 16 * a) * DP_LD + 4 * tx) = make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]);
  __syncthreads();
  zero(acc);
  mm_nt(acc, t3, t1, ty, tx);                                   // X1 T^T        (columns tx + 16 b)
  __syncthreads();                                              // t0 (d_T), t1 (T), t3 (X1) are free from here
  // ---- element-wise on the owned elements: M1 (+ its transpose) -> t0, M2 -> t3, M2^T -> t1; row / column sums
  {
    const float* dqk = p.d_qk + cc.chunk * DP_C * DP_C;
    float e_col[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int i = ty + 16 * a;
      float e_row = 0.f, b_row = 0.f;
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int j = tx + 16 * b;
        const float dec = i >= j ? expf(vec.G[i] - vec.G[j]) : 0.f;
        const float dl = i > j ? -acc[a][b] : 0.f;
        const float m1 = dl * vec.beta[i] * dec;
        const float m2 = dqk[i * DP_C + j] * dec;
        const float e = m1 * A[a][b] + m2 * QK[a][b];          // d_L L + M2 QK
        e_row += e;
        e_col[b] += e;
        b_row += dl * dec * A[a][b];
        if (i > j) { t0[i * DP_LD + j] = m1; t0[j * DP_LD + i] = m1; }
        if (i == j) t0[i * DP_LD + j] = 0.f;
        t3[i * DP_LD + j] = m2;
        t1[j * DP_LD + i] = m2;
      }
      e_row = row_sum16(e_row);
      b_row = row_sum16(b_row);
      if (tx == 0) { vec.v3[i] = e_row; vec.v4[i] = b_row; }
    }
    // column sums of E: partials per ty in S0, then 64 threads add the 16 partials
#pragma unroll
    for (int b = 0; b < 4; ++b) S0[ty * DP_LD + tx + 16 * b] = e_col[b];
  }
  __syncthreads();
  if (tid < DP_C) {
    float s = 0.f;
    for (int y = 0; y < 16; ++y) s += S0[y * DP_LD + tid];
    vec.v3[tid] -= s;                                           // dG so far: row sum - column sum of E
  }
  __syncthreads();

  // ---- per D slice: dq, dk (with respect to the normalised rows), kept in the outputs until the row dots are known
  float rk1[4] = {0.f, 0.f, 0.f, 0.f}, rq1[4] = {0.f, 0.f, 0.f, 0.f}, rt1[4] = {0.f, 0.f, 0.f, 0.f};
  float dotq[4] = {0.f, 0.f, 0.f, 0.f}, dotk[4] = {0.f, 0.f, 0.f, 0.f};
  for (int s = 0; s < p.D; s += DP_C) {
    load_tokens(S0, p.k, p.in_bf16, elem0 + s, row_stride, cc.rows, vec.rk);
    load_tokens(S1, p.q, p.in_bf16, elem0 + s, row_stride, cc.rows, vec.rq);
    __syncthreads();
    float adq[4][4], adk[4][4];
    zero(adq);
    zero(adk);
    mm_nn(adq, t3, S0, ty, tx);                                 // M2 k
    mm_nn(adk, t0, S0, ty, tx);                                 // (M1 + M1^T) k
    mm_nn(adk, t1, S1, ty, tx);                                 // M2^T q
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int i = ty + 16 * a;
      const float4 dqi = *reinterpret_cast<const float4*>(p.d_qin + (cc.chunk * DP_C + i) * p.D + s + 4 * tx);
      const float4 qq = *reinterpret_cast<const float4*>(S1 + i * DP_LD + 4 * tx);
      const float eg = vec.eg[i];
      adq[a][0] = fmaf(dqi.x, eg, adq[a][0]); adq[a][1] = fmaf(dqi.y, eg, adq[a][1]);
      adq[a][2] = fmaf(dqi.z, eg, adq[a][2]); adq[a][3] = fmaf(dqi.w, eg, adq[a][3]);
      rq1[a] += dqi.x * qq.x + dqi.y * qq.y + dqi.z * qq.z + dqi.w * qq.w;
      dotq[a] += adq[a][0] * qq.x + adq[a][1] * qq.y + adq[a][2] * qq.z + adq[a][3] * qq.w;
      if (i < cc.rows)
        *reinterpret_cast<float4*>(p.dq + elem0 + i * row_stride + s + 4 * tx) = make_float4(adq[a][0], adq[a][1], adq[a][2], adq[a][3]);
    }
    __syncthreads();
    load_chunk(S1, p.d_w + cc.chunk * DP_C * p.D + s, p.D, nullptr);
    __syncthreads();
    zero(adq);
    mm_nn(adq, t2, S1, ty, tx);                                 // d_kbg = T^T d_w
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int i = ty + 16 * a;
      const float4 dkt = *reinterpret_cast<const float4*>(p.d_kt + (cc.chunk * DP_C + i) * p.D + s + 4 * tx);
      const float4 kk = *reinterpret_cast<const float4*>(S0 + i * DP_LD + 4 * tx);
      const float be = vec.beta[i] * vec.eg[i], te = vec.to_end[i];
      rk1[a] += adq[a][0] * kk.x + adq[a][1] * kk.y + adq[a][2] * kk.z + adq[a][3] * kk.w;
      rt1[a] += dkt.x * kk.x + dkt.y * kk.y + dkt.z * kk.z + dkt.w * kk.w;
      adk[a][0] += adq[a][0] * be + dkt.x * te; adk[a][1] += adq[a][1] * be + dkt.y * te;
      adk[a][2] += adq[a][2] * be + dkt.z * te; adk[a][3] += adq[a][3] * be + dkt.w * te;
      dotk[a] += adk[a][0] * kk.x + adk[a][1] * kk.y + adk[a][2] * kk.z + adk[a][3] * kk.w;
      if (i < cc.rows)
        *reinterpret_cast<float4*>(p.dk + elem0 + i * row_stride + s + 4 * tx) = make_float4(adk[a][0], adk[a][1], adk[a][2], adk[a][3]);
    }
    __syncthreads();
  }
  // ---- per Dv slice: dv = beta T^T d_u
  float rvb[4] = {0.f, 0.f, 0.f, 0.f};
  for (int s = 0; s < p.Dv; s += DP_C) {
    load_chunk(S0, p.d_u + cc.chunk * DP_C * p.Dv + s, p.Dv, nullptr);
    load_tokens(S1, p.v, p.in_bf16, velem0 + s, vrow_stride, cc.rows, nullptr);
    __syncthreads();
    zero(acc);
    mm_nn(acc, t2, S0, ty, tx);
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int i = ty + 16 * a;
      const float4 vv = *reinterpret_cast<const float4*>(S1 + i * DP_LD + 4 * tx);
      const float be = vec.beta[i];
      rvb[a] += acc[a][0] * vv.x + acc[a][1] * vv.y + acc[a][2] * vv.z + acc[a][3] * vv.w;
      if (i < cc.rows)
        *reinterpret_cast<float4*>(p.dv + velem0 + i * vrow_stride + s + 4 * tx) =
            make_float4(acc[a][0] * be, acc[a][1] * be, acc[a][2] * be, acc[a][3] * be);
    }
    __syncthreads();
  }
  // ---- row sums across the 16 threads of a row -> per-row vectors (v0: dot_q, v1: dot_k, v2: d_kt.k e^{..})
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int i = ty + 16 * a;
    const float s_rk1 = row_sum16(rk1[a]), s_rq1 = row_sum16(rq1[a]), s_rt1 = row_sum16(rt1[a]);
    const float s_dq = row_sum16(dotq[a]), s_dk = row_sum16(dotk[a]), s_vb = row_sum16(rvb[a]);
    if (tx == 0) {
      const float eg = vec.eg[i], r_kt = s_rt1 * vec.to_end[i];
      vec.v0[i] = s_dq;
      vec.v1[i] = s_dk;
      vec.v2[i] = r_kt;
      vec.v4[i] += eg * s_rk1 + s_vb;                                           // dbeta
      vec.v3[i] += vec.beta[i] * eg * s_rk1 + eg * s_rq1 - r_kt;                // dG
    }
  }
  __syncthreads();
  if (tid < DP_C) {
    // dG_last also collects every row's d_kt term and gamma's gradient; dg = reverse running sum of dG
    float tail = p.d_gamma[cc.chunk] * vec.eg[DP_C - 1];
    for (int j = 0; j < DP_C; ++j) tail += vec.v2[j];
    float s = tail;
    for (int j = DP_C - 1; j >= tid; --j) s += vec.v3[j];
    if (tid < cc.rows) {
      const int64_t at = (cc.tok0 + tid) * p.H + cc.h;
      p.dbeta[at] = vec.v4[tid];
      if (p.dg != nullptr) p.dg[at] = s;
    }
  }
  // ---- backward of the row normalisation (and of q's scale), on the values this CTA wrote above
  const float inv_s2 = p.l2norm ? 1.f / (p.scale * p.scale) : 0.f;
  const float k_on = p.l2norm ? 1.f : 0.f;
  for (int s = 0; s < p.D; s += DP_C) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int f = tid + DP_THREADS * e, r = f >> 4, c4 = (f & 15) * 4;
      if (r >= cc.rows) continue;
      const int64_t at = elem0 + r * row_stride + s + c4;
      const float4 qr = load4(p.q, at, p.in_bf16), kr = load4(p.k, at, p.in_bf16);
      float4 gq = *reinterpret_cast<const float4*>(p.dq + at), gk = *reinterpret_cast<const float4*>(p.dk + at);
      const float rq = vec.rq[r], rk = vec.rk[r];
      const float cq = vec.v0[r] * inv_s2 * rq, ck = vec.v1[r] * k_on * rk;    // (dot / scale^2) * (q_s / q),  dot * (k_n / k)
      gq = make_float4(rq * (gq.x - cq * qr.x), rq * (gq.y - cq * qr.y), rq * (gq.z - cq * qr.z), rq * (gq.w - cq * qr.w));
      gk = make_float4(rk * (gk.x - ck * kr.x), rk * (gk.y - ck * kr.y), rk * (gk.z - ck * kr.z), rk * (gk.w - ck * kr.w));
      *reinterpret_cast<float4*>(p.dq + at) = gq;
      *reinterpret_cast<float4*>(p.dk + at) = gk;
    }
  }
}

static int delta_prep_check(const DeltaPrepParams& p, int BH) {
  if (BH <= 0 || BH > 65535 || p.T <= 0 || p.H <= 0 || BH % p.H != 0 || p.n != (p.T + DP_C - 1) / DP_C) return TTCD_ERR_ARG;
  if (p.D < DP_C || p.D % DP_C != 0 || p.Dv < DP_C || p.Dv % DP_C != 0) return TTCD_ERR_ARG;
  return TTCD_OK;
}

}  // namespace ttcd

// q, k [B, T, H, D], v [B, T, H, Dv] contiguous, bf16 (in_bf16 = 1) or fp32; beta, g [B, T, H] fp32 (g may be null).
// Outputs fp32 in chunk layout, n = ceil(T / 64) chunks per (batch, head): w, kt, q_in [B*H, n, 64, D]; u [B*H, n, 64, Dv];
// qk [B*H, n, 64, 64]; gamma [B*H, n].  Rows beyond T act as beta = 0, g = 0.  D, Dv multiples of 64.
TTCD_EXPORT int ttcd_delta_prep_fwd(const void* q, const void* k, const void* v, const float* beta, const float* g, float* w,
                                    float* u, float* kt, float* q_in, float* qk, float* gamma, int B, int T, int H, int D,
                                    int Dv, float scale, int l2norm, int in_bf16, void* stream_ptr) {
  ttcd::DeltaPrepParams p = {};
  p.q = q; p.k = k; p.v = v; p.beta = beta; p.g = g;
  p.T = T; p.H = H; p.D = D; p.Dv = Dv; p.n = (T + ttcd::DP_C - 1) / ttcd::DP_C;
  p.scale = scale; p.l2norm = l2norm; p.in_bf16 = in_bf16;
  p.w = w; p.u = u; p.kt = kt; p.q_in = q_in; p.qk = qk; p.gamma = gamma;
  const int rc = ttcd::delta_prep_check(p, B * H);
  if (rc != TTCD_OK) return rc;
  static bool configured = false;
  if (!configured) {
    TTCD_CUDA_CHECK(cudaFuncSetAttribute(ttcd::delta_prep_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ttcd::DP_SMEM_FWD));
    configured = true;
  }
  ttcd::delta_prep_fwd_kernel<<<dim3(p.n, B * H), ttcd::DP_THREADS, ttcd::DP_SMEM_FWD, static_cast<cudaStream_t>(stream_ptr)>>>(p);
  return static_cast<int>(cudaGetLastError());
}

// Gradients of the six forward outputs (fp32, chunk layout) -> dq, dk [B, T, H, D], dv [B, T, H, Dv], dbeta, dg [B, T, H]
// (fp32; dg may be null when there is no gate).
TTCD_EXPORT int ttcd_delta_prep_bwd(const void* q, const void* k, const void* v, const float* beta, const float* g,
                                    const float* d_w, const float* d_u, const float* d_kt, const float* d_qin,
                                    const float* d_qk, const float* d_gamma, float* dq, float* dk, float* dv, float* dbeta,
                                    float* dg, int B, int T, int H, int D, int Dv, float scale, int l2norm, int in_bf16,
                                    void* stream_ptr) {
  ttcd::DeltaPrepParams p = {};
  p.q = q; p.k = k; p.v = v; p.beta = beta; p.g = g;
  p.T = T; p.H = H; p.D = D; p.Dv = Dv; p.n = (T + ttcd::DP_C - 1) / ttcd::DP_C;
  p.scale = scale; p.l2norm = l2norm; p.in_bf16 = in_bf16;
  p.d_w = d_w; p.d_u = d_u; p.d_kt = d_kt; p.d_qin = d_qin; p.d_qk = d_qk; p.d_gamma = d_gamma;
  p.dq = dq; p.dk = dk; p.dv = dv; p.dbeta = dbeta; p.dg = dg;
  const int rc = ttcd::delta_prep_check(p, B * H);
  if (rc != TTCD_OK) return rc;
  static bool configured = false;
  if (!configured) {
    TTCD_CUDA_CHECK(cudaFuncSetAttribute(ttcd::delta_prep_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ttcd::DP_SMEM_BWD));
    configured = true;
  }
  ttcd::delta_prep_bwd_kernel<<<dim3(p.n, B * H), ttcd::DP_THREADS, ttcd::DP_SMEM_BWD, static_cast<cudaStream_t>(stream_ptr)>>>(p);
  return static_cast<int>(cudaGetLastError());
}
