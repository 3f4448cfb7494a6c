// The chunk-local part of the (gated) delta rule, forward and backward, one CTA per (batch, head, 64-token chunk)
// (sm_100a; the 64 x 64 x 64 products run on the tensor cores as TF32 mma.sync tiles with fp32 accumulation, out of
// fp32 tiles in shared memory; the triangular inverse and all element-wise work stay fp32.  The products of a chunk are
// too small for a tcgen05 pipeline; the point of the kernels is to replace some forty element-wise / batched-GEMM /
// triangular-solve launches over fp32 [B,H,T,D] tensors by one pass that reads q, k, v once).
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
constexpr int DP_LDA = 68;                // row stride (floats) of a tile read as the A operand, or row-wise as B (X Y^T)
constexpr int DP_LDB = 72;                // row stride of a tile read column-wise as the B operand (M X)
constexpr int DP_TILE_A = DP_C * DP_LDA;
constexpr int DP_TILE_B = DP_C * DP_LDB;
constexpr int DP_THREADS = 256;
constexpr int DP_VEC = 8 * DP_C + 8 * 2 * DP_C;     // 8 per-row vectors + 8 pairs of partial row sums
constexpr int DP_SMEM_FWD = (3 * DP_TILE_A + 2 * DP_TILE_B + DP_VEC) * 4;
constexpr int DP_SMEM_BWD = (3 * DP_TILE_A + 3 * DP_TILE_B + DP_VEC) * 4;

struct DeltaPrepParams {
  const void* q; const void* k; const void* v;      // [B, T, H, D | Dv], bf16 or fp32 (in_bf16)
  const float* beta; const float* g;                // [B, T, H]; g null: no gate
  int T, H, D, Dv, n;                               // n = chunks per sequence
  float scale; int l2norm; int in_bf16;
  bf16 *w, *kt;                                     // forward outputs, chunk layout [B*H, n, 64, *]: the chain's tile operands in bf16,
  float *u, *q_in, *qk, *gamma;                     // the rest fp32
  const float *d_w, *d_u, *d_kt, *d_qin, *d_qk, *d_gamma;
  float *dq, *dk, *dv, *dbeta, *dg;                 // backward outputs, token layout [B, T, H, *] fp32
};

// ---- 64 x 64 x 64 products as TF32 m16n8k8 tiles -----------------------------------------------------------------
// Warp (wr, wc) of the 4 x 2 warp grid owns rows 16 wr .. +15 and columns 32 wc .. +31 (four n-tiles of 8); lane
// (g = lane / 4, c = lane % 4) holds, of n-tile t, the elements (r0, j), (r0, j + 1), (r1, j), (r1, j + 1) with
// r0 = 16 wr + g, r1 = r0 + 8, j = 32 wc + 8 t + 2 c  ->  acc[t][0..3].
struct Own {
  int r0, r1, wr, wc, g, c;
  __device__ Own() {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    wr = warp >> 1; wc = warp & 1; g = lane >> 2; c = lane & 3;
    r0 = 16 * wr + g; r1 = r0 + 8;
  }
  __device__ __forceinline__ int col(int t) const { return 32 * wc + 8 * t + 2 * c; }
};
__device__ __forceinline__ uint32_t tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void load_a(uint32_t (&a)[4], const float* X, const Own& o, int k0) {
  a[0] = tf32(X[o.r0 * DP_LDA + k0 + o.c]);
  a[1] = tf32(X[o.r1 * DP_LDA + k0 + o.c]);
  a[2] = tf32(X[o.r0 * DP_LDA + k0 + o.c + 4]);
  a[3] = tf32(X[o.r1 * DP_LDA + k0 + o.c + 4]);
}
// B operands that were rounded to TF32 when their tile was written (ROUNDED_B) are fed as they are.
// acc += X Y^T:  acc(i, j) += sum_d X[i][d] Y[j][d]      (both tiles with row stride DP_LDA)
template <bool ROUNDED_B>
__device__ __forceinline__ void mm_nt(float (&acc)[4][4], const float* X, const float* Y, const Own& o) {
#pragma unroll 2
  for (int k0 = 0; k0 < DP_C; k0 += 8) {
    uint32_t a[4];
    load_a(a, X, o, k0);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float* y = Y + (32 * o.wc + 8 * t + o.g) * DP_LDA + k0 + o.c;
      if (ROUNDED_B) mma_tf32(acc[t], a, __float_as_uint(y[0]), __float_as_uint(y[4]));
      else mma_tf32(acc[t], a, tf32(y[0]), tf32(y[4]));
    }
  }
}
// acc += M X:    acc(i, j) += sum_k M[i][k] X[k][j]      (M with row stride DP_LDA, X with DP_LDB)
template <bool ROUNDED_B>
__device__ __forceinline__ void mm_nn(float (&acc)[4][4], const float* M, const float* X, const Own& o) {
#pragma unroll 2
  for (int k0 = 0; k0 < DP_C; k0 += 8) {
    uint32_t a[4];
    load_a(a, M, o, k0);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float* x = X + (k0 + o.c) * DP_LDB + 32 * o.wc + 8 * t + o.g;
      if (ROUNDED_B) mma_tf32(acc[t], a, __float_as_uint(x[0]), __float_as_uint(x[4 * DP_LDB]));
      else mma_tf32(acc[t], a, tf32(x[0]), tf32(x[4 * DP_LDB]));
    }
  }
}
__device__ __forceinline__ void zero(float (&acc)[4][4]) {
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
}
// sum over the four lanes (c) that share the rows r0, r1 of a warp; every one of them gets the total
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  return v;
}
// a thread's sums over its columns of rows r0 / r1 -> the warp-column's slot of a pair of partial row sums
__device__ __forceinline__ void put_row_partials(float* pair, const Own& o, float s0, float s1) {
  s0 = quad_sum(s0);
  s1 = quad_sum(s1);
  if (o.c == 0) { pair[o.wc * DP_C + o.r0] = s0; pair[o.wc * DP_C + o.r1] = s1; }
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
// A tile travels in two halves so that its global loads can be in flight while the previous tile is multiplied:
// fetch_* issues the loads into registers, store_* (after the barrier that frees the shared-memory tile) converts,
// scales and writes them.
struct RawTile { uint4 w[4]; };
__device__ __forceinline__ float4 round4(float4 x) {
  return make_float4(__uint_as_float(tf32(x.x)), __uint_as_float(tf32(x.y)), __uint_as_float(tf32(x.z)), __uint_as_float(tf32(x.w)));
}
// token layout [.., T, H, width]: row r of the chunk is token t0 + r (zero beyond `rows`)
__device__ __forceinline__ void fetch_tokens(RawTile& t, const void* src, bool bf, int64_t elem0, int64_t row_stride, int rows) {
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int f = threadIdx.x + DP_THREADS * e, r = f >> 4, c4 = (f & 15) * 4;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < rows) {
      if (bf) {
        const uint2 h = *reinterpret_cast<const uint2*>(static_cast<const bf16*>(src) + elem0 + r * row_stride + c4);
        v.x = h.x; v.y = h.y;
      } else {
        v = *reinterpret_cast<const uint4*>(static_cast<const float*>(src) + elem0 + r * row_stride + c4);
      }
    }
    t.w[e] = v;
  }
}
// ROUND: the tile is stored rounded to TF32 (it is only multiplied, as an operand of the products)
template <bool ROUND>
__device__ __forceinline__ void store_tokens(float* dst, int ld, const RawTile& t, bool bf, const float* mul) {
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int f = threadIdx.x + DP_THREADS * e, r = f >> 4, c4 = (f & 15) * 4;
    const uint4 v = t.w[e];
    float4 x;
    if (bf) {
      const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&v.x);
      const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&v.y);
      x = make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
    } else {
      x = make_float4(__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z), __uint_as_float(v.w));
    }
    const float m = mul != nullptr ? mul[r] : 1.f;
    x = make_float4(x.x * m, x.y * m, x.z * m, x.w * m);
    *reinterpret_cast<float4*>(dst + r * ld + c4) = ROUND ? round4(x) : x;
  }
}
// chunk layout [.., 64, width] fp32 (all 64 rows exist), stored rounded to TF32
__device__ __forceinline__ void fetch_chunk(RawTile& t, const float* src, int width) {
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int f = threadIdx.x + DP_THREADS * e, r = f >> 4, c4 = (f & 15) * 4;
    t.w[e] = *reinterpret_cast<const uint4*>(src + static_cast<int64_t>(r) * width + c4);
  }
}
__device__ __forceinline__ void store_chunk(float* dst, int ld, const RawTile& t) {
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int f = threadIdx.x + DP_THREADS * e, r = f >> 4, c4 = (f & 15) * 4;
    const uint4 v = t.w[e];
    *reinterpret_cast<float4*>(dst + r * ld + c4) =
        round4(make_float4(__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z), __uint_as_float(v.w)));
  }
}

// per-row vectors and pairs of partial row sums (one half per warp column) in shared memory
struct DeltaVec {
  float *beta, *G, *eg, *to_end, *rq, *rk, *m0, *m1;
  float* pair[8];
  __device__ explicit DeltaVec(float* p)
      : beta(p), G(p + 64), eg(p + 128), to_end(p + 192), rq(p + 256), rk(p + 320), m0(p + 384), m1(p + 448) {
#pragma unroll
    for (int i = 0; i < 8; ++i) pair[i] = p + 512 + 128 * i;
  }
  __device__ __forceinline__ float total(int i, int row) const { return pair[i][row] + pair[i][DP_C + row]; }
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
    vec.m0[tid] = (ok && p.g != nullptr) ? p.g[at] : 0.f;
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
    for (int j = 0; j <= tid; ++j) s += vec.m0[j];
    vec.G[tid] = s;
  }
  __syncthreads();
  if (tid < DP_C) {
    vec.eg[tid] = expf(vec.G[tid]);
    vec.to_end[tid] = expf(vec.G[DP_C - 1] - vec.G[tid]);
  }
  __syncthreads();
}

// A = k k^T and QK = q k^T over all D (in the threads' accumulator layout); S0, S1: two scratch tiles
__device__ __forceinline__ void chunk_grams(const DeltaPrepParams& p, const ChunkCoord& cc, const DeltaVec& vec, float* S0,
                                            float* S1, float (&A)[4][4], float (&QK)[4][4], const Own& o) {
  zero(A);
  zero(QK);
  const int64_t row_stride = static_cast<int64_t>(p.H) * p.D;
  const int64_t elem0 = (cc.tok0 * p.H + cc.h) * p.D;
  RawTile rk, rq;
  fetch_tokens(rk, p.k, p.in_bf16, elem0, row_stride, cc.rows);
  fetch_tokens(rq, p.q, p.in_bf16, elem0, row_stride, cc.rows);
  for (int s = 0; s < p.D; s += DP_C) {
    store_tokens<true>(S0, DP_LDA, rk, p.in_bf16, vec.rk);
    store_tokens<true>(S1, DP_LDA, rq, p.in_bf16, vec.rq);
    __syncthreads();
    if (s + DP_C < p.D) {
      fetch_tokens(rk, p.k, p.in_bf16, elem0 + s + DP_C, row_stride, cc.rows);
      fetch_tokens(rq, p.q, p.in_bf16, elem0 + s + DP_C, row_stride, cc.rows);
    }
    mm_nt<true>(A, S0, S0, o);
    mm_nt<true>(QK, S1, S0, o);
    __syncthreads();
  }
}

// T = (I + L)^-1 by forward substitution, column by column: column c belongs to the four lanes 4 c .. 4 c + 3 of one
// warp, which split the sum over earlier rows.  Writes T (Tm) and, if asked, its transpose (TTm).  fp32 throughout.
__device__ __forceinline__ void chunk_inverse(const float* Lm, float* Tm, float* TTm) {
  const int c = threadIdx.x >> 2, part = threadIdx.x & 3;
  for (int i = 0; i < DP_C; ++i) {
    float s = 0.f;
    for (int j = c + part; j < i; j += 4) s = fmaf(Lm[i * DP_LDA + j], Tm[j * DP_LDA + c], s);
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    if (part == 0) {
      const float t = i == c ? 1.f : (i > c ? -s : 0.f);
      Tm[i * DP_LDA + c] = t;
      if (TTm != nullptr) TTm[c * DP_LDA + i] = t;
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
  float* Tm = Lm + DP_TILE_A;
  float* Tu = Tm + DP_TILE_A;            // T with the columns scaled for u
  float* S0 = Tu + DP_TILE_A;
  float* S1 = S0 + DP_TILE_B;
  const DeltaVec vec(S1 + DP_TILE_B);
  const int tid = threadIdx.x;
  const Own o;
  const ChunkCoord cc = chunk_coord(p);

  chunk_rows(p, cc, vec);
  float A[4][4], QK[4][4];
  chunk_grams(p, cc, vec, S0, S1, A, QK, o);
  const int64_t row_stride = static_cast<int64_t>(p.H) * p.D, vrow_stride = static_cast<int64_t>(p.H) * p.Dv;
  const int64_t elem0 = (cc.tok0 * p.H + cc.h) * p.D, velem0 = (cc.tok0 * p.H + cc.h) * p.Dv;
  RawTile ra, rb;                        // the next tiles, in flight while the current ones are worked on
  fetch_tokens(ra, p.k, p.in_bf16, elem0, row_stride, cc.rows);
  fetch_tokens(rb, p.q, p.in_bf16, elem0, row_stride, cc.rows);
  // L (strictly lower) into shared memory, qk = lower(dec QK) into S1 for a coalesced copy out
#pragma unroll
  for (int t = 0; t < 4; ++t)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = e < 2 ? o.r0 : o.r1, j = o.col(t) + (e & 1);
      const float dec = i >= j ? expf(vec.G[i] - vec.G[j]) : 0.f;
      Lm[i * DP_LDA + j] = i > j ? vec.beta[i] * dec * A[t][e] : 0.f;
      S1[i * DP_LDB + j] = dec * QK[t][e];
    }
  __syncthreads();
  {
    float* out = p.qk + cc.chunk * DP_C * DP_C;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int f = tid + DP_THREADS * e, r = f >> 4, c4 = (f & 15) * 4;
      *reinterpret_cast<float4*>(out + r * DP_C + c4) = *reinterpret_cast<const float4*>(S1 + r * DP_LDB + c4);
    }
    if (tid == 0) p.gamma[cc.chunk] = vec.eg[DP_C - 1];
  }
  chunk_inverse(Lm, Tm, nullptr);
  __syncthreads();
  // fold the row factors of the right-hand sides into the columns of T:  w = (T diag(beta e^G)) k,  u = (T diag(beta)) v
#pragma unroll
  for (int e = 0; e < 16; ++e) {
    const int f = tid + DP_THREADS * e, i = f >> 6, j = f & 63;
    const float t = Tm[i * DP_LDA + j];
    Lm[i * DP_LDA + j] = t * vec.beta[j] * vec.eg[j];
    Tu[i * DP_LDA + j] = t * vec.beta[j];
  }
  __syncthreads();
  const float* Tw = Lm;
  for (int s = 0; s < p.D; s += DP_C) {
    store_tokens<false>(S0, DP_LDB, ra, p.in_bf16, vec.rk);     // exact: kt, q_in are written from these
    store_tokens<false>(S1, DP_LDB, rb, p.in_bf16, vec.rq);
    __syncthreads();
    if (s + DP_C < p.D) {
      fetch_tokens(ra, p.k, p.in_bf16, elem0 + s + DP_C, row_stride, cc.rows);
      fetch_tokens(rb, p.q, p.in_bf16, elem0 + s + DP_C, row_stride, cc.rows);
    } else {
      fetch_tokens(ra, p.v, p.in_bf16, velem0, vrow_stride, cc.rows);
    }
    // kt = e^{G_last - G} k, q_in = e^G q (element-wise, in the loaders' layout)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int f = tid + DP_THREADS * e, r = f >> 4, c4 = (f & 15) * 4;
      const float4 kk = *reinterpret_cast<const float4*>(S0 + r * DP_LDB + c4);
      const float4 qq = *reinterpret_cast<const float4*>(S1 + r * DP_LDB + c4);
      const float te = vec.to_end[r], eg = vec.eg[r];
      const int64_t at = (cc.chunk * DP_C + r) * p.D + s + c4;
      const __nv_bfloat162 k01 = __floats2bfloat162_rn(kk.x * te, kk.y * te), k23 = __floats2bfloat162_rn(kk.z * te, kk.w * te);
      *reinterpret_cast<uint2*>(p.kt + at) = make_uint2(*reinterpret_cast<const uint32_t*>(&k01), *reinterpret_cast<const uint32_t*>(&k23));
      *reinterpret_cast<float4*>(p.q_in + at) = make_float4(qq.x * eg, qq.y * eg, qq.z * eg, qq.w * eg);
    }
    float acc[4][4];
    zero(acc);
    mm_nn<false>(acc, Tw, S0, o);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      *reinterpret_cast<__nv_bfloat162*>(p.w + (cc.chunk * DP_C + o.r0) * p.D + s + o.col(t)) = __floats2bfloat162_rn(acc[t][0], acc[t][1]);
      *reinterpret_cast<__nv_bfloat162*>(p.w + (cc.chunk * DP_C + o.r1) * p.D + s + o.col(t)) = __floats2bfloat162_rn(acc[t][2], acc[t][3]);
    }
    __syncthreads();
  }
  for (int s = 0; s < p.Dv; s += DP_C) {
    store_tokens<true>(S0, DP_LDB, ra, p.in_bf16, nullptr);
    __syncthreads();
    if (s + DP_C < p.Dv) fetch_tokens(ra, p.v, p.in_bf16, velem0 + s + DP_C, vrow_stride, cc.rows);
    float acc[4][4];
    zero(acc);
    mm_nn<true>(acc, Tu, S0, o);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      *reinterpret_cast<float2*>(p.u + (cc.chunk * DP_C + o.r0) * p.Dv + s + o.col(t)) = make_float2(acc[t][0], acc[t][1]);
      *reinterpret_cast<float2*>(p.u + (cc.chunk * DP_C + o.r1) * p.Dv + s + o.col(t)) = make_float2(acc[t][2], acc[t][3]);
    }
    __syncthreads();
  }
}

// =====================================================================================================
// backward
// =====================================================================================================
// pairs of partial row sums
enum { PR_E = 0, PR_B = 1, PR_RK1 = 2, PR_RQ1 = 3, PR_RT1 = 4, PR_DOTQ = 5, PR_DOTK = 6, PR_VB = 7 };

__global__ void __launch_bounds__(DP_THREADS, 2) delta_prep_bwd_kernel(const DeltaPrepParams p) {
  extern __shared__ __align__(16) float dp_smem[];
  float* t0 = dp_smem;                   // L -> d_T (read column-wise) -> M1 + M1^T
  float* t1 = t0 + DP_TILE_B;            // T -> M2^T
  float* t2 = t1 + DP_TILE_A;            // T^T
  float* t3 = t2 + DP_TILE_A;            // T^T d_T -> M2
  float* S0 = t3 + DP_TILE_A;
  float* S1 = S0 + DP_TILE_B;
  const DeltaVec vec(S1 + DP_TILE_B);
  const int tid = threadIdx.x;
  const Own o;
  const ChunkCoord cc = chunk_coord(p);
  const int64_t row_stride = static_cast<int64_t>(p.H) * p.D, vrow_stride = static_cast<int64_t>(p.H) * p.Dv;
  const int64_t elem0 = (cc.tok0 * p.H + cc.h) * p.D, velem0 = (cc.tok0 * p.H + cc.h) * p.Dv;

  chunk_rows(p, cc, vec);
  float A[4][4], QK[4][4];
  chunk_grams(p, cc, vec, S0, S1, A, QK, o);
#pragma unroll
  for (int t = 0; t < 4; ++t)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = e < 2 ? o.r0 : o.r1, j = o.col(t) + (e & 1);
      t0[i * DP_LDA + j] = i > j ? vec.beta[i] * expf(vec.G[i] - vec.G[j]) * A[t][e] : 0.f;
    }
  if (tid < DP_C) { vec.m0[tid] = vec.beta[tid] * vec.eg[tid] * vec.rk[tid]; vec.m1[tid] = vec.beta[tid]; }
  RawTile ra, rb;                        // the next tiles, in flight while the current ones are worked on
  const int nd = p.D / DP_C, nv = p.Dv / DP_C;
  // tile pair `it` of the d_T sum: (d_w, beta e^G k) slices first, then (d_u, beta v) slices
  auto fetch_dT = [&](int it) {
    if (it < nd) {
      fetch_chunk(ra, p.d_w + cc.chunk * DP_C * p.D + it * DP_C, p.D);
      fetch_tokens(rb, p.k, p.in_bf16, elem0 + it * DP_C, row_stride, cc.rows);
    } else {
      fetch_chunk(ra, p.d_u + cc.chunk * DP_C * p.Dv + (it - nd) * DP_C, p.Dv);
      fetch_tokens(rb, p.v, p.in_bf16, velem0 + (it - nd) * DP_C, vrow_stride, cc.rows);
    }
  };
  fetch_dT(0);
  __syncthreads();
  chunk_inverse(t0, t1, t2);
  __syncthreads();

  // ---- d_T = d_w (beta e^G k)^T + d_u (beta v)^T
  float acc[4][4];
  zero(acc);
  for (int it = 0; it < nd + nv; ++it) {
    store_chunk(S0, DP_LDA, ra);
    store_tokens<true>(S1, DP_LDA, rb, p.in_bf16, it < nd ? vec.m0 : vec.m1);
    __syncthreads();
    if (it + 1 < nd + nv) {
      fetch_dT(it + 1);
    } else {                             // the first tiles of the dq / dk loop, in flight over the d_L phase
      fetch_tokens(ra, p.k, p.in_bf16, elem0, row_stride, cc.rows);
      fetch_tokens(rb, p.q, p.in_bf16, elem0, row_stride, cc.rows);
    }
    mm_nt<true>(acc, S0, S1, o);
    __syncthreads();
  }
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    *reinterpret_cast<uint2*>(t0 + o.r0 * DP_LDB + o.col(t)) = make_uint2(tf32(acc[t][0]), tf32(acc[t][1]));     // B operand below
    *reinterpret_cast<uint2*>(t0 + o.r1 * DP_LDB + o.col(t)) = make_uint2(tf32(acc[t][2]), tf32(acc[t][3]));
  }
  __syncthreads();
  // ---- d_L = -strict_lower(T^T d_T T^T)
  zero(acc);
  mm_nn<true>(acc, t2, t0, o);                                  // X1 = T^T d_T
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    *reinterpret_cast<float2*>(t3 + o.r0 * DP_LDA + o.col(t)) = make_float2(acc[t][0], acc[t][1]);
    *reinterpret_cast<float2*>(t3 + o.r1 * DP_LDA + o.col(t)) = make_float2(acc[t][2], acc[t][3]);
  }
  __syncthreads();
  zero(acc);
  mm_nt<false>(acc, t3, t1, o);                                 // X1 T^T  (T is kept exact)
  __syncthreads();                                              // t0 (d_T), t1 (T), t3 (X1) are free from here
  // ---- element-wise on the owned elements: M1 (+ its transpose) -> t0, M2 -> t3, M2^T -> t1; row / column sums
  {
    const float* dqk = p.d_qk + cc.chunk * DP_C * DP_C;
    float e_row[2] = {0.f, 0.f}, b_row[2] = {0.f, 0.f};
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      float e_col[2] = {0.f, 0.f};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = e < 2 ? o.r0 : o.r1, j = o.col(t) + (e & 1);
        const float dec = i >= j ? expf(vec.G[i] - vec.G[j]) : 0.f;
        const float dl = i > j ? -acc[t][e] : 0.f;
        const float m1 = dl * vec.beta[i] * dec;
        const float m2 = dqk[i * DP_C + j] * dec;
        const float ee = m1 * A[t][e] + m2 * QK[t][e];         // d_L L + M2 QK
        e_row[e >> 1] += ee;
        e_col[e & 1] += ee;
        b_row[e >> 1] += dl * dec * A[t][e];
        if (i > j) { t0[i * DP_LDA + j] = m1; t0[j * DP_LDA + i] = m1; }
        if (i == j) t0[i * DP_LDA + j] = 0.f;
        t3[i * DP_LDA + j] = m2;
        t1[j * DP_LDA + i] = m2;
      }
      // column sums of E over the warp's 16 rows -> S0[wr][j], added up by 64 threads below
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float v = e_col[h];
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        v += __shfl_xor_sync(0xffffffffu, v, 8);
        v += __shfl_xor_sync(0xffffffffu, v, 16);
        if (o.g == 0) S0[o.wr * DP_LDB + o.col(t) + h] = v;
      }
    }
    put_row_partials(vec.pair[PR_E], o, e_row[0], e_row[1]);
    put_row_partials(vec.pair[PR_B], o, b_row[0], b_row[1]);
  }
  __syncthreads();
  if (tid < DP_C) {
    float s = 0.f;
    for (int y = 0; y < 4; ++y) s += S0[y * DP_LDB + tid];
    vec.m0[tid] = vec.total(PR_E, tid) - s;                     // dG so far: row sum - column sum of E
  }
  __syncthreads();

  // ---- per D slice: dq, dk (with respect to the normalised rows), kept in the outputs until the row dots are known
  float rk1[2] = {0.f, 0.f}, rq1[2] = {0.f, 0.f}, rt1[2] = {0.f, 0.f}, dotq[2] = {0.f, 0.f}, dotk[2] = {0.f, 0.f};
  RawTile rc;
  for (int s = 0; s < p.D; s += DP_C) {
    store_tokens<true>(S0, DP_LDB, ra, p.in_bf16, vec.rk);
    store_tokens<true>(S1, DP_LDB, rb, p.in_bf16, vec.rq);
    __syncthreads();
    fetch_chunk(rc, p.d_w + cc.chunk * DP_C * p.D + s, p.D);     // needed after the first epilogue
    float adq[4][4], adk[4][4];
    zero(adq);
    zero(adk);
    mm_nn<true>(adq, t3, S0, o);                                // M2 k
    mm_nn<true>(adk, t0, S0, o);                                // (M1 + M1^T) k
    mm_nn<true>(adk, t1, S1, o);                                // M2^T q
#pragma unroll
    for (int t = 0; t < 4; ++t)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int i = h ? o.r1 : o.r0, j = o.col(t);
        const float2 dqi = *reinterpret_cast<const float2*>(p.d_qin + (cc.chunk * DP_C + i) * p.D + s + j);
        const float2 qq = *reinterpret_cast<const float2*>(S1 + i * DP_LDB + j);
        const float eg = vec.eg[i];
        const float x0 = fmaf(dqi.x, eg, adq[t][2 * h]), x1 = fmaf(dqi.y, eg, adq[t][2 * h + 1]);
        rq1[h] += dqi.x * qq.x + dqi.y * qq.y;
        dotq[h] += x0 * qq.x + x1 * qq.y;
        if (i < cc.rows) *reinterpret_cast<float2*>(p.dq + elem0 + i * row_stride + s + j) = make_float2(x0, x1);
      }
    __syncthreads();
    store_chunk(S1, DP_LDB, rc);
    __syncthreads();
    if (s + DP_C < p.D) {
      fetch_tokens(ra, p.k, p.in_bf16, elem0 + s + DP_C, row_stride, cc.rows);
      fetch_tokens(rb, p.q, p.in_bf16, elem0 + s + DP_C, row_stride, cc.rows);
    } else {                             // the first tiles of the dv loop
      fetch_chunk(ra, p.d_u + cc.chunk * DP_C * p.Dv, p.Dv);
      fetch_tokens(rb, p.v, p.in_bf16, velem0, vrow_stride, cc.rows);
    }
    zero(adq);
    mm_nn<true>(adq, t2, S1, o);                                // d_kbg = T^T d_w
#pragma unroll
    for (int t = 0; t < 4; ++t)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int i = h ? o.r1 : o.r0, j = o.col(t);
        const float2 dkt = *reinterpret_cast<const float2*>(p.d_kt + (cc.chunk * DP_C + i) * p.D + s + j);
        const float2 kk = *reinterpret_cast<const float2*>(S0 + i * DP_LDB + j);
        const float be = vec.beta[i] * vec.eg[i], te = vec.to_end[i];
        const float d0 = adq[t][2 * h], d1 = adq[t][2 * h + 1];
        rk1[h] += d0 * kk.x + d1 * kk.y;
        rt1[h] += dkt.x * kk.x + dkt.y * kk.y;
        const float x0 = adk[t][2 * h] + d0 * be + dkt.x * te, x1 = adk[t][2 * h + 1] + d1 * be + dkt.y * te;
        dotk[h] += x0 * kk.x + x1 * kk.y;
        if (i < cc.rows) *reinterpret_cast<float2*>(p.dk + elem0 + i * row_stride + s + j) = make_float2(x0, x1);
      }
    __syncthreads();
  }
  // ---- per Dv slice: dv = beta T^T d_u
  float rvb[2] = {0.f, 0.f};
  for (int s = 0; s < p.Dv; s += DP_C) {
    store_chunk(S0, DP_LDB, ra);
    store_tokens<true>(S1, DP_LDB, rb, p.in_bf16, nullptr);
    __syncthreads();
    if (s + DP_C < p.Dv) {
      fetch_chunk(ra, p.d_u + cc.chunk * DP_C * p.Dv + s + DP_C, p.Dv);
      fetch_tokens(rb, p.v, p.in_bf16, velem0 + s + DP_C, vrow_stride, cc.rows);
    }
    zero(acc);
    mm_nn<true>(acc, t2, S0, o);
#pragma unroll
    for (int t = 0; t < 4; ++t)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int i = h ? o.r1 : o.r0, j = o.col(t);
        const float2 vv = *reinterpret_cast<const float2*>(S1 + i * DP_LDB + j);
        const float be = vec.beta[i];
        rvb[h] += acc[t][2 * h] * vv.x + acc[t][2 * h + 1] * vv.y;
        if (i < cc.rows)
          *reinterpret_cast<float2*>(p.dv + velem0 + i * vrow_stride + s + j) = make_float2(acc[t][2 * h] * be, acc[t][2 * h + 1] * be);
      }
    __syncthreads();
  }
  put_row_partials(vec.pair[PR_RK1], o, rk1[0], rk1[1]);
  put_row_partials(vec.pair[PR_RQ1], o, rq1[0], rq1[1]);
  put_row_partials(vec.pair[PR_RT1], o, rt1[0], rt1[1]);
  put_row_partials(vec.pair[PR_DOTQ], o, dotq[0], dotq[1]);
  put_row_partials(vec.pair[PR_DOTK], o, dotk[0], dotk[1]);
  put_row_partials(vec.pair[PR_VB], o, rvb[0], rvb[1]);
  __syncthreads();
  // ---- per-row results: dbeta, dG (m0), the d_kt term of every row (m1)
  float dbeta_i = 0.f;
  if (tid < DP_C) {
    const float eg = vec.eg[tid], s_rk1 = vec.total(PR_RK1, tid);
    const float r_kt = vec.total(PR_RT1, tid) * vec.to_end[tid];
    dbeta_i = vec.total(PR_B, tid) + eg * s_rk1 + vec.total(PR_VB, tid);
    vec.m0[tid] += vec.beta[tid] * eg * s_rk1 + eg * vec.total(PR_RQ1, tid) - r_kt;
    vec.m1[tid] = r_kt;
  }
  __syncthreads();
  if (tid < DP_C) {
    // dG_last also collects every row's d_kt term and gamma's gradient; dg = reverse running sum of dG
    float s = p.d_gamma[cc.chunk] * vec.eg[DP_C - 1];
    for (int j = 0; j < DP_C; ++j) s += vec.m1[j];
    for (int j = DP_C - 1; j >= tid; --j) s += vec.m0[j];
    if (tid < cc.rows) {
      const int64_t at = (cc.tok0 + tid) * p.H + cc.h;
      p.dbeta[at] = dbeta_i;
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
      const float cq = vec.total(PR_DOTQ, r) * inv_s2 * rq, ck = vec.total(PR_DOTK, r) * k_on * rk;
      gq = make_float4(rq * (gq.x - cq * qr.x), rq * (gq.y - cq * qr.y), rq * (gq.z - cq * qr.z), rq * (gq.w - cq * qr.w));
      gk = make_float4(rk * (gk.x - ck * kr.x), rk * (gk.y - ck * kr.y), rk * (gk.z - ck * kr.z), rk * (gk.w - ck * kr.w));
      *reinterpret_cast<float4*>(p.dq + at) = gq;
      *reinterpret_cast<float4*>(p.dk + at) = gk;
    }
  }
}

// ---- layout changes between token rows [B, T, H, W] and chunk rows [B*H, n*64, W] (fp32), one 16-byte group per thread
__global__ void __launch_bounds__(256) delta_rows_kernel(const void* src, void* dst, int T, int H, int n, int W, int64_t groups,
                                                         int to_tokens, int token_bf16) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= groups) return;
  const int wq = W / 4;
  const int c4 = static_cast<int>(idx % wq) * 4;
  const int64_t row = idx / wq;                                  // chunk row: (b * H + h) * n * 64 + t
  const int t = static_cast<int>(row % (static_cast<int64_t>(n) * DP_C));
  const int64_t bh = row / (static_cast<int64_t>(n) * DP_C);
  const int64_t tok = ((bh / H) * T + t) * H + bh % H;           // token row: (b * T + t) * H + h
  if (to_tokens) {
    if (t >= T) return;
    const float4 x = *reinterpret_cast<const float4*>(static_cast<const float*>(src) + row * W + c4);
    if (token_bf16) {
      const __nv_bfloat162 lo = __floats2bfloat162_rn(x.x, x.y), hi = __floats2bfloat162_rn(x.z, x.w);
      uint2 raw;
      raw.x = *reinterpret_cast<const uint32_t*>(&lo);
      raw.y = *reinterpret_cast<const uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(static_cast<bf16*>(dst) + tok * W + c4) = raw;
    } else {
      *reinterpret_cast<float4*>(static_cast<float*>(dst) + tok * W + c4) = x;
    }
  } else {
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
    if (t < T) x = load4(src, tok * W + c4, token_bf16 != 0);
    *reinterpret_cast<float4*>(static_cast<float*>(dst) + row * W + c4) = x;
  }
}

static int delta_prep_check(const DeltaPrepParams& p, int BH) {
  if (BH <= 0 || BH > 65535 || p.T <= 0 || p.H <= 0 || BH % p.H != 0 || p.n != (p.T + DP_C - 1) / DP_C) return TTCD_ERR_ARG;
  if (p.D < DP_C || p.D % DP_C != 0 || p.Dv < DP_C || p.Dv % DP_C != 0) return TTCD_ERR_ARG;
  return TTCD_OK;
}

}  // namespace ttcd

// q, k [B, T, H, D], v [B, T, H, Dv] contiguous, bf16 (in_bf16 = 1) or fp32; beta, g [B, T, H] fp32 (g may be null).
// Outputs in chunk layout, n = ceil(T / 64) chunks per (batch, head): w, kt [B*H, n, 64, D] bf16 (the chain kernel's tile
// operands); fp32: q_in [B*H, n, 64, D], u [B*H, n, 64, Dv], qk [B*H, n, 64, 64], gamma [B*H, n].  Rows beyond T act as beta = 0, g = 0.  D, Dv multiples of 64.
TTCD_EXPORT int ttcd_delta_prep_fwd(const void* q, const void* k, const void* v, const float* beta, const float* g, bf16* w,
                                    float* u, bf16* kt, float* q_in, float* qk, float* gamma, int B, int T, int H, int D,
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

// Chunk rows [B*H, n*64, W] fp32 -> token rows [B, T, H, W] (bf16 or fp32; rows beyond T are dropped), or the reverse
// (rows beyond T zero).  W a multiple of 4; both buffers 16-byte aligned.
TTCD_EXPORT int ttcd_delta_rows(const void* src, void* dst, int B, int T, int H, int W, int to_tokens, int token_bf16,
                                void* stream_ptr) {
  if (B <= 0 || T <= 0 || H <= 0 || W <= 0 || W % 4 != 0) return TTCD_ERR_ARG;
  const int n = (T + ttcd::DP_C - 1) / ttcd::DP_C;
  const int64_t groups = static_cast<int64_t>(B) * H * n * ttcd::DP_C * (W / 4);
  const int64_t blocks = (groups + 255) / 256;
  if (blocks > 0x7fffffffLL) return TTCD_ERR_SIZE;
  ttcd::delta_rows_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      src, dst, T, H, n, W, groups, to_tokens, token_bf16);
  return static_cast<int>(cudaGetLastError());
}
