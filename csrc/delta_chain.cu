// The chunk-to-chunk chain of the (gated) delta rule (sm_100a; plain fp32 FMA work, no tensor cores: the products are
// 64 x D x 32 per chunk and column slice, the point of the kernel is to run the n dependent steps in ONE launch).
//
// For one (batch, head) pair, S [D, Dv] the running state and i the chunk index:
//
//   forward  (i ascending):  states[i] = S;  y_i = x_i - a_i S;          S = gamma_i S + b_i^T y_i
//            a = w (WY factor), b = kt (keys scaled to the chunk end), x = u, y = vn
//   backward (i descending): states[i] = dS; y_i = x_i + a_i dS;         dS = gamma_i dS + add_i - b_i^T y_i
//            a = kt, b = w, x = d_vn (from downstream), add = d_states (from downstream), y = total d_vn
//
// (the role of chunk_gated_delta_rule_fwd_h / chunk_gated_delta_rule_bwd_dhu in fla/ops/common/chunk_delta_h.py).
// The columns of S never mix, so a CTA owns 32 of them for the whole sequence: grid (Dv / 32, batch * heads).  Per
// chunk the CTA stages a_i and b_i [64, D] in shared memory; thread (warp, lane) owns column `lane`, rows
// warp + 8 r of y and rows warp * (D / 8) + r of S (kept in registers across chunks, mirrored in shared memory for
// the other warps).  No waits on other CTAs or on asynchronous copies: nothing here can spin.
#include "common.cuh"

namespace ttcd {

constexpr int DC_C = 64;         // rows of a chunk
constexpr int DC_COLS = 32;      // state columns per CTA
constexpr int DC_THREADS = 256;  // 8 warps

struct DeltaChainParams {
  const float* a; const float* b; const float* gamma; const float* x; const float* add; const float* s_init;
  float* y; float* states; float* s_last;
  int n, D, Dv;
  float sign_a, sign_b;          // y = x + sign_a a S;  S = gamma S + add + sign_b b^T y
  int reverse;
};

template <int R>                 // R = D / 8: rows of S owned by one thread
__global__ void __launch_bounds__(DC_THREADS) delta_chain_kernel(const DeltaChainParams p) {
  constexpr int D = R * 8;
  extern __shared__ __align__(16) float dc_smem[];
  float* As = dc_smem;                       // [64][D]
  float* Bs = As + DC_C * D;                 // [64][D]
  float* Ss = Bs + DC_C * D;                 // [D][32]
  float* Ys = Ss + D * DC_COLS;              // [64][32]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col0 = blockIdx.x * DC_COLS;
  const int64_t bh = blockIdx.y;
  const int Dv = p.Dv;
  const float* a_base = p.a + bh * p.n * DC_C * D;
  const float* b_base = p.b + bh * p.n * DC_C * D;
  const float* x_base = p.x + bh * p.n * DC_C * Dv + col0 + lane;
  float* y_base = p.y + bh * p.n * DC_C * Dv + col0 + lane;
  float* st_base = p.states + bh * p.n * D * Dv + col0 + lane;
  const float* add_base = p.add != nullptr ? p.add + bh * p.n * D * Dv + col0 + lane : nullptr;

  float s[R];                                // S[warp * R + r][lane]
#pragma unroll
  for (int r = 0; r < R; ++r) s[r] = p.s_init[(bh * D + warp * R + r) * Dv + col0 + lane];

  for (int step = 0; step < p.n; ++step) {
    const int i = p.reverse ? p.n - 1 - step : step;
    // ---- stage a_i, b_i; publish S (to shared memory for the y products, to global memory as states[i])
    const float4* ga = reinterpret_cast<const float4*>(a_base + static_cast<int64_t>(i) * DC_C * D);
    const float4* gb = reinterpret_cast<const float4*>(b_base + static_cast<int64_t>(i) * DC_C * D);
    for (int v = threadIdx.x; v < DC_C * D / 4; v += DC_THREADS) {
      reinterpret_cast<float4*>(As)[v] = __ldg(ga + v);
      reinterpret_cast<float4*>(Bs)[v] = __ldg(gb + v);
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      Ss[(warp * R + r) * DC_COLS + lane] = s[r];
      st_base[(static_cast<int64_t>(i) * D + warp * R + r) * Dv] = s[r];
    }
    __syncthreads();
    // ---- y rows warp + 8 q:  y = x + sign_a * (a S)
    float acc[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) acc[q] = 0.f;
    for (int d = 0; d < D; d += 4) {
      const float s0 = Ss[(d + 0) * DC_COLS + lane], s1 = Ss[(d + 1) * DC_COLS + lane];
      const float s2 = Ss[(d + 2) * DC_COLS + lane], s3 = Ss[(d + 3) * DC_COLS + lane];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float4 av = *reinterpret_cast<const float4*>(As + (warp + 8 * q) * D + d);     // same address across the warp
        acc[q] = fmaf(av.x, s0, fmaf(av.y, s1, fmaf(av.z, s2, fmaf(av.w, s3, acc[q]))));
      }
    }
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const int c = warp + 8 * q;
      const int64_t off = (static_cast<int64_t>(i) * DC_C + c) * Dv;
      const float yv = x_base[off] + p.sign_a * acc[q];
      y_base[off] = yv;
      Ys[c * DC_COLS + lane] = yv;
    }
    __syncthreads();
    // ---- S rows warp * R + r:  S = gamma S + add + sign_b * (b^T y)
    float upd[R];
#pragma unroll
    for (int r = 0; r < R; ++r) upd[r] = 0.f;
    for (int c = 0; c < DC_C; ++c) {
      const float yv = Ys[c * DC_COLS + lane];
      const float* brow = Bs + c * D + warp * R;
#pragma unroll
      for (int r = 0; r < R; r += 4) {
        const float4 bv = *reinterpret_cast<const float4*>(brow + r);
        upd[r] = fmaf(bv.x, yv, upd[r]);
        upd[r + 1] = fmaf(bv.y, yv, upd[r + 1]);
        upd[r + 2] = fmaf(bv.z, yv, upd[r + 2]);
        upd[r + 3] = fmaf(bv.w, yv, upd[r + 3]);
      }
    }
    const float gm = p.gamma[bh * p.n + i];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float v = gm * s[r] + p.sign_b * upd[r];
      if (add_base != nullptr) v += add_base[(static_cast<int64_t>(i) * D + warp * R + r) * Dv];
      s[r] = v;
    }
    __syncthreads();                           // As / Bs / Ss / Ys are rewritten by the next step
  }
#pragma unroll
  for (int r = 0; r < R; ++r) p.s_last[(bh * D + warp * R + r) * Dv + col0 + lane] = s[r];
}

template <int R>
static int launch_delta_chain(const DeltaChainParams& p, int BH, cudaStream_t stream) {
  constexpr int D = R * 8;
  constexpr int smem = (2 * DC_C * D + D * DC_COLS + DC_C * DC_COLS) * static_cast<int>(sizeof(float));
  auto kern = delta_chain_kernel<R>;
  static bool configured = false;
  if (!configured) {
    TTCD_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  kern<<<dim3(p.Dv / DC_COLS, BH), DC_THREADS, smem, stream>>>(p);
  return static_cast<int>(cudaGetLastError());
}

static int delta_chain_dispatch(const DeltaChainParams& p, int BH, cudaStream_t stream) {
  if (BH <= 0 || p.n <= 0 || p.Dv <= 0 || p.Dv % DC_COLS != 0 || BH > 65535) return TTCD_ERR_ARG;
  switch (p.D) {
    case 32: return launch_delta_chain<4>(p, BH, stream);
    case 64: return launch_delta_chain<8>(p, BH, stream);
    case 128: return launch_delta_chain<16>(p, BH, stream);
    case 256: return launch_delta_chain<32>(p, BH, stream);
    default: return TTCD_ERR_ARG;
  }
}

}  // namespace ttcd

// All tensors fp32, contiguous: w, kt [BH][n][64][D]; u, vn [BH][n][64][Dv]; gamma [BH][n]; s0, s_final [BH][D][Dv];
// states [BH][n][D][Dv] (the state entering each chunk).  D in {32, 64, 128, 256}, Dv a multiple of 32.
TTCD_EXPORT int ttcd_delta_chain_fwd(const float* w, const float* u, const float* kt, const float* gamma, const float* s0,
                                     float* vn, float* states, float* s_final, int BH, int n, int D, int Dv,
                                     void* stream_ptr) {
  ttcd::DeltaChainParams p;
  p.a = w; p.b = kt; p.gamma = gamma; p.x = u; p.add = nullptr; p.s_init = s0;
  p.y = vn; p.states = states; p.s_last = s_final;
  p.n = n; p.D = D; p.Dv = Dv; p.sign_a = -1.f; p.sign_b = 1.f; p.reverse = 0;
  return ttcd::delta_chain_dispatch(p, BH, static_cast<cudaStream_t>(stream_ptr));
}

// Reverse chain: d_vn, d_states, d_final are the gradients arriving at vn, states and the final state; writes the total
// gradient of vn (d_vn_tot), the gradient of the state LEAVING each chunk (ds_next [BH][n][D][Dv]) and of s0.
TTCD_EXPORT int ttcd_delta_chain_bwd(const float* w, const float* kt, const float* gamma, const float* d_vn,
                                     const float* d_states, const float* d_final, float* d_vn_tot, float* ds_next,
                                     float* d_s0, int BH, int n, int D, int Dv, void* stream_ptr) {
  ttcd::DeltaChainParams p;
  p.a = kt; p.b = w; p.gamma = gamma; p.x = d_vn; p.add = d_states; p.s_init = d_final;
  p.y = d_vn_tot; p.states = ds_next; p.s_last = d_s0;
  p.n = n; p.D = D; p.Dv = Dv; p.sign_a = 1.f; p.sign_b = -1.f; p.reverse = 1;
  return ttcd::delta_chain_dispatch(p, BH, static_cast<cudaStream_t>(stream_ptr));
}
