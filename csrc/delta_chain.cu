// The chunk-to-chunk chain of the (gated) delta rule (sm_100a; the two products of a step, 64 x D x 32 each, run on the
// tensor cores as TF32 mma.sync tiles with fp32 accumulation: they are far too small for a tcgen05 pipeline; the point
// of the kernel is to run the n dependent steps in ONE launch with the state resident in registers).
//
// For one (batch, head) pair, S [D, Dv] the running state and i the chunk index:
//
//   forward  (i ascending):  states[i] = S;  y_i = x_i - a_i S;          S = gamma_i S + b_i^T y_i
//            a = w (WY factor), b = kt (keys scaled to the chunk end), x = u, y = vn
//   backward (i descending): states[i] = dS; y_i = x_i + a_i dS;         dS = gamma_i dS + add_i - b_i^T y_i
//            a = kt, b = w, x = d_vn (from downstream), add = d_states (from downstream), y = total d_vn
//
// (the role of chunk_gated_delta_rule_fwd_h / chunk_gated_delta_rule_bwd_dhu in fla/ops/common/chunk_delta_h.py).
// The columns of S never mix, so a CTA owns 32 of them (64 for D = 256, where a_i and b_i are large and every column
// slice re-reads them) for the whole sequence: grid (Dv / columns, batch * heads).  Per chunk the CTA stages a_i and
// b_i [64, D] (bf16) in shared memory with asynchronous 16-byte copies that overlap the publication of S.  S [D, columns]
// lives in the accumulator registers of the second product (D / 32 m16n8 tiles per warp) across chunks, in fp32, and is
// mirrored in shared memory, rounded to bf16, as the B operand of the first; y is rounded the same way for the second.
// Every operand of a product is thus a bf16 value (an exact TF32 operand after a 16-bit shift; the precision the
// reference's Triton kernels multiply at), the sums and the state stay fp32, and two CTAs fit an SM at every D.
// The only asynchronous copies are the CTA's own cp.async groups (waited for with wait_group); nothing here waits on
// another CTA, so nothing can spin.
#include "common.cuh"

namespace ttcd {

constexpr int DC_C = 64;         // rows of a chunk
constexpr int DC_THREADS = 256;  // 8 warps

struct DeltaChainParams {
  const bf16* a; const bf16* b;   // bf16: exact TF32 operands after a 16-bit shift, half the staging traffic
  const float* gamma; const float* x; const float* add; const float* s_init;
  float* y; float* states; float* s_last;
  int n, D, Dv;
  float sign_a, sign_b;          // y = x + sign_a a S;  S = gamma S + add + sign_b b^T y
  int reverse;
  // optional: per chunk, the sum over this CTA's columns of dot_with[i] * (S entering the step)  ->  dot_out[bh][i][blockIdx.x]
  // (the reverse chain uses it for the gradient of gamma: dot_with = the forward states)
  const float* dot_with; float* dot_out;
};

__device__ __forceinline__ uint32_t dc_bf16_bits(const bf16* p) {   // a bf16 value as a TF32 operand
  return static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(p)) << 16;
}
__device__ __forceinline__ void dc_cp_async16(void* dst_smem, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void dc_cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void dc_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int D, int DC_COLS>
__global__ void __launch_bounds__(DC_THREADS, (D <= 128 ? 4 : 2)) delta_chain_kernel(const DeltaChainParams p) {
  constexpr int LDT = D + 8;                 // bf16 row stride of the a_i / b_i tiles: rows 4 banks apart, 16-byte rows
  constexpr int DC_LDS = DC_COLS + 8;        // bf16 row stride of the [*, columns] tiles read column-wise as B operands
  constexpr int NTM = DC_COLS / 8;           // n-tiles per m-tile of S
  constexpr int TPW = (D / 16) * NTM / 8;    // m16n8 tiles of S per warp: tile id = warp * TPW + x -> (id / NTM, id % NTM)
  constexpr int NT = TPW >= NTM ? NTM : TPW; // ... of which NT share an m-tile
  constexpr int MT = TPW / NT;
  constexpr int YT = DC_COLS / 16;           // n-tiles of y per warp
  extern __shared__ __align__(16) float dc_smem[];
  bf16* As = reinterpret_cast<bf16*>(dc_smem);              // [64][LDT]
  bf16* Bs = As + DC_C * LDT;                               // [64][LDT]
  bf16* Ss = Bs + DC_C * LDT;                               // [D][columns + 8]   S as the B operand of a S
  bf16* Ys = Ss + D * DC_LDS;                               // [64][columns + 8]  sign_b * y as the B operand of b^T y
  float* red = reinterpret_cast<float*>(Ys + DC_C * DC_LDS);    // [8] per-warp partial sums of the optional dot product
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, c = lane & 3;
  const int col0 = blockIdx.x * DC_COLS;
  const int64_t bh = blockIdx.y;
  const int Dv = p.Dv;
  const bf16* a_base = p.a + bh * p.n * DC_C * D;
  const bf16* b_base = p.b + bh * p.n * DC_C * D;
  const float* x_base = p.x + bh * p.n * DC_C * Dv + col0;
  float* y_base = p.y + bh * p.n * DC_C * Dv + col0;
  float* st_base = p.states + bh * p.n * D * Dv + col0;
  const float* add_base = p.add != nullptr ? p.add + bh * p.n * D * Dv + col0 : nullptr;
  const float* dot_base = p.dot_with != nullptr ? p.dot_with + bh * p.n * D * Dv + col0 : nullptr;
  // the warp's tiles of S: m-tile mt0 + m (rows 16 (mt0 + m) + g, + 8), n-tiles nt0 .. nt0 + NT - 1 (columns 8 nt + 2 c, + 1)
  const int mt0 = (warp * TPW) / NTM, nt0 = (warp * TPW) % NTM;
  // the warp's YT tiles of y: m-tile warp / 2, n-tiles YT (warp % 2) ..
  const int ymt = warp >> 1, ynt0 = YT * (warp & 1);

  float s[MT][NT][4];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      const int row = 16 * (mt0 + m) + g, col = 8 * (nt0 + t) + 2 * c;
      const float2 lo = *reinterpret_cast<const float2*>(p.s_init + (bh * D + row) * Dv + col0 + col);
      const float2 hi = *reinterpret_cast<const float2*>(p.s_init + (bh * D + row + 8) * Dv + col0 + col);
      s[m][t][0] = lo.x; s[m][t][1] = lo.y; s[m][t][2] = hi.x; s[m][t][3] = hi.y;
    }

  for (int step = 0; step < p.n; ++step) {
    const int i = p.reverse ? p.n - 1 - step : step;
    // ---- stage a_i, b_i; publish S (to shared memory for the y products, to global memory as states[i])
    const uint4* ga = reinterpret_cast<const uint4*>(a_base + static_cast<int64_t>(i) * DC_C * D);
    const uint4* gb = reinterpret_cast<const uint4*>(b_base + static_cast<int64_t>(i) * DC_C * D);
    for (int v = threadIdx.x; v < DC_C * D / 8; v += DC_THREADS) {
      const int row = v / (D / 8), c8 = (v % (D / 8)) * 8;
      dc_cp_async16(As + row * LDT + c8, ga + v);
      dc_cp_async16(Bs + row * LDT + c8, gb + v);
    }
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        const int row = 16 * (mt0 + m) + g, col = 8 * (nt0 + t) + 2 * c;
        const float2 lo = make_float2(s[m][t][0], s[m][t][1]), hi = make_float2(s[m][t][2], s[m][t][3]);
        *reinterpret_cast<__nv_bfloat162*>(Ss + row * DC_LDS + col) = __floats2bfloat162_rn(lo.x, lo.y);      // B operand, rounded once
        *reinterpret_cast<__nv_bfloat162*>(Ss + (row + 8) * DC_LDS + col) = __floats2bfloat162_rn(hi.x, hi.y);
        *reinterpret_cast<float2*>(st_base + (static_cast<int64_t>(i) * D + row) * Dv + col) = lo;
        *reinterpret_cast<float2*>(st_base + (static_cast<int64_t>(i) * D + row + 8) * Dv + col) = hi;
      }
    if (dot_base != nullptr) {
      float part = 0.f;
#pragma unroll
      for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          const int row = 16 * (mt0 + m) + g, col = 8 * (nt0 + t) + 2 * c;
          const float2 lo = *reinterpret_cast<const float2*>(dot_base + (static_cast<int64_t>(i) * D + row) * Dv + col);
          const float2 hi = *reinterpret_cast<const float2*>(dot_base + (static_cast<int64_t>(i) * D + row + 8) * Dv + col);
          part += s[m][t][0] * lo.x + s[m][t][1] * lo.y + s[m][t][2] * hi.x + s[m][t][3] * hi.y;
        }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
      if (lane == 0) red[warp] = part;
    }
    dc_cp_async_wait_all();
    __syncthreads();
    if (dot_base != nullptr && threadIdx.x == 0) {
      float tot = 0.f;
#pragma unroll
      for (int wv = 0; wv < DC_THREADS / 32; ++wv) tot += red[wv];
      p.dot_out[(bh * p.n + i) * (Dv / 32) + blockIdx.x] = tot;        // rows of Dv / 32 slots (zero-filled by the caller)
    }
    // ---- y = x + sign_a * (a S): the warp's YT 16 x 8 tiles
    {
      float acc[YT][4];
#pragma unroll
      for (int t = 0; t < YT; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f;
      const bf16* arow = As + (16 * ymt + g) * LDT + c;
      const bf16* sb0 = Ss + c * DC_LDS + 8 * ynt0 + g;
#pragma unroll 4
      for (int k0 = 0; k0 < D; k0 += 8) {
        uint32_t a[4];
        a[0] = dc_bf16_bits(arow + k0); a[1] = dc_bf16_bits(arow + 8 * LDT + k0);
        a[2] = dc_bf16_bits(arow + k0 + 4); a[3] = dc_bf16_bits(arow + 8 * LDT + k0 + 4);
#pragma unroll
        for (int t = 0; t < YT; ++t) {
          const bf16* sb = sb0 + k0 * DC_LDS + 8 * t;
          dc_mma(acc[t], a, dc_bf16_bits(sb), dc_bf16_bits(sb + 4 * DC_LDS));
        }
      }
#pragma unroll
      for (int t = 0; t < YT; ++t)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int row = 16 * ymt + g + 8 * h, col = 8 * (ynt0 + t) + 2 * c;
          const int64_t off = (static_cast<int64_t>(i) * DC_C + row) * Dv + col;
          const float2 xv = *reinterpret_cast<const float2*>(x_base + off);
          const float2 yv = make_float2(xv.x + p.sign_a * acc[t][2 * h], xv.y + p.sign_a * acc[t][2 * h + 1]);
          *reinterpret_cast<float2*>(y_base + off) = yv;
          *reinterpret_cast<__nv_bfloat162*>(Ys + row * DC_LDS + col) = __floats2bfloat162_rn(p.sign_b * yv.x, p.sign_b * yv.y);
        }
    }
    __syncthreads();
    // ---- S = gamma S + add + sign_b * (b^T y), accumulated in place
    const float gm = p.gamma[bh * p.n + i];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        const int row = 16 * (mt0 + m) + g, col = 8 * (nt0 + t) + 2 * c;
        float2 lo = make_float2(0.f, 0.f), hi = make_float2(0.f, 0.f);
        if (add_base != nullptr) {
          lo = *reinterpret_cast<const float2*>(add_base + (static_cast<int64_t>(i) * D + row) * Dv + col);
          hi = *reinterpret_cast<const float2*>(add_base + (static_cast<int64_t>(i) * D + row + 8) * Dv + col);
        }
        s[m][t][0] = fmaf(gm, s[m][t][0], lo.x); s[m][t][1] = fmaf(gm, s[m][t][1], lo.y);
        s[m][t][2] = fmaf(gm, s[m][t][2], hi.x); s[m][t][3] = fmaf(gm, s[m][t][3], hi.y);
      }
      const bf16* bcol = Bs + c * LDT + 16 * (mt0 + m) + g;              // b^T as the A operand: A[d][k] = b[k][d]
#pragma unroll 4
      for (int k0 = 0; k0 < DC_C; k0 += 8) {
        uint32_t a[4];
        a[0] = dc_bf16_bits(bcol + k0 * LDT); a[1] = dc_bf16_bits(bcol + k0 * LDT + 8);
        a[2] = dc_bf16_bits(bcol + (k0 + 4) * LDT); a[3] = dc_bf16_bits(bcol + (k0 + 4) * LDT + 8);
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          const bf16* yb = Ys + (k0 + c) * DC_LDS + 8 * (nt0 + t) + g;
          dc_mma(s[m][t], a, dc_bf16_bits(yb), dc_bf16_bits(yb + 4 * DC_LDS));
        }
      }
    }
    __syncthreads();                           // As / Bs / Ss / Ys are rewritten by the next step
  }
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      const int row = 16 * (mt0 + m) + g, col = 8 * (nt0 + t) + 2 * c;
      *reinterpret_cast<float2*>(p.s_last + (bh * D + row) * Dv + col0 + col) = make_float2(s[m][t][0], s[m][t][1]);
      *reinterpret_cast<float2*>(p.s_last + (bh * D + row + 8) * Dv + col0 + col) = make_float2(s[m][t][2], s[m][t][3]);
    }
}

template <int D, int COLS>
static int launch_delta_chain(const DeltaChainParams& p, int BH, cudaStream_t stream) {
  constexpr int smem = (2 * DC_C * (D + 8) + D * (COLS + 8) + DC_C * (COLS + 8)) * static_cast<int>(sizeof(bf16)) +
                       8 * static_cast<int>(sizeof(float));
  auto kern = delta_chain_kernel<D, COLS>;
  static bool configured = false;
  if (!configured) {
    TTCD_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  kern<<<dim3(p.Dv / COLS, BH), DC_THREADS, smem, stream>>>(p);
  return static_cast<int>(cudaGetLastError());
}

static int delta_chain_dispatch(const DeltaChainParams& p, int BH, cudaStream_t stream) {
  if (BH <= 0 || p.n <= 0 || p.Dv <= 0 || p.Dv % 32 != 0 || BH > 65535) return TTCD_ERR_ARG;
  switch (p.D) {
    case 32: return launch_delta_chain<32, 32>(p, BH, stream);
    case 64: return launch_delta_chain<64, 32>(p, BH, stream);
    case 128: return launch_delta_chain<128, 32>(p, BH, stream);
    case 256: return p.Dv % 64 == 0 ? launch_delta_chain<256, 64>(p, BH, stream) : launch_delta_chain<256, 32>(p, BH, stream);
    default: return TTCD_ERR_ARG;
  }
}

}  // namespace ttcd

// Contiguous tensors: w, kt [BH][n][64][D] bf16; fp32: u, vn [BH][n][64][Dv]; gamma [BH][n]; s0, s_final [BH][D][Dv];
// states [BH][n][D][Dv] (the state entering each chunk).  D in {32, 64, 128, 256}, Dv a multiple of 32.
TTCD_EXPORT int ttcd_delta_chain_fwd(const bf16* w, const float* u, const bf16* kt, const float* gamma, const float* s0,
                                     float* vn, float* states, float* s_final, int BH, int n, int D, int Dv,
                                     void* stream_ptr) {
  ttcd::DeltaChainParams p;
  p.a = w; p.b = kt; p.gamma = gamma; p.x = u; p.add = nullptr; p.s_init = s0;
  p.y = vn; p.states = states; p.s_last = s_final;
  p.n = n; p.D = D; p.Dv = Dv; p.sign_a = -1.f; p.sign_b = 1.f; p.reverse = 0;
  p.dot_with = nullptr; p.dot_out = nullptr;
  return ttcd::delta_chain_dispatch(p, BH, static_cast<cudaStream_t>(stream_ptr));
}

// Reverse chain: d_vn, d_states, d_final are the gradients arriving at vn, states and the final state; writes the total
// gradient of vn (d_vn_tot), the gradient of the state LEAVING each chunk (ds_next [BH][n][D][Dv]) and of s0.  With
// `states` (the forward states) it also writes d_gamma_parts [BH][n][Dv / 32] (zero-filled by the caller): per chunk and
// column slice of a CTA, the sum of states * ds_next (the gradient of the chunk's decay is the sum over a row).
TTCD_EXPORT int ttcd_delta_chain_bwd(const bf16* w, const bf16* kt, const float* gamma, const float* d_vn,
                                     const float* d_states, const float* d_final, float* d_vn_tot, float* ds_next,
                                     float* d_s0, const float* states, float* d_gamma_parts, int BH, int n, int D, int Dv,
                                     void* stream_ptr) {
  ttcd::DeltaChainParams p;
  p.a = kt; p.b = w; p.gamma = gamma; p.x = d_vn; p.add = d_states; p.s_init = d_final;
  p.y = d_vn_tot; p.states = ds_next; p.s_last = d_s0;
  p.n = n; p.D = D; p.Dv = Dv; p.sign_a = 1.f; p.sign_b = -1.f; p.reverse = 1;
  p.dot_with = d_gamma_parts != nullptr ? states : nullptr; p.dot_out = d_gamma_parts;
  return ttcd::delta_chain_dispatch(p, BH, static_cast<cudaStream_t>(stream_ptr));
}
