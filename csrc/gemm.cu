// Persistent, warp-specialised bf16 GEMM for sm_100a.
//
//   C[b][m][n] = alpha * rowscale[m] * sum_k A[b][m][k] * B[b][n][k]  (+ beta * Cin[b][m][n])
//
// A is given either K-major ([M, K] row-major) or MN-major ([K, M] row-major); likewise B
// ([N, K] or [K, N]).  That covers y = x W^T, dx = dy W, dW = dy^T x and their batched forms
// without any transposition pass.
//
// One CTA per SM; tile 128 x BN x 64.  Warp 0 streams operand tiles with TMA (128-byte swizzle,
// no multicast) through a 4-stage mbarrier ring, one thread of warp 1 issues tcgen05.mma into a
// double-buffered TMEM accumulator (2 x BN fp32 columns), warps 2-5 drain the other accumulator
// with tcgen05.ld and write C, so the epilogue of tile i overlaps the main loop of tile i+1.
// Replaces the reference's cuBLAS calls behind nn.Linear / torch.matmul
// (custom_models/ipttcd/modeling_ipttcdv9_lowcopy_scanfuse.py:113-200).
#include "common.cuh"

namespace ttcd {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_THREADS = 192;

struct GemmParams {
  int64_t M, N, K, batch;
  int64_t ldc, stride_c;     // elements
  int64_t tiles_m, tiles_n;  // per batch
  float alpha, beta;
  const bf16* row_scale;     // optional [batch*M]
  int a_bcast, b_bcast;      // operand shared by every batch entry (its tensor map has batch 1)
  int m_fastest;             // raster order inside a batch entry: consecutive tiles walk M (the B panel is the big one)
  float2* lse_part;          // optional [batch*M][tiles_n]: per row and column tile (max, sum of exp(x - max)) of the
                             // bf16-rounded outputs, for a log-sum-exp over the row without another pass (bf16 out only)
};

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // epilogue staging for TMA stores: 4 warps x 2 buffers x (32 rows x 128 bytes), 128-byte swizzled
  static constexpr int EPI_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int EPI_BYTES = 4 * 2 * 4096;
  static constexpr int BAR_OFFSET = EPI_OFFSET + EPI_BYTES;
  // full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], tmem base word, abort flag
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16;
};

template <int BN, int STAGES, bool A_MN, bool B_MN, typename OutT, bool HAS_CIN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
            const __grid_constant__ CUtensorMap tma_c, OutT* __restrict__ C, const OutT* __restrict__ Cin,
            const GemmParams p) {
  using S = GemmSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: required by the 128-byte swizzle pattern shared by TMA and UMMA.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + S::BAR_OFFSET;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + S::BAR_OFFSET + (2 * STAGES + 4) * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = 2 * BN;  // 256 or 512: power of two

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 4);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int64_t tiles_per_batch = p.tiles_m * p.tiles_n;
  const int64_t total_tiles = tiles_per_batch * p.batch;
  const int num_kb = static_cast<int>((p.K + GEMM_BK - 1) / GEMM_BK);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int64_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int b = static_cast<int>(tile / tiles_per_batch);
        const int64_t r = tile % tiles_per_batch;
        const int m0 = static_cast<int>(p.m_fastest ? r % p.tiles_m : r / p.tiles_n) * GEMM_BM;
        const int n0 = static_cast<int>(p.m_fastest ? r / p.tiles_m : r % p.tiles_n) * BN;
        const int za = p.a_bcast ? 0 : b, zb = p.b_bcast ? 0 : b;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, 101)) { ok = false; break; }
          const uint32_t sa = smem_base + stage * S::STAGE_BYTES;
          const uint32_t sb = sa + S::A_BYTES;
          mbar_expect_tx(full_bar(stage), S::STAGE_BYTES);
          const int k0 = kb * GEMM_BK;
          if (!A_MN) {
            tma_load_3d(sa, &tma_a, full_bar(stage), k0, m0, za);
          } else {
#pragma unroll
            for (int h = 0; h < GEMM_BM / 64; ++h)
              tma_load_3d(sa + h * (GEMM_BK * 128), &tma_a, full_bar(stage), m0 + h * 64, k0, za);
          }
          if (!B_MN) {
            tma_load_3d(sb, &tma_b, full_bar(stage), k0, n0, zb);
          } else {
#pragma unroll
            for (int h = 0; h < BN / 64; ++h)
              tma_load_3d(sb + h * (GEMM_BK * 128), &tma_b, full_bar(stage), n0 + h * 64, k0, zb);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // abort path: give copies already in flight a bounded time to land before smem is released
        for (int s = 0; s < STAGES; ++s) mbar_drain(full_bar(s), 0), mbar_drain(full_bar(s), 1);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(GEMM_BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase[2] = {0, 0};
      int acc = 0;
      bool ok = true;
      for (int64_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(tempty_bar(acc), acc_phase[acc] ^ 1u, abort_flag, 102)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, 103)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_base + stage * S::STAGE_BYTES;
          const uint32_t sb = sa + S::A_BYTES;
#pragma unroll
          for (int k = 0; k < GEMM_BK / 16; ++k) {
            // K-major: 16 k-elements = 32 bytes inside the swizzled row; MN-major: 16 k-rows = 2 KiB.
            const uint64_t ad = A_MN ? umma_desc_sw128(sa + k * 2048, GEMM_BK * 128, 1024)
                                     : umma_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t bd = B_MN ? umma_desc_sw128(sb + k * 2048, GEMM_BK * 128, 1024)
                                     : umma_desc_sw128(sb + k * 32, 16, 1024);
            umma_ss(d_tmem, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));  // frees the smem stage when these MMAs retire
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(tfull_bar(acc));  // accumulator complete
        acc_phase[acc] ^= 1u;
        acc ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;  // TMEM lane quarter this warp may access
    uint32_t acc_phase[2] = {0, 0};
    int acc = 0;
    bool ok = true;
    for (int64_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      const int b = static_cast<int>(tile / tiles_per_batch);
      const int64_t r = tile % tiles_per_batch;
      const int64_t m0 = (p.m_fastest ? r % p.tiles_m : r / p.tiles_n) * GEMM_BM;
      const int64_t n0 = (p.m_fastest ? r / p.tiles_m : r % p.tiles_n) * BN;
      if (!mbar_wait(tfull_bar(acc), acc_phase[acc], abort_flag, 104)) { ok = false; break; }
      tc_fence_after_sync();
      const int64_t row = m0 + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      float rs = p.alpha;
      if (p.row_scale != nullptr && row_ok) rs *= __bfloat162float(p.row_scale[b * p.M + row]);
      OutT* crow = C + b * p.stride_c + row * p.ldc;
      const OutT* cin_row = HAS_CIN ? (Cin + b * p.stride_c + row * p.ldc) : nullptr;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      if constexpr (sizeof(OutT) == 2) {
        // bf16 output: TMEM -> registers -> swizzled shared memory -> TMA store of a 32-row x 64-column box
        // (full 128-byte lines, clipped at the matrix edges by the tensor map); two staging buffers per warp.
        uint8_t* stage = smem + S::EPI_OFFSET + quarter * 8192;
        int chunk = 0;
        const bool want_lse = p.lse_part != nullptr;
        float run_m = -INFINITY, run_s = 0.f;
#pragma unroll 1
        for (int c = 0; c < BN; c += 64, ++chunk) {
          uint32_t v0[32], v1[32];
          tmem_ld32(t_row + c, v0);
          tmem_ld32(t_row + c + 32, v1);
          if (lane == 0) tma_store_wait_read1();      // the store issued two chunks ago has released this buffer
          __syncwarp();
          tmem_ld_wait();
          uint8_t* buf = stage + (chunk & 1) * 4096;
          const int64_t col = n0 + c;
#pragma unroll
          for (int j = 0; j < 64; j += 8) {
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(j < 32 ? v0[(j & 31) + e] : v1[(j & 31) + e]) * rs;
            if constexpr (HAS_CIN) {
              if (row_ok && col + j + 8 <= p.N) {
                const uint4 cv = *reinterpret_cast<const uint4*>(cin_row + col + j);
                const uint32_t cw[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 t = unpack_bf16(cw[e]);
                  f[2 * e] += p.beta * t.x;
                  f[2 * e + 1] += p.beta * t.y;
                }
              } else if (row_ok) {
                for (int e = 0; e < 8 && col + j + e < p.N; ++e) f[e] += p.beta * __bfloat162float(cin_row[col + j + e]);
              }
            }
            uint4 o;
            o.x = pack_bf16(f[0], f[1]);
            o.y = pack_bf16(f[2], f[3]);
            o.z = pack_bf16(f[4], f[5]);
            o.w = pack_bf16(f[6], f[7]);
            *reinterpret_cast<uint4*>(buf + sw128_offset(lane, j >> 3)) = o;
            if (want_lse) {
              // running (max, sum) over this thread's row, on the values as the consumer will read them (bf16)
              const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
              float r[8];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 t = unpack_bf16(ow[e]);
                r[2 * e] = col + j + 2 * e < p.N ? t.x : -INFINITY;
                r[2 * e + 1] = col + j + 2 * e + 1 < p.N ? t.y : -INFINITY;
              }
              float mx = r[0];
#pragma unroll
              for (int e = 1; e < 8; ++e) mx = fmaxf(mx, r[e]);
              if (mx > run_m) {
                run_s *= __expf(run_m - mx);
                run_m = mx;
              }
              if (run_m != -INFINITY) {
#pragma unroll
                for (int e = 0; e < 8; ++e) run_s += __expf(r[e] - run_m);
              }
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && col < p.N) {
            tma_store_3d(&tma_c, smem_u32(buf), static_cast<int>(col), static_cast<int>(m0 + quarter * 32), b);
            tma_store_commit();
          }
        }
        if (want_lse && row_ok) p.lse_part[(b * p.M + row) * p.tiles_n + n0 / BN] = make_float2(run_m, run_s);
      } else {
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t v[32];
          tmem_ld32(t_row + c, v);
          tmem_ld_wait();
          const int64_t col = n0 + c;
          if (row_ok && col < p.N) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (col + j + 4 <= p.N) {
                float4 o;
                o.x = __uint_as_float(v[j]) * rs;
                o.y = __uint_as_float(v[j + 1]) * rs;
                o.z = __uint_as_float(v[j + 2]) * rs;
                o.w = __uint_as_float(v[j + 3]) * rs;
                if constexpr (HAS_CIN) {
                  const float4 cv = *reinterpret_cast<const float4*>(cin_row + col + j);
                  o.x += p.beta * cv.x; o.y += p.beta * cv.y; o.z += p.beta * cv.z; o.w += p.beta * cv.w;
                }
                *reinterpret_cast<float4*>(crow + col + j) = o;
              } else {
                for (int e = 0; e < 4 && col + j + e < p.N; ++e) {
                  float f = __uint_as_float(v[j + e]) * rs;
                  if constexpr (HAS_CIN) f += p.beta * cin_row[col + j + e];
                  crow[col + j + e] = f;
                }
              }
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
      acc_phase[acc] ^= 1u;
      acc ^= 1;
    }
    if (sizeof(OutT) == 2 && lane == 0) tma_store_wait0();   // staging buffers stay valid until the stores ran
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int BN, int STAGES, bool A_MN, bool B_MN, typename OutT, bool HAS_CIN>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, void* c, const void* cin,
                       const GemmParams& p, cudaStream_t stream) {
  using S = GemmSmem<BN, STAGES>;
  auto kern = gemm_kernel<BN, STAGES, A_MN, B_MN, OutT, HAS_CIN>;
  constexpr int smem_bytes = S::TOTAL + 1024;
  static bool configured = false;  // per instantiation; attribute is per function, device-independent here
  if (!configured) {
    TTCD_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    configured = true;
  }
  const int64_t total = p.tiles_m * p.tiles_n * p.batch;
  const int grid = static_cast<int>(total < sm_count() ? total : sm_count());
  kern<<<grid, GEMM_THREADS, smem_bytes, stream>>>(ta, tb, tc, static_cast<OutT*>(c), static_cast<const OutT*>(cin), p);
  return static_cast<int>(cudaGetLastError());
}

template <int BN, int STAGES, bool A_MN, bool B_MN>
static int dispatch_out(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, void* c, const void* cin,
                        const GemmParams& p, int out_fp32, cudaStream_t stream) {
  const bool has_cin = cin != nullptr && p.beta != 0.f;
  if (out_fp32) {
    return has_cin ? launch_gemm<BN, STAGES, A_MN, B_MN, float, true>(ta, tb, tc, c, cin, p, stream)
                   : launch_gemm<BN, STAGES, A_MN, B_MN, float, false>(ta, tb, tc, c, cin, p, stream);
  }
  return has_cin ? launch_gemm<BN, STAGES, A_MN, B_MN, bf16, true>(ta, tb, tc, c, cin, p, stream)
                 : launch_gemm<BN, STAGES, A_MN, B_MN, bf16, false>(ta, tb, tc, c, cin, p, stream);
}

template <int BN, int STAGES>
static int dispatch_major(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, void* c, const void* cin,
                          const GemmParams& p, int a_mn, int b_mn, int out_fp32, cudaStream_t stream) {
  if (!a_mn && !b_mn) return dispatch_out<BN, STAGES, false, false>(ta, tb, tc, c, cin, p, out_fp32, stream);
  if (!a_mn && b_mn) return dispatch_out<BN, STAGES, false, true>(ta, tb, tc, c, cin, p, out_fp32, stream);
  if (a_mn && !b_mn) return dispatch_out<BN, STAGES, true, false>(ta, tb, tc, c, cin, p, out_fp32, stream);
  return dispatch_out<BN, STAGES, true, true>(ta, tb, tc, c, cin, p, out_fp32, stream);
}

}  // namespace ttcd

TTCD_DEFINE_STATUS_READER(gemm)

// a: [batch][M][K] (a_mn = 0, row stride lda) or [batch][K][M] (a_mn = 1).  b likewise with N.
// c / c_in: [batch][M][N], row stride ldc, bf16 or fp32 (out_fp32).  Strides in elements.
// c_in may alias c.  row_scale: optional bf16 [batch*M].
static int gemm_bf16_impl(const void* a, const void* b, void* c, const void* c_in, const void* row_scale,
                         long long M, long long N, long long K, long long batch, long long lda,
                         long long ldb, long long ldc, long long stride_a, long long stride_b,
                         long long stride_c, int a_mn, int b_mn, int out_fp32, float alpha, float beta,
                         float* lse_part, void* stream_ptr) {
  using namespace ttcd;
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return TTCD_ERR_ARG;
  if (lse_part != nullptr && (out_fp32 || (reinterpret_cast<uintptr_t>(lse_part) & 7u))) return TTCD_ERR_ARG;
  const int elem_c = out_fp32 ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(c) & 15u) || (ldc * elem_c) % 16 != 0 || (stride_c * elem_c) % 16 != 0)
    return TTCD_ERR_ARG;
  if (c_in != nullptr && (reinterpret_cast<uintptr_t>(c_in) & 15u)) return TTCD_ERR_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  // every TMA box must fit inside its tensor: the caller pads tiny problems up to these minima
  if (M < GEMM_BM || N < 128 || K < GEMM_BK) return TTCD_ERR_ARG;
  const int BN = N >= 256 ? 256 : 128;
  CUtensorMap ta, tb;
  int rc;
  const int a_bcast = (batch > 1 && stride_a == 0) ? 1 : 0;
  const int b_bcast = (batch > 1 && stride_b == 0) ? 1 : 0;
  const long long batch_a = a_bcast ? 1 : batch, batch_b = b_bcast ? 1 : batch;
  if (!a_mn) rc = make_tmap_bf16_3d(&ta, a, K, M, batch_a, lda, stride_a, 64, GEMM_BM);
  else       rc = make_tmap_bf16_3d(&ta, a, M, K, batch_a, lda, stride_a, 64, GEMM_BK);
  if (rc != TTCD_OK) return rc;
  if (!b_mn) rc = make_tmap_bf16_3d(&tb, b, K, N, batch_b, ldb, stride_b, 64, BN);
  else       rc = make_tmap_bf16_3d(&tb, b, N, K, batch_b, ldb, stride_b, 64, GEMM_BK);
  if (rc != TTCD_OK) return rc;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.batch = batch;
  p.ldc = ldc; p.stride_c = stride_c;
  p.tiles_m = (M + GEMM_BM - 1) / GEMM_BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.alpha = alpha; p.beta = beta;
  p.row_scale = static_cast<const bf16*>(row_scale);
  p.a_bcast = a_bcast; p.b_bcast = b_bcast;
  // the operand panel that is re-streamed once per step of the outer tile loop should be the smaller one (it then
  // lives in the 126 MB L2): walk M fastest when the B panel (N x K) is the larger
  p.m_fastest = N > M ? 1 : 0;
  p.lse_part = reinterpret_cast<float2*>(lse_part);
  CUtensorMap tc = ta;      // fp32 outputs are written with plain stores and never touch this map
  if (!out_fp32) {
    rc = make_tmap_bf16_3d(&tc, c, N, M, batch, ldc, stride_c, 64, 32);
    if (rc != TTCD_OK) return rc;
  }
  if (BN == 256) return dispatch_major<256, 4>(ta, tb, tc, c, c_in, p, a_mn, b_mn, out_fp32, stream);
  return dispatch_major<128, 6>(ta, tb, tc, c, c_in, p, a_mn, b_mn, out_fp32, stream);
}

TTCD_EXPORT int ttcd_gemm_bf16(const void* a, const void* b, void* c, const void* c_in, const void* row_scale,
                               long long M, long long N, long long K, long long batch, long long lda,
                               long long ldb, long long ldc, long long stride_a, long long stride_b,
                               long long stride_c, int a_mn, int b_mn, int out_fp32, float alpha, float beta,
                               void* stream_ptr) {
  return gemm_bf16_impl(a, b, c, c_in, row_scale, M, N, K, batch, lda, ldb, ldc, stride_a, stride_b, stride_c, a_mn, b_mn,
                        out_fp32, alpha, beta, nullptr, stream_ptr);
}

// Same GEMM (bf16 output) that also leaves, per output row and column tile, the pair (max, sum of exp(x - max)) of the
// row's values in that tile, taken on the bf16-rounded outputs: lse_part is fp32 [batch*M][tiles_n][2] with
// tiles_n = ceil(N / 256) (N >= 256) or ceil(N / 128).  A consumer merges the tiles_n pairs of a row into its
// log-sum-exp without reading the row (the cross-entropy row kernel does).
TTCD_EXPORT int ttcd_gemm_bf16_lse(const void* a, const void* b, void* c, long long M, long long N, long long K,
                                   long long lda, long long ldb, long long ldc, int a_mn, int b_mn, float alpha,
                                   float* lse_part, void* stream_ptr) {
  if (lse_part == nullptr) return TTCD_ERR_ARG;
  return gemm_bf16_impl(a, b, c, nullptr, nullptr, M, N, K, 1, lda, ldb, ldc, 0, 0, M * ldc, a_mn, b_mn, 0, alpha, 0.f,
                        lse_part, stream_ptr);
}
