// Sliding-window causal attention forward for sm_100a, single- or dual-window.
//
// One CTA handles 128 query rows of one (batch, head).  K/V blocks of 64 keys stream through a
// 2-slot TMA ring (128-byte swizzle, no multicast); S = Q K^T and O += P V run on tcgen05 with the
// accumulators in TMEM (two S buffers of 64 columns + one O buffer of D columns = 256 columns, so
// two CTAs share an SM and one CTA's softmax overlaps the other's MMAs).  Four softmax warps own
// one query row per thread (TMEM lane == row, so row reductions need no shuffles); a fifth warp's
// elected lane issues every TMA copy and MMA.
//
// Dual-window mode computes the student output (window w_S) and the teacher output (window w_T)
// in ONE pass over K/V: the key blocks inside the student window are accumulated first, the
// normalised accumulator is written out as the student result, and accumulation simply continues
// over the teacher-only keys with the same running max / sum (online-softmax rescale identity).
// Blocks that straddle the student boundary are visited once per phase with complementary masks.
// Packed batches (several sequences in one row, the role of flash_attn_varlen_func in fla/layers/attn.py:229-270):
// a per-token `seg_start` array bounds each query's keys to its own sequence, and the key-block range of a tile is
// clipped to the sequences that the tile touches.
// This replaces the two flash-attn calls of the reference's TTT layers
// (custom_models/ipttcd/modeling_ipttcdv9.py:686-690) and its forward-only Triton kernel
// (profiling/fused_dual_attn.py:34-241).
#include "common.cuh"

namespace ttcd {

constexpr int ATT_BM = 128;
constexpr int ATT_BN = 64;
constexpr int ATT_THREADS = 160;
constexpr float RESCALE_THRESHOLD = 8.0f;  // log2 units: lazy accumulator rescale

struct AttnFwdParams {
  bf16* o_t; bf16* o_s;          // [B, Tq, H, D]; o_s null => single window
  float* lse_t; float* lse_s;    // [B, H, Tq]
  int Tq, Tk, H, HK;
  int w_t, w_s;                  // window sizes in keys (w_s is the only window in single mode)
  float scale_log2;              // softmax scale * log2(e)
  // context parallel: keys [0, halo_len) are the tail of the PREVIOUS rank's sequence shard and are read
  // straight from that rank's memory (rows halo_row0.. of its K/V buffers); keys >= halo_len are local
  int halo_len, halo_row0;
  // packed sequences (null: none): per token, the first token of its sequence
  const int* seg_start;
};

template <int D>
struct AttnSmem {
  static constexpr int DB = D / 64;                       // 64-column sub-blocks of the head dim
  static constexpr int Q_REGION = ATT_BM * 128;           // bytes of one [128 x 64] swizzled region
  static constexpr int KV_REGION = ATT_BN * 128;          // bytes of one [64 x 64] swizzled region
  static constexpr int Q_BYTES = DB * Q_REGION;
  static constexpr int KV_BYTES = DB * KV_REGION;
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + Q_BYTES;           // 2 slots
  static constexpr int V_OFF = K_OFF + 2 * KV_BYTES;      // 2 slots
  static constexpr int BAR_OFF = V_OFF + 2 * KV_BYTES;
  // bar_q, k_full[2], v_full[2], s_full[2], s_free[2], p_full, pv_done  = 11 barriers
  static constexpr int NBARS = 11;
  static constexpr int TOTAL = BAR_OFF + NBARS * 8 + 16;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D, bool DUAL>
__global__ void __launch_bounds__(ATT_THREADS, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                const __grid_constant__ CUtensorMap tma_v, const __grid_constant__ CUtensorMap tma_kh,
                const __grid_constant__ CUtensorMap tma_vh, const AttnFwdParams p) {
  using S = AttnSmem<D>;
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bars = sbase + S::BAR_OFF;
  const uint32_t bar_q = bars;
  auto k_full = [&](int s) { return bars + 8u * (1 + s); };
  auto v_full = [&](int s) { return bars + 8u * (3 + s); };
  auto s_full = [&](int s) { return bars + 8u * (5 + s); };
  auto s_free = [&](int s) { return bars + 8u * (7 + s); };
  const uint32_t p_full = bars + 8u * 9;
  const uint32_t pv_done = bars + 8u * 10;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + S::BAR_OFF + S::NBARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int h = blockIdx.x;
  const int m0 = blockIdx.y * ATT_BM;
  const int b = blockIdx.z;
  const int kvh = h / (p.H / p.HK);
  const int off = p.Tk - p.Tq;  // bottom-right alignment
  const int qlo = m0 + off;
  const int qhi = m0 + ATT_BM - 1 + off;

  // packed sequences: first key of the sequence of the tile's first / last row (sequence starts do not decrease)
  const bool packed = p.seg_start != nullptr;
  const int seg_first = packed ? p.seg_start[m0] + off : 0;
  const int seg_last = packed ? p.seg_start[min(m0 + ATT_BM - 1, p.Tq - 1)] + off : 0;
  // key-block schedule: phase A = keys inside the student (or only) window, phase B = teacher-only keys
  const int a_hi = min(qhi, p.Tk - 1);
  const int a_lo = max(max(0, qlo - p.w_s + 1), seg_first);
  const int a_blk_hi = a_hi / ATT_BN;
  const int a_blk_lo = a_lo / ATT_BN;
  const int n_a = a_blk_hi - a_blk_lo + 1;
  int n_b = 0, b_blk_hi = 0;
  if (DUAL) {
    const int b_hi = min(qhi - p.w_s, p.Tk - 1);
    const int b_lo = max(max(0, qlo - p.w_t + 1), seg_first);
    if (p.w_t > p.w_s && b_hi >= b_lo) {
      b_blk_hi = b_hi / ATT_BN;
      n_b = b_blk_hi - b_lo / ATT_BN + 1;
    }
  }
  const int n_blocks = n_a + n_b;
  auto block_key0 = [&](int i) { return (i < n_a ? (a_blk_hi - i) : (b_blk_hi - (i - n_a))) * ATT_BN; };

  if (threadIdx.x == 0) {
    if ((sbase & 1023u) != 0) {  // swizzled tiles need a 1024-byte aligned base
      atomicCAS(&g_status, 0, 299);
      *abort_flag = 1;
    } else {
      *abort_flag = 0;
    }
    mbar_init(bar_q, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(k_full(s), 1);
      mbar_init(v_full(s), 1);
      mbar_init(s_full(s), 1);
      mbar_init(s_free(s), 4);
    }
    mbar_init(p_full, 4);
    mbar_init(pv_done, 1);
    mbar_fence_init();
  }
  if (warp == 4) {
    tmem_alloc(smem_u32(tmem_slot), 256);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 2 * ATT_BN;
  const bool healthy = (*abort_flag == 0);

  if (warp == 4 && healthy) {
    // ---------------------------------------------------------------- control lane: TMA + MMA
    if (elect_one()) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(ATT_BM, ATT_BN, false, false);
      constexpr uint32_t idesc_o = umma_idesc_bf16(ATT_BM, D, false, true);
      auto load_k = [&](int i) {
        const int slot = i & 1;
        mbar_expect_tx(k_full(slot), S::KV_BYTES);
        const int key0 = block_key0(i);
        const bool halo = key0 < p.halo_len;   // plain (non-multicast) TMA load from the peer's memory
        const CUtensorMap* map = halo ? &tma_kh : &tma_k;
        const int row = halo ? p.halo_row0 + key0 : key0 - p.halo_len;
        for (int d = 0; d < S::DB; ++d)
          tma_load_3d(sbase + S::K_OFF + slot * S::KV_BYTES + d * S::KV_REGION, map, k_full(slot),
                      kvh * D + d * 64, row, b);
      };
      auto load_v = [&](int i) {
        const int slot = i & 1;
        mbar_expect_tx(v_full(slot), S::KV_BYTES);
        const int key0 = block_key0(i);
        const bool halo = key0 < p.halo_len;
        const CUtensorMap* map = halo ? &tma_vh : &tma_v;
        const int row = halo ? p.halo_row0 + key0 : key0 - p.halo_len;
        for (int d = 0; d < S::DB; ++d)
          tma_load_3d(sbase + S::V_OFF + slot * S::KV_BYTES + d * S::KV_REGION, map, v_full(slot),
                      kvh * D + d * 64, row, b);
      };
      // descriptors as (low word + constant step, constant high word): one add per k-step on this thread
      constexpr uint32_t HI = umma_desc_hi_sw128(1024);
      const uint32_t q_lo = umma_desc_lo(sbase + S::Q_OFF, 16);
      auto issue_s = [&](int i) {
        const uint32_t k_lo = umma_desc_lo(sbase + S::K_OFF + (i & 1) * S::KV_BYTES, 16);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t qo = ((k / 4) * S::Q_REGION + (k % 4) * 32) >> 4;
          const uint32_t ko = ((k / 4) * S::KV_REGION + (k % 4) * 32) >> 4;
          umma_ss(tmem_base + (i & 1) * ATT_BN, umma_desc_join(q_lo + qo, HI), umma_desc_join(k_lo + ko, HI), idesc_s,
                  k != 0 ? 1u : 0u);
        }
        umma_commit(s_full(i & 1));
      };
      auto issue_pv = [&](int i) {
        // V as the MN-major B operand: 64 keys of the contraction, the next 64 columns KV_REGION bytes on
        const uint32_t v_lo = umma_desc_lo(sbase + S::V_OFF + (i & 1) * S::KV_BYTES, S::KV_REGION);
        const uint32_t acc = i != 0;
        // P (bf16) was written back over the S columns it was computed from: a tensor-memory A operand
#pragma unroll
        for (int k = 0; k < ATT_BN / 16; ++k)
          umma_ts(tmem_o, tmem_base + (i & 1) * ATT_BN + k * 8, umma_desc_join(v_lo + k * (2048 >> 4), HI), idesc_o,
                  acc | (k != 0));
        umma_commit(pv_done);
      };

      bool ok = true;
      mbar_expect_tx(bar_q, S::Q_BYTES);
#pragma unroll
      for (int d = 0; d < S::DB; ++d)
        tma_load_3d(sbase + S::Q_OFF + d * S::Q_REGION, &tma_q, bar_q, h * D + d * 64, m0, b);
      load_k(0);
      load_v(0);
      if (n_blocks > 1) load_k(1);
      ok = ok && mbar_wait(bar_q, 0, abort_flag, 201) && mbar_wait(k_full(0), 0, abort_flag, 202);
      if (ok) {
        tc_fence_after_sync();
        issue_s(0);
      }
      for (int i = 0; i < n_blocks && ok; ++i) {
        if (i + 1 < n_blocks) {
          ok = mbar_wait(k_full((i + 1) & 1), ((i + 1) >> 1) & 1, abort_flag, 203);
          if (ok && i >= 1) ok = mbar_wait(s_free((i + 1) & 1), ((i - 1) >> 1) & 1, abort_flag, 204);
          if (!ok) break;
          tc_fence_after_sync();
          issue_s(i + 1);
        }
        if (i + 2 < n_blocks) {
          ok = mbar_wait(s_full(i & 1), (i >> 1) & 1, abort_flag, 205);  // S(i) done: its K slot is free
          if (!ok) break;
          load_k(i + 2);
        }
        if (i + 1 < n_blocks) {
          if (i >= 1) ok = mbar_wait(pv_done, (i - 1) & 1, abort_flag, 206);  // PV(i-1) done: V slot free
          if (!ok) break;
          load_v(i + 1);
        }
        ok = mbar_wait(p_full, i & 1, abort_flag, 207) && mbar_wait(v_full(i & 1), (i >> 1) & 1, abort_flag, 208);
        if (!ok) break;
        tc_fence_after_sync();
        issue_pv(i);
      }
      if (!ok) {
        mbar_drain(bar_q, 0);
        for (int s = 0; s < 2; ++s) {
          mbar_drain(k_full(s), 0); mbar_drain(k_full(s), 1);
          mbar_drain(v_full(s), 0); mbar_drain(v_full(s), 1);
        }
      }
    }
  } else if (warp < 4 && healthy) {
    // ---------------------------------------------------------------- softmax warps: thread == query row
    const int row = warp * 32 + lane;          // row inside the tile == TMEM lane
    const int qpos = qlo + row;
    const int seg_lo = (packed && m0 + row < p.Tq) ? p.seg_start[m0 + row] + off : 0;   // first key of this row's sequence
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    float m_ref = -INFINITY;   // running reference max (log2 domain), possibly stale by < threshold
    float l_sum = 0.f;
    bool ok = true;
    // warp-uniform bounded wait: the .sync.aligned TMEM instructions below need all 32 lanes
    auto wait_all = [&](uint32_t bar, uint32_t parity, int code) {
      const bool r = mbar_wait(bar, parity, abort_flag, code);
      return __all_sync(0xffffffffu, r) != 0;
    };

    // write one normalised output row + its LSE
    auto write_out = [&](bf16* o_ptr, float* lse_ptr) {
      const float inv_l = l_sum > 0.f ? 1.f / l_sum : 0.f;
      const bool store = (m0 + row) < p.Tq;
      bf16* orow = o_ptr + ((static_cast<int64_t>(b) * p.Tq + (m0 + row)) * p.H + h) * D;
#pragma unroll
      for (int c = 0; c < D; c += 32) {
        uint32_t v[32];
        tmem_ld32(tmem_o + lane_addr + c, v);
        tmem_ld_wait();
        if (store) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 o;
            o.x = pack_bf16(__uint_as_float(v[j]) * inv_l, __uint_as_float(v[j + 1]) * inv_l);
            o.y = pack_bf16(__uint_as_float(v[j + 2]) * inv_l, __uint_as_float(v[j + 3]) * inv_l);
            o.z = pack_bf16(__uint_as_float(v[j + 4]) * inv_l, __uint_as_float(v[j + 5]) * inv_l);
            o.w = pack_bf16(__uint_as_float(v[j + 6]) * inv_l, __uint_as_float(v[j + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + c + j) = o;
          }
        }
      }
      if (store && lse_ptr != nullptr) {
        const float lse = l_sum > 0.f ? (m_ref + log2f(l_sum)) * 0.6931471805599453f : -INFINITY;
        lse_ptr[(static_cast<int64_t>(b) * p.H + h) * p.Tq + (m0 + row)] = lse;
      }
    };

    for (int i = 0; i < n_blocks && ok; ++i) {
      if (DUAL && i == n_a) {
        // student snapshot: every PV of phase A must have landed in TMEM
        ok = wait_all(pv_done, (i - 1) & 1, 211);
        if (!ok) break;
        tc_fence_after_sync();
        write_out(p.o_s, p.lse_s);
      }
      const bool phase_b = DUAL && i >= n_a;
      const int key0 = block_key0(i);
      ok = wait_all(s_full(i & 1), (i >> 1) & 1, 212);
      if (!ok) break;
      tc_fence_after_sync();
      uint32_t sv[ATT_BN];
      {
        uint32_t t0[32], t1[32];
        tmem_ld32(tmem_base + lane_addr + (i & 1) * ATT_BN, t0);
        tmem_ld32(tmem_base + lane_addr + (i & 1) * ATT_BN + 32, t1);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) { sv[j] = t0[j]; sv[32 + j] = t1[j]; }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free(i & 1));

      // visibility window of this row in this phase: keys in (lo_excl, hi_incl]
      int hi_incl, lo_excl;
      if (!phase_b) { hi_incl = qpos; lo_excl = qpos - p.w_s; }
      else          { hi_incl = qpos - p.w_s; lo_excl = qpos - p.w_t; }
      const bool full = (key0 + ATT_BN - 1 <= (phase_b ? qlo - p.w_s : qlo)) &&
                        (key0 > (phase_b ? qhi - p.w_t : qhi - p.w_s)) && (key0 >= seg_last);
      float mx = -INFINITY;
      if (full) {
#pragma unroll
        for (int j = 0; j < ATT_BN; ++j) {
          const float s = __uint_as_float(sv[j]) * p.scale_log2;
          sv[j] = __float_as_uint(s);
          mx = fmaxf(mx, s);
        }
      } else {
#pragma unroll
        for (int j = 0; j < ATT_BN; ++j) {
          const int key = key0 + j;
          const bool vis = key <= hi_incl && key > lo_excl && key >= seg_lo;
          const float s = vis ? __uint_as_float(sv[j]) * p.scale_log2 : -INFINITY;
          sv[j] = __float_as_uint(s);
          mx = fmaxf(mx, s);
        }
      }
      // lazy rescale: move the reference max only when it grows by more than the threshold
      const float m_new = fmaxf(m_ref, mx);
      const bool need = (m_new > m_ref + RESCALE_THRESHOLD) || (m_ref == -INFINITY && m_new > -INFINITY);
      if (i > 0) {
        // P buffer and (if rescaling) the O accumulator are free once PV(i-1) has completed
        ok = wait_all(pv_done, (i - 1) & 1, 213);
        if (!ok) break;
        tc_fence_after_sync();
        if (__any_sync(0xffffffffu, need)) {
          const float f = need ? (m_ref == -INFINITY ? 0.f : fast_exp2(m_ref - m_new)) : 1.f;
#pragma unroll
          for (int c = 0; c < D; c += 32) {
            uint32_t v[32];
            tmem_ld32(tmem_o + lane_addr + c, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * f);
            tmem_st32(tmem_o + lane_addr + c, v);
          }
          tmem_st_wait();
          l_sum *= f;
        }
      }
      if (need) m_ref = m_new;
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
      float psum = 0.f;
      uint32_t ppk[ATT_BN / 2];
#pragma unroll
      for (int c = 0; c < ATT_BN / 8; ++c) {
        float e[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          e[j] = fast_exp2(__uint_as_float(sv[c * 8 + j]) - m_use);
          psum += e[j];
        }
        ppk[4 * c] = pack_bf16(e[0], e[1]);
        ppk[4 * c + 1] = pack_bf16(e[2], e[3]);
        ppk[4 * c + 2] = pack_bf16(e[4], e[5]);
        ppk[4 * c + 3] = pack_bf16(e[6], e[7]);
      }
      l_sum += psum;
      tmem_st32(tmem_base + lane_addr + (i & 1) * ATT_BN, ppk);   // this lane's own S columns, already in registers
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok && n_blocks > 0) {
      ok = wait_all(pv_done, (n_blocks - 1) & 1, 214);
      if (ok) {
        tc_fence_after_sync();
        if (DUAL && n_b == 0) write_out(p.o_s, p.lse_s);  // equal windows: student == teacher
        if (DUAL) write_out(p.o_t, p.lse_t);
        else write_out(p.o_t, p.lse_t);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 256);
  }
}

template <int D, bool DUAL>
static int launch_attn_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                           const CUtensorMap& tkh, const CUtensorMap& tvh, const AttnFwdParams& p, int B,
                           cudaStream_t stream) {
  using S = AttnSmem<D>;
  auto kern = attn_fwd_kernel<D, DUAL>;
  static bool configured = false;
  if (!configured) {
    TTCD_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL));
    configured = true;
  }
  dim3 grid(p.H, (p.Tq + ATT_BM - 1) / ATT_BM, B);
  kern<<<grid, ATT_THREADS, S::TOTAL, stream>>>(tq, tk, tv, tkh, tvh, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace ttcd

TTCD_DEFINE_STATUS_READER(attn)

// q: [B, Tq, *] with token stride ldq and batch stride sq (elements), head h at column h*D.
// k, v: [B, Tk_local, *] likewise with HK heads.  o_t (and o_s, lse_s when dual) are contiguous
// [B, Tq, H, D] / [B, H, Tq].  window <= 0 means unlimited (full causal).
// Context parallel: k_halo / v_halo point at the previous rank's K / V buffers (same layout and strides,
// halo_rows rows); its last halo_len rows are prepended to the local keys.  halo_len % 128 == 0.
// seg_start (int32 [Tq], or null): packed sequences in one row (needs B == 1, Tq == Tk, no halo); for every token the
// first token of its sequence.
TTCD_EXPORT int ttcd_attn_fwd_cp(const void* q, const void* k, const void* v, const void* k_halo, const void* v_halo,
                                 void* o_t, void* o_s, float* lse_t, float* lse_s, int B, int Tq, int Tk_local, int H,
                                 int HK, int D, long long ldq, long long ldk, long long ldv, long long sq, long long sk,
                                 long long sv, int halo_len, int halo_rows, int window_t, int window_s, float scale,
                                 const int* seg_start, void* stream_ptr) {
  using namespace ttcd;
  const int Tk = Tk_local + halo_len;
  if (seg_start != nullptr && (B != 1 || Tq != Tk_local || halo_len != 0)) return TTCD_ERR_ARG;
  if (B <= 0 || Tq < ATT_BM || Tk_local < Tq || H <= 0 || HK <= 0 || H % HK != 0 || (D != 64 && D != 128))
    return TTCD_ERR_ARG;
  if (halo_len < 0 || halo_len % 128 != 0 || (halo_len > 0 && (k_halo == nullptr || v_halo == nullptr || halo_rows < halo_len)))
    return TTCD_ERR_ARG;
  const bool dual = o_s != nullptr;
  CUtensorMap tq, tk, tv, tkh, tvh;
  int rc = make_tmap_bf16_3d(&tq, q, static_cast<uint64_t>(H) * D, Tq, B, ldq, sq, 64, ATT_BM);
  if (rc != TTCD_OK) return rc;
  rc = make_tmap_bf16_3d(&tk, k, static_cast<uint64_t>(HK) * D, Tk_local, B, ldk, sk, 64, ATT_BN);
  if (rc != TTCD_OK) return rc;
  rc = make_tmap_bf16_3d(&tv, v, static_cast<uint64_t>(HK) * D, Tk_local, B, ldv, sv, 64, ATT_BN);
  if (rc != TTCD_OK) return rc;
  tkh = tk;
  tvh = tv;
  if (halo_len > 0) {
    rc = make_tmap_bf16_3d(&tkh, k_halo, static_cast<uint64_t>(HK) * D, halo_rows, B, ldk, sk, 64, ATT_BN);
    if (rc != TTCD_OK) return rc;
    rc = make_tmap_bf16_3d(&tvh, v_halo, static_cast<uint64_t>(HK) * D, halo_rows, B, ldv, sv, 64, ATT_BN);
    if (rc != TTCD_OK) return rc;
  }
  const int big = 1 << 30;
  AttnFwdParams p;
  p.o_t = static_cast<bf16*>(o_t); p.o_s = static_cast<bf16*>(o_s);
  p.lse_t = lse_t; p.lse_s = lse_s;
  p.Tq = Tq; p.Tk = Tk; p.H = H; p.HK = HK;
  p.w_t = window_t > 0 ? window_t : big;
  p.w_s = window_s > 0 ? window_s : big;
  if (!dual) p.w_s = p.w_t;  // single-window mode runs phase A only, with the one window
  p.scale_log2 = scale * 1.4426950408889634f;
  p.seg_start = seg_start;
  p.halo_len = halo_len;
  p.halo_row0 = halo_rows - halo_len;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  if (D == 128) return dual ? launch_attn_fwd<128, true>(tq, tk, tv, tkh, tvh, p, B, stream)
                            : launch_attn_fwd<128, false>(tq, tk, tv, tkh, tvh, p, B, stream);
  return dual ? launch_attn_fwd<64, true>(tq, tk, tv, tkh, tvh, p, B, stream)
              : launch_attn_fwd<64, false>(tq, tk, tv, tkh, tvh, p, B, stream);
}

TTCD_EXPORT int ttcd_attn_fwd(const void* q, const void* k, const void* v, void* o_t, void* o_s, float* lse_t,
                              float* lse_s, int B, int Tq, int Tk, int H, int HK, int D, long long ldq,
                              long long ldk, long long ldv, long long sq, long long sk, long long sv,
                              int window_t, int window_s, float scale, const int* seg_start, void* stream_ptr) {
  return ttcd_attn_fwd_cp(q, k, v, nullptr, nullptr, o_t, o_s, lse_t, lse_s, B, Tq, Tk, H, HK, D, ldq, ldk, ldv, sq, sk,
                          sv, 0, 0, window_t, window_s, scale, seg_start, stream_ptr);
}
