// Sliding-window attention backward for sm_100a (single- and dual-window), two kernels, no atomics:
//
//   attn_bwd_dkdv : one CTA per (128-key block, kv head, batch); loops over the query blocks (64 rows)
//                   and the query heads of the GQA group that can see those keys.  Per step it forms
//                   S^T = K Q^T and dP^T = V dO^T on tcgen05 (keys on the TMEM lanes), the element-wise warps
//                   turn them into P^T and dS^T, and dV += P^T dO, dK += dS^T Q accumulate in TMEM.
//   attn_bwd_dq   : one CTA per (128-query block, head, batch); loops over the key blocks (64 keys) of
//                   the teacher window, recomputes S / dP and accumulates dQ += dS K in TMEM.
//
// Dual window goes through ONE softmax: inside the student window P_S = r P_T with the per-row ratio
// r = exp(lse_T - lse_S), so the student's gradient stream folds into the teacher's (dO' = dO_T + r dO_S,
// delta' = delta_T + r delta_S, formed once per layer by attn_combine_kernel); every block step then uses either
// (dO', delta', keys inside the student window) or (dO_T, delta_T, keys outside it), and the blocks that straddle
// the window edge take one step of each.
//
// Roles per CTA: 16 element-wise warps in two groups that take alternate steps (group g works on TMEM set g, so the
// element-wise work of step i+1 starts as soon as its S / dP are there), one warp whose elected thread issues every
// tcgen05.mma / tcgen05.commit, one warp whose elected thread issues every TMA copy.  The S / dP accumulators are
// double-buffered in TMEM; P^T / dS^T go back into tensor memory over the columns they were computed from and feed
// the accumulate MMAs as TMEM A operands; operand tiles come through a 4-5 slot TMA ring (128-byte swizzle, no
// multicast) with per-slot "free" barriers.  One swizzled tile serves as a K-major operand of one MMA and an
// MN-major operand of another (Q and dO in dkdv, K in dq), so nothing is transposed in memory.
//
// Packed batches (several sequences in one row): per-token `seg_start` / `seg_end` arrays bound the visible keys of
// a query to its own sequence inside the kernels (the role of flash_attn_varlen_func in fla/layers/attn.py:229-270),
// and the block ranges are clipped to the sequences that a tile touches.
//
// The reference has no fused dual-window backward: training there runs two flash-attn backward passes whose
// dq/dk/dv are summed by autograd (custom_models/ipttcd/modeling_ipttcdv9.py:686-690;
// profiling/FUSED_ATTENTION_DESIGN.md:68-69).
// every role of these kernels waits long enough per step for parked waits to pay (measured: 13.8 vs 14.3 ms)
#define TTCD_PARK_ALL_WAITS 1
#include "common.cuh"

#include <algorithm>

namespace ttcd {

// 16 element-wise warps + 1 tensor-core issue warp + 1 TMA producer warp (one elected thread each: a thread that
// issued the copies as well spent more clocks per step on them than the tensor core needs for the step).  A warp
// may only touch the TMEM lanes of its quarter (warp % 4); two warps per quarter split the 64 S columns of a step,
// and the two groups of eight warps take alternate steps.
constexpr int BWD_EW_WARPS = 16;
constexpr int BWD_THREADS = (BWD_EW_WARPS + 2) * 32;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void named_barrier_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// TMEM column offset (inside an S / dP column group of 64) of the 8 packed bf16 columns that hold k-step `k` (16
// rows of the contraction): each of the two warps of a lane quarter packs its 32 columns in place into 16
__device__ __forceinline__ constexpr uint32_t ts_packed_off(int k) {
  return static_cast<uint32_t>(32 * (k / 2) + 8 * (k % 2));
}

// Division of a step index by a per-CTA constant (steps per head, ring slots) without the integer-division
// sequence: exact for n, d < 65536 with magic = 2^32 / d + 1.  The control thread runs this several times between
// two tensor-core issues, where every instruction of latency is idle tensor time.
struct FastDiv {
  uint32_t d, magic;
  __device__ __forceinline__ explicit FastDiv(int div) : d(static_cast<uint32_t>(div < 1 ? 1 : div)), magic(0xffffffffu / d + 1u) {}
  __device__ __forceinline__ int div(int n) const {
    return (n < 65536 && d < 65536u && d > 1u) ? static_cast<int>(__umulhi(static_cast<uint32_t>(n), magic))
                                     : static_cast<int>(static_cast<uint32_t>(n) / d);
  }
  __device__ __forceinline__ int mod(int n) const { return n - div(n) * static_cast<int>(d); }
};

struct AttnBwdParams {
  const float* lse_t;                           // [B, H, Tq] natural log (teacher / only window)
  const float* delta_t;                         // [B, H, Tq] rowsum(dO_T * O_T)
  const float* delta_c;                         // dual: delta' = delta_T + r delta_S
  bf16* dq; bf16* dk; bf16* dv;                 // [B,Tq,H,D], [B,Tk,HK,D], [B,Tk,HK,D]
  int Tq, Tk, H, HK;
  int w_t, w_s;
  float scale, scale_log2;
  // context parallel: keys [0, halo_len) live in the previous rank's K/V buffers (rows halo_row0..)
  int halo_len, halo_row0;
  // dV may be written into a wider row (the packed q|k|v gradient of a fused projection): row and batch strides
  // in elements; 0 = contiguous [B, Tk, HK, D]
  int64_t ld_dv, sb_dv;
  // dual window: the second dO tensor map addresses dO', `delta_c` holds delta' (see the file header)
  int combine;
  // packed sequences (null: none): per token, the first token of its sequence and one past its last
  const int* seg_start; const int* seg_end;
  // check of the bounded waits: the dK/dV producer leaves out the K/V copies, so that the wait for them runs out
  int skip_kv_load;
};

// 32 fp32 accumulator columns (times `scale`) -> 32 bf16 written to global memory (64 contiguous bytes)
__device__ __forceinline__ void store_out32(bf16* dst, const uint32_t (&a)[32], float scale = 1.f) {
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    uint4 o;
    o.x = pack_bf16(__uint_as_float(a[j]) * scale, __uint_as_float(a[j + 1]) * scale);
    o.y = pack_bf16(__uint_as_float(a[j + 2]) * scale, __uint_as_float(a[j + 3]) * scale);
    o.z = pack_bf16(__uint_as_float(a[j + 4]) * scale, __uint_as_float(a[j + 5]) * scale);
    o.w = pack_bf16(__uint_as_float(a[j + 6]) * scale, __uint_as_float(a[j + 7]) * scale);
    *reinterpret_cast<uint4*>(dst + j) = o;
  }
}

// Element-wise core of the dK/dV step for one thread: NC query columns of one key row.
//   stats: shared-memory block [-lse*log2e | delta | first token of the query's sequence (int bits)], 64 each,
//          already offset to this thread's first column.
//   p = 2^(s*c - lse),  dS (unscaled) = p (dP - delta);  visible pairs:  qpos - hi < key <= qpos - lo
//   (and key >= the query's sequence start when PACKED).
// MASKED = false is the common case of a block that is fully visible.
// Packed fp32 pairs (two lanes per FFMA / FMUL): the element-wise phase is bound by instruction issue.
template <bool MASKED, bool PACKED, int NC>
__device__ __forceinline__ void dkdv_elementwise(const uint32_t (&sv)[NC], const uint32_t (&dpt)[NC], const float* stats,
                                                 float scale_log2, int key, int qpos0, int lo, int hi, bool key_ok,
                                                 uint32_t (&ptp)[NC / 2], uint32_t (&dsp)[NC / 2]) {
  const float2 sc2 = make_float2(scale_log2, scale_log2), neg1 = make_float2(-1.f, -1.f);
#pragma unroll
  for (int c = 0; c < NC; c += 4) {
    const float4 nl = *reinterpret_cast<const float4*>(stats + c);
    const float4 dl = *reinterpret_cast<const float4*>(stats + 64 + c);
    int4 sg = make_int4(0, 0, 0, 0);
    if (MASKED && PACKED) sg = *reinterpret_cast<const int4*>(stats + 128 + c);
#pragma unroll
    for (int hp = 0; hp < 2; ++hp) {
      const int j0 = c + 2 * hp;
      const float2 n2 = hp ? make_float2(nl.z, nl.w) : make_float2(nl.x, nl.y);
      const float2 l2 = hp ? make_float2(dl.z, dl.w) : make_float2(dl.x, dl.y);
      const float2 x2 = __ffma2_rn(make_float2(__uint_as_float(sv[j0]), __uint_as_float(sv[j0 + 1])), sc2, n2);
      float2 p2 = make_float2(ex2(x2.x), ex2(x2.y));
      if (MASKED) {
        const int qpos = qpos0 + j0;
        const int s0 = hp ? sg.z : sg.x, s1 = hp ? sg.w : sg.y;
        if (!(key_ok && key <= qpos - lo && key > qpos - hi && key >= s0)) p2.x = 0.f;
        if (!(key_ok && key <= qpos + 1 - lo && key > qpos + 1 - hi && key >= s1)) p2.y = 0.f;
      }
      const float2 dd = __ffma2_rn(l2, neg1, make_float2(__uint_as_float(dpt[j0]), __uint_as_float(dpt[j0 + 1])));
      const float2 d2 = __fmul2_rn(p2, dd);
      ptp[j0 / 2] = pack_bf16(p2.x, p2.y);
      dsp[j0 / 2] = pack_bf16(d2.x, d2.y);
    }
  }
}

// Element-wise core of the dQ step: NC key columns of one query row (statistics live in registers); visible pairs
// qpos - hi < key <= qpos - lo and key >= seg_lo (the first key of the query's sequence; 0 without packing).
template <bool MASKED, int NC>
__device__ __forceinline__ void dq_elementwise(const uint32_t (&sv)[NC], const uint32_t (&dpt)[NC], float scale_log2,
                                               float nlse, float del, int qpos, int key0, int lo, int hi, int seg_lo,
                                               uint32_t (&dsp)[NC / 2]) {
  const float2 sc2 = make_float2(scale_log2, scale_log2), n2 = make_float2(nlse, nlse);
  const float2 nd2 = make_float2(-del, -del);
#pragma unroll
  for (int c = 0; c < NC; c += 2) {
    const float2 x2 = __ffma2_rn(make_float2(__uint_as_float(sv[c]), __uint_as_float(sv[c + 1])), sc2, n2);
    float2 p2 = make_float2(ex2(x2.x), ex2(x2.y));
    if (MASKED) {
      const int key = key0 + c;
      if (!(key <= qpos - lo && key > qpos - hi && key >= seg_lo)) p2.x = 0.f;
      if (!(key + 1 <= qpos - lo && key + 1 > qpos - hi && key + 1 >= seg_lo)) p2.y = 0.f;
    }
    const float2 dd = __fadd2_rn(make_float2(__uint_as_float(dpt[c]), __uint_as_float(dpt[c + 1])), nd2);
    const float2 d2 = __fmul2_rn(p2, dd);
    dsp[c / 2] = pack_bf16(d2.x, d2.y);
  }
}

// =================================================================================================
// dK / dV
// =================================================================================================
template <int D>
struct DkdvCfg {
  static constexpr int DB = D / 64;
  static constexpr int NSETS = 2;               // S/dP accumulator sets in TMEM
  static constexpr int NSLOTS = 4;              // Q/dO tile ring: a tile load has two steps to arrive
  static constexpr int SET_COLS = 128;
  static constexpr int KEY_REGION = 128 * 128;  // [128 keys x 64 d] swizzled
  static constexpr int ROW_REGION = 64 * 128;   // [64 rows x 64 d] swizzled
  static constexpr int TILE_BYTES = DB * ROW_REGION;
  static constexpr int NTILES = 2;              // Q, dO per slot
  static constexpr int K_OFF = 0;
  static constexpr int V_OFF = K_OFF + DB * KEY_REGION;
  static constexpr int RING_OFF = V_OFF + DB * KEY_REGION;            // NSLOTS x NTILES x TILE_BYTES
  static constexpr int VEC_OFF = RING_OFF + NSLOTS * NTILES * TILE_BYTES;   // 4 slots x 4 vectors x 64 words
  static constexpr int BAR_OFF = VEC_OFF + 4 * 4 * 64 * 4;
  // kv_full, tiles_full[NSLOTS], sdp_full[NSETS], ew_done[2], all_done, slot_free[NSLOTS]
  static constexpr int NBARS = 1 + NSLOTS + NSETS + 2 + 1 + NSLOTS;
  static constexpr int TOTAL = BAR_OFF + NBARS * 8 + 16;
};

template <int D>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                     const __grid_constant__ CUtensorMap tma_v, const __grid_constant__ CUtensorMap tma_dot,
                     const __grid_constant__ CUtensorMap tma_doc, const __grid_constant__ CUtensorMap tma_kh,
                     const __grid_constant__ CUtensorMap tma_vh, const AttnBwdParams p) {
  using C = DkdvCfg<D>;
  constexpr int NEW = BWD_EW_WARPS;
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bars = sbase + C::BAR_OFF;
  const uint32_t kv_full = bars;
  auto tiles_full = [&](int s) { return bars + 8u * (1 + s); };
  auto sdp_full = [&](int s) { return bars + 8u * (1 + C::NSLOTS + s); };
  auto ew_done = [&](int g) { return bars + 8u * (1 + C::NSLOTS + C::NSETS + g); };
  const uint32_t all_done = ew_done(2);
  auto slot_free = [&](int s) { return all_done + 8u * (1 + s); };   // the MMAs that read ring slot s have completed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::BAR_OFF + C::NBARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* vecs = reinterpret_cast<float*>(smem + C::VEC_OFF);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * 128;
  const int kvh = blockIdx.y;
  const int b = blockIdx.z;
  const int G = p.H / p.HK;
  const int off = p.Tk - p.Tq;
  const bool packed = p.seg_start != nullptr;

  // query rows that can see keys [n0, n0+127] through the teacher window (and, packed, inside their sequences)
  const int row_lo = max(0, n0 - off);
  int row_hi = min(p.Tq - 1, n0 + 127 + p.w_t - 1 - off);
  if (packed) row_hi = min(row_hi, p.seg_end[min(n0 + 127, p.Tk - 1)] - 1 - off);
  const int jb_lo = row_lo / 64;
  const int nqb = row_hi >= row_lo ? (row_hi / 64 - jb_lo + 1) : 0;
  // dual window: query blocks [jb_lo, jb1) only hold pairs inside the student window, (jb2, ..] only pairs
  // outside it, [jb1, jb2] straddle its edge and take two steps (student part, then teacher-only part)
  const bool combine = p.combine != 0;
  int pre = nqb, nb = 0, jb1 = 0;
  if (combine && nqb > 0) {
    auto fdiv = [](int a, int d) { return a >= 0 ? a / d : -((-a + d - 1) / d); };
    const int first_t = fdiv(n0 + p.w_s - off - 63 + 63, 64);        // ceil((n0 + w_s - off - 63) / 64)
    const int last_s = fdiv(n0 + 126 + p.w_s - off, 64);
    jb1 = min(max(first_t, jb_lo), jb_lo + nqb);
    const int jb2 = min(last_s, jb_lo + nqb - 1);
    pre = jb1 - jb_lo;
    nb = max(0, jb2 - jb1 + 1);
  }
  const int steps = nqb + nb;
  const int n_iters = steps * G;

  if (threadIdx.x == 0) {
    *abort_flag = ((sbase & 1023u) != 0) ? 1 : 0;
    if (*abort_flag) atomicCAS(&g_status, 0, 399);
    mbar_init(kv_full, 1);
    for (int s = 0; s < C::NSLOTS; ++s) mbar_init(tiles_full(s), 1);
    for (int s = 0; s < C::NSETS; ++s) mbar_init(sdp_full(s), 1);
    mbar_init(ew_done(0), 8);
    mbar_init(ew_done(1), 8);
    mbar_init(all_done, 1);
    for (int s = 0; s < C::NSLOTS; ++s) mbar_init(slot_free(s), 1);
    mbar_fence_init();
  }
  if (warp == NEW) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_dk = tmem_base, t_dv = tmem_base + 128;
  auto t_set = [&](int it) { return tmem_base + 256 + (it & 1) * C::SET_COLS; };  // S^T | dP^T
  const bool healthy = (*abort_flag == 0);

  const FastDiv by_steps(steps);
  auto iter_head = [&](int it) { return kvh * G + by_steps.div(it); };
  auto iter_block = [&](int it) {          // query block of step `it`
    const int s = by_steps.mod(it);
    if (s < pre) return jb_lo + s;
    if (s < pre + 2 * nb) return jb1 + (s - pre) / 2;
    return jb_lo + s - nb;
  };
  auto iter_inner = [&](int it) {          // dual: 1 = student part (dO', delta'), 0 = teacher-only part
    if (!combine) return 0;
    const int s = by_steps.mod(it);
    if (s < pre) return 1;
    if (s < pre + 2 * nb) return ((s - pre) & 1) ? 0 : 1;
    return 0;
  };
  auto iter_row0 = [&](int it) { return iter_block(it) * 64; };
  auto slot_base = [&](int it) { return sbase + C::RING_OFF + (it & (C::NSLOTS - 1)) * C::NTILES * C::TILE_BYTES; };
  static_assert((C::NSLOTS & (C::NSLOTS - 1)) == 0, "ring slots: power of two");

  if (warp == NEW + 1 && healthy && n_iters > 0) {
    // ---- TMA producer: K/V of this key block once, then the Q / dO tiles of every step through the ring
    if (elect_one()) {
      auto load_tiles = [&](int it) {
        const int slot = it & (C::NSLOTS - 1);
        const int h = iter_head(it), r0 = iter_row0(it);
        const uint32_t base = slot_base(it);
        mbar_expect_tx(tiles_full(slot), C::TILE_BYTES * 2);
    #pragma unroll
        for (int d = 0; d < C::DB; ++d) {
          tma_load_3d(base + d * C::ROW_REGION, &tma_q, tiles_full(slot), h * D + d * 64, r0, b);
          tma_load_3d(base + C::TILE_BYTES + d * C::ROW_REGION, iter_inner(it) ? &tma_doc : &tma_dot, tiles_full(slot),
                      h * D + d * 64, r0, b);
        }
      };
      bool ok = true;
      if (!p.skip_kv_load) {
        mbar_expect_tx(kv_full, 2 * C::DB * C::KEY_REGION);
#pragma unroll
        for (int d = 0; d < C::DB; ++d) {
          const bool halo = n0 < p.halo_len;  // plain TMA loads from the previous rank's memory
          const int krow = halo ? p.halo_row0 + n0 : n0 - p.halo_len;
          tma_load_3d(sbase + C::K_OFF + d * C::KEY_REGION, halo ? &tma_kh : &tma_k, kv_full, kvh * D + d * 64, krow, b);
          tma_load_3d(sbase + C::V_OFF + d * C::KEY_REGION, halo ? &tma_vh : &tma_v, kv_full, kvh * D + d * 64, krow, b);
        }
      }
      for (int it = 0; it < n_iters && ok; ++it) {
        if (it >= C::NSLOTS) {              // the slot's previous tiles (step it - NSLOTS) have been consumed
          ok = mbar_wait_parked(slot_free(it & (C::NSLOTS - 1)), ((it / C::NSLOTS) - 1) & 1, abort_flag, 304);
          if (!ok) break;
        }
        load_tiles(it);
      }
      // stay until every copy has been consumed (or the CTA gave up): no copy may be in flight at exit
      if (ok) ok = mbar_wait_parked(all_done, 0, abort_flag, 306);
      if (!ok) {
        if (!p.skip_kv_load) mbar_drain(kv_full, 0);
        for (int s = 0; s < C::NSLOTS; ++s) { mbar_drain(tiles_full(s), 0); mbar_drain(tiles_full(s), 1); }
      }
    }
  } else if (warp == NEW && healthy && n_iters > 0) {
    // ---- tensor-core issue
    if (elect_one()) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 64, false, false);  // [keys x q] = A(K-major) B(K-major)
      constexpr uint32_t idesc_acc = umma_idesc_bf16(128, D, false, true);   // [keys x D] = A(TMEM) B(MN-major)
      // descriptors as (low word + constant step, constant high word): one add per k-step on this thread
      constexpr uint32_t HI = umma_desc_hi_sw128(1024);
      const uint32_t k_lo = umma_desc_lo(sbase + C::K_OFF, 16), v_lo = umma_desc_lo(sbase + C::V_OFF, 16);
      auto issue_sdp = [&](int it) {
        const uint32_t sq = slot_base(it);
        const uint32_t q_lo = umma_desc_lo(sq, 16), do_lo = q_lo + (C::TILE_BYTES >> 4);
        const uint32_t ts = t_set(it);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t ko = ((k / 4) * C::KEY_REGION + (k % 4) * 32) >> 4;
          const uint32_t ro = ((k / 4) * C::ROW_REGION + (k % 4) * 32) >> 4;
          umma_ss(ts, umma_desc_join(k_lo + ko, HI), umma_desc_join(q_lo + ro, HI), idesc_s, k != 0);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t ko = ((k / 4) * C::KEY_REGION + (k % 4) * 32) >> 4;
          const uint32_t ro = ((k / 4) * C::ROW_REGION + (k % 4) * 32) >> 4;
          umma_ss(ts + 64, umma_desc_join(v_lo + ko, HI), umma_desc_join(do_lo + ro, HI), idesc_s, k != 0);
        }
        umma_commit(sdp_full(it & 1));
      };
      auto issue_acc = [&](int it) {
        const uint32_t sq = slot_base(it);
        // Q / dO tiles as MN-major B operands: 64 rows of the contraction, the next 64 columns ROW_REGION bytes on
        const uint32_t qm_lo = umma_desc_lo(sq, C::ROW_REGION), dom_lo = qm_lo + (C::TILE_BYTES >> 4);
        const uint32_t acc = it != 0;
        const uint32_t ts = t_set(it);
#pragma unroll
        for (int k = 0; k < 4; ++k)       // 16 queries = 8 packed columns at the start of their warp's column group
          umma_ts(t_dv, ts + ts_packed_off(k), umma_desc_join(dom_lo + k * (2048 >> 4), HI), idesc_acc, acc | (k != 0));
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_ts(t_dk, ts + 64 + ts_packed_off(k), umma_desc_join(qm_lo + k * (2048 >> 4), HI), idesc_acc, acc | (k != 0));
      };

      bool ok = mbar_wait(kv_full, 0, abort_flag, 301);
      if (ok) ok = mbar_wait(tiles_full(0), 0, abort_flag, 302);
      if (ok) { tc_fence_after_sync(); issue_sdp(0); }
      for (int it = 0; it < n_iters && ok; ++it) {
        // S/dP for the step the element-wise warps will need next
        const int nxt = it + 1;
        if (nxt < n_iters) {
          ok = mbar_wait(tiles_full(nxt & (C::NSLOTS - 1)), (nxt / C::NSLOTS) & 1, abort_flag, 303);
          if (!ok) break;
          tc_fence_after_sync();
          issue_sdp(nxt);  // its TMEM set was last read by the accumulate MMAs of step nxt - 2, issued before
        }
        ok = mbar_wait(ew_done(it & 1), (it >> 1) & 1, abort_flag, 305);
        if (!ok) break;
        tc_fence_after_sync();
        issue_acc(it);
        umma_commit(slot_free(it & (C::NSLOTS - 1)));   // the producer may refill this step's ring slot
      }
      if (ok) umma_commit(all_done);      // every accumulate MMA has completed when this arrives
    }
  } else if (warp < NEW && healthy) {
    constexpr int NC = 16;                      // S^T columns (queries) per pass; a thread owns 32 of a step
    const int grp = warp >> 3;                  // takes steps grp, grp + 2, ...
    const int quarter = warp & 3, part = (warp >> 2) & 1;
    const int krow = quarter * 32 + lane;       // key row inside the block == TMEM lane
    const int key = n0 + krow;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const int ctid = threadIdx.x & 255;         // thread of the group: fetches one row statistic per step
    // statistics slot of a step: the two groups own two slots each
    auto vslot_of = [&](int it) { return vecs + ((it & 1) * 2 + ((it >> 1) & 1)) * 256; };
    bool ok = true;
    auto wait_all = [&](uint32_t bar, uint32_t parity, int code) {
      const bool r = mbar_wait_parked(bar, parity, abort_flag, code);
      return __all_sync(0xffffffffu, r) != 0;
    };
    // per-row statistics of a query block: [-lse*log2e | delta | sequence start], 64 each; this thread fetches
    // element (which, r) of the block used by step `it`.  The load is issued here and its value is first touched
    // by finish_stat at the end of the step, so that its latency is not waited out here.
    const int which = ctid >> 6;
    auto fetch_stat = [&](int it) -> float {
      const int row = iter_row0(it) + (ctid & 63);
      const int64_t idx = (static_cast<int64_t>(b) * p.H + iter_head(it)) * p.Tq + row;
      if (which == 0) return row < p.Tq ? p.lse_t[idx] : INFINITY;          // p = 0 past the end (after the negation)
      if (which == 1) return row < p.Tq ? (iter_inner(it) ? p.delta_c : p.delta_t)[idx] : 0.f;
      if (which == 2 && packed) return __int_as_float(p.seg_start[min(row, p.Tq - 1)] + off);
      return 0.f;
    };
    auto finish_stat = [&](float raw) { return which == 0 ? -raw * LOG2E : raw; };
    const int it0 = grp;
    if (it0 < n_iters) vslot_of(it0)[ctid] = finish_stat(fetch_stat(it0));
    for (int it = it0; it < n_iters && ok; it += 2) {
      const int r0 = iter_row0(it);
      const float* vslot = vslot_of(it);
      const float next_stat = (it + 2 < n_iters) ? fetch_stat(it + 2) : 0.f;  // in flight during this step
      named_barrier_sync(1 + grp, 256);
      ok = wait_all(sdp_full(it & 1), (it >> 1) & 1, 311);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t ts = t_set(it) + lane_addr + part * 32;      // set == grp
      const int qlo_b = r0 + off, qhi_b = r0 + 63 + off;
      const bool key_ok = key < p.Tk;
      // visible pairs of this step:  qpos - hi < key <= qpos - lo  (dual: student part, then teacher-only part)
      const int inner = iter_inner(it);
      const int lo = combine ? (inner ? 0 : p.w_s) : 0, hi = combine ? (inner ? p.w_s : p.w_t) : p.w_t;
      // fully visible block: every (key, query) pair passes
      bool full = (n0 + 127 <= qlo_b - lo) && (n0 > qhi_b - hi) && (n0 + 127 < p.Tk);
      if (packed) full = full && (n0 >= __float_as_int(vslot[128 + 63]));     // sequence starts do not decrease
#pragma unroll
      for (int h = 0; h < 2; ++h) {             // two passes of 16 columns keep the registers low
        uint32_t sv[NC], dpt[NC];
        tmem_ld_n<NC>(ts + h * NC, sv);
        tmem_ld_n<NC>(ts + 64 + h * NC, dpt);
        tmem_ld_wait();
        uint32_t ptp[NC / 2], dsp[NC / 2];
        const float* stats = vslot + part * 32 + h * NC;
        const int qpos0 = r0 + part * 32 + h * NC + off;
        if (full)
          dkdv_elementwise<false, false, NC>(sv, dpt, stats, p.scale_log2, key, qpos0, lo, hi, key_ok, ptp, dsp);
        else if (packed)
          dkdv_elementwise<true, true, NC>(sv, dpt, stats, p.scale_log2, key, qpos0, lo, hi, key_ok, ptp, dsp);
        else
          dkdv_elementwise<true, false, NC>(sv, dpt, stats, p.scale_log2, key, qpos0, lo, hi, key_ok, ptp, dsp);
        // packed over the first half of this thread's own S^T / dP^T columns, all of which (up to this pass) are read
        tmem_st_n<NC / 2>(ts + h * (NC / 2), ptp);
        tmem_st_n<NC / 2>(ts + 64 + h * (NC / 2), dsp);
      }
      tmem_st_wait();
      if (it + 2 < n_iters) vslot_of(it + 2)[ctid] = finish_stat(next_stat);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(ew_done(it & 1));
    }
    // epilogue: dK, dV -> global (this thread: key row `krow`, one half of the D columns; group 0 writes dK and
    // group 1 dV)
    if (ok) {
      if (n_iters > 0) ok = wait_all(all_done, 0, 313);
      if (ok) {
        const int half = part;
        const bool do_k = grp == 0, do_v = grp == 1;
        tc_fence_after_sync();
        const bool store = key < p.Tk;
        const int64_t rowoff = ((static_cast<int64_t>(b) * p.Tk + key) * p.HK + kvh) * D;
        const int64_t voff = p.ld_dv != 0 ? static_cast<int64_t>(b) * p.sb_dv + static_cast<int64_t>(key) * p.ld_dv +
                                                static_cast<int64_t>(kvh) * D
                                          : rowoff;
        constexpr int COLS = D / 2;
#pragma unroll
        for (int c = 0; c < COLS; c += 32) {
          uint32_t a[32];
          if (n_iters > 0) {
            tmem_ld32((do_k ? t_dk : t_dv) + lane_addr + half * COLS + c, a);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) a[j] = 0u;
          }
          if (store && do_k) store_out32(p.dk + rowoff + half * COLS + c, a, p.scale);  // dS was kept unscaled
          if (store && do_v) store_out32(p.dv + voff + half * COLS + c, a);
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == NEW) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// =================================================================================================
// dQ
// =================================================================================================
template <int D, bool DUAL>
struct DqCfg {
  static constexpr int DB = D / 64;
  static constexpr int NSLOTS = DUAL ? 4 : 5;      // K/V ring: a tile load has NSLOTS - 2 steps to arrive
  static constexpr int SET_COLS = 128;
  static constexpr int Q_REGION = 128 * 128;
  static constexpr int KV_REGION = 64 * 128;
  static constexpr int KV_BYTES = DB * KV_REGION;
  static constexpr int Q_OFF = 0;
  static constexpr int DOT_OFF = Q_OFF + DB * Q_REGION;
  static constexpr int DOC_OFF = DOT_OFF + DB * Q_REGION;                 // dO': only used when DUAL
  static constexpr int RING_OFF = DOC_OFF + (DUAL ? DB * Q_REGION : 0);   // NSLOTS x (K, V)
  static constexpr int BAR_OFF = RING_OFF + NSLOTS * 2 * KV_BYTES;
  // q_full, kv_full[NSLOTS], sdp_full[2], ew_done[2], a_ready, all_done, slot_free[NSLOTS]
  static constexpr int NBARS = 1 + NSLOTS + 2 + 2 + 2 + NSLOTS;
  // 128 (dQ) + 2 x 128 (S | dP sets) leaves 128 columns: Q and one dO as bf16 A operands in tensor memory (single
  // window: dO; dual window: dO', used by the steps inside the student window; the teacher-only steps read dO_T from
  // shared memory)
  static constexpr int A_COLS = D / 2;
  static constexpr int TOTAL = BAR_OFF + NBARS * 8 + 16;
};

template <int D, bool DUAL>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                   const __grid_constant__ CUtensorMap tma_v, const __grid_constant__ CUtensorMap tma_dot,
                   const __grid_constant__ CUtensorMap tma_doc, const __grid_constant__ CUtensorMap tma_kh,
                   const __grid_constant__ CUtensorMap tma_vh, const AttnBwdParams p) {
  using C = DqCfg<D, DUAL>;
  constexpr int NEW = BWD_EW_WARPS;
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bars = sbase + C::BAR_OFF;
  const uint32_t q_full = bars;
  auto kv_full = [&](int s) { return bars + 8u * (1 + s); };
  auto sdp_full = [&](int s) { return bars + 8u * (1 + C::NSLOTS + s); };
  auto ew_done = [&](int g) { return bars + 8u * (3 + C::NSLOTS + g); };
  const uint32_t a_ready = ew_done(2);
  const uint32_t all_done = a_ready + 8u;
  auto slot_free = [&](int s) { return all_done + 8u * (1 + s); };   // the MMAs that read ring slot s have completed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::BAR_OFF + C::NBARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x;
  const int m0 = blockIdx.y * 128;
  const int b = blockIdx.z;
  const int kvh = h / (p.H / p.HK);
  const int off = p.Tk - p.Tq;
  const int qlo = m0 + off, qhi = m0 + 127 + off;
  const bool packed = p.seg_start != nullptr;
  // packed sequences: first key of the sequence of the tile's first / last row (sequence starts do not decrease)
  const int seg_first = packed ? p.seg_start[m0] + off : 0;
  const int seg_last = packed ? p.seg_start[min(m0 + 127, p.Tq - 1)] + off : 0;
  const int key_hi = min(qhi, p.Tk - 1);
  const int key_lo = max(max(0, qlo - p.w_t + 1), seg_first);
  const int blk_lo = key_lo / 64;
  const int nblk = key_hi / 64 - blk_lo + 1;
  // dual window: key blocks [blk_lo, kb1) hold only teacher-only pairs, (kb2, ..] only pairs inside the student
  // window, [kb1, kb2] straddle its edge and take two steps
  const bool combine = DUAL && p.combine != 0;
  int pre = nblk, nb = 0, kb1 = 0;
  if (combine) {
    auto fdiv = [](int a, int d) { return a >= 0 ? a / d : -((-a + d - 1) / d); };
    kb1 = min(max(fdiv(qlo - p.w_s + 1, 64), blk_lo), blk_lo + nblk);
    const int kb2 = min(fdiv(qhi - p.w_s, 64), blk_lo + nblk - 1);
    pre = kb1 - blk_lo;
    nb = max(0, kb2 - kb1 + 1);
  }
  const int n_iters = nblk + nb;
  auto iter_block = [&](int it) {
    if (it < pre) return blk_lo + it;
    if (it < pre + 2 * nb) return kb1 + (it - pre) / 2;
    return blk_lo + it - nb;
  };
  auto iter_inner = [&](int it) {          // 1 = pairs inside the student window (dO', delta'), 0 = teacher-only pairs
    if (!combine) return 0;
    if (it < pre) return 0;
    if (it < pre + 2 * nb) return (it - pre) & 1;
    return 1;
  };
  auto iter_key0 = [&](int it) { return iter_block(it) * 64; };
  const FastDiv by_slots(C::NSLOTS);
  auto slot_base = [&](int it) { return sbase + C::RING_OFF + by_slots.mod(it) * 2 * C::KV_BYTES; };

  if (threadIdx.x == 0) {
    *abort_flag = ((sbase & 1023u) != 0) ? 1 : 0;
    if (*abort_flag) atomicCAS(&g_status, 0, 398);
    mbar_init(q_full, 1);
    for (int s = 0; s < C::NSLOTS; ++s) mbar_init(kv_full(s), 1);
    mbar_init(sdp_full(0), 1);
    mbar_init(sdp_full(1), 1);
    mbar_init(ew_done(0), 8);
    mbar_init(ew_done(1), 8);
    mbar_init(a_ready, NEW);
    mbar_init(all_done, 1);
    for (int s = 0; s < C::NSLOTS; ++s) mbar_init(slot_free(s), 1);
    mbar_fence_init();
  }
  if (warp == NEW) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_dq = tmem_base;
  // every mode: dS goes back into tensor memory over the S columns it was computed from (bf16 pairs) and feeds the
  // dQ MMA as its TMEM A operand; the S MMA that next writes those columns is issued after that dQ MMA
  const uint32_t t_qa = tmem_base + 128 + 2 * C::SET_COLS;      // [384, 384 + D/2): Q, then dO (dual: dO')
  const uint32_t t_doa = t_qa + C::A_COLS;
  auto t_set = [&](int it) { return tmem_base + 128 + (it & 1) * C::SET_COLS; };  // S | dP
  const bool healthy = (*abort_flag == 0);

  if (warp == NEW + 1 && healthy) {
    // ---- TMA producer: this query block's Q / dO once, then the K / V tiles of every step through the ring
    if (elect_one()) {
      auto load_kv = [&](int it) {
        const int slot = by_slots.mod(it);
        const uint32_t base = slot_base(it);
        mbar_expect_tx(kv_full(slot), 2 * C::KV_BYTES);
        const int key0 = iter_key0(it);
        const bool halo = key0 < p.halo_len;
        const int krow = halo ? p.halo_row0 + key0 : key0 - p.halo_len;
        for (int d = 0; d < C::DB; ++d) {
          tma_load_3d(base + d * C::KV_REGION, halo ? &tma_kh : &tma_k, kv_full(slot), kvh * D + d * 64, krow, b);
          tma_load_3d(base + C::KV_BYTES + d * C::KV_REGION, halo ? &tma_vh : &tma_v, kv_full(slot), kvh * D + d * 64, krow, b);
        }
      };
      bool ok = true;
      mbar_expect_tx(q_full, C::DB * C::Q_REGION * (DUAL ? 3 : 2));
#pragma unroll
      for (int d = 0; d < C::DB; ++d) {
        tma_load_3d(sbase + C::Q_OFF + d * C::Q_REGION, &tma_q, q_full, h * D + d * 64, m0, b);
        tma_load_3d(sbase + C::DOT_OFF + d * C::Q_REGION, &tma_dot, q_full, h * D + d * 64, m0, b);
        if (DUAL) tma_load_3d(sbase + C::DOC_OFF + d * C::Q_REGION, &tma_doc, q_full, h * D + d * 64, m0, b);
      }
      for (int it = 0; it < n_iters && ok; ++it) {
        if (it >= C::NSLOTS) {              // the slot's previous tiles (step it - NSLOTS) have been consumed
          ok = mbar_wait_parked(slot_free(by_slots.mod(it)), (by_slots.div(it) - 1) & 1, abort_flag, 324);
          if (!ok) break;
        }
        load_kv(it);
      }
      // stay until every copy has been consumed (or the CTA gave up): no copy may be in flight at exit
      if (ok) ok = mbar_wait_parked(all_done, 0, abort_flag, 327);
      if (!ok) {
        mbar_drain(q_full, 0);
        for (int s = 0; s < C::NSLOTS; ++s) { mbar_drain(kv_full(s), 0); mbar_drain(kv_full(s), 1); }
      }
    }
  } else if (warp == NEW && healthy) {
    // ---- tensor-core issue
    if (elect_one()) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 64, false, false);
      constexpr uint32_t idesc_acc = umma_idesc_bf16(128, D, false, true);
      // descriptors as (low word + constant step, constant high word): one add per k-step on this thread
      constexpr uint32_t HI = umma_desc_hi_sw128(1024);
      const uint32_t dot_lo = umma_desc_lo(sbase + C::DOT_OFF, 16);
      auto issue_sdp = [&](int it) {
        const uint32_t sk = slot_base(it);
        const uint32_t k_lo = umma_desc_lo(sk, 16), v_lo = k_lo + (C::KV_BYTES >> 4);
        const uint32_t ts = t_set(it);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t ko = ((k / 4) * C::KV_REGION + (k % 4) * 32) >> 4;
          umma_ts(ts, t_qa + k * 8, umma_desc_join(k_lo + ko, HI), idesc_s, k != 0);
        }
        if (!DUAL || iter_inner(it)) {
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint32_t ko = ((k / 4) * C::KV_REGION + (k % 4) * 32) >> 4;
            umma_ts(ts + 64, t_doa + k * 8, umma_desc_join(v_lo + ko, HI), idesc_s, k != 0);
          }
        } else {
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint32_t qo = ((k / 4) * C::Q_REGION + (k % 4) * 32) >> 4;
            const uint32_t ko = ((k / 4) * C::KV_REGION + (k % 4) * 32) >> 4;
            umma_ss(ts + 64, umma_desc_join(dot_lo + qo, HI), umma_desc_join(v_lo + ko, HI), idesc_s, k != 0);
          }
        }
        umma_commit(sdp_full(it & 1));
      };
      bool ok = true;
      ok = mbar_wait(q_full, 0, abort_flag, 321) && mbar_wait(kv_full(0), 0, abort_flag, 322);
      if (ok) ok = mbar_wait(a_ready, 0, abort_flag, 326);      // Q and dO copied into tensor memory
      if (ok) { tc_fence_after_sync(); issue_sdp(0); }
      for (int it = 0; it < n_iters && ok; ++it) {
        if (it + 1 < n_iters) {
          ok = mbar_wait(kv_full(by_slots.mod(it + 1)), by_slots.div(it + 1) & 1, abort_flag, 323);
          if (!ok) break;
          tc_fence_after_sync();
          issue_sdp(it + 1);  // its TMEM set was last read by the dQ MMA of step it - 1, issued before
        }
        ok = mbar_wait(ew_done(it & 1), (it >> 1) & 1, abort_flag, 325);
        if (!ok) break;
        tc_fence_after_sync();
        // the K tile as the MN-major B operand: 64 keys of the contraction, the next 64 columns KV_REGION bytes on
        const uint32_t km_lo = umma_desc_lo(slot_base(it), C::KV_REGION);
        const uint32_t acc = it != 0;
#pragma unroll
        for (int k = 0; k < 4; ++k)  // dS as the TMEM A operand: 16 keys = 8 packed columns
          umma_ts(t_dq, t_set(it) + ts_packed_off(k), umma_desc_join(km_lo + k * (2048 >> 4), HI), idesc_acc, acc | (k != 0));
        umma_commit(slot_free(by_slots.mod(it)));   // the producer may refill this step's ring slot
      }
      if (ok) umma_commit(all_done);      // every dQ MMA has completed when this arrives
    }
  } else if (warp < NEW && healthy) {
    constexpr int NC = 16;                      // S columns (keys) per pass; a thread owns 32 of a step
    const int grp = warp >> 3;                  // takes steps grp, grp + 2, ...
    const int quarter = warp & 3, part = (warp >> 2) & 1;
    const int qrow = quarter * 32 + lane;
    const int row = m0 + qrow;
    const int qpos = row + off;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const bool row_ok = row < p.Tq;
    const int64_t sidx = (static_cast<int64_t>(b) * p.H + h) * p.Tq + row;
    const float nlse_t = row_ok ? -p.lse_t[sidx] * LOG2E : -INFINITY;
    const float del_t = row_ok ? p.delta_t[sidx] : 0.f;
    const float del_c = (DUAL && row_ok) ? p.delta_c[sidx] : 0.f;
    const int seg_lo = (packed && row_ok) ? p.seg_start[row] + off : 0;
    bool ok = true;
    auto wait_all = [&](uint32_t bar, uint32_t parity, int code) {
      const bool r = mbar_wait_parked(bar, parity, abort_flag, code);
      return __all_sync(0xffffffffu, r) != 0;
    };
    {
      // Q and dO rows: shared memory (128-byte swizzled, 64 columns per region) -> packed bf16 pairs in TMEM
      constexpr int DO_SRC = DUAL ? C::DOC_OFF : C::DOT_OFF;
      ok = wait_all(q_full, 0, 334);
      if (ok) {
        for (int u = part + 2 * grp; u < C::DB * 2; u += NEW / 4) {      // units of 32 columns (16 packed) of a row
          const int reg = u >> 1, hc = u & 1;
          uint32_t qa[16], da[16];
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const uint4 a = *reinterpret_cast<const uint4*>(smem + C::Q_OFF + reg * C::Q_REGION + sw128_offset(qrow, hc * 4 + c));
            const uint4 g = *reinterpret_cast<const uint4*>(smem + DO_SRC + reg * C::Q_REGION + sw128_offset(qrow, hc * 4 + c));
            qa[4 * c] = a.x; qa[4 * c + 1] = a.y; qa[4 * c + 2] = a.z; qa[4 * c + 3] = a.w;
            da[4 * c] = g.x; da[4 * c + 1] = g.y; da[4 * c + 2] = g.z; da[4 * c + 3] = g.w;
          }
          tmem_st16(t_qa + lane_addr + reg * 32 + hc * 16, qa);
          tmem_st16(t_doa + lane_addr + reg * 32 + hc * 16, da);
        }
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(a_ready);
      }
    }
    for (int it = grp; it < n_iters && ok; it += 2) {
      const int key0 = iter_key0(it) + part * 32;
      ok = wait_all(sdp_full(it & 1), (it >> 1) & 1, 331);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t ts = t_set(it) + lane_addr + part * 32;
      const int kb0 = iter_key0(it);
      // visible pairs of this step:  qpos - hi < key <= qpos - lo  (dual: teacher-only part or student part)
      const int inner = iter_inner(it);
      const int lo = combine ? (inner ? 0 : p.w_s) : 0, hi = combine ? (inner ? p.w_s : p.w_t) : p.w_t;
      const float del = (combine && inner) ? del_c : del_t;
      const bool full = (kb0 + 63 <= qlo - lo) && (kb0 > qhi - hi) && (kb0 >= seg_last);
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {          // two passes of 16 columns keep the registers low
        uint32_t sv[NC], dpt[NC];
        tmem_ld_n<NC>(ts + hh * NC, sv);
        tmem_ld_n<NC>(ts + 64 + hh * NC, dpt);
        tmem_ld_wait();
        uint32_t dsp[NC / 2];
        const int kpos0 = key0 + hh * NC;
        if (full)
          dq_elementwise<false, NC>(sv, dpt, p.scale_log2, nlse_t, del, qpos, kpos0, lo, hi, seg_lo, dsp);
        else
          dq_elementwise<true, NC>(sv, dpt, p.scale_log2, nlse_t, del, qpos, kpos0, lo, hi, seg_lo, dsp);
        tmem_st_n<NC / 2>(ts + hh * (NC / 2), dsp);    // over this thread's own S columns (already read)
      }
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(ew_done(it & 1));
    }
    if (ok) {
      ok = wait_all(all_done, 0, 333);
      if (ok && grp == 0) {               // two warps per quarter write dQ out, half the columns each
        const int half = part;
        tc_fence_after_sync();
        constexpr int COLS = D / 2;
        const int64_t rowoff = ((static_cast<int64_t>(b) * p.Tq + row) * p.H + h) * D;
#pragma unroll
        for (int c = 0; c < COLS; c += 32) {
          uint32_t a[32];
          tmem_ld32(t_dq + lane_addr + half * COLS + c, a);
          tmem_ld_wait();
          if (row_ok) store_out32(p.dq + rowoff + half * COLS + c, a, p.scale);  // dS was kept unscaled
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == NEW) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[b,h,t] = sum_d dO[b,t,h,d] * O[b,t,h,d]; D / 8 lanes per (b,t,h) row, 16-byte loads
__global__ void __launch_bounds__(256) attn_delta_kernel(const bf16* __restrict__ o, const bf16* __restrict__ d_o,
                                                         float* __restrict__ delta, int64_t B, int T, int H, int D) {
  const int lpr = D / 8;                                   // lanes per row: 16 (D = 128) or 8 (D = 64)
  const int rpw = 32 / lpr;                                // rows per warp
  const int lane = threadIdx.x & 31, sub = lane % lpr, grp = lane / lpr;
  const int64_t warp_id = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t item = warp_id * rpw + grp;
  const bool live = item < B * T * H;
  float acc = 0.f;
  if (live) {
    const uint4 a = *reinterpret_cast<const uint4*>(o + item * D + sub * 8);
    const uint4 g = *reinterpret_cast<const uint4*>(d_o + item * D + sub * 8);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = unpack_bf16(aw[i]), y = unpack_bf16(gw[i]);
      acc += x.x * y.x + x.y * y.y;
    }
  }
  for (int off = lpr / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (live && sub == 0) {
    const int h = static_cast<int>(item % H);
    const int64_t bt = item / H;
    delta[((bt / T) * H + h) * T + (bt % T)] = acc;
  }
}

// One pass over both outputs and their gradients for the combined dual backward: delta_t = rowsum(dO_T * O_T),
// r = exp(lse_T - lse_S), delta' = delta_t + r * rowsum(dO_S * O_S), dO' = dO_T + r * dO_S (bf16).
__global__ void __launch_bounds__(256) attn_combine_kernel(const bf16* __restrict__ o_t, const bf16* __restrict__ do_t,
                                                           const bf16* __restrict__ o_s, const bf16* __restrict__ do_s,
                                                           const float* __restrict__ lse_t, const float* __restrict__ lse_s,
                                                           float* __restrict__ delta_t, float* __restrict__ delta_p,
                                                           bf16* __restrict__ do_p, int64_t B, int T, int H, int D) {
  const int lpr = D / 8;
  const int rpw = 32 / lpr;
  const int lane = threadIdx.x & 31, sub = lane % lpr, grp = lane / lpr;
  const int64_t warp_id = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t item = warp_id * rpw + grp;
  const bool live = item < B * T * H;
  float acc_t = 0.f, acc_s = 0.f, r = 0.f;
  int64_t stat = 0;
  float gt[8], gs[8];
  if (live) {
    const int h = static_cast<int>(item % H);
    const int64_t bt = item / H;
    stat = ((bt / T) * H + h) * T + (bt % T);
    r = __expf(lse_t[stat] - lse_s[stat]);
    const int64_t off = item * D + sub * 8;
    const uint4 a = *reinterpret_cast<const uint4*>(o_t + off);
    const uint4 g = *reinterpret_cast<const uint4*>(do_t + off);
    const uint4 c = *reinterpret_cast<const uint4*>(o_s + off);
    const uint4 e = *reinterpret_cast<const uint4*>(do_s + off);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, gw[4] = {g.x, g.y, g.z, g.w};
    const uint32_t cw[4] = {c.x, c.y, c.z, c.w}, ew[4] = {e.x, e.y, e.z, e.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = unpack_bf16(aw[i]), y = unpack_bf16(gw[i]);
      const float2 u = unpack_bf16(cw[i]), w = unpack_bf16(ew[i]);
      acc_t += x.x * y.x + x.y * y.y;
      acc_s += u.x * w.x + u.y * w.y;
      gt[2 * i] = y.x; gt[2 * i + 1] = y.y;
      gs[2 * i] = w.x; gs[2 * i + 1] = w.y;
    }
    uint4 outv;
    outv.x = pack_bf16(fmaf(r, gs[0], gt[0]), fmaf(r, gs[1], gt[1]));
    outv.y = pack_bf16(fmaf(r, gs[2], gt[2]), fmaf(r, gs[3], gt[3]));
    outv.z = pack_bf16(fmaf(r, gs[4], gt[4]), fmaf(r, gs[5], gt[5]));
    outv.w = pack_bf16(fmaf(r, gs[6], gt[6]), fmaf(r, gs[7], gt[7]));
    *reinterpret_cast<uint4*>(do_p + off) = outv;
  }
  for (int off = lpr / 2; off > 0; off >>= 1) {
    acc_t += __shfl_xor_sync(0xffffffffu, acc_t, off);
    acc_s += __shfl_xor_sync(0xffffffffu, acc_s, off);
  }
  if (live && sub == 0) {
    delta_t[stat] = acc_t;
    delta_p[stat] = fmaf(r, acc_s, acc_t);
  }
}

struct BwdMaps {
  CUtensorMap q64, q128, k64, k128, v64, v128, dot64, dot128, doc64, doc128, kh64, kh128, vh64, vh128;
};

template <int D, bool DUAL>
static int launch_bwd(const BwdMaps& m, const AttnBwdParams& p, int B, cudaStream_t stream) {
  auto k1 = attn_bwd_dkdv_kernel<D>;
  auto k2 = attn_bwd_dq_kernel<D, DUAL>;
  constexpr int smem1 = DkdvCfg<D>::TOTAL, smem2 = DqCfg<D, DUAL>::TOTAL;
  static_assert(smem1 <= 232448 && smem2 <= 232448, "shared memory budget exceeded");
  static bool configured = false;
  if (!configured) {
    TTCD_CUDA_CHECK(cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, smem1));
    TTCD_CUDA_CHECK(cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2));
    configured = true;
  }
  dim3 g1((p.Tk + 127) / 128, p.HK, B);
  k1<<<g1, BWD_THREADS, smem1, stream>>>(m.q64, m.k128, m.v128, m.dot64, m.doc64, m.kh128, m.vh128, p);
  TTCD_CUDA_CHECK(cudaGetLastError());
  dim3 g2(p.H, (p.Tq + 127) / 128, B);
  k2<<<g2, BWD_THREADS, smem2, stream>>>(m.q128, m.k64, m.v64, m.dot128, m.doc128, m.kh64, m.vh64, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace ttcd

TTCD_DEFINE_STATUS_READER(attn_bwd)

// delta = rowsum(dO * O): o, d_o contiguous [B, T, H, D]; delta [B, H, T] fp32.
TTCD_EXPORT int ttcd_attn_delta(const void* o, const void* d_o, float* delta, long long B, int T, int H, int D,
                                void* stream_ptr) {
  using namespace ttcd;
  if ((D != 64 && D != 128) || B <= 0) return TTCD_ERR_ARG;
  const long long items = B * T * H;
  const long long rows_per_block = 8 * (32 / (D / 8));
  attn_delta_kernel<<<static_cast<unsigned>((items + rows_per_block - 1) / rows_per_block), 256, 0,
                      static_cast<cudaStream_t>(stream_ptr)>>>(
      static_cast<const bf16*>(o), static_cast<const bf16*>(d_o), delta, B, T, H, D);
  return static_cast<int>(cudaGetLastError());
}

// Inputs of the dual-window backward in one pass: o_*, do_* contiguous [B, T, H, D] bf16, lse_* [B, H, T] fp32;
// writes delta_t, delta_c ([B, H, T] fp32) and do_c ([B, T, H, D] bf16): dO' = dO_T + r dO_S,
// delta' = delta_T + r delta_S with r = exp(lse_T - lse_S).
TTCD_EXPORT int ttcd_attn_bwd_combine(const void* o_t, const void* do_t, const void* o_s, const void* do_s,
                                      const float* lse_t, const float* lse_s, float* delta_t, float* delta_c, void* do_c,
                                      long long B, int T, int H, int D, void* stream_ptr) {
  using namespace ttcd;
  if ((D != 64 && D != 128) || B <= 0) return TTCD_ERR_ARG;
  const long long items = B * T * H;
  const long long rows_per_block = 8 * (32 / (D / 8));
  attn_combine_kernel<<<static_cast<unsigned>((items + rows_per_block - 1) / rows_per_block), 256, 0,
                        static_cast<cudaStream_t>(stream_ptr)>>>(
      static_cast<const bf16*>(o_t), static_cast<const bf16*>(do_t), static_cast<const bf16*>(o_s),
      static_cast<const bf16*>(do_s), lse_t, lse_s, delta_t, delta_c, static_cast<bf16*>(do_c), B, T, H, D);
  return static_cast<int>(cudaGetLastError());
}

// Gradients of (dual-window) attention.
//   q/k/v strided as in ttcd_attn_fwd_cp; do_t contiguous [B, Tq, H, D]; lse_t, delta_t [B, H, Tq] fp32.
//   Dual window: do_c / delta_c are the combined stream made by ttcd_attn_bwd_combine (null => single window).
//   dq [B,Tq,H,D], dk [B, halo_len + Tk_local, HK, D] bf16 contiguous: the first halo_len rows are the gradients
//   of the previous rank's keys.  dv likewise, or, with ld_dv != 0, rows ld_dv elements apart and batches sb_dv
//   apart (the packed q|k|v gradient of a fused projection); both multiples of 8, dv 16-byte aligned.
//   seg_start / seg_end (int32 [Tq], or null): packed sequences in one row (needs B == 1, Tq == Tk, no halo);
//   for every token the first token of its sequence and one past its last.
//   flags: bit 0 = leave out the K/V copies of the dK/dV kernel (check of the bounded waits: the call returns with
//   a status code after the wait budget and its outputs are undefined).
TTCD_EXPORT int ttcd_attn_bwd_cp(const void* q, const void* k, const void* v, const void* k_halo, const void* v_halo,
                                 const void* do_t, const void* do_c, const float* lse_t, const float* delta_t,
                                 const float* delta_c, void* dq, void* dk, void* dv, int B, int Tq, int Tk_local, int H,
                                 int HK, int D, long long ldq, long long ldk, long long ldv, long long sq, long long sk,
                                 long long sv, long long ld_dv, long long sb_dv, int halo_len, int halo_rows,
                                 int window_t, int window_s, float scale, const int* seg_start, const int* seg_end,
                                 int flags, void* stream_ptr) {
  using namespace ttcd;
  if (B <= 0 || Tq < 128 || Tk_local < Tq || H <= 0 || HK <= 0 || H % HK != 0 || (D != 64 && D != 128)) return TTCD_ERR_ARG;
  if (halo_len < 0 || halo_len % 128 != 0 || (halo_len > 0 && (k_halo == nullptr || v_halo == nullptr || halo_rows < halo_len)))
    return TTCD_ERR_ARG;
  if (ld_dv < 0 || sb_dv < 0 || ld_dv % 8 != 0 || sb_dv % 8 != 0) return TTCD_ERR_ARG;
  if (ld_dv != 0 && (reinterpret_cast<uintptr_t>(dv) & 15u)) return TTCD_ERR_ARG;
  const bool dual = do_c != nullptr;
  if (dual && delta_c == nullptr) return TTCD_ERR_ARG;
  if ((seg_start == nullptr) != (seg_end == nullptr)) return TTCD_ERR_ARG;
  if (seg_start != nullptr && (B != 1 || Tq != Tk_local || halo_len != 0)) return TTCD_ERR_ARG;
  BwdMaps m;
  const uint64_t qi = static_cast<uint64_t>(H) * D, ki = static_cast<uint64_t>(HK) * D;
  int rc = TTCD_OK;
  auto mk = [&](CUtensorMap* map, const void* ptr, uint64_t inner, int rows, long long ld, long long sb, int box) {
    if (rc == TTCD_OK) rc = make_tmap_bf16_3d(map, ptr, inner, rows, B, ld, sb, 64, box);
  };
  mk(&m.q64, q, qi, Tq, ldq, sq, 64);         mk(&m.q128, q, qi, Tq, ldq, sq, 128);
  mk(&m.k64, k, ki, Tk_local, ldk, sk, 64);   mk(&m.k128, k, ki, Tk_local, ldk, sk, 128);
  mk(&m.v64, v, ki, Tk_local, ldv, sv, 64);   mk(&m.v128, v, ki, Tk_local, ldv, sv, 128);
  mk(&m.dot64, do_t, qi, Tq, qi, qi * Tq, 64);   mk(&m.dot128, do_t, qi, Tq, qi, qi * Tq, 128);
  const void* doc = dual ? do_c : do_t;
  mk(&m.doc64, doc, qi, Tq, qi, qi * Tq, 64);    mk(&m.doc128, doc, qi, Tq, qi, qi * Tq, 128);
  m.kh64 = m.k64; m.kh128 = m.k128; m.vh64 = m.v64; m.vh128 = m.v128;
  if (halo_len > 0) {
    mk(&m.kh64, k_halo, ki, halo_rows, ldk, sk, 64);   mk(&m.kh128, k_halo, ki, halo_rows, ldk, sk, 128);
    mk(&m.vh64, v_halo, ki, halo_rows, ldv, sv, 64);   mk(&m.vh128, v_halo, ki, halo_rows, ldv, sv, 128);
  }
  if (rc != TTCD_OK) return rc;
  const int big = 1 << 30;
  AttnBwdParams p;
  p.lse_t = lse_t; p.delta_t = delta_t; p.delta_c = dual ? delta_c : delta_t;
  p.dq = static_cast<bf16*>(dq); p.dk = static_cast<bf16*>(dk); p.dv = static_cast<bf16*>(dv);
  p.Tq = Tq; p.Tk = Tk_local + halo_len; p.H = H; p.HK = HK;
  p.w_t = window_t > 0 ? window_t : big;
  p.w_s = (dual && window_s > 0) ? window_s : p.w_t;
  p.scale = scale; p.scale_log2 = scale * LOG2E;
  p.halo_len = halo_len; p.halo_row0 = halo_rows - halo_len;
  p.ld_dv = ld_dv; p.sb_dv = sb_dv;
  p.combine = dual ? 1 : 0;
  p.seg_start = seg_start; p.seg_end = seg_end;
  p.skip_kv_load = flags & 1;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  if (D == 128) return dual ? launch_bwd<128, true>(m, p, B, stream) : launch_bwd<128, false>(m, p, B, stream);
  return dual ? launch_bwd<64, true>(m, p, B, stream) : launch_bwd<64, false>(m, p, B, stream);
}

TTCD_EXPORT int ttcd_attn_bwd(const void* q, const void* k, const void* v, const void* do_t, const void* do_c,
                              const float* lse_t, const float* delta_t, const float* delta_c, void* dq, void* dk,
                              void* dv, int B, int Tq, int Tk, int H, int HK, int D, long long ldq, long long ldk,
                              long long ldv, long long sq, long long sk, long long sv, long long ld_dv, long long sb_dv,
                              int window_t, int window_s, float scale, const int* seg_start, const int* seg_end, int flags,
                              void* stream_ptr) {
  return ttcd_attn_bwd_cp(q, k, v, nullptr, nullptr, do_t, do_c, lse_t, delta_t, delta_c, dq, dk, dv, B, Tq, Tk, H, HK, D,
                          ldq, ldk, ldv, sq, sk, sv, ld_dv, sb_dv, 0, 0, window_t, window_s, scale, seg_start, seg_end,
                          flags, stream_ptr);
}
