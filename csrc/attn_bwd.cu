// Sliding-window attention backward for sm_100a (single- and dual-window), two kernels, no atomics:
//
//   attn_bwd_dkdv : one CTA per (128-key block, kv head, batch); loops over the query blocks (64 rows)
//                   and the query heads of the GQA group that can see those keys.  Per step it forms
//                   S^T = K Q^T and dP^T = V dO^T on tcgen05 (keys on the TMEM lanes), eight warps turn
//                   them into P^T and dS^T in shared memory, and dV += P^T dO, dK += dS^T Q accumulate
//                   in TMEM.  In dual-window mode the student and teacher gradients are summed here:
//                   dS = P_T (dP_T - delta_T) + P_S (dP_S - delta_S),  dV += P_T^T dO_T + P_S^T dO_S.
//   attn_bwd_dq   : one CTA per (128-query block, head, batch); loops over the key blocks (64 keys) of
//                   the teacher window, recomputes S / dP and accumulates dQ += dS K in TMEM.
//
// Both stream operand tiles with TMA (128-byte swizzle, no multicast) through 2-slot rings and reuse
// one swizzled tile as a K-major operand of one MMA and an MN-major operand of another (Q and dO in
// dkdv, K in dq), so nothing is transposed in memory.  The reference has no fused dual-window
// backward at all: training there runs two flash-attn backward passes whose dq/dk/dv are summed by
// autograd (custom_models/ipttcd/modeling_ipttcdv9.py:686-690; profiling/FUSED_ATTENTION_DESIGN.md:68-69).
#include "common.cuh"

namespace ttcd {

constexpr int BWD_THREADS = 288;  // 8 compute warps + 1 control warp
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void named_barrier_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

struct AttnBwdParams {
  const float* lse_t; const float* lse_s;      // [B, H, Tq] natural log
  const float* delta_t; const float* delta_s;  // [B, H, Tq] rowsum(dO * O)
  bf16* dq; bf16* dk; bf16* dv;                 // [B,Tq,H,D], [B,Tk,HK,D], [B,Tk,HK,D]
  int Tq, Tk, H, HK;
  int w_t, w_s;
  float scale, scale_log2;
};

// 32 accumulator columns of one TMEM lane -> 32 bf16 (one 64-byte half row) of a K-major SW128 tile
__device__ __forceinline__ void store_half_row(uint8_t* tile, int row, int half, const float (&v)[32]) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint4 pk;
    pk.x = pack_bf16(v[c * 8 + 0], v[c * 8 + 1]);
    pk.y = pack_bf16(v[c * 8 + 2], v[c * 8 + 3]);
    pk.z = pack_bf16(v[c * 8 + 4], v[c * 8 + 5]);
    pk.w = pack_bf16(v[c * 8 + 6], v[c * 8 + 7]);
    *reinterpret_cast<uint4*>(tile + sw128_offset(row, half * 4 + c)) = pk;
  }
}

// =================================================================================================
// dK / dV
// =================================================================================================
template <int D>
struct DkdvSmem {
  static constexpr int DB = D / 64;
  static constexpr int KEY_REGION = 128 * 128;  // [128 keys x 64 d] swizzled
  static constexpr int ROW_REGION = 64 * 128;   // [64 rows x 64 d] swizzled
  static constexpr int K_OFF = 0;
  static constexpr int V_OFF = K_OFF + DB * KEY_REGION;
  static constexpr int Q_OFF = V_OFF + DB * KEY_REGION;          // 2 slots
  static constexpr int DOT_OFF = Q_OFF + 2 * DB * ROW_REGION;    // 2 slots
  static constexpr int DOS_OFF = DOT_OFF + 2 * DB * ROW_REGION;  // 2 slots
  static constexpr int PT_OFF = DOS_OFF + 2 * DB * ROW_REGION;   // [128 x 64] bf16
  static constexpr int PS_OFF = PT_OFF + KEY_REGION;
  static constexpr int DS_OFF = PS_OFF + KEY_REGION;
  static constexpr int VEC_OFF = DS_OFF + KEY_REGION;            // 2 slots x 4 vectors x 64 floats
  static constexpr int BAR_OFF = VEC_OFF + 2 * 4 * 64 * 4;
  static constexpr int NBARS = 6;  // kv_full, tiles_full[2], sdp_full, ew_done, acc_done
  static constexpr int TOTAL = BAR_OFF + NBARS * 8 + 16;
  static constexpr int TILE_BYTES = DB * ROW_REGION;
};

template <int D, bool DUAL>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                     const __grid_constant__ CUtensorMap tma_v, const __grid_constant__ CUtensorMap tma_dot,
                     const __grid_constant__ CUtensorMap tma_dos, const AttnBwdParams p) {
  using S = DkdvSmem<D>;
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bars = sbase + S::BAR_OFF;
  const uint32_t kv_full = bars;
  auto tiles_full = [&](int s) { return bars + 8u * (1 + s); };
  const uint32_t sdp_full = bars + 8u * 3;
  const uint32_t ew_done = bars + 8u * 4;
  const uint32_t acc_done = bars + 8u * 5;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + S::BAR_OFF + S::NBARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* vecs = reinterpret_cast<float*>(smem + S::VEC_OFF);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * 128;
  const int kvh = blockIdx.y;
  const int b = blockIdx.z;
  const int G = p.H / p.HK;
  const int off = p.Tk - p.Tq;

  // query rows that can see keys [n0, n0+127] through the teacher window
  const int row_lo = max(0, n0 - off);
  const int row_hi = min(p.Tq - 1, n0 + 127 + p.w_t - 1 - off);
  const int jb_lo = row_lo / 64;
  const int nqb = row_hi >= row_lo ? (row_hi / 64 - jb_lo + 1) : 0;
  const int n_iters = nqb * G;

  if (threadIdx.x == 0) {
    *abort_flag = ((sbase & 1023u) != 0) ? 1 : 0;
    if (*abort_flag) atomicCAS(&g_status, 0, 399);
    mbar_init(kv_full, 1);
    mbar_init(tiles_full(0), 1);
    mbar_init(tiles_full(1), 1);
    mbar_init(sdp_full, 1);
    mbar_init(ew_done, 8);
    mbar_init(acc_done, 1);
    mbar_fence_init();
  }
  if (warp == 8) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_dk = tmem_base, t_dv = tmem_base + 128, t_s = tmem_base + 256, t_dpt = tmem_base + 320,
                 t_dps = tmem_base + 384;
  const bool healthy = (*abort_flag == 0);

  auto iter_head = [&](int it) { return kvh * G + it / nqb; };
  auto iter_row0 = [&](int it) { return (jb_lo + it % nqb) * 64; };
  auto iter_student = [&](int it) {
    const int qlo_b = iter_row0(it) + off;
    return DUAL && (qlo_b < n0 + 127 + p.w_s);
  };

  if (warp == 8 && healthy && n_iters > 0) {
    if (elect_one()) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 64, false, false);  // [keys x q] = A(K-major) B(K-major)
      constexpr uint32_t idesc_acc = umma_idesc_bf16(128, D, false, true);   // [keys x D] = A(K-major) B(MN-major)
      auto load_tiles = [&](int it) {
        const int slot = it & 1;
        const int h = iter_head(it), r0 = iter_row0(it);
        const bool st = iter_student(it);
        mbar_expect_tx(tiles_full(slot), S::TILE_BYTES * (st ? 3 : 2));
#pragma unroll
        for (int d = 0; d < S::DB; ++d) {
          tma_load_3d(sbase + S::Q_OFF + slot * S::TILE_BYTES + d * S::ROW_REGION, &tma_q, tiles_full(slot),
                      h * D + d * 64, r0, b);
          tma_load_3d(sbase + S::DOT_OFF + slot * S::TILE_BYTES + d * S::ROW_REGION, &tma_dot, tiles_full(slot),
                      h * D + d * 64, r0, b);
          if (st)
            tma_load_3d(sbase + S::DOS_OFF + slot * S::TILE_BYTES + d * S::ROW_REGION, &tma_dos, tiles_full(slot),
                        h * D + d * 64, r0, b);
        }
      };
      bool ok = true;
      mbar_expect_tx(kv_full, 2 * S::DB * S::KEY_REGION);
#pragma unroll
      for (int d = 0; d < S::DB; ++d) {
        tma_load_3d(sbase + S::K_OFF + d * S::KEY_REGION, &tma_k, kv_full, kvh * D + d * 64, n0, b);
        tma_load_3d(sbase + S::V_OFF + d * S::KEY_REGION, &tma_v, kv_full, kvh * D + d * 64, n0, b);
      }
      load_tiles(0);
      ok = mbar_wait(kv_full, 0, abort_flag, 301);
      for (int it = 0; it < n_iters && ok; ++it) {
        const int slot = it & 1;
        const bool st = iter_student(it);
        ok = mbar_wait(tiles_full(slot), (it >> 1) & 1, abort_flag, 302);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t sq = sbase + S::Q_OFF + slot * S::TILE_BYTES;
        const uint32_t sdot = sbase + S::DOT_OFF + slot * S::TILE_BYTES;
        const uint32_t sdos = sbase + S::DOS_OFF + slot * S::TILE_BYTES;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t ko = (k / 4) * S::KEY_REGION + (k % 4) * 32;
          const uint32_t ro = (k / 4) * S::ROW_REGION + (k % 4) * 32;
          umma_ss(t_s, umma_desc_sw128(sbase + S::K_OFF + ko, 16, 1024), umma_desc_sw128(sq + ro, 16, 1024), idesc_s,
                  k != 0);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t ko = (k / 4) * S::KEY_REGION + (k % 4) * 32;
          const uint32_t ro = (k / 4) * S::ROW_REGION + (k % 4) * 32;
          umma_ss(t_dpt, umma_desc_sw128(sbase + S::V_OFF + ko, 16, 1024), umma_desc_sw128(sdot + ro, 16, 1024),
                  idesc_s, k != 0);
        }
        if (st) {
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint32_t ko = (k / 4) * S::KEY_REGION + (k % 4) * 32;
            const uint32_t ro = (k / 4) * S::ROW_REGION + (k % 4) * 32;
            umma_ss(t_dps, umma_desc_sw128(sbase + S::V_OFF + ko, 16, 1024), umma_desc_sw128(sdos + ro, 16, 1024),
                    idesc_s, k != 0);
          }
        }
        umma_commit(sdp_full);
        if (it + 1 < n_iters) {
          // slot (it+1)&1 was last read by the accumulate MMAs of iteration it-1
          if (it >= 1) ok = mbar_wait(acc_done, (it - 1) & 1, abort_flag, 303);
          if (!ok) break;
          load_tiles(it + 1);
        }
        ok = mbar_wait(ew_done, it & 1, abort_flag, 304);
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < 4; ++k) {  // contraction over the 64 query rows
          umma_ss(t_dv, umma_desc_sw128(sbase + S::PT_OFF + k * 32, 16, 1024),
                  umma_desc_sw128(sdot + k * 2048, S::ROW_REGION, 1024), idesc_acc, (it | k) != 0);
        }
        if (st) {
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_ss(t_dv, umma_desc_sw128(sbase + S::PS_OFF + k * 32, 16, 1024),
                    umma_desc_sw128(sdos + k * 2048, S::ROW_REGION, 1024), idesc_acc, 1u);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          umma_ss(t_dk, umma_desc_sw128(sbase + S::DS_OFF + k * 32, 16, 1024),
                  umma_desc_sw128(sq + k * 2048, S::ROW_REGION, 1024), idesc_acc, (it | k) != 0);
        }
        umma_commit(acc_done);
      }
      if (!ok) {
        mbar_drain(kv_full, 0);
        for (int s = 0; s < 2; ++s) { mbar_drain(tiles_full(s), 0); mbar_drain(tiles_full(s), 1); }
      }
    }
  } else if (warp < 8 && healthy) {
    const int quarter = warp & 3, half = warp >> 2;
    const int krow = quarter * 32 + lane;       // key row inside the block == TMEM lane
    const int key = n0 + krow;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const int ctid = threadIdx.x;               // 0..255
    bool ok = true;
    auto wait_all = [&](uint32_t bar, uint32_t parity, int code) {
      const bool r = mbar_wait(bar, parity, abort_flag, code);
      return __all_sync(0xffffffffu, r) != 0;
    };
    for (int it = 0; it < n_iters && ok; ++it) {
      const int h = iter_head(it), r0 = iter_row0(it);
      const bool st = iter_student(it);
      float* vslot = vecs + (it & 1) * 256;
      {
        // per-row statistics of this query block: [lse_t*log2e | delta_t | lse_s*log2e | delta_s]
        const int which = ctid >> 6, r = ctid & 63;
        const int row = r0 + r;
        const int64_t idx = (static_cast<int64_t>(b) * p.H + h) * p.Tq + row;
        float val = 0.f;
        if (row < p.Tq) {
          if (which == 0) val = p.lse_t[idx] * LOG2E;
          else if (which == 1) val = p.delta_t[idx];
          else if (DUAL && st && which == 2) val = p.lse_s[idx] * LOG2E;
          else if (DUAL && st && which == 3) val = p.delta_s[idx];
        } else if (which == 0 || which == 2) {
          val = INFINITY;  // rows past the end contribute p = 0
        }
        vslot[which * 64 + r] = val;
      }
      named_barrier_sync(1, 256);
      ok = wait_all(sdp_full, it & 1, 311);
      if (!ok) break;
      tc_fence_after_sync();
      uint32_t sv[32], dpt[32], dps[32];
      tmem_ld32(t_s + lane_addr + half * 32, sv);
      tmem_ld32(t_dpt + lane_addr + half * 32, dpt);
      if (st) tmem_ld32(t_dps + lane_addr + half * 32, dps);
      tmem_ld_wait();
      if (it >= 1) {
        ok = wait_all(acc_done, (it - 1) & 1, 312);  // P / dS tiles free again
        if (!ok) break;
      }
      float pt[32], ps[32], ds[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const int col = half * 32 + c;
        const int qpos = r0 + col + off;
        const float s2 = __uint_as_float(sv[c]) * p.scale_log2;
        const bool vis_t = key <= qpos && key > qpos - p.w_t && key < p.Tk;
        const float p_t = vis_t ? ex2(s2 - vslot[col]) : 0.f;
        float d = p_t * (__uint_as_float(dpt[c]) - vslot[64 + col]);
        pt[c] = p_t;
        if (DUAL && st) {
          const bool vis_s = key <= qpos && key > qpos - p.w_s && key < p.Tk;
          const float p_s = vis_s ? ex2(s2 - vslot[128 + col]) : 0.f;
          d += p_s * (__uint_as_float(dps[c]) - vslot[192 + col]);
          ps[c] = p_s;
        }
        ds[c] = d * p.scale;
      }
      store_half_row(smem + S::PT_OFF, krow, half, pt);
      if (DUAL && st) store_half_row(smem + S::PS_OFF, krow, half, ps);
      store_half_row(smem + S::DS_OFF, krow, half, ds);
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(ew_done);
    }
    // epilogue: dK, dV -> global (this thread: key row `krow`, column half of D)
    if (ok) {
      if (n_iters > 0) ok = wait_all(acc_done, (n_iters - 1) & 1, 313);
      if (ok) {
        tc_fence_after_sync();
        const bool store = key < p.Tk;
        const int64_t rowoff = ((static_cast<int64_t>(b) * p.Tk + key) * p.HK + kvh) * D;
        constexpr int COLS = D / 2;  // per thread
#pragma unroll
        for (int c = 0; c < COLS; c += 32) {
          uint32_t a[32], v[32];
          if (n_iters > 0) {
            tmem_ld32(t_dk + lane_addr + half * COLS + c, a);
            tmem_ld32(t_dv + lane_addr + half * COLS + c, v);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) a[j] = v[j] = 0u;
          }
          if (store) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 o;
              o.x = pack_bf16(__uint_as_float(a[j]), __uint_as_float(a[j + 1]));
              o.y = pack_bf16(__uint_as_float(a[j + 2]), __uint_as_float(a[j + 3]));
              o.z = pack_bf16(__uint_as_float(a[j + 4]), __uint_as_float(a[j + 5]));
              o.w = pack_bf16(__uint_as_float(a[j + 6]), __uint_as_float(a[j + 7]));
              *reinterpret_cast<uint4*>(p.dk + rowoff + half * COLS + c + j) = o;
              o.x = pack_bf16(__uint_as_float(v[j]), __uint_as_float(v[j + 1]));
              o.y = pack_bf16(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
              o.z = pack_bf16(__uint_as_float(v[j + 4]), __uint_as_float(v[j + 5]));
              o.w = pack_bf16(__uint_as_float(v[j + 6]), __uint_as_float(v[j + 7]));
              *reinterpret_cast<uint4*>(p.dv + rowoff + half * COLS + c + j) = o;
            }
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// =================================================================================================
// dQ
// =================================================================================================
template <int D>
struct DqSmem {
  static constexpr int DB = D / 64;
  static constexpr int Q_REGION = 128 * 128;
  static constexpr int KV_REGION = 64 * 128;
  static constexpr int Q_OFF = 0;
  static constexpr int DOT_OFF = Q_OFF + DB * Q_REGION;
  static constexpr int DOS_OFF = DOT_OFF + DB * Q_REGION;
  static constexpr int K_OFF = DOS_OFF + DB * Q_REGION;      // 2 slots
  static constexpr int V_OFF = K_OFF + 2 * DB * KV_REGION;   // 2 slots
  static constexpr int DS_OFF = V_OFF + 2 * DB * KV_REGION;  // [128 x 64] bf16
  static constexpr int BAR_OFF = DS_OFF + Q_REGION;
  static constexpr int NBARS = 6;  // q_full, kv_full[2], sdp_full, ew_done, acc_done
  static constexpr int TOTAL = BAR_OFF + NBARS * 8 + 16;
  static constexpr int KV_BYTES = DB * KV_REGION;
};

template <int D, bool DUAL>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                   const __grid_constant__ CUtensorMap tma_v, const __grid_constant__ CUtensorMap tma_dot,
                   const __grid_constant__ CUtensorMap tma_dos, const AttnBwdParams p) {
  using S = DqSmem<D>;
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bars = sbase + S::BAR_OFF;
  const uint32_t q_full = bars;
  auto kv_full = [&](int s) { return bars + 8u * (1 + s); };
  const uint32_t sdp_full = bars + 8u * 3;
  const uint32_t ew_done = bars + 8u * 4;
  const uint32_t acc_done = bars + 8u * 5;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + S::BAR_OFF + S::NBARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x;
  const int m0 = blockIdx.y * 128;
  const int b = blockIdx.z;
  const int kvh = h / (p.H / p.HK);
  const int off = p.Tk - p.Tq;
  const int qlo = m0 + off, qhi = m0 + 127 + off;
  const int key_hi = min(qhi, p.Tk - 1);
  const int key_lo = max(0, qlo - p.w_t + 1);
  const int blk_lo = key_lo / 64;
  const int n_iters = key_hi / 64 - blk_lo + 1;
  auto iter_key0 = [&](int it) { return (blk_lo + it) * 64; };
  auto iter_student = [&](int it) { return DUAL && (iter_key0(it) + 63 > qlo - p.w_s); };

  if (threadIdx.x == 0) {
    *abort_flag = ((sbase & 1023u) != 0) ? 1 : 0;
    if (*abort_flag) atomicCAS(&g_status, 0, 398);
    mbar_init(q_full, 1);
    mbar_init(kv_full(0), 1);
    mbar_init(kv_full(1), 1);
    mbar_init(sdp_full, 1);
    mbar_init(ew_done, 8);
    mbar_init(acc_done, 1);
    mbar_fence_init();
  }
  if (warp == 8) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_dq = tmem_base, t_s = tmem_base + 128, t_dpt = tmem_base + 192, t_dps = tmem_base + 256;
  const bool healthy = (*abort_flag == 0);

  if (warp == 8 && healthy) {
    if (elect_one()) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 64, false, false);
      constexpr uint32_t idesc_acc = umma_idesc_bf16(128, D, false, true);
      auto load_kv = [&](int it) {
        const int slot = it & 1;
        mbar_expect_tx(kv_full(slot), 2 * S::KV_BYTES);
#pragma unroll
        for (int d = 0; d < S::DB; ++d) {
          tma_load_3d(sbase + S::K_OFF + slot * S::KV_BYTES + d * S::KV_REGION, &tma_k, kv_full(slot),
                      kvh * D + d * 64, iter_key0(it), b);
          tma_load_3d(sbase + S::V_OFF + slot * S::KV_BYTES + d * S::KV_REGION, &tma_v, kv_full(slot),
                      kvh * D + d * 64, iter_key0(it), b);
        }
      };
      bool ok = true;
      mbar_expect_tx(q_full, S::DB * S::Q_REGION * (DUAL ? 3 : 2));
#pragma unroll
      for (int d = 0; d < S::DB; ++d) {
        tma_load_3d(sbase + S::Q_OFF + d * S::Q_REGION, &tma_q, q_full, h * D + d * 64, m0, b);
        tma_load_3d(sbase + S::DOT_OFF + d * S::Q_REGION, &tma_dot, q_full, h * D + d * 64, m0, b);
        if (DUAL) tma_load_3d(sbase + S::DOS_OFF + d * S::Q_REGION, &tma_dos, q_full, h * D + d * 64, m0, b);
      }
      load_kv(0);
      ok = mbar_wait(q_full, 0, abort_flag, 321);
      for (int it = 0; it < n_iters && ok; ++it) {
        const int slot = it & 1;
        const bool st = iter_student(it);
        ok = mbar_wait(kv_full(slot), (it >> 1) & 1, abort_flag, 322);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t sk = sbase + S::K_OFF + slot * S::KV_BYTES;
        const uint32_t sv = sbase + S::V_OFF + slot * S::KV_BYTES;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t qo = (k / 4) * S::Q_REGION + (k % 4) * 32;
          const uint32_t ko = (k / 4) * S::KV_REGION + (k % 4) * 32;
          umma_ss(t_s, umma_desc_sw128(sbase + S::Q_OFF + qo, 16, 1024), umma_desc_sw128(sk + ko, 16, 1024), idesc_s,
                  k != 0);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t qo = (k / 4) * S::Q_REGION + (k % 4) * 32;
          const uint32_t ko = (k / 4) * S::KV_REGION + (k % 4) * 32;
          umma_ss(t_dpt, umma_desc_sw128(sbase + S::DOT_OFF + qo, 16, 1024), umma_desc_sw128(sv + ko, 16, 1024),
                  idesc_s, k != 0);
        }
        if (st) {
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint32_t qo = (k / 4) * S::Q_REGION + (k % 4) * 32;
            const uint32_t ko = (k / 4) * S::KV_REGION + (k % 4) * 32;
            umma_ss(t_dps, umma_desc_sw128(sbase + S::DOS_OFF + qo, 16, 1024), umma_desc_sw128(sv + ko, 16, 1024),
                    idesc_s, k != 0);
          }
        }
        umma_commit(sdp_full);
        if (it + 1 < n_iters) {
          if (it >= 1) ok = mbar_wait(acc_done, (it - 1) & 1, abort_flag, 323);
          if (!ok) break;
          load_kv(it + 1);
        }
        ok = mbar_wait(ew_done, it & 1, abort_flag, 324);
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < 4; ++k)  // contraction over the 64 keys of the block
          umma_ss(t_dq, umma_desc_sw128(sbase + S::DS_OFF + k * 32, 16, 1024),
                  umma_desc_sw128(sk + k * 2048, S::KV_REGION, 1024), idesc_acc, (it | k) != 0);
        umma_commit(acc_done);
      }
      if (!ok) {
        mbar_drain(q_full, 0);
        for (int s = 0; s < 2; ++s) { mbar_drain(kv_full(s), 0); mbar_drain(kv_full(s), 1); }
      }
    }
  } else if (warp < 8 && healthy) {
    const int quarter = warp & 3, half = warp >> 2;
    const int qrow = quarter * 32 + lane;
    const int row = m0 + qrow;
    const int qpos = row + off;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const bool row_ok = row < p.Tq;
    const int64_t sidx = (static_cast<int64_t>(b) * p.H + h) * p.Tq + row;
    const float lse_t2 = row_ok ? p.lse_t[sidx] * LOG2E : INFINITY;
    const float del_t = row_ok ? p.delta_t[sidx] : 0.f;
    const float lse_s2 = (DUAL && row_ok) ? p.lse_s[sidx] * LOG2E : INFINITY;
    const float del_s = (DUAL && row_ok) ? p.delta_s[sidx] : 0.f;
    bool ok = true;
    auto wait_all = [&](uint32_t bar, uint32_t parity, int code) {
      const bool r = mbar_wait(bar, parity, abort_flag, code);
      return __all_sync(0xffffffffu, r) != 0;
    };
    for (int it = 0; it < n_iters && ok; ++it) {
      const bool st = iter_student(it);
      const int key0 = iter_key0(it) + half * 32;
      ok = wait_all(sdp_full, it & 1, 331);
      if (!ok) break;
      tc_fence_after_sync();
      uint32_t sv[32], dpt[32], dps[32];
      tmem_ld32(t_s + lane_addr + half * 32, sv);
      tmem_ld32(t_dpt + lane_addr + half * 32, dpt);
      if (st) tmem_ld32(t_dps + lane_addr + half * 32, dps);
      tmem_ld_wait();
      if (it >= 1) {
        ok = wait_all(acc_done, (it - 1) & 1, 332);
        if (!ok) break;
      }
      float ds[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const int key = key0 + c;
        const float s2 = __uint_as_float(sv[c]) * p.scale_log2;
        const bool vis_t = key <= qpos && key > qpos - p.w_t;
        float d = vis_t ? ex2(s2 - lse_t2) * (__uint_as_float(dpt[c]) - del_t) : 0.f;
        if (DUAL && st) {
          const bool vis_s = key <= qpos && key > qpos - p.w_s;
          d += vis_s ? ex2(s2 - lse_s2) * (__uint_as_float(dps[c]) - del_s) : 0.f;
        }
        ds[c] = d * p.scale;
      }
      store_half_row(smem + S::DS_OFF, qrow, half, ds);
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(ew_done);
    }
    if (ok) {
      ok = wait_all(acc_done, (n_iters - 1) & 1, 333);
      if (ok) {
        tc_fence_after_sync();
        constexpr int COLS = D / 2;
        const int64_t rowoff = ((static_cast<int64_t>(b) * p.Tq + row) * p.H + h) * D;
#pragma unroll
        for (int c = 0; c < COLS; c += 32) {
          uint32_t a[32];
          tmem_ld32(t_dq + lane_addr + half * COLS + c, a);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 o;
              o.x = pack_bf16(__uint_as_float(a[j]), __uint_as_float(a[j + 1]));
              o.y = pack_bf16(__uint_as_float(a[j + 2]), __uint_as_float(a[j + 3]));
              o.z = pack_bf16(__uint_as_float(a[j + 4]), __uint_as_float(a[j + 5]));
              o.w = pack_bf16(__uint_as_float(a[j + 6]), __uint_as_float(a[j + 7]));
              *reinterpret_cast<uint4*>(p.dq + rowoff + half * COLS + c + j) = o;
            }
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[b,h,t] = sum_d dO[b,t,h,d] * O[b,t,h,d]; one warp per (b,t,h)
__global__ void __launch_bounds__(256) attn_delta_kernel(const bf16* __restrict__ o, const bf16* __restrict__ d_o,
                                                         float* __restrict__ delta, int64_t B, int T, int H, int D) {
  const int lane = threadIdx.x & 31;
  const int64_t item = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= B * T * H) return;
  const int h = static_cast<int>(item % H);
  const int64_t bt = item / H;
  float acc = 0.f;
  for (int d = lane * 2; d < D; d += 64) {
    const float2 a = unpack_bf16(*reinterpret_cast<const uint32_t*>(o + item * D + d));
    const float2 g = unpack_bf16(*reinterpret_cast<const uint32_t*>(d_o + item * D + d));
    acc += a.x * g.x + a.y * g.y;
  }
  acc = warp_sum(acc);
  if (lane == 0) delta[((bt / T) * H + h) * T + (bt % T)] = acc;
}

template <int D, bool DUAL>
static int launch_bwd(const CUtensorMap& tq64, const CUtensorMap& tq128, const CUtensorMap& tk64,
                      const CUtensorMap& tk128, const CUtensorMap& tv64, const CUtensorMap& tv128,
                      const CUtensorMap& tdot64, const CUtensorMap& tdot128, const CUtensorMap& tdos64,
                      const CUtensorMap& tdos128, const AttnBwdParams& p, int B, cudaStream_t stream) {
  auto k1 = attn_bwd_dkdv_kernel<D, DUAL>;
  auto k2 = attn_bwd_dq_kernel<D, DUAL>;
  static bool configured = false;
  if (!configured) {
    TTCD_CUDA_CHECK(cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, DkdvSmem<D>::TOTAL));
    TTCD_CUDA_CHECK(cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, DqSmem<D>::TOTAL));
    configured = true;
  }
  dim3 g1((p.Tk + 127) / 128, p.HK, B);
  k1<<<g1, BWD_THREADS, DkdvSmem<D>::TOTAL, stream>>>(tq64, tk128, tv128, tdot64, tdos64, p);
  TTCD_CUDA_CHECK(cudaGetLastError());
  dim3 g2(p.H, (p.Tq + 127) / 128, B);
  k2<<<g2, BWD_THREADS, DqSmem<D>::TOTAL, stream>>>(tq128, tk64, tv64, tdot128, tdos128, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace ttcd

// delta = rowsum(dO * O): o, d_o contiguous [B, T, H, D]; delta [B, H, T] fp32.
TTCD_EXPORT int ttcd_attn_delta(const void* o, const void* d_o, float* delta, long long B, int T, int H, int D,
                                void* stream_ptr) {
  using namespace ttcd;
  if (D % 2 != 0 || B <= 0) return TTCD_ERR_ARG;
  const long long items = B * T * H;
  attn_delta_kernel<<<static_cast<unsigned>((items + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      static_cast<const bf16*>(o), static_cast<const bf16*>(d_o), delta, B, T, H, D);
  return static_cast<int>(cudaGetLastError());
}

// Gradients of (dual-window) attention.  q/k/v strided as in ttcd_attn_fwd; do_t/do_s contiguous
// [B, Tq, H, D] (do_s null => single window); dq [B,Tq,H,D], dk/dv [B,Tk,HK,D] bf16 contiguous.
TTCD_EXPORT int ttcd_attn_bwd(const void* q, const void* k, const void* v, const void* do_t, const void* do_s,
                              const float* lse_t, const float* lse_s, const float* delta_t, const float* delta_s,
                              void* dq, void* dk, void* dv, int B, int Tq, int Tk, int H, int HK, int D,
                              long long ldq, long long ldk, long long ldv, long long sq, long long sk, long long sv,
                              int window_t, int window_s, float scale, void* stream_ptr) {
  using namespace ttcd;
  if (B <= 0 || Tq <= 0 || Tk < Tq || H <= 0 || HK <= 0 || H % HK != 0 || (D != 64 && D != 128)) return TTCD_ERR_ARG;
  const bool dual = do_s != nullptr;
  CUtensorMap tq64, tq128, tk64, tk128, tv64, tv128, tdot64, tdot128, tdos64, tdos128;
  const uint64_t qi = static_cast<uint64_t>(H) * D, ki = static_cast<uint64_t>(HK) * D;
  int rc = TTCD_OK;
  auto mk = [&](CUtensorMap* m, const void* ptr, uint64_t inner, int rows, long long ld, long long sb, int box) {
    if (rc == TTCD_OK) rc = make_tmap_bf16_3d(m, ptr, inner, rows, B, ld, sb, 64, box);
  };
  mk(&tq64, q, qi, Tq, ldq, sq, 64);   mk(&tq128, q, qi, Tq, ldq, sq, 128);
  mk(&tk64, k, ki, Tk, ldk, sk, 64);   mk(&tk128, k, ki, Tk, ldk, sk, 128);
  mk(&tv64, v, ki, Tk, ldv, sv, 64);   mk(&tv128, v, ki, Tk, ldv, sv, 128);
  mk(&tdot64, do_t, qi, Tq, qi, qi * Tq, 64);   mk(&tdot128, do_t, qi, Tq, qi, qi * Tq, 128);
  const void* dos = dual ? do_s : do_t;
  mk(&tdos64, dos, qi, Tq, qi, qi * Tq, 64);    mk(&tdos128, dos, qi, Tq, qi, qi * Tq, 128);
  if (rc != TTCD_OK) return rc;
  const int big = 1 << 30;
  AttnBwdParams p;
  p.lse_t = lse_t; p.lse_s = lse_s; p.delta_t = delta_t; p.delta_s = delta_s;
  p.dq = static_cast<bf16*>(dq); p.dk = static_cast<bf16*>(dk); p.dv = static_cast<bf16*>(dv);
  p.Tq = Tq; p.Tk = Tk; p.H = H; p.HK = HK;
  p.w_t = window_t > 0 ? window_t : big;
  p.w_s = window_s > 0 ? window_s : big;
  if (!dual) p.w_s = p.w_t;
  p.scale = scale; p.scale_log2 = scale * LOG2E;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  if (D == 128)
    return dual ? launch_bwd<128, true>(tq64, tq128, tk64, tk128, tv64, tv128, tdot64, tdot128, tdos64, tdos128, p, B, stream)
                : launch_bwd<128, false>(tq64, tq128, tk64, tk128, tv64, tv128, tdot64, tdot128, tdos64, tdos128, p, B, stream);
  return dual ? launch_bwd<64, true>(tq64, tq128, tk64, tk128, tv64, tv128, tdot64, tdot128, tdos64, tdos128, p, B, stream)
              : launch_bwd<64, false>(tq64, tq128, tk64, tk128, tv64, tv128, tdot64, tdot128, tdos64, tdos128, p, B, stream);
}
