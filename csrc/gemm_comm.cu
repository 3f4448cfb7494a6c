// Tensor-core GEMMs fused with their collective over NVLink peer memory (sm_100a), for tensor /
// sequence parallel linears.  One kernel does both the transfer and the math, tile by tile:
//
//   ag_gemm :  C[M_total, N] = allgather_rows(X_shard)[M_total, K] * W^T
//              Rank r owns rows [r*M_shard, (r+1)*M_shard) of X in its symmetric buffer.  Inside the
//              kernel one elected thread per CTA pulls the peers' row blocks into a local gathered
//              buffer with bulk async copies (peer global -> shared -> local global, each remote byte
//              crosses NVLink once) and publishes a per-row-block flag; the TMA producer of the GEMM
//              starts with the rank's own rows (no wait) and takes a peer's row block as soon as its
//              flag is up.  The gathered buffer is left behind for the weight-gradient GEMM.
//
//   gemm_rs :  Y_shard[M_shard, N] = reduce_scatter_rows( X[M_total, K_local] * W^T )
//              Every rank computes the row blocks of the OTHER ranks first and PUSHES each finished tile
//              (bf16) straight into its owner's memory: the epilogue warps transpose the tile through
//              shared memory so that every store instruction writes 512 contiguous bytes of one row over
//              NVLink (posted writes: no round trip), then raise the tile's flag in the owner's flag array.
//              The rank's own row blocks are computed last; their epilogue waits for the peers' flags
//              (local memory), adds the peers' tiles in a fixed order (deterministic) and writes the final
//              bf16 output.  No separate reduction pass, no pull across the link, and the NVLink traffic
//              overlaps the tensor-core work of the remaining tiles.
//
//   wgather_gemm :  C[M, N] = X[M, K] * W^T with W a slice of a sharded flat parameter buffer (ZeRO-3 / FSDP):
//              every rank keeps 1/world of a block's parameters; the first GEMM that consumes them (the fused
//              q|k|v projection) gathers the WHOLE block inside the kernel: one elected thread per CTA pulls 64 KB
//              units of the peers' shards (and of the rank's own) into the local gathered buffer with bulk async
//              copies, the units that hold W first, and raises a flag per unit; the TMA producer waits for the
//              flags of the units under the W rows of its tile.  The rest of the block's parameters land while
//              the tensor cores work and are there, by stream order, for the block's other kernels.
//
// All kernels: persistent, one CTA per SM, 128x256x64 tiles, 3-stage TMA ring (never multicast),
// tcgen05.mma into a double-buffered TMEM accumulator.  Every wait (mbarrier or flag) is bounded; on
// expiry the kernel records a code in the status word, drains its copies, frees TMEM and returns.
// They replace NCCL all-gather / reduce-scatter + cuBLAS behind the reference's tensor-parallel plan
// (flame/models/parallelize_fla.py:118-208, 283-287: ColwiseParallel / RowwiseParallel, async-TP).
#include "common.cuh"

#include <algorithm>

namespace ttcd {

constexpr int GC_BM = 128, GC_BN = 256, GC_BK = 64, GC_STAGES = 3, GC_THREADS = 320;
constexpr int GC_A_BYTES = GC_BM * GC_BK * 2;
constexpr int GC_B_BYTES = GC_BN * GC_BK * 2;
constexpr int GC_STAGE_BYTES = GC_A_BYTES + GC_B_BYTES;
constexpr int GC_RING_BYTES = GC_STAGES * GC_STAGE_BYTES;
constexpr int GC_COPY_SLOTS = 4, GC_COPY_LOOK = 2, GC_COPY_BYTES = 16384;
constexpr int GC_MAX_RANKS = 8;
// barriers: full[3] empty[3] tfull[2] tempty[2] copy[4]
constexpr int GC_NBARS = 2 * GC_STAGES + 4 + GC_COPY_SLOTS;

struct GcPeers {
  void* p[GC_MAX_RANKS];
};

constexpr int GC_RS_THREADS = 224;                  // producer, MMA issue, four epilogue warps, flag warp
constexpr int GC_RS_STAGING = 4 * 32 * GC_BN * 2;   // per epilogue warp: 32 rows x 256 bf16 for the transpose

struct GcParams {
  int rank, world, epoch;
  int mbps;            // 128-row blocks per rank shard
  int tiles_n;         // N / 256
  int num_kb;          // K / 64
  int lag;             // gemm_rs: rounds by which this rank's own row blocks trail the pushes (1..mbps)
  int64_t m_shard, N, K;
  int64_t ldc;         // row stride of the output (elements)
  uint64_t wait_ns;    // budget of one flag wait
  // ag_gemm
  bf16* gathered;      // [world*m_shard, K] local
  int* ready;          // [world*mbps] local flags
  // wgather_gemm
  int64_t shard_bytes;   // bytes of one rank's shard of the flat buffer (multiple of the 64 KB unit)
  int64_t w_byte_off;    // byte offset of W inside the flat buffer
  int units;             // 64 KB units in the flat buffer (world * shard_bytes / 64 KB)
  uint8_t* flat;         // local gathered flat buffer
  // gemm_rs
  bf16* partial;       // this rank's symmetric receive buffer [(world-1)*m_shard, N]: slot d-1 holds what rank
                       // (rank + d) % world computed for this rank's rows
  int* part_flags;     // this rank's symmetric flags [(world-1)*mbps*tiles_n], same slot order
};

__device__ __forceinline__ void gc_st_release_sys(int* addr, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void gc_st_release_gpu(int* addr, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int gc_ld_acquire_sys(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ int gc_ld_acquire_gpu(const int* addr) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void gc_fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Bounded wait until *flag >= epoch.  SYS: the flag lives in a peer's memory.
template <bool SYS>
__device__ __forceinline__ bool gc_wait_flag(const int* flag, int epoch, uint64_t wait_ns, volatile int* abort_flag,
                                             int code) {
  if ((SYS ? gc_ld_acquire_sys(flag) : gc_ld_acquire_gpu(flag)) >= epoch) return true;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t it = 1;; ++it) {
    if ((SYS ? gc_ld_acquire_sys(flag) : gc_ld_acquire_gpu(flag)) >= epoch) return true;
    if ((it & 0xf) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > wait_ns) {
        *abort_flag = 1;
        atomicCAS(&g_status, 0, code);
        return false;
      }
      __nanosleep(SYS ? 400 : 100);
    }
  }
}

__device__ __forceinline__ void gc_bulk_g2s(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
               "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void gc_bulk_s2g(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(reinterpret_cast<uint64_t>(dst)),
               "r"(src_smem), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void gc_bulk_wait_read1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }

struct GcTile {
  int owner, mb, nt;
  int64_t row0;   // first row in the [world*m_shard] index space
};
// Tile t of the persistent schedule.
//   own_first (ag_gemm): the rank's own shard leads, then the peers' shards one after the other (their rows arrive
//   while the own rows are multiplied).
//   else (gemm_rs): rounds.  Round r holds row block r of every OTHER rank (pushed to its owner) and row block r - lag
//   of this rank (whose peers' tiles were pushed `lag` rounds earlier, so its epilogue does not wait for them); the
//   first `lag` rounds only push, the last `lag` rounds only finish own blocks.  lag = mbps puts all own blocks last;
//   a smaller lag keeps the link busy for more of the kernel.
__device__ __forceinline__ GcTile gc_tile(int64_t t, const GcParams& p, bool own_first) {
  GcTile c;
  const int64_t mi = t / p.tiles_n;
  c.nt = static_cast<int>(t % p.tiles_n);
  int s;
  if (own_first) {
    s = static_cast<int>(mi / p.mbps);
    c.mb = static_cast<int>(mi % p.mbps);
  } else {
    const int others = p.world - 1, lag = p.lag;
    const int64_t head = static_cast<int64_t>(lag) * others;                       // rounds [0, lag): pushes only
    const int64_t mid = static_cast<int64_t>(p.mbps - lag) * p.world;               // rounds [lag, mbps): pushes + own
    if (mi < head) {
      s = static_cast<int>(mi % others);
      c.mb = static_cast<int>(mi / others);
    } else if (mi < head + mid) {
      const int64_t m2 = mi - head;
      s = static_cast<int>(m2 % p.world);
      const int round = lag + static_cast<int>(m2 / p.world);
      c.mb = s < others ? round : round - lag;
    } else {
      s = others;
      c.mb = p.mbps - lag + static_cast<int>(mi - head - mid);
    }
  }
  c.owner = (p.rank + s + (own_first ? 0 : 1)) % p.world;
  c.row0 = static_cast<int64_t>(c.owner) * p.m_shard + static_cast<int64_t>(c.mb) * GC_BM;
  return c;
}

struct GcSmem {
  uint8_t* base;
  uint32_t base_u32, bar_base;
  uint32_t* tmem_slot;
  volatile int* abort_flag;
  int* epi_count;
  __device__ __forceinline__ uint32_t full(int s) const { return bar_base + 8u * s; }
  __device__ __forceinline__ uint32_t empty(int s) const { return bar_base + 8u * (GC_STAGES + s); }
  __device__ __forceinline__ uint32_t tfull(int b) const { return bar_base + 8u * (2 * GC_STAGES + b); }
  __device__ __forceinline__ uint32_t tempty(int b) const { return bar_base + 8u * (2 * GC_STAGES + 2 + b); }
  __device__ __forceinline__ uint32_t copy(int s) const { return bar_base + 8u * (2 * GC_STAGES + 4 + s); }
};

template <int EXTRA_BYTES>
__device__ __forceinline__ GcSmem gc_setup(uint8_t* raw) {
  GcSmem s;
  s.base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  s.base_u32 = smem_u32(s.base);
  s.bar_base = s.base_u32 + GC_RING_BYTES + EXTRA_BYTES;
  uint8_t* tail = s.base + GC_RING_BYTES + EXTRA_BYTES + GC_NBARS * 8;
  s.tmem_slot = reinterpret_cast<uint32_t*>(tail);
  s.abort_flag = reinterpret_cast<volatile int*>(tail + 4);
  s.epi_count = reinterpret_cast<int*>(tail + 8);
  if (threadIdx.x == 0) {
    for (int i = 0; i < GC_STAGES; ++i) {
      mbar_init(s.full(i), 1);
      mbar_init(s.empty(i), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(s.tfull(b), 1);
      mbar_init(s.tempty(b), 4);
    }
    for (int i = 0; i < GC_COPY_SLOTS; ++i) mbar_init(s.copy(i), 1);
    *s.abort_flag = 0;
    for (int i = 0; i < 4; ++i) s.epi_count[i] = 0;
    mbar_fence_init();
  }
  if ((threadIdx.x >> 5) == 1) {
    tmem_alloc(smem_u32(s.tmem_slot), 2 * GC_BN);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  return s;
}

// One elected thread: tcgen05.mma over the ring for `my_tiles` tiles.
template <bool B_MN>
__device__ __forceinline__ void gc_mma_role(const GcSmem& s, uint32_t tmem_base, int64_t total_tiles, int num_kb) {
  constexpr uint32_t idesc = umma_idesc_bf16(GC_BM, GC_BN, false, B_MN);
  int stage = 0, acc = 0;
  uint32_t phase = 0, acc_phase[2] = {0, 0};
  for (int64_t tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
    if (!mbar_wait(s.tempty(acc), acc_phase[acc] ^ 1u, s.abort_flag, 612)) return;
    tc_fence_after_sync();
    const uint32_t d_tmem = tmem_base + acc * GC_BN;
    for (int kb = 0; kb < num_kb; ++kb) {
      if (!mbar_wait(s.full(stage), phase, s.abort_flag, 613)) return;
      tc_fence_after_sync();
      const uint32_t sa = s.base_u32 + stage * GC_STAGE_BYTES;
      const uint32_t sb = sa + GC_A_BYTES;
#pragma unroll
      for (int k = 0; k < GC_BK / 16; ++k) {
        const uint64_t ad = umma_desc_sw128(sa + k * 32, 16, 1024);
        const uint64_t bd = B_MN ? umma_desc_sw128(sb + k * 2048, GC_BK * 128, 1024) : umma_desc_sw128(sb + k * 32, 16, 1024);
        umma_ss(d_tmem, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
      }
      umma_commit(s.empty(stage));
      if (++stage == GC_STAGES) { stage = 0; phase ^= 1u; }
    }
    umma_commit(s.tfull(acc));
    acc_phase[acc] ^= 1u;
    acc ^= 1;
  }
}

__device__ __forceinline__ void gc_load_b(bool b_mn, uint32_t sb, const CUtensorMap* tma_b, uint32_t bar, int k0, int n0) {
  if (!b_mn) {
    tma_load_3d(sb, tma_b, bar, k0, n0, 0);
  } else {
#pragma unroll
    for (int h = 0; h < GC_BN / 64; ++h) tma_load_3d(sb + h * (GC_BK * 128), tma_b, bar, n0 + h * 64, k0, 0);
  }
}

// Epilogue helper: 32 accumulator columns of one TMEM lane -> bf16 row segment (optionally + fp32 addend).
__device__ __forceinline__ void gc_store_row32(const uint32_t (&v)[32], bf16* dst, const float* add) {
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    float f[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(v[j + e]);
    if (add != nullptr) {
      const float4 a0 = *reinterpret_cast<const float4*>(add + j);
      const float4 a1 = *reinterpret_cast<const float4*>(add + j + 4);
      f[0] += a0.x; f[1] += a0.y; f[2] += a0.z; f[3] += a0.w;
      f[4] += a1.x; f[5] += a1.y; f[6] += a1.z; f[7] += a1.w;
    }
    uint4 o;
    o.x = pack_bf16(f[0], f[1]);
    o.y = pack_bf16(f[2], f[3]);
    o.z = pack_bf16(f[4], f[5]);
    o.w = pack_bf16(f[6], f[7]);
    *reinterpret_cast<uint4*>(dst + j) = o;
  }
}

// ================================================================================================
// all-gather -> GEMM
// ================================================================================================
template <bool B_MN>
__global__ void __launch_bounds__(GC_THREADS, 1)
ag_gemm_kernel(const __grid_constant__ CUtensorMap tma_own, const __grid_constant__ CUtensorMap tma_ag,
               const __grid_constant__ CUtensorMap tma_b, const GcPeers peer_x, bf16* __restrict__ C, const GcParams p) {
  extern __shared__ uint8_t smem_raw[];
  constexpr int STAGING = GC_COPY_SLOTS * GC_COPY_BYTES;
  const GcSmem s = gc_setup<STAGING>(smem_raw);
  const uint32_t tmem_base = *s.tmem_slot;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t total_tiles = static_cast<int64_t>(p.world) * p.mbps * p.tiles_n;

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int64_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const GcTile c = gc_tile(tile, p, true);
        const bool own = c.owner == p.rank;
        if (!own) {
          if (!gc_wait_flag<false>(p.ready + c.owner * p.mbps + c.mb, p.epoch, p.wait_ns, s.abort_flag, 620)) break;
          gc_fence_proxy_async();   // the rows were written through the async proxy of another CTA
        }
        const int arow = own ? c.mb * GC_BM : static_cast<int>(c.row0);
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(s.empty(stage), phase ^ 1u, s.abort_flag, 611)) { ok = false; break; }
          const uint32_t sa = s.base_u32 + stage * GC_STAGE_BYTES;
          mbar_expect_tx(s.full(stage), GC_STAGE_BYTES);
          tma_load_3d(sa, own ? &tma_own : &tma_ag, s.full(stage), kb * GC_BK, arow, 0);
          gc_load_b(B_MN, sa + GC_A_BYTES, &tma_b, s.full(stage), kb * GC_BK, c.nt * GC_BN);
          if (++stage == GC_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (*s.abort_flag)
        for (int i = 0; i < GC_STAGES; ++i) mbar_drain(s.full(i), 0), mbar_drain(s.full(i), 1);
    }
  } else if (warp == 1) {
    if (elect_one()) gc_mma_role<B_MN>(s, tmem_base, total_tiles, p.num_kb);
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue
    const int quarter = warp & 3;
    uint32_t acc_phase[2] = {0, 0};
    int acc = 0;
    for (int64_t tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      const GcTile c = gc_tile(tile, p, true);
      if (!mbar_wait(s.tfull(acc), acc_phase[acc], s.abort_flag, 614)) break;
      tc_fence_after_sync();
      bf16* crow = C + (c.row0 + quarter * 32 + lane) * p.ldc + static_cast<int64_t>(c.nt) * GC_BN;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * GC_BN;
#pragma unroll 1
      for (int col = 0; col < GC_BN; col += 32) {
        uint32_t v[32];
        tmem_ld32(t_row + col, v);
        tmem_ld_wait();
        gc_store_row32(v, crow + col, nullptr);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(s.tempty(acc));
      acc_phase[acc] ^= 1u;
      acc ^= 1;
    }
  } else if (warp == 6) {
    // ------------------------------------------------------------------ gather: peer rows -> local buffer
    if (elect_one()) {
      const uint32_t stage_base = s.base_u32 + GC_RING_BYTES;
      const int64_t unit_bytes = static_cast<int64_t>(GC_BM) * p.K * 2;
      const int n_chunks = static_cast<int>(unit_bytes / GC_COPY_BYTES);
      const int64_t units = static_cast<int64_t>(p.world - 1) * p.mbps;
      uint32_t g = 0;   // running chunk counter: slot = g % SLOTS, parity = (g / SLOTS) & 1
      bool ok = true;
      for (int64_t u = blockIdx.x; u < units && ok; u += gridDim.x) {
        const int sidx = static_cast<int>(u / p.mbps) + 1, mb = static_cast<int>(u % p.mbps);
        const int owner = (p.rank + sidx) % p.world;
        const uint8_t* src = static_cast<const uint8_t*>(peer_x.p[owner]) + static_cast<int64_t>(mb) * unit_bytes;
        uint8_t* dst = reinterpret_cast<uint8_t*>(p.gathered) +
                       (static_cast<int64_t>(owner) * p.m_shard + static_cast<int64_t>(mb) * GC_BM) * p.K * 2;
        for (int i = 0; i < n_chunks + GC_COPY_LOOK; ++i) {
          if (i < n_chunks) {
            gc_bulk_wait_read1();   // the store that last used this slot has finished reading it
            const uint32_t slot = (g + i) % GC_COPY_SLOTS;
            mbar_expect_tx(s.copy(slot), GC_COPY_BYTES);
            gc_bulk_g2s(stage_base + slot * GC_COPY_BYTES, src + static_cast<int64_t>(i) * GC_COPY_BYTES, GC_COPY_BYTES,
                        s.copy(slot));
          }
          if (i >= GC_COPY_LOOK) {
            const uint32_t j = g + i - GC_COPY_LOOK;
            const uint32_t slot = j % GC_COPY_SLOTS;
            if (!mbar_wait(s.copy(slot), (j / GC_COPY_SLOTS) & 1u, s.abort_flag, 621)) { ok = false; break; }
            gc_bulk_s2g(dst + static_cast<int64_t>(i - GC_COPY_LOOK) * GC_COPY_BYTES, stage_base + slot * GC_COPY_BYTES,
                        GC_COPY_BYTES);
            tma_store_commit();
          }
        }
        if (!ok) break;
        g += n_chunks;
        tma_store_wait0();          // the row block is complete in local memory
        gc_fence_proxy_async();
        __threadfence();
        gc_st_release_gpu(p.ready + owner * p.mbps + mb, p.epoch);
      }
      if (!ok) {
        for (int i = 0; i < GC_COPY_SLOTS; ++i) mbar_drain(s.copy(i), 0), mbar_drain(s.copy(i), 1);
      }
      tma_store_wait0();
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 2 * GC_BN);
  }
}

// ================================================================================================
// sharded-parameter gather -> GEMM
// ================================================================================================
constexpr int GC_UNIT_BYTES = GC_COPY_SLOTS * GC_COPY_BYTES;     // 64 KB: flag granularity of the gathered buffer

template <bool B_MN>
__global__ void __launch_bounds__(GC_THREADS, 1)
wgather_gemm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                    const GcPeers shards, bf16* __restrict__ C, const GcParams p) {
  extern __shared__ uint8_t smem_raw[];
  constexpr int STAGING = GC_COPY_SLOTS * GC_COPY_BYTES;
  const GcSmem s = gc_setup<STAGING>(smem_raw);
  const uint32_t tmem_base = *s.tmem_slot;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t tiles_m = p.m_shard / GC_BM;
  const int64_t total_tiles = tiles_m * p.tiles_n;
  // bytes of W under one n-tile of the output: B_MN = false: W is [N, K], 256 rows; B_MN = true: W is [K, N] and an
  // n-tile touches every row, so all of W must be there
  const int64_t w_bytes = p.N * p.K * 2;
  const int u_w0 = static_cast<int>(p.w_byte_off / GC_UNIT_BYTES);
  const int u_w1 = static_cast<int>((p.w_byte_off + w_bytes - 1) / GC_UNIT_BYTES);      // inclusive

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int ready_hi = u_w0 - 1;        // units [u_w0, ready_hi] are known to be there
      for (int64_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int mi = static_cast<int>(tile / p.tiles_n), nt = static_cast<int>(tile % p.tiles_n);
        const int64_t hi_byte = B_MN ? p.w_byte_off + w_bytes - 1
                                     : p.w_byte_off + (static_cast<int64_t>(nt + 1) * GC_BN) * p.K * 2 - 1;
        const int need = static_cast<int>(hi_byte / GC_UNIT_BYTES);       // the units arrive in ascending order of W
        while (ready_hi < need) {
          if (!gc_wait_flag<false>(p.ready + ready_hi + 1, p.epoch, p.wait_ns, s.abort_flag, 650)) { ok = false; break; }
          ++ready_hi;
        }
        if (!ok) break;
        gc_fence_proxy_async();       // the rows were written through the async proxy of another CTA
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(s.empty(stage), phase ^ 1u, s.abort_flag, 651)) { ok = false; break; }
          const uint32_t sa = s.base_u32 + stage * GC_STAGE_BYTES;
          mbar_expect_tx(s.full(stage), GC_STAGE_BYTES);
          tma_load_3d(sa, &tma_a, s.full(stage), kb * GC_BK, mi * GC_BM, 0);
          gc_load_b(B_MN, sa + GC_A_BYTES, &tma_b, s.full(stage), kb * GC_BK, nt * GC_BN);
          if (++stage == GC_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (*s.abort_flag)
        for (int i = 0; i < GC_STAGES; ++i) mbar_drain(s.full(i), 0), mbar_drain(s.full(i), 1);
    }
  } else if (warp == 1) {
    if (elect_one()) gc_mma_role<B_MN>(s, tmem_base, total_tiles, p.num_kb);
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue
    const int quarter = warp & 3;
    uint32_t acc_phase[2] = {0, 0};
    int acc = 0;
    for (int64_t tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      const int mi = static_cast<int>(tile / p.tiles_n), nt = static_cast<int>(tile % p.tiles_n);
      if (!mbar_wait(s.tfull(acc), acc_phase[acc], s.abort_flag, 654)) break;
      tc_fence_after_sync();
      bf16* crow = C + (static_cast<int64_t>(mi) * GC_BM + quarter * 32 + lane) * p.ldc + static_cast<int64_t>(nt) * GC_BN;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * GC_BN;
#pragma unroll 1
      for (int col = 0; col < GC_BN; col += 32) {
        uint32_t v[32];
        tmem_ld32(t_row + col, v);
        tmem_ld_wait();
        gc_store_row32(v, crow + col, nullptr);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(s.tempty(acc));
      acc_phase[acc] ^= 1u;
      acc ^= 1;
    }
  } else if (warp == 6) {
    // ------------------------------------------------------------------ gather: every rank's shard -> local flat buffer
    // Units are taken in the order [units of W, ascending] then [the other units of the block]; unit j of that
    // order goes to CTA j % gridDim.x, so the W units are spread over the first CTAs and land first.
    if (elect_one()) {
      const uint32_t stage_base = s.base_u32 + GC_RING_BYTES;
      const int n_w = u_w1 - u_w0 + 1;
      uint32_t g = 0;   // running chunk counter: slot = g % SLOTS, parity = (g / SLOTS) & 1
      bool ok = true;
      for (int j = blockIdx.x; j < p.units && ok; j += gridDim.x) {
        // order: W units first; then units [0, u_w0); then units (u_w1, units)
        const int unit = j < n_w ? u_w0 + j : (j - n_w < u_w0 ? j - n_w : j);
        const int64_t byte0 = static_cast<int64_t>(unit) * GC_UNIT_BYTES;
        const int owner = static_cast<int>(byte0 / p.shard_bytes);
        const uint8_t* src = static_cast<const uint8_t*>(shards.p[owner]) + (byte0 - static_cast<int64_t>(owner) * p.shard_bytes);
        uint8_t* dst = p.flat + byte0;
        constexpr int n_chunks = GC_COPY_SLOTS;
        for (int i = 0; i < n_chunks + GC_COPY_LOOK; ++i) {
          if (i < n_chunks) {
            gc_bulk_wait_read1();   // the store that last used this slot has finished reading it
            const uint32_t slot = (g + i) % GC_COPY_SLOTS;
            mbar_expect_tx(s.copy(slot), GC_COPY_BYTES);
            gc_bulk_g2s(stage_base + slot * GC_COPY_BYTES, src + static_cast<int64_t>(i) * GC_COPY_BYTES, GC_COPY_BYTES,
                        s.copy(slot));
          }
          if (i >= GC_COPY_LOOK) {
            const uint32_t jj = g + i - GC_COPY_LOOK;
            const uint32_t slot = jj % GC_COPY_SLOTS;
            if (!mbar_wait(s.copy(slot), (jj / GC_COPY_SLOTS) & 1u, s.abort_flag, 652)) { ok = false; break; }
            gc_bulk_s2g(dst + static_cast<int64_t>(i - GC_COPY_LOOK) * GC_COPY_BYTES, stage_base + slot * GC_COPY_BYTES,
                        GC_COPY_BYTES);
            tma_store_commit();
          }
        }
        if (!ok) break;
        g += n_chunks;
        tma_store_wait0();          // the unit is complete in local memory
        gc_fence_proxy_async();
        __threadfence();
        gc_st_release_gpu(p.ready + unit, p.epoch);
      }
      if (!ok) {
        for (int i = 0; i < GC_COPY_SLOTS; ++i) mbar_drain(s.copy(i), 0), mbar_drain(s.copy(i), 1);
      }
      tma_store_wait0();
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 2 * GC_BN);
  }
}

// ================================================================================================
// GEMM -> reduce-scatter
// ================================================================================================
template <bool B_MN>
__global__ void __launch_bounds__(GC_RS_THREADS, 1)
gemm_rs_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
               const GcPeers peer_part, const GcPeers peer_flags, bf16* __restrict__ out, const GcParams p) {
  extern __shared__ uint8_t smem_raw[];
  const GcSmem s = gc_setup<GC_RS_STAGING>(smem_raw);
  const uint32_t tmem_base = *s.tmem_slot;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t total_tiles = static_cast<int64_t>(p.world) * p.mbps * p.tiles_n;

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int64_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const GcTile c = gc_tile(tile, p, false);
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(s.empty(stage), phase ^ 1u, s.abort_flag, 631)) { ok = false; break; }
          const uint32_t sa = s.base_u32 + stage * GC_STAGE_BYTES;
          mbar_expect_tx(s.full(stage), GC_STAGE_BYTES);
          tma_load_3d(sa, &tma_a, s.full(stage), kb * GC_BK, static_cast<int>(c.row0), 0);
          gc_load_b(B_MN, sa + GC_A_BYTES, &tma_b, s.full(stage), kb * GC_BK, c.nt * GC_BN);
          if (++stage == GC_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (*s.abort_flag)
        for (int i = 0; i < GC_STAGES; ++i) mbar_drain(s.full(i), 0), mbar_drain(s.full(i), 1);
    }
  } else if (warp == 1) {
    if (elect_one()) gc_mma_role<B_MN>(s, tmem_base, total_tiles, p.num_kb);
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue
    const int quarter = warp & 3;
    uint32_t acc_phase[2] = {0, 0};
    int acc = 0;
    uint8_t* stage = s.base + GC_RING_BYTES + quarter * (32 * GC_BN * 2);     // this warp's 32 x 512-byte rows
    volatile int* pushed = s.epi_count;      // per epilogue warp: tiles of other ranks whose stores it has issued
    int n_pushed = 0;
    for (int64_t tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      const GcTile c = gc_tile(tile, p, false);
      const bool own = c.owner == p.rank;
      if (!mbar_wait(s.tfull(acc), acc_phase[acc], s.abort_flag, 634)) break;
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * GC_BN;
      const int64_t col0 = static_cast<int64_t>(c.nt) * GC_BN;
      if (!own) {
        // another rank's rows.  TMEM lane == row, so a thread holds one row; a store instruction of the warp should
        // cover one row's 512 contiguous bytes instead (NVLink writes of whole lines): transpose through shared
        // memory, 16-byte chunk c of row r at chunk position c ^ r (conflict-free both ways)
#pragma unroll 1
        for (int col = 0; col < GC_BN; col += 32) {
          uint32_t v[32];
          tmem_ld32(t_row + col, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 o;
            o.x = pack_bf16(__uint_as_float(v[8 * j]), __uint_as_float(v[8 * j + 1]));
            o.y = pack_bf16(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
            o.z = pack_bf16(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
            o.w = pack_bf16(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
            const int chunk = col / 8 + j;
            *reinterpret_cast<uint4*>(stage + lane * 512 + ((chunk ^ lane) & 31) * 16) = o;
          }
        }
        // the accumulator has left TMEM: hand the buffer back to the MMA warp before the remote stores
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(s.tempty(acc));
        const int slot = (p.rank - c.owner - 1 + p.world) % p.world;
        bf16* dst = static_cast<bf16*>(peer_part.p[c.owner]) +
                    (static_cast<int64_t>(slot) * p.m_shard + static_cast<int64_t>(c.mb) * GC_BM + quarter * 32) * p.N + col0 +
                    lane * 8;
#pragma unroll 4
        for (int r = 0; r < 32; ++r) {
          const uint4 val = *reinterpret_cast<const uint4*>(stage + r * 512 + ((lane ^ r) & 31) * 16);
          *reinterpret_cast<uint4*>(dst + static_cast<int64_t>(r) * p.N) = val;
        }
        // The stores are posted; waiting here for their acknowledgement (a system-scope fence) would stall this warp
        // for a link round trip per tile.  Instead the warp only publishes, at CTA scope, that its stores of this
        // tile are issued; the flag warp fences at system scope and raises the tile's flag in the owner's memory
        // (release semantics are cumulative over what it observed).
        __syncwarp();                 // the staging rows are free for the next tile
        if (lane == 0) {
          __threadfence_block();
          pushed[quarter] = ++n_pushed;          // one counter per epilogue warp: the warps may be two tiles apart
        }
        acc_phase[acc] ^= 1u;
        acc ^= 1;
        continue;
      }
      // this rank's rows: wait for the peers' tiles (pushed into local memory), add them in slot order, write the output
      bool ready = true;
      for (int d = 0; d + 1 < p.world && ready; ++d) {
        const int* flag = p.part_flags + (d * p.mbps + c.mb) * p.tiles_n + c.nt;
        int r = 1;
        if (lane == 0) r = gc_wait_flag<true>(flag, p.epoch, p.wait_ns, s.abort_flag, 635) ? 1 : 0;   // written by a peer GPU
        ready = __shfl_sync(0xffffffffu, r, 0) != 0;
        if (ready) (void)gc_ld_acquire_sys(flag);   // every lane orders its reads of the tile after the flag
      }
      if (!ready) break;
      const int64_t lrow = static_cast<int64_t>(c.mb) * GC_BM + quarter * 32 + lane;
      bf16* orow = out + lrow * p.ldc + col0;
      const bf16* prow = p.partial + lrow * p.N + col0;
      const int64_t slot_stride = p.m_shard * p.N;
#pragma unroll 1
      for (int col = 0; col < GC_BN; col += 32) {
        uint32_t v[32];
        tmem_ld32(t_row + col, v);
        // peers' tiles: the loads of slot d + 1 are in flight while slot d is added (fixed order: deterministic)
        uint4 cur[4], nxt[4];
        auto load_slot = [&](uint4 (&dstv)[4], int d) {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            dstv[j] = *reinterpret_cast<const uint4*>(prow + static_cast<int64_t>(d) * slot_stride + col + 8 * j);
        };
        if (p.world > 1) load_slot(cur, 0);
        tmem_ld_wait();
#pragma unroll
        for (int d = 0; d < GC_MAX_RANKS - 1; ++d) {
          if (d + 1 < p.world) {
            if (d + 2 < p.world) load_slot(nxt, d + 1);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t w[4] = {cur[j].x, cur[j].y, cur[j].z, cur[j].w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 t = unpack_bf16(w[e]);
                v[8 * j + 2 * e] = __float_as_uint(__uint_as_float(v[8 * j + 2 * e]) + t.x);
                v[8 * j + 2 * e + 1] = __float_as_uint(__uint_as_float(v[8 * j + 2 * e + 1]) + t.y);
              }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) cur[j] = nxt[j];
          }
        }
        gc_store_row32(v, orow + col, nullptr);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(s.tempty(acc));
      acc_phase[acc] ^= 1u;
      acc ^= 1;
    }
  } else if (warp == 6 && p.world > 1) {
    // ------------------------------------------------------------------ flag warp
    // Walks this CTA's tiles of other ranks in schedule order; when all four epilogue warps have issued the stores
    // of a tile, makes them visible system-wide and raises the tile's flag at its owner.
    if (lane == 0) {
      volatile int* pushed = s.epi_count;
      int done = 0;
      for (int64_t tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
        const GcTile c = gc_tile(tile, p, false);
        if (c.owner == p.rank) continue;
        ++done;
        const uint64_t t0 = globaltimer_ns();
        bool ok = true;
        while (pushed[0] < done || pushed[1] < done || pushed[2] < done || pushed[3] < done) {
          if (*s.abort_flag) { ok = false; break; }
          if (globaltimer_ns() - t0 > p.wait_ns) {      // the epilogue warps never got there: give up like they did
            *s.abort_flag = 1;
            atomicCAS(&g_status, 0, 636);
            ok = false;
            break;
          }
          __nanosleep(100);
        }
        if (!ok) break;
        __threadfence_system();
        const int slot = (p.rank - c.owner - 1 + p.world) % p.world;
        gc_st_release_sys(static_cast<int*>(peer_flags.p[c.owner]) + (slot * p.mbps + c.mb) * p.tiles_n + c.nt, p.epoch);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 2 * GC_BN);
  }
}

static GcPeers gc_peers(const long long* ptrs, int world) {
  GcPeers pp{};
  for (int r = 0; r < world && r < GC_MAX_RANKS; ++r) pp.p[r] = reinterpret_cast<void*>(ptrs[r]);
  return pp;
}

static int gc_check(int rank, int world, long long m_shard, long long N, long long K) {
  if (world < 1 || world > GC_MAX_RANKS || rank < 0 || rank >= world) return TTCD_ERR_ARG;
  if (m_shard <= 0 || m_shard % GC_BM != 0 || N <= 0 || N % GC_BN != 0 || K <= 0 || K % GC_BK != 0) return TTCD_ERR_ARG;
  if (m_shard * world > 0x7fffffffLL) return TTCD_ERR_ARG;
  return TTCD_OK;
}

template <typename Kern>
static int gc_configure(Kern kern, int smem_bytes) {
  return static_cast<int>(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
}

}  // namespace ttcd

TTCD_DEFINE_STATUS_READER(gemm_comm)
using namespace ttcd;

// C[world*m_shard, N] (row stride ldc) = gather_r(x_r)[world*m_shard, K] * W^T.
// x_ptrs[r]: rank r's bf16 [m_shard, K] block in peer-addressable memory (x_ptrs[rank] is local).
// w: [N, K] (b_mn = 0) or [K, N] (b_mn = 1), row stride ldw.  gathered: local bf16 [world*m_shard, K]; on
// return the peers' rows are in it (the rank's own rows are NOT copied).  ready: local int[world*mbps], must
// hold values < epoch.  All peers must have finished writing their x block before the launch (barrier).
TTCD_EXPORT int ttcd_ag_gemm(const long long* x_ptrs, const void* w, void* c, void* gathered, int* ready, int rank,
                             int world, long long m_shard, long long N, long long K, long long ldw, long long ldc,
                             int b_mn, int epoch, long long wait_ns, void* stream_ptr) {
  int rc = gc_check(rank, world, m_shard, N, K);
  if (rc != TTCD_OK) return rc;
  if ((static_cast<long long>(GC_BM) * K * 2) % GC_COPY_BYTES != 0 || (ldc * 2) % 16 != 0) return TTCD_ERR_ARG;
  CUtensorMap t_own, t_ag, t_b;
  rc = make_tmap_bf16_3d(&t_own, reinterpret_cast<const void*>(x_ptrs[rank]), K, m_shard, 1, K, 0, 64, GC_BM);
  if (rc != TTCD_OK) return rc;
  rc = make_tmap_bf16_3d(&t_ag, gathered, K, m_shard * world, 1, K, 0, 64, GC_BM);
  if (rc != TTCD_OK) return rc;
  rc = b_mn ? make_tmap_bf16_3d(&t_b, w, N, K, 1, ldw, 0, 64, GC_BK) : make_tmap_bf16_3d(&t_b, w, K, N, 1, ldw, 0, 64, GC_BN);
  if (rc != TTCD_OK) return rc;
  GcParams p{};
  p.rank = rank; p.world = world; p.epoch = epoch;
  p.mbps = static_cast<int>(m_shard / GC_BM); p.tiles_n = static_cast<int>(N / GC_BN); p.num_kb = static_cast<int>(K / GC_BK);
  p.m_shard = m_shard; p.N = N; p.K = K; p.ldc = ldc;
  p.wait_ns = wait_ns > 0 ? static_cast<uint64_t>(wait_ns) : 10000000000ull;
  p.gathered = static_cast<bf16*>(gathered); p.ready = ready;
  constexpr int smem_bytes = GC_RING_BYTES + GC_COPY_SLOTS * GC_COPY_BYTES + GC_NBARS * 8 + 32 + 1024;
  const long long total = static_cast<long long>(world) * p.mbps * p.tiles_n;
  const int grid = static_cast<int>(std::min<long long>(total, sm_count()));
  cudaStream_t st = static_cast<cudaStream_t>(stream_ptr);
  if (b_mn) {
    TTCD_CUDA_CHECK(static_cast<cudaError_t>(gc_configure(ag_gemm_kernel<true>, smem_bytes)));
    ag_gemm_kernel<true><<<grid, GC_THREADS, smem_bytes, st>>>(t_own, t_ag, t_b, gc_peers(x_ptrs, world), static_cast<bf16*>(c), p);
  } else {
    TTCD_CUDA_CHECK(static_cast<cudaError_t>(gc_configure(ag_gemm_kernel<false>, smem_bytes)));
    ag_gemm_kernel<false><<<grid, GC_THREADS, smem_bytes, st>>>(t_own, t_ag, t_b, gc_peers(x_ptrs, world), static_cast<bf16*>(c), p);
  }
  return static_cast<int>(cudaGetLastError());
}

// out[m_shard, N] (row stride ldc) = rows [rank*m_shard, (rank+1)*m_shard) of sum_r ( x_r[world*m_shard, K] * w_r^T ).
// x: local bf16 [world*m_shard, K] (row stride ldx); w: [N, K] or [K, N] (b_mn).  partial_ptrs[r] / flag_ptrs[r]:
// rank r's symmetric receive buffer (bf16 [(world-1)*m_shard, N]) and flags (int[(world-1)*mbps*tiles_n], values <
// epoch): the peers' tiles of rank r's rows arrive there.  Every rank must have finished the previous call that used
// these buffers before this launch (barrier): peers start writing into them at once.
// lag_blocks: see gc_tile (<= 0: the rank's own row blocks come last).
TTCD_EXPORT int ttcd_gemm_rs(const void* x, const void* w, void* out, const long long* partial_ptrs,
                             const long long* flag_ptrs, int rank, int world, long long m_shard, long long N, long long K,
                             long long ldx, long long ldw, long long ldc, int b_mn, int epoch, long long wait_ns,
                             int lag_blocks, void* stream_ptr) {
  int rc = gc_check(rank, world, m_shard, N, K);
  if (rc != TTCD_OK) return rc;
  if ((ldc * 2) % 16 != 0) return TTCD_ERR_ARG;
  CUtensorMap t_a, t_b;
  rc = make_tmap_bf16_3d(&t_a, x, K, m_shard * world, 1, ldx, 0, 64, GC_BM);
  if (rc != TTCD_OK) return rc;
  rc = b_mn ? make_tmap_bf16_3d(&t_b, w, N, K, 1, ldw, 0, 64, GC_BK) : make_tmap_bf16_3d(&t_b, w, K, N, 1, ldw, 0, 64, GC_BN);
  if (rc != TTCD_OK) return rc;
  GcParams p{};
  p.rank = rank; p.world = world; p.epoch = epoch;
  p.mbps = static_cast<int>(m_shard / GC_BM); p.tiles_n = static_cast<int>(N / GC_BN); p.num_kb = static_cast<int>(K / GC_BK);
  p.m_shard = m_shard; p.N = N; p.K = K; p.ldc = ldc;
  p.wait_ns = wait_ns > 0 ? static_cast<uint64_t>(wait_ns) : 10000000000ull;
  p.partial = reinterpret_cast<bf16*>(partial_ptrs[rank]);
  p.part_flags = reinterpret_cast<int*>(flag_ptrs[rank]);
  // lag_blocks <= 0: all own row blocks last
  p.lag = (lag_blocks <= 0 || lag_blocks > p.mbps || world == 1) ? p.mbps : lag_blocks;
  constexpr int smem_bytes = GC_RING_BYTES + GC_RS_STAGING + GC_NBARS * 8 + 32 + 1024;
  const long long total = static_cast<long long>(world) * p.mbps * p.tiles_n;
  const int grid = static_cast<int>(std::min<long long>(total, sm_count()));
  cudaStream_t st = static_cast<cudaStream_t>(stream_ptr);
  if (b_mn) {
    TTCD_CUDA_CHECK(static_cast<cudaError_t>(gc_configure(gemm_rs_kernel<true>, smem_bytes)));
    gemm_rs_kernel<true><<<grid, GC_RS_THREADS, smem_bytes, st>>>(t_a, t_b, gc_peers(partial_ptrs, world),
                                                                  gc_peers(flag_ptrs, world), static_cast<bf16*>(out), p);
  } else {
    TTCD_CUDA_CHECK(static_cast<cudaError_t>(gc_configure(gemm_rs_kernel<false>, smem_bytes)));
    gemm_rs_kernel<false><<<grid, GC_RS_THREADS, smem_bytes, st>>>(t_a, t_b, gc_peers(partial_ptrs, world),
                                                                   gc_peers(flag_ptrs, world), static_cast<bf16*>(out), p);
  }
  return static_cast<int>(cudaGetLastError());
}

namespace ttcd {
// flat[r * shard_elems + i] = shards.p[r][i]: the stand-alone statement of the parameter all-gather (plain peer loads),
// used where no GEMM of a fitting shape consumes the block first (backward re-gather, odd widths).
__global__ void __launch_bounds__(256) peer_gather_kernel(GcPeers shards, int world, int64_t shard_vecs, uint4* __restrict__ flat) {
  const int64_t total = shard_vecs * world;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / shard_vecs);
    flat[i] = static_cast<const uint4*>(shards.p[r])[i - static_cast<int64_t>(r) * shard_vecs];
  }
}
}  // namespace ttcd

// flat (local bf16 [world * shard_elems]) <- every rank's shard (shard_ptrs[r]: bf16 [shard_elems], peer-addressable).
TTCD_EXPORT int ttcd_peer_gather(void* flat, const long long* shard_ptrs, int world, long long shard_elems, void* stream_ptr) {
  if (world < 1 || world > GC_MAX_RANKS || shard_elems <= 0 || shard_elems % 8 != 0) return TTCD_ERR_ARG;
  const long long vecs = shard_elems / 8;
  const unsigned grid = static_cast<unsigned>(std::min<long long>((vecs * world + 255) / 256, 148LL * 8));
  peer_gather_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream_ptr)>>>(gc_peers(shard_ptrs, world), world, vecs,
                                                                              static_cast<uint4*>(flat));
  return static_cast<int>(cudaGetLastError());
}

// C[M, N] (row stride ldc) = x[M, K] (row stride ldx) * W^T, W = flat + w_elem_off: [N, K] contiguous (b_mn = 0) or
// [K, N] contiguous (b_mn = 1), where flat (local bf16 [world * shard_elems]) is filled INSIDE the kernel from every
// rank's shard (shard_ptrs[r], peer-addressable; shard_ptrs[rank] is local).  ready: local int[world * shard_elems * 2 /
// 65536], values < epoch; on return every unit's flag is at epoch and the whole flat buffer is gathered.
// M % 128 == 0, N % 256 == 0, K % 64 == 0, shard_elems * 2 % 65536 == 0, w_elem_off % 8 == 0.
// All peers must have finished writing their shards before the launch (barrier or stream order after the optimizer).
TTCD_EXPORT int ttcd_wgather_gemm(const void* x, void* c, void* flat, const long long* shard_ptrs, int* ready, int rank,
                                  int world, long long M, long long N, long long K, long long ldx, long long ldc,
                                  long long w_elem_off, long long shard_elems, int b_mn, int epoch, long long wait_ns,
                                  void* stream_ptr) {
  int rc = gc_check(rank, world, M, N, K);
  if (rc != TTCD_OK) return rc;
  if ((ldc * 2) % 16 != 0 || (ldx * 2) % 16 != 0 || w_elem_off % 8 != 0 || w_elem_off < 0) return TTCD_ERR_ARG;
  if (shard_elems <= 0 || (shard_elems * 2) % GC_UNIT_BYTES != 0) return TTCD_ERR_ARG;
  if (w_elem_off + N * K > shard_elems * world) return TTCD_ERR_ARG;
  const bf16* w = static_cast<const bf16*>(flat) + w_elem_off;
  CUtensorMap t_a, t_b;
  rc = make_tmap_bf16_3d(&t_a, x, K, M, 1, ldx, 0, 64, GC_BM);
  if (rc != TTCD_OK) return rc;
  rc = b_mn ? make_tmap_bf16_3d(&t_b, w, N, K, 1, N, 0, 64, GC_BK) : make_tmap_bf16_3d(&t_b, w, K, N, 1, K, 0, 64, GC_BN);
  if (rc != TTCD_OK) return rc;
  GcParams p{};
  p.rank = rank; p.world = world; p.epoch = epoch;
  p.tiles_n = static_cast<int>(N / GC_BN); p.num_kb = static_cast<int>(K / GC_BK);
  p.m_shard = M; p.N = N; p.K = K; p.ldc = ldc;
  p.wait_ns = wait_ns > 0 ? static_cast<uint64_t>(wait_ns) : 10000000000ull;
  p.ready = ready;
  p.shard_bytes = shard_elems * 2; p.w_byte_off = w_elem_off * 2;
  p.units = static_cast<int>(shard_elems * 2 * world / GC_UNIT_BYTES);
  p.flat = static_cast<uint8_t*>(flat);
  constexpr int smem_bytes = GC_RING_BYTES + GC_COPY_SLOTS * GC_COPY_BYTES + GC_NBARS * 8 + 32 + 1024;
  // every CTA must be resident at once (the producers wait for units that other CTAs gather): one CTA per SM at most
  const long long total = (M / GC_BM) * p.tiles_n;
  const int grid = static_cast<int>(std::min<long long>(std::max<long long>(total, 1), sm_count()));
  cudaStream_t st = static_cast<cudaStream_t>(stream_ptr);
  if (b_mn) {
    TTCD_CUDA_CHECK(static_cast<cudaError_t>(gc_configure(wgather_gemm_kernel<true>, smem_bytes)));
    wgather_gemm_kernel<true><<<grid, GC_THREADS, smem_bytes, st>>>(t_a, t_b, gc_peers(shard_ptrs, world), static_cast<bf16*>(c), p);
  } else {
    TTCD_CUDA_CHECK(static_cast<cudaError_t>(gc_configure(wgather_gemm_kernel<false>, smem_bytes)));
    wgather_gemm_kernel<false><<<grid, GC_THREADS, smem_bytes, st>>>(t_a, t_b, gc_peers(shard_ptrs, world), static_cast<bf16*>(c), p);
  }
  return static_cast<int>(cudaGetLastError());
}
