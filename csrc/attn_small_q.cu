// Attention for a few query rows over a long key/value cache (sm_100a): the decode step (one row) and short
// continuations (up to 127 rows), where a 128-row tensor-core tile would be almost empty and the work is one
// pass over the cached keys and values.
//
//   pass 1 (attn_small_q_partial): grid (key splits, kv heads, batch).  A CTA stages its <= 256 keys and values in
//           shared memory with 16-byte loads (rows padded by 16 bytes: conflict-free row-per-lane reads), then each
//           warp takes (query row, head of the GQA group) pairs: lanes own keys for Q.K (fp32, the query in shared
//           memory), the warp reduces max / sum, lanes own head-dim slices for P.V.  Writes the partial output and
//           its (max, sum) per split.
//   pass 2 (attn_small_q_merge): one warp per (batch, head, row) folds the splits with the log-sum-exp identity.
//
// Causal mask with bottom-right alignment (query row r sits at key position Tk - Tq + r) and an optional sliding
// window, as flash_attn_func(causal=True, window_size=(W-1, 0)) applies them on the cached decode path of the
// reference (fla/layers/attn.py:215-226, 271-282).  Forward only.
#include "common.cuh"

namespace ttcd {

constexpr int SQ_KEYS = 256;       // keys per split
constexpr int SQ_WARPS = 8;

template <int D>
struct SmallQSmem {
  static constexpr int ROW_BYTES = D * 2 + 16;                    // padded K / V row
  static constexpr int K_OFF = 0;
  static constexpr int V_OFF = K_OFF + SQ_KEYS * ROW_BYTES;
  static constexpr int Q_OFF = V_OFF + SQ_KEYS * ROW_BYTES;       // SQ_WARPS query rows, fp32
  static constexpr int P_OFF = Q_OFF + SQ_WARPS * D * 4;          // SQ_WARPS x SQ_KEYS probabilities, fp32
  static constexpr int TOTAL = P_OFF + SQ_WARPS * SQ_KEYS * 4;
};

struct SmallQParams {
  const bf16* q; const bf16* k; const bf16* v;
  float* part_o;        // [B, H, Tq, splits, D]
  float* part_ml;       // [B, H, Tq, splits, 2]  (max in log2 units, sum)
  const int* kv_len;    // optional device word: the number of valid keys (<= Tk); read at launch time
  int B, Tq, Tk, H, HK, splits, window;
  int64_t ldq, ldk, ldv, sq, sk, sv;
  float scale_log2;
};

template <int D>
__global__ void __launch_bounds__(SQ_WARPS * 32) attn_small_q_partial_kernel(const SmallQParams p) {
  using S = SmallQSmem<D>;
  extern __shared__ __align__(16) uint8_t smem[];
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.H / p.HK;
  const int key0 = split * SQ_KEYS;
  // a cache with a device-side fill count: splits past the count stage nothing and report an empty partial
  const int Tk = p.kv_len != nullptr ? min(max(*p.kv_len, p.Tq), p.Tk) : p.Tk;
  const int nkeys = min(SQ_KEYS, Tk - key0);
  constexpr int VPR = D / 8;                                     // 16-byte vectors per row
  // ---- stage K and V rows of this split
  for (int i = threadIdx.x; i < nkeys * VPR; i += blockDim.x) {
    const int r = i / VPR, c = i % VPR;
    const int64_t krow = static_cast<int64_t>(b) * p.sk + static_cast<int64_t>(key0 + r) * p.ldk + kvh * D + c * 8;
    const int64_t vrow = static_cast<int64_t>(b) * p.sv + static_cast<int64_t>(key0 + r) * p.ldv + kvh * D + c * 8;
    *reinterpret_cast<uint4*>(smem + S::K_OFF + r * S::ROW_BYTES + c * 16) = *reinterpret_cast<const uint4*>(p.k + krow);
    *reinterpret_cast<uint4*>(smem + S::V_OFF + r * S::ROW_BYTES + c * 16) = *reinterpret_cast<const uint4*>(p.v + vrow);
  }
  __syncthreads();
  float* qs = reinterpret_cast<float*>(smem + S::Q_OFF) + warp * D;
  float* ps = reinterpret_cast<float*>(smem + S::P_OFF) + warp * SQ_KEYS;
  const int npairs = p.Tq * G;
  for (int pair = warp; pair < npairs; pair += SQ_WARPS) {
    const int row = pair / G, h = kvh * G + pair % G;
    const int qpos = Tk - p.Tq + row;
    const int lo_excl = p.window > 0 ? qpos - p.window : -1;
    // the query row -> shared memory as fp32
    const bf16* qrow = p.q + static_cast<int64_t>(b) * p.sq + static_cast<int64_t>(row) * p.ldq + h * D;
    for (int d = lane; d < D; d += 32) qs[d] = __bfloat162float(qrow[d]);
    __syncwarp();
    // ---- scores: lane owns keys lane, lane + 32, ...
    float sc[SQ_KEYS / 32];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < SQ_KEYS / 32; ++j) {
      const int r = lane + 32 * j, key = key0 + r;
      float acc = 0.f;
      if (r < nkeys && key <= qpos && key > lo_excl) {
        const uint8_t* krow = smem + S::K_OFF + r * S::ROW_BYTES;
#pragma unroll 4
        for (int c = 0; c < VPR; ++c) {
          const uint4 raw = *reinterpret_cast<const uint4*>(krow + c * 16);
          const float4 qa = *reinterpret_cast<const float4*>(qs + c * 8), qb = *reinterpret_cast<const float4*>(qs + c * 8 + 4);
          const float2 k0 = unpack_bf16(raw.x), k1 = unpack_bf16(raw.y), k2 = unpack_bf16(raw.z), k3 = unpack_bf16(raw.w);
          acc = fmaf(k0.x, qa.x, acc); acc = fmaf(k0.y, qa.y, acc);
          acc = fmaf(k1.x, qa.z, acc); acc = fmaf(k1.y, qa.w, acc);
          acc = fmaf(k2.x, qb.x, acc); acc = fmaf(k2.y, qb.y, acc);
          acc = fmaf(k3.x, qb.z, acc); acc = fmaf(k3.y, qb.w, acc);
        }
        acc *= p.scale_log2;
      } else {
        acc = -INFINITY;
      }
      sc[j] = acc;
      mx = fmaxf(mx, acc);
    }
    mx = warp_max(mx);
    const float m_use = mx == -INFINITY ? 0.f : mx;
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < SQ_KEYS / 32; ++j) {
      const float e = exp2f(sc[j] - m_use);          // exp2(-inf) = 0 for masked keys
      ps[lane + 32 * j] = e;
      sum += e;
    }
    sum = warp_sum(sum);
    __syncwarp();
    // ---- output: lane owns D / 32 consecutive head-dim elements
    constexpr int DPL = D / 32;
    float o[DPL];
#pragma unroll
    for (int e = 0; e < DPL; ++e) o[e] = 0.f;
    for (int r = 0; r < nkeys; ++r) {
      const float pr = ps[r];
      const bf16* vrow = reinterpret_cast<const bf16*>(smem + S::V_OFF + r * S::ROW_BYTES) + lane * DPL;
      if (DPL == 4) {
        const uint2 raw = *reinterpret_cast<const uint2*>(vrow);
        const float2 a = unpack_bf16(raw.x), c = unpack_bf16(raw.y);
        o[0] = fmaf(pr, a.x, o[0]); o[1] = fmaf(pr, a.y, o[1]);
        o[DPL - 2] = fmaf(pr, c.x, o[DPL - 2]); o[DPL - 1] = fmaf(pr, c.y, o[DPL - 1]);
      } else {
        const float2 a = unpack_bf16(*reinterpret_cast<const uint32_t*>(vrow));
        o[0] = fmaf(pr, a.x, o[0]); o[1] = fmaf(pr, a.y, o[1]);
      }
    }
    const int64_t pidx = ((static_cast<int64_t>(b) * p.H + h) * p.Tq + row) * p.splits + split;
#pragma unroll
    for (int e = 0; e < DPL; ++e) p.part_o[pidx * D + lane * DPL + e] = o[e];
    if (lane == 0) {
      p.part_ml[pidx * 2] = mx;
      p.part_ml[pidx * 2 + 1] = sum;
    }
    __syncwarp();
  }
}

// out[b, row, h, :] = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M)
template <int D>
__global__ void __launch_bounds__(256) attn_small_q_merge_kernel(const float* __restrict__ part_o,
                                                                 const float* __restrict__ part_ml, bf16* __restrict__ out,
                                                                 int64_t items, int Tq, int H, int splits) {
  const int lane = threadIdx.x & 31;
  const int64_t item = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);   // (b, h, row)
  if (item >= items) return;
  constexpr int DPL = D / 32;
  float M = -INFINITY;
  for (int s = lane; s < splits; s += 32) M = fmaxf(M, part_ml[(item * splits + s) * 2]);
  M = warp_max(M);
  float o[DPL], l = 0.f;
#pragma unroll
  for (int e = 0; e < DPL; ++e) o[e] = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float m = part_ml[(item * splits + s) * 2];
    if (m == -INFINITY) continue;
    const float w = exp2f(m - M);
    l = fmaf(part_ml[(item * splits + s) * 2 + 1], w, l);
#pragma unroll
    for (int e = 0; e < DPL; ++e) o[e] = fmaf(part_o[(item * splits + s) * D + lane * DPL + e], w, o[e]);
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  const int row = static_cast<int>(item % Tq);
  const int64_t bh = item / Tq;
  const int h = static_cast<int>(bh % H);
  const int64_t b = bh / H;
  bf16* dst = out + ((b * Tq + row) * H + h) * D + lane * DPL;
#pragma unroll
  for (int e = 0; e < DPL; ++e) dst[e] = __float2bfloat16(o[e] * inv);
}

template <int D>
static int launch_small_q(const SmallQParams& p, bf16* out, cudaStream_t stream) {
  using S = SmallQSmem<D>;
  auto k1 = attn_small_q_partial_kernel<D>;
  static bool configured = false;
  if (!configured) {
    TTCD_CUDA_CHECK(cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL));
    configured = true;
  }
  k1<<<dim3(p.splits, p.HK, p.B), SQ_WARPS * 32, S::TOTAL, stream>>>(p);
  TTCD_CUDA_CHECK(cudaGetLastError());
  const int64_t items = static_cast<int64_t>(p.B) * p.H * p.Tq;
  attn_small_q_merge_kernel<D><<<static_cast<unsigned>((items + 7) / 8), 256, 0, stream>>>(p.part_o, p.part_ml, out, items,
                                                                                        p.Tq, p.H, p.splits);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace ttcd

// q [B, Tq, *] (token stride ldq, batch stride sq, head h at column h*D), k / v [B, Tk, *] likewise with HK heads,
// 16-byte aligned rows; out contiguous [B, Tq, H, D] bf16.  part_o fp32 [B, H, Tq, splits, D] and part_ml fp32
// [B, H, Tq, splits, 2] are caller-provided scratch; splits must equal ceil(Tk / 256).  window <= 0: unlimited.
// kv_len (may be null): a device int holding how many of the Tk key rows are filled, read when the kernel runs, so
// that a captured launch follows a cache that grows between replays; the causal alignment then counts from it.
TTCD_EXPORT int ttcd_attn_small_q(const void* q, const void* k, const void* v, void* out, float* part_o, float* part_ml,
                                  int B, int Tq, int Tk, int H, int HK, int D, long long ldq, long long ldk, long long ldv,
                                  long long sq, long long sk, long long sv, int window, float scale, int splits,
                                  const int* kv_len, void* stream_ptr) {
  using namespace ttcd;
  if (B <= 0 || Tq <= 0 || Tq >= 128 || Tk < Tq || H <= 0 || HK <= 0 || H % HK != 0 || (D != 64 && D != 128))
    return TTCD_ERR_ARG;
  if (splits != (Tk + SQ_KEYS - 1) / SQ_KEYS || ldk % 8 != 0 || ldv % 8 != 0 || sk % 8 != 0 || sv % 8 != 0) return TTCD_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(k) & 15u) || (reinterpret_cast<uintptr_t>(v) & 15u)) return TTCD_ERR_ARG;
  SmallQParams p;
  p.q = static_cast<const bf16*>(q); p.k = static_cast<const bf16*>(k); p.v = static_cast<const bf16*>(v);
  p.part_o = part_o; p.part_ml = part_ml; p.kv_len = kv_len;
  p.B = B; p.Tq = Tq; p.Tk = Tk; p.H = H; p.HK = HK; p.splits = splits; p.window = window;
  p.ldq = ldq; p.ldk = ldk; p.ldv = ldv; p.sq = sq; p.sk = sk; p.sv = sv;
  p.scale_log2 = scale * 1.4426950408889634f;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  return D == 128 ? launch_small_q<128>(p, static_cast<bf16*>(out), stream)
                  : launch_small_q<64>(p, static_cast<bf16*>(out), stream);
}
