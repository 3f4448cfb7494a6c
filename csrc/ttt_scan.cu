// Fast-weight chunk scan helpers (sm_100a).  The scan of IP-TTCD's TTT layers
//
//     dW_j = P_j^T zhat_j,   W_i = W_down + lr * sum_{j<i} dW_j,   Y_i = zout_i W_i^T
//
// (custom_models/ipttcd/modeling_ipttcdv9_lowcopy_scanfuse.py:117-204) runs its three contractions as
// batched tcgen05 GEMM launches (csrc/gemm.cu); the two kernels here are the streaming passes between them:
//
//   ttt_prefix_weights : exclusive prefix over chunks of the fp32 updates fused with the add of the slow weight
//                        (and of a context-parallel start state) and the cast to the bf16 operand of the Y GEMM
//   ttt_suffix_grads   : backward of that prefix: reverse exclusive sum of the per-chunk weight gradients,
//                        scaled by lr and cast to bf16 (operand of the dP / dzhat GEMMs), plus the slow-weight
//                        gradient (sum over all chunks and batch entries)
//
// One thread owns 8 consecutive weight elements for the whole chunk loop: every input is read once and
// every output written once with 16/32-byte accesses.  They replace torch.cumsum + per-chunk adds + casts
// (and, in backward, flip-cumsum-flip) of the reference.
#include "common.cuh"

namespace ttcd {

__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void store8_bf16(bf16* p, const float (&v)[8], float scale) {
  uint4 o;
  o.x = pack_bf16(v[0] * scale, v[1] * scale);
  o.y = pack_bf16(v[2] * scale, v[3] * scale);
  o.z = pack_bf16(v[4] * scale, v[5] * scale);
  o.w = pack_bf16(v[6] * scale, v[7] * scale);
  *reinterpret_cast<uint4*>(p) = o;
}

// d_w: [B, n_upd, R] fp32 (n_upd = T - 1, or T when a later sequence shard continues the scan; only the first T - 1
// are used here); w_down: [R] bf16; w_init: [B, R] fp32 or null (start state from earlier shards, already scaled);
// states: [B, T, R] bf16
__global__ void __launch_bounds__(256) ttt_prefix_weights_kernel(const float* __restrict__ d_w, const bf16* __restrict__ w_down,
                                                                 const float* __restrict__ w_init, bf16* __restrict__ states,
                                                                 float lr, int B, int T, int64_t R, int n_upd) {
  const int64_t nvec = R / 8;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < nvec * B;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int b = static_cast<int>(idx / nvec);
    const int64_t e = (idx % nvec) * 8;
    float acc[8];
    {
      const uint4 raw = *reinterpret_cast<const uint4*>(w_down + e);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 t = unpack_bf16(w[i]);
        acc[2 * i] = t.x;
        acc[2 * i + 1] = t.y;
      }
    }
    if (w_init != nullptr) {
      float a[8];
      load8(w_init + static_cast<int64_t>(b) * R + e, a);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += a[i];
    }
    bf16* out = states + static_cast<int64_t>(b) * T * R + e;
    const float* in = d_w + static_cast<int64_t>(b) * n_upd * R + e;
    store8_bf16(out, acc, 1.f);
    for (int j = 0; j + 1 < T; ++j) {
      float d[8];
      load8(in + static_cast<int64_t>(j) * R, d);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = fmaf(lr, d[i], acc[i]);
      store8_bf16(out + static_cast<int64_t>(j + 1) * R, acc, 1.f);
    }
  }
}

// d_states: [B, T, R] fp32; g: [B, n_upd, R] bf16 (g_j = lr * (g_init + sum_{i>j} d_states_i)); d_w_down: [R] fp32
// (sum over b, i).  g_init: [B, R] fp32 or null: what later sequence shards hand back for this shard's summed update;
// n_upd = T - 1, or T when this shard's last chunk also updates (then g_{T-1} = lr * g_init).
__global__ void __launch_bounds__(256) ttt_suffix_grads_kernel(const float* __restrict__ d_states, bf16* __restrict__ g,
                                                               float* __restrict__ d_w_down, const float* __restrict__ g_init,
                                                               float lr, int B, int T, int64_t R, int n_upd) {
  const int64_t nvec = R / 8;
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec;
       v += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t e = v * 8;
    float total[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int b = 0; b < B; ++b) {
      const float* in = d_states + static_cast<int64_t>(b) * T * R + e;
      bf16* out = g + static_cast<int64_t>(b) * n_upd * R + e;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      float local[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (g_init != nullptr) load8(g_init + static_cast<int64_t>(b) * R + e, acc);
      if (n_upd == T) store8_bf16(out + static_cast<int64_t>(T - 1) * R, acc, lr);
      for (int i = T - 1; i >= 1; --i) {
        float d[8];
        load8(in + static_cast<int64_t>(i) * R, d);
#pragma unroll
        for (int k = 0; k < 8; ++k) { acc[k] += d[k]; local[k] += d[k]; }
        store8_bf16(out + static_cast<int64_t>(i - 1) * R, acc, lr);
      }
      float d0[8];
      load8(in, d0);
#pragma unroll
      for (int k = 0; k < 8; ++k) total[k] += local[k] + d0[k];
    }
    *reinterpret_cast<float4*>(d_w_down + e) = make_float4(total[0], total[1], total[2], total[3]);
    *reinterpret_cast<float4*>(d_w_down + e + 4) = make_float4(total[4], total[5], total[6], total[7]);
  }
}

}  // namespace ttcd

using namespace ttcd;

static unsigned ttt_grid(long long nvec) {
  const long long blocks = (nvec + 255) / 256;
  return static_cast<unsigned>(blocks < 1 ? 1 : (blocks > 148LL * 8 ? 148LL * 8 : blocks));
}

TTCD_EXPORT int ttcd_ttt_prefix_weights(const float* d_w, const void* w_down, const float* w_init, void* states, float lr,
                                        int B, int T, long long R, int n_upd, void* stream_ptr) {
  if (B <= 0 || T <= 0 || R <= 0 || R % 8 != 0 || (n_upd != T - 1 && n_upd != T)) return TTCD_ERR_ARG;
  ttt_prefix_weights_kernel<<<ttt_grid(R / 8 * B), 256, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      d_w, static_cast<const bf16*>(w_down), w_init, static_cast<bf16*>(states), lr, B, T, R, n_upd);
  return static_cast<int>(cudaGetLastError());
}

TTCD_EXPORT int ttcd_ttt_suffix_grads(const float* d_states, void* g, float* d_w_down, const float* g_init, float lr, int B,
                                      int T, long long R, int n_upd, void* stream_ptr) {
  if (B <= 0 || T <= 0 || R <= 0 || R % 8 != 0 || (n_upd != T - 1 && n_upd != T)) return TTCD_ERR_ARG;
  ttt_suffix_grads_kernel<<<ttt_grid(R / 8), 256, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      d_states, static_cast<bf16*>(g), d_w_down, g_init, lr, B, T, R, n_upd);
  return static_cast<int>(cudaGetLastError());
}
