// Mixture-of-experts routing in two launches (plus one for the backward pass).
//
//   gate_topk_kernel      one warp per token: (capped) router logits -> scores (softmax or
//                         sigmoid) -> the k best experts and their scores, the token's
//                         log-sum-exp (router z-loss) and per-CTA partial sums of the scores per
//                         expert (the "density proxy" of the load-balance loss);
//   gate_positions_kernel one CTA per routing group: for every (token, choice) its position in
//                         the chosen expert's capacity buffer, in the priority order of the
//                         reference -- every token's first choice in token order, then every
//                         second choice, ... -- with -1 beyond the capacity; also the number of
//                         tokens per (choice, expert) and the reduced score sums.  Positions come
//                         from a warp match (rank among the lanes with the same expert), a
//                         per-warp histogram and a scan over the warps, so they are exact and
//                         deterministic without sorting;
//   gate_bwd_kernel       one warp per token: gradient of the logits from the gradients of the
//                         k gathered scores, of the per-expert score sums and of the log-sum-exp.
//
// What it replaces in the reference: jax.lax.top_k, one-hot + cumsum positions and the aux-loss
// reductions of axlearn/common/mixture_of_experts.py:461-724 (Top2Gating), :727-1098
// (TopKGating), :791-804, :966-1008; they lower to a chain of XLA sort / scan / reduce fusions.
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace axb {

constexpr int kGateMaxPerLane = 8;    // experts per lane: E <= 256
constexpr int kGateMaxK = 8;
constexpr int kGateWarps = 8;         // warps (tokens in flight) per CTA of the per-token kernels
constexpr int kPosThreads = 1024;
constexpr int kPosWarps = kPosThreads / 32;

struct GateParams {
  const float* logits;  // [G, S, E]
  int G, S, E, K;
  float cap;            // tanh logit cap, 0 = none
  int sigmoid;          // score function: 0 softmax, 1 sigmoid
};

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Loads one token's (capped) logits into lane-strided registers and returns max and sum-exp.
__device__ __forceinline__ void load_token(const float* row, int E, float cap, int lane, float (&x)[kGateMaxPerLane],
                                           float& mx, float& lse) {
  mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < kGateMaxPerLane; ++i) {
    const int e = lane + 32 * i;
    float v = -INFINITY;
    if (e < E) {
      v = row[e];
      if (cap > 0.f) v = cap * tanhf(v / cap);
    }
    x[i] = v;
    mx = fmaxf(mx, v);
  }
  mx = warp_max(mx);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < kGateMaxPerLane; ++i) s += (lane + 32 * i < E) ? expf(x[i] - mx) : 0.f;
  lse = mx + logf(warp_sum(s));
}

__global__ void __launch_bounds__(kGateWarps * 32)
gate_topk_kernel(GateParams p, int* __restrict__ index, float* __restrict__ gate, float* __restrict__ lse_out,
                 float* __restrict__ proxy_part, int tokens_per_cta) {
  __shared__ float red[kGateWarps][kGateMaxPerLane * 32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = blockIdx.y;
  const int s_lo = blockIdx.x * tokens_per_cta, s_hi = min(p.S, s_lo + tokens_per_cta);
  float acc[kGateMaxPerLane];
#pragma unroll
  for (int i = 0; i < kGateMaxPerLane; ++i) acc[i] = 0.f;
  for (int s = s_lo + warp; s < s_hi; s += kGateWarps) {
    const int64_t tok = static_cast<int64_t>(g) * p.S + s;
    float x[kGateMaxPerLane], mx, lse;
    load_token(p.logits + tok * p.E, p.E, p.cap, lane, x, mx, lse);
    float score[kGateMaxPerLane];
#pragma unroll
    for (int i = 0; i < kGateMaxPerLane; ++i) {
      const bool on = lane + 32 * i < p.E;
      score[i] = !on ? -INFINITY : (p.sigmoid ? 1.f / (1.f + expf(-x[i])) : expf(x[i] - lse));
      acc[i] += on ? score[i] : 0.f;
    }
    if (lane == 0) lse_out[tok] = lse;
    // k rounds of warp arg-max; ties go to the smaller expert id (as a stable top-k does).
    for (int j = 0; j < p.K; ++j) {
      float best = -INFINITY;
      int best_e = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < kGateMaxPerLane; ++i) {
        const int e = lane + 32 * i;
        if (score[i] > best) best = score[i], best_e = e;  // ascending e within a lane: first wins
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
        if (ob > best || (ob == best && oe < best_e)) best = ob, best_e = oe;
      }
      if (lane == 0) {
        index[tok * p.K + j] = best_e;
        gate[tok * p.K + j] = best;
      }
#pragma unroll
      for (int i = 0; i < kGateMaxPerLane; ++i)
        if (lane + 32 * i == best_e) score[i] = -INFINITY;  // taken
    }
  }
  // Per-CTA partial sums of the scores, reduced over the warps in a fixed order.
#pragma unroll
  for (int i = 0; i < kGateMaxPerLane; ++i) red[warp][lane + 32 * i] = acc[i];
  __syncthreads();
  for (int e = threadIdx.x; e < p.E; e += blockDim.x) {
    float t = 0.f;
    for (int w = 0; w < kGateWarps; ++w) t += red[w][e];
    proxy_part[(static_cast<int64_t>(g) * gridDim.x + blockIdx.x) * p.E + e] = t;
  }
}

__global__ void __launch_bounds__(kPosThreads)
gate_positions_kernel(const int* __restrict__ index, int* __restrict__ slot, int* __restrict__ counts,
                      const float* __restrict__ proxy_part, float* __restrict__ proxy, int S, int E, int K,
                      int capacity, int parts) {
  extern __shared__ int sm[];
  int* hist = sm;                      // [kPosWarps][E] per-warp counts of the current chunk
  int* run = sm + kPosWarps * E;       // [E] tokens already placed in each expert
  const int g = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    run[e] = 0;
    float t = 0.f;
    for (int c = 0; c < parts; ++c) t += proxy_part[(static_cast<int64_t>(g) * parts + c) * E + e];
    proxy[static_cast<int64_t>(g) * E + e] = t;
  }
  __syncthreads();
  for (int j = 0; j < K; ++j) {
    int before = 0;  // value of run[e] at the start of this choice, to report counts[j][e]
    if (threadIdx.x < E) before = run[threadIdx.x];
    for (int s0 = 0; s0 < S; s0 += kPosThreads) {
      for (int i = threadIdx.x; i < kPosWarps * E; i += blockDim.x) hist[i] = 0;
      __syncthreads();
      const int s = s0 + threadIdx.x;
      const bool live = s < S;
      const int64_t at = (static_cast<int64_t>(g) * S + s) * K + j;
      const int e = live ? index[at] : -1 - lane;  // dead lanes match nobody
      const unsigned peers = __match_any_sync(0xffffffffu, e);
      const int rank = __popc(peers & ((1u << lane) - 1u));
      if (live && rank == 0) hist[warp * E + e] = __popc(peers);
      __syncthreads();
      // Exclusive scan over the warps, one expert per thread; leaves the chunk total in run[].
      if (threadIdx.x < E) {
        int t = run[threadIdx.x];
        for (int w = 0; w < kPosWarps; ++w) {
          const int c = hist[w * E + threadIdx.x];
          hist[w * E + threadIdx.x] = t;
          t += c;
        }
        run[threadIdx.x] = t;
      }
      __syncthreads();
      if (live) {
        const int pos = hist[warp * E + e] + rank;
        slot[at] = pos < capacity ? pos : -1;
      }
      __syncthreads();
    }
    if (threadIdx.x < E) counts[(static_cast<int64_t>(g) * K + j) * E + threadIdx.x] = run[threadIdx.x] - before;
  }
}

__global__ void __launch_bounds__(kGateWarps * 32)
gate_bwd_kernel(GateParams p, const int* __restrict__ index, const float* __restrict__ lse_in,
                const float* __restrict__ d_gate, const float* __restrict__ d_proxy, const float* __restrict__ d_lse,
                float* __restrict__ d_logits) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t total = static_cast<int64_t>(p.G) * p.S;
  for (int64_t tok = blockIdx.x * static_cast<int64_t>(kGateWarps) + warp; tok < total;
       tok += static_cast<int64_t>(gridDim.x) * kGateWarps) {
    const int g = static_cast<int>(tok / p.S);
    const float* row = p.logits + tok * p.E;
    const float lse = lse_in[tok];
    float raw[kGateMaxPerLane], x[kGateMaxPerLane], soft[kGateMaxPerLane], dscore[kGateMaxPerLane];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < kGateMaxPerLane; ++i) {
      const int e = lane + 32 * i;
      const bool on = e < p.E;
      raw[i] = on ? row[e] : 0.f;
      x[i] = (p.cap > 0.f) ? p.cap * tanhf(raw[i] / p.cap) : raw[i];
      soft[i] = on ? expf(x[i] - lse) : 0.f;
      float d = (on && d_proxy != nullptr) ? d_proxy[static_cast<int64_t>(g) * p.E + e] : 0.f;
      for (int j = 0; j < p.K; ++j)
        if (on && index[tok * p.K + j] == e) d += d_gate[tok * p.K + j];
      dscore[i] = d;
      dot += soft[i] * d;
    }
    dot = warp_sum(dot);
    const float dl = d_lse != nullptr ? d_lse[tok] : 0.f;
#pragma unroll
    for (int i = 0; i < kGateMaxPerLane; ++i) {
      const int e = lane + 32 * i;
      if (e >= p.E) continue;
      float dx;
      if (p.sigmoid) {
        const float sg = 1.f / (1.f + expf(-x[i]));
        dx = dscore[i] * sg * (1.f - sg) + dl * soft[i];
      } else {
        dx = soft[i] * (dscore[i] - dot) + dl * soft[i];
      }
      if (p.cap > 0.f) {
        const float th = x[i] / p.cap;
        dx *= 1.f - th * th;
      }
      d_logits[tok * p.E + e] = dx;
    }
  }
}

}  // namespace axb

// Number of per-CTA partial rows `proxy_part` must hold per group.
extern "C" int axb_moe_gate_parts(int S) {
  const int per_cta = 256;
  return (S + per_cta - 1) / per_cta;
}

// logits [G, S, E] fp32 -> index / gate / slot [G, S, K], counts [G, K, E], proxy [G, E], lse [G, S];
// proxy_part: scratch [G, axb_moe_gate_parts(S), E] floats.  E <= 256, K <= 8, K <= E.
extern "C" int axb_moe_gate_fwd(const float* logits, int* index, float* gate, int* slot, int* counts, float* proxy,
                                float* lse, float* proxy_part, int G, int S, int E, int K, int capacity,
                                float logit_cap, int sigmoid, cudaStream_t stream) {
  using namespace axb;
  if (E < 1 || E > 32 * kGateMaxPerLane || K < 1 || K > kGateMaxK || K > E || G < 1 || S < 1) return -10;
  GateParams p{logits, G, S, E, K, logit_cap, sigmoid};
  const int per_cta = 256;
  const int parts = (S + per_cta - 1) / per_cta;
  dim3 grid(parts, G);
  gate_topk_kernel<<<grid, kGateWarps * 32, 0, stream>>>(p, index, gate, lse, proxy_part, per_cta);
  const size_t smem = (static_cast<size_t>(kPosWarps) * E + E) * sizeof(int);
  gate_positions_kernel<<<G, kPosThreads, smem, stream>>>(index, slot, counts, proxy_part, proxy, S, E, K, capacity,
                                                          parts);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// d_logits [G, S, E] from d_gate [G, S, K], d_proxy [G, E] (may be null), d_lse [G, S] (may be null).
extern "C" int axb_moe_gate_bwd(const float* logits, const int* index, const float* lse, const float* d_gate,
                                const float* d_proxy, const float* d_lse, float* d_logits, int G, int S, int E, int K,
                                float logit_cap, int sigmoid, cudaStream_t stream) {
  using namespace axb;
  if (E < 1 || E > 32 * kGateMaxPerLane || K < 1 || K > kGateMaxK) return -10;
  GateParams p{logits, G, S, E, K, logit_cap, sigmoid};
  const int64_t total = static_cast<int64_t>(G) * S;
  int blocks = static_cast<int>((total + kGateWarps - 1) / kGateWarps);
  if (blocks > 148 * 8) blocks = 148 * 8;
  gate_bwd_kernel<<<blocks, kGateWarps * 32, 0, stream>>>(p, index, lse, d_gate, d_proxy, d_lse, d_logits);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
