// Flash attention forward, third generation.
//
// Same data flow as flash_fwd_v2.cu (two 128-row query tiles per CTA, scores and probabilities
// in tensor memory, P*V and the next Q*K^T of one tile running while the other tile's softmax
// works), with two changes:
//   * every 128-row tile has EIGHT softmax warps instead of four: the two warps that share a
//     TMEM lane quarter split the 128 score columns in halves, exchange their row maxima and
//     row sums through shared memory and a 64-thread named barrier.  A warp's instruction
//     stream per key tile is half as long, and each SM sub-partition always has two softmax
//     warps of the active tile to interleave, which is what hides the latency between
//     tcgen05.ld, the max/exp chain and tcgen05.st;
//   * masking beyond "causal": segment ids (packed sequences), a sliding window and a tanh
//     logit cap are applied inside the kernel, and key tiles that no row of a query tile can
//     see (left of the window, other segments) are skipped on both sides of the range.
//
// Per CTA (640 threads): warp 0 TMA producer, warp 1 MMA issuer (warps 2-3 idle: they keep the
// softmax warps aligned to warpgroups), warps 4..11 softmax of tile A, warps 12..19 of tile B.  TMEM (512 columns): S_A/P_A 0..127, S_B/P_B 128..255,
// O_A 256.., O_B 384...  P (bf16 pairs): keys 0-63 overlay score columns 0-31, keys 64-127
// score columns 64-95 (each softmax warp writes over columns it read itself).
//
// Reference kernels being replaced: axlearn/common/flash_attention/gpu_attention.py:114-243
// (segment ids :179-205, block skipping by mask_fn) and the cuDNN call at :792-926.
#include <stdlib.h>

#include "host_utils.cuh"
#include "sm100.cuh"

namespace axb {

int make_bthd_map(CUtensorMap* map, const void* base, int B, int L, int N, int H, int box_rows);

constexpr int kF3Threads = 640;
// 640 threads launch with 96 registers each.  The first warpgroup (producer, MMA issuer, two idle
// warps) gives registers back and the sixteen softmax warps take them, so that a softmax thread
// can hold all 64 scores of its half row at once: both tensor-memory loads of a key tile are in
// flight together, and the exponentials are computed from registers instead of a second load.
constexpr int kF3LaunchRegs = 96, kF3LightRegs = 64, kF3SoftmaxRegs = 104;
static_assert(128 * kF3LightRegs + 512 * kF3SoftmaxRegs <= kF3Threads * kF3LaunchRegs,
              "setmaxnreg split exceeds the launch allocation");
constexpr uint32_t kGaveUp = 0x7fc0dead;  // NaN payload: "my wait on the score tile timed out"

struct FlashFwd3Params {
  void* out;
  float* lse;
  const int* q_seg;    // [B, T] or null
  const int* k_seg;    // [B, S] or null
  const int2* ranges;  // [B, ceil(T/128)]: key tiles [x, y) that share a segment id with the query tile
  int B, T, S, N, Nkv, H;
  float sc;            // multiplier applied to a (transformed) score before exp2
  float cap_in;        // softmax_scale / cap          (logit cap: z = s * cap_in)
  float cap_out;       // cap * log2(e); 0 = no cap    (score in log2 units = tanh(z) * cap_out)
  int causal, q_offset, window;  // window < 0: none; else keys older than row_pos - window are hidden
  int* status;
};

template <int H>
struct F3Smem {
  static constexpr int kSub = 16384;
  static constexpr int kTile = (H / 64) * kSub;
  static constexpr int kQ = 0;                  // two tiles
  static constexpr int kK = kQ + 2 * kTile;     // two stages
  static constexpr int kV = kK + 2 * kTile;     // two stages
  static constexpr int kMax = kV + 2 * kTile;   // float [2 parity][2 tiles][2 halves][128]
  static constexpr int kSum = kMax + 4096;      // float [2 tiles][2 halves][128]
  static constexpr int kBar = kSum + 2048;
  static constexpr int kTotal = kBar + 256 + 1024;
};

__device__ __forceinline__ void pair_barrier(int id) {
  asm volatile("bar.sync %0, 64;" ::"r"(id) : "memory");
}

__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Two-wide fp32 arithmetic (one issue slot for two lanes of work on the FMA pipe).
__device__ __forceinline__ uint64_t f32x2(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void f32x2_split(uint64_t v, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// e[u] = 2^(s[u] * sc - m) for eight scores; the scaling runs two values per instruction.
//
// Evaluating a share of the exponentials with a polynomial on the FMA pipe (round-to-nearest
// split, degree-3 minimax, exponent add; two-wide FMAs, about 5.5 issue slots per value) was
// measured on B200 at 25 % / 37 % / 50 % of the values: 886 / 836 / 831 TFLOP/s against 910 with
// the exponential unit alone (b4, T 4096, 32 heads, d 128).  The softmax warps are short of issue
// slots and latency, not of exponential throughput, so every exponential stays on the unit.
__device__ __forceinline__ void exp2_batch8(const uint32_t* s, uint64_t sc2, uint64_t nm2, float (&e)[8]) {
  float a[8];
#pragma unroll
  for (int u = 0; u < 8; u += 2)
    f32x2_split(fma2(f32x2(__uint_as_float(s[u]), __uint_as_float(s[u + 1])), sc2, nm2), a[u], a[u + 1]);
#pragma unroll
  for (int u = 0; u < 8; ++u) e[u] = ex2_approx(a[u]);
}

// kGeneral: segment ids / sliding window / logit cap are honoured (every tile takes the masking
// path when segment ids are present).  The plain instantiation only masks diagonal and ragged
// tiles.
template <int H, bool kGeneral>
__global__ void __launch_bounds__(kF3Threads, 1)
flash_fwd3_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                  const __grid_constant__ CUtensorMap tmap_v, FlashFwd3Params p) {
  using L = F3Smem<H>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBar);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* it_done = bars + 3;   // [2]: MMA iteration g (ring index) releases V stage g & 1 and
                                  //      K stage (g + 1) & 1 with ONE commit on it_done[g & 1];
                                  //      the prologue counts as iteration -1
  uint64_t* v_full = bars + 5;    // [2]
  uint64_t* s_full = bars + 9;    // [2] per query tile
  uint64_t* p_full = bars + 11;   // [2] per query tile, 8 arrivals
  uint64_t* pv_done = bars + 13;  // [2] per query tile, completes once
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  float* ex_max = reinterpret_cast<float*>(smem + L::kMax);
  float* ex_sum = reinterpret_cast<float*>(smem + L::kSum);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pair = gridDim.x - 1 - blockIdx.x;  // heavy (late) query tiles first
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / (p.N / p.Nkv);
  const int t0 = pair * 256;
  const int n_qt = (p.T + 127) / 128;

  // Key tiles [lo, hi) each query tile needs.
  int lo[2], hi[2];
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    const int tx = t0 + x * 128;
    int l = 0, h = 0;
    if (tx < p.T) {
      int kv_len = p.S;
      if (p.causal) kv_len = min(p.S, tx + 128 + p.q_offset);
      h = kv_len > 0 ? (kv_len + 127) / 128 : 0;
      if (kGeneral) {
        if (p.window >= 0) l = max(0, tx + p.q_offset - p.window) / 128;
        if (p.ranges != nullptr) {
          const int2 r = p.ranges[batch * n_qt + pair * 2 + x];
          l = max(l, r.x);
          h = min(h, r.y);
        }
      }
      if (l >= h) l = h = 0;
    }
    lo[x] = l, hi[x] = h;
  }
  const bool act0 = hi[0] > lo[0], act1 = hi[1] > lo[1];
  const int g_lo = act0 ? (act1 ? min(lo[0], lo[1]) : lo[0]) : lo[1];
  const int g_hi = max(hi[0], hi[1]);
  const bool any = act0 || act1;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&it_done[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 8);
      mbar_init(&pv_done[i], 1);
    }
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 4) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");  // kF3LightRegs
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one() && any) {
      mbar_arrive_expect_tx(q_full, 2 * L::kTile);
#pragma unroll
      for (int x = 0; x < 2; ++x)
#pragma unroll
        for (int j = 0; j < H / 64; ++j)
          tma_load_4d(smem + L::kQ + x * L::kTile + j * L::kSub, &tmap_q, q_full, j * 64, head,
                      t0 + x * 128, batch);
      for (int it = g_lo; it < g_hi; ++it) {
        const int g = it - g_lo;
        const int st = g & 1;
        // K(g) reuses the stage of K(g - 2), last read by the scores issued in iteration g - 3;
        // V(g) reuses the stage of V(g - 2), last read in iteration g - 2.  Completion number k
        // of it_done[1] belongs to iteration 2k - 1, of it_done[0] to iteration 2k.
        if (g >= 2) {
          const int k_need = (g & 1) ? (g - 3) / 2 : (g - 2) / 2;
          if (!mbar_wait(&it_done[(g + 1) & 1], k_need & 1, p.status, kStatusWaitTimeoutProducer)) break;
        }
        mbar_arrive_expect_tx(&k_full[st], L::kTile);
#pragma unroll
        for (int j = 0; j < H / 64; ++j)
          tma_load_4d(smem + L::kK + st * L::kTile + j * L::kSub, &tmap_k, &k_full[st], j * 64, kv_head,
                      it * 128, batch);
        if (g >= 2) {
          const int v_need = (g & 1) ? (g - 1) / 2 : (g - 2) / 2;
          if (!mbar_wait(&it_done[g & 1], v_need & 1, p.status, kStatusWaitTimeoutProducer)) break;
        }
        mbar_arrive_expect_tx(&v_full[st], L::kTile);
#pragma unroll
        for (int j = 0; j < H / 64; ++j)
          tma_load_4d(smem + L::kV + st * L::kTile + j * L::kSub, &tmap_v, &v_full[st], j * 64, kv_head,
                      it * 128, batch);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one() && any) {
      constexpr uint32_t idesc_qk = umma_idesc_f16(128, 128, 1, 1, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_f16(128, H, 1, 1, 0, 1);
      bool ok = mbar_wait(q_full, 0, p.status, kStatusWaitTimeoutMma);
      // Descriptors are assembled from a per-operand low word plus an immediate: the high word
      // (stride between 8-row groups, version, swizzle mode) is the same constant for every
      // operand, so the issuer keeps a handful of registers instead of one 64-bit value per MMA.
      constexpr uint32_t kDescHi = ((1024u >> 4) & 0x3FFF) | (1u << 14) | (2u << 29);
      auto desc_lo = [](uint32_t addr, uint32_t lbo) { return ((addr >> 4) & 0x3FFFu) | (((lbo >> 4) & 0x3FFFu) << 16); };
      auto desc = [](uint32_t lo) {
        uint64_t d;
        asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(kDescHi));
        return d;
      };
      auto issue_qk = [&](int x, int st) {
        const uint32_t q_lo = desc_lo(smem_u32(smem + L::kQ + x * L::kTile), 16);
        const uint32_t k_lo = desc_lo(smem_u32(smem + L::kK + st * L::kTile), 16);
#pragma unroll
        for (int kk = 0; kk < H / 16; ++kk) {
          const uint32_t off = ((kk >> 2) * L::kSub + (kk & 3) * 32) >> 4;
          tc_mma_f16(tmem_base + x * 128, desc(q_lo + off), desc(k_lo + off), idesc_qk, kk > 0 ? 1u : 0u);
        }
        tc_commit(&s_full[x]);
      };
      auto issue_pv = [&](int x, int st, bool first) {
        const uint32_t v_lo = desc_lo(smem_u32(smem + L::kV + st * L::kTile), L::kSub);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          // 16 keys per step: 8 TMEM columns of packed bf16 pairs; 16 V rows = 2048 B.
          // keys 0-63 (first half's probabilities) at columns 0-31, keys 64-127 at columns 64-95
          tc_mma_f16_ts(tmem_base + 256 + x * 128, tmem_base + x * 128 + (kk >> 2) * 64 + (kk & 3) * 8,
                        desc(v_lo + ((kk * 2048) >> 4)), idesc_pv, (!first || kk > 0) ? 1u : 0u);
        }
      };
      // Prologue: scores of the first key tile for the query tiles that start there.
      if (ok) ok = mbar_wait(&k_full[0], 0, p.status, kStatusWaitTimeoutMma);
      if (ok) {
        tc_fence_after_sync();
        for (int x = 0; x < 2; ++x)
          if (hi[x] > lo[x] && lo[x] == g_lo) issue_qk(x, 0);
        tc_commit(&it_done[1]);
      }
      for (int it = g_lo; it < g_hi && ok; ++it) {
        const int g = it - g_lo;
        const int st = g & 1;
        const uint32_t ph = (g >> 1) & 1;
        const bool has_next = it + 1 < g_hi;
        if (!mbar_wait(&v_full[st], ph, p.status, kStatusWaitTimeoutMma)) break;
        if (has_next) {
          if (!mbar_wait(&k_full[st ^ 1], ((g + 1) >> 1) & 1, p.status, kStatusWaitTimeoutMma)) break;
        }
        tc_fence_after_sync();
        for (int x = 0; x < 2 && ok; ++x) {
          if (it >= lo[x] && it < hi[x]) {
            if (!mbar_wait(&p_full[x], (it - lo[x]) & 1, p.status, kStatusWaitTimeoutMma)) {
              ok = false;
              break;
            }
            tc_fence_after_sync();
            issue_pv(x, st, it == lo[x]);
            if (it + 1 < hi[x]) issue_qk(x, st ^ 1);
            else tc_commit(&pv_done[x]);
          } else if (it + 1 == lo[x] && it + 1 < hi[x]) {
            issue_qk(x, st ^ 1);  // first score tile of a query tile that starts later
          }
        }
        if (!ok) break;
        tc_commit(&it_done[st]);
      }
    }
  }
  } else {
    // ------------------------------------------------------------------ softmax / epilogue
    asm volatile("setmaxnreg.inc.sync.aligned.u32 104;");  // kF3SoftmaxRegs
    const int idx = warp - 4;
    const int x = idx >> 3;               // query tile
    const int half = (idx >> 2) & 1;      // which 64 score columns / which half of the O columns
    const int quarter = warp & 3;         // TMEM lane quarter accessible to this warp
    const int r_in = quarter * 32 + lane;
    const int row = t0 + x * 128 + r_in;
    const int row_pos = row + p.q_offset;
    const int bar_id = 1 + x * 4 + quarter;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_base + x * 128 + half * 64;
    const uint32_t p_addr = tmem_base + lane_base + x * 128 + half * 64;  // P pairs over the own scores
    const uint32_t o_addr = tmem_base + lane_base + 256 + x * 128 + half * (H / 2);
    float* my_max = ex_max + (x * 2 + half) * 128 + r_in;
    float* other_max = ex_max + (x * 2 + (half ^ 1)) * 128 + r_in;
    const int my_lo = lo[x], my_hi = hi[x];
    // Visible key range of this row (general mode) and its segment id.
    int c_lo = 0, c_hi = p.S - 1, seg = 0;
    if (p.causal) c_hi = min(c_hi, row_pos);
    const int* kseg_row = nullptr;
    if (kGeneral) {
      if (p.window >= 0) c_lo = max(0, row_pos - p.window);
      if (p.q_seg != nullptr) {
        seg = row < p.T ? p.q_seg[static_cast<int64_t>(batch) * p.T + row] : -1;
        kseg_row = p.k_seg + static_cast<int64_t>(batch) * p.S;
      }
    }
    const uint32_t c_span = static_cast<uint32_t>(c_hi - c_lo);
    float m_ref = -INFINITY, l_sum = 0.f;
    bool ok = true;
    for (int it = my_lo; it < my_hi && ok; ++it) {
      const int kpar = (it - my_lo) & 1;
      // A wait that gives up must not leave the partner warp alone at the named barrier: both
      // halves always reach it, and a failed wait travels through the exchange slot.
      const bool got = mbar_wait_warp(&s_full[x], kpar, p.status, kStatusWaitTimeoutEpilogue);
      const int s0 = it * 128 + half * 64;  // first key column of this thread
      // All 64 scores of this thread's half row are loaded at once (two loads in flight, one
      // wait) and stay in registers for both passes.  Masks and the logit cap are applied once.
      uint32_t r0[32], r1[32];
      auto mask_scores = [&](int hh, uint32_t (&r)[32]) {
        const int c0 = s0 + hh * 32;
        const uint32_t ninf = __float_as_uint(-INFINITY);
        if (kGeneral) {
          if (p.cap_out != 0.f) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              r[j] = __float_as_uint(tanh_approx(__uint_as_float(r[j]) * p.cap_in) * p.cap_out);
          }
          if ((c0 < c_lo) || (c0 + 31 > c_hi)) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (static_cast<uint32_t>(c0 + j - c_lo) > c_span || c_hi < c_lo) r[j] = ninf;
          }
          if (kseg_row != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int c = c0 + j;
              const int ks = c < p.S ? __ldg(kseg_row + c) : -2;
              if (ks != seg) r[j] = ninf;
            }
          }
        } else {
          const int tile_t0 = t0 + x * 128;
          if ((p.causal && c0 + 31 > tile_t0 + p.q_offset) || (c0 + 32 > p.S)) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (c0 + j > c_hi) r[j] = ninf;
          }
        }
      };
      auto row_max = [&](const uint32_t (&r)[32]) {
        // Four independent chains of three-input maxima.
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          mx0 = max3(mx0, __uint_as_float(r[j]), __uint_as_float(r[j + 1]));
          mx1 = max3(mx1, __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
          mx2 = max3(mx2, __uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
          mx3 = max3(mx3, __uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
        }
        return fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      };
      float tmax = -INFINITY;
      if (got) {
        tc_fence_after_sync();
        tmem_ld_32x32(s_addr, r0);
        tmem_ld_32x32(s_addr + 32, r1);
        tmem_ld_wait();
        mask_scores(0, r0);
        mask_scores(1, r1);
        tmax = fmaxf(row_max(r0), row_max(r1));
      }
      my_max[kpar * 512] = got ? tmax : __uint_as_float(kGaveUp);
      pair_barrier(bar_id);
      const float other = other_max[kpar * 512];
      if (!got || __any_sync(0xffffffffu, __float_as_uint(other) == kGaveUp)) {
        ok = false;
        break;
      }
      tmax = fmaxf(tmax, other) * p.sc;  // sc > 0, so max commutes with scaling
      float alpha = 1.f;
      bool rescale = false;
      if (tmax > m_ref + 8.f) {
        if (m_ref != -INFINITY) {
          alpha = exp2f(m_ref - tmax);
          rescale = true;
        }
        m_ref = tmax;
      }
      if (__any_sync(0xffffffffu, rescale)) {
        // s_full of this tile was committed after the previous P*V of this query tile, so O is
        // quiescent; each half rescales its own O columns.
#pragma unroll 1
        for (int c = 0; c < H / 2; c += 16) {  // 16 columns at a time: the 64 scores stay in registers
          uint32_t o[16];
          tmem_ld_32x16(o_addr + c, o);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
          tmem_st_32x16(o_addr + c, o);
        }
        l_sum *= alpha;
      }
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
      // Probabilities rounded to bf16, packed two per register, 32 columns (16 registers) at a
      // time; each chunk travels to tensor memory while the next one is computed.  This thread's
      // probabilities overlay the first 32 columns of its OWN 64 score columns (the chunk being
      // written was consumed just before, the other chunk lies beyond), so the two halves of a
      // row never touch each other's columns.
      const uint64_t sc2 = f32x2(p.sc, p.sc), nm2 = f32x2(-m_use, -m_use);
      uint64_t acc0 = f32x2(0.f, 0.f), acc1 = acc0;   // row sums, two lanes each
      auto write_probs = [&](int hh, const uint32_t (&r)[32]) {
        uint32_t q[16];
#pragma unroll
        for (int j0 = 0; j0 < 32; j0 += 8) {
          float e[8];
          exp2_batch8(r + j0, sc2, nm2, e);
#pragma unroll
          for (int u = 0; u < 4; ++u) q[(j0 >> 1) + u] = pack_bf16x2(e[2 * u], e[2 * u + 1]);
          acc0 = add2(acc0, add2(f32x2(e[0], e[1]), f32x2(e[2], e[3])));
          acc1 = add2(acc1, add2(f32x2(e[4], e[5]), f32x2(e[6], e[7])));
        }
        tmem_st_32x16(p_addr + hh * 16, q);
      };
      write_probs(0, r0);
      write_probs(1, r1);
      float l0, l1, l2, l3;
      f32x2_split(acc0, l0, l1);
      f32x2_split(acc1, l2, l3);
      l0 += l2;
      l1 += l3;
      l_sum += l0 + l1;
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[x]);
    }
    const int nt = my_hi - my_lo;
    if (ok && nt > 0) {
      ok = mbar_wait_warp(&pv_done[x], 0, p.status, kStatusWaitTimeoutEpilogue);
      tc_fence_after_sync();
    }
    // Total row sum = the two halves' partial sums.
    ex_sum[(x * 2 + half) * 128 + r_in] = l_sum;
    pair_barrier(bar_id);
    l_sum += ex_sum[(x * 2 + (half ^ 1)) * 128 + r_in];
    if (ok && row < p.T) {
      __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) +
                            ((static_cast<int64_t>(batch) * p.T + row) * p.N + head) * H + half * (H / 2);
      if (half == 0) {
        p.lse[(static_cast<int64_t>(batch) * p.N + head) * p.T + row] =
            (l_sum > 0.f) ? (m_ref * 0.6931471805599453f + logf(l_sum)) : -INFINITY;
      }
      if (nt == 0) {
        for (int c = 0; c < H / 2; c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(0, 0, 0, 0);
      }
    }
    if (ok && nt > 0) {
      const float inv_l = l_sum > 0.f ? 1.f / l_sum : 0.f;
      __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) +
                            ((static_cast<int64_t>(batch) * p.T + row) * p.N + head) * H + half * (H / 2);
#pragma unroll 1
      for (int c = 0; c < H / 2; c += 32) {
        uint32_t o[32];
        tmem_ld_32x32(o_addr + c, o);
        tmem_ld_wait();
        if (row < p.T) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(o[8 * g + 0]) * inv_l, __uint_as_float(o[8 * g + 1]) * inv_l);
            v.y = pack_bf16x2(__uint_as_float(o[8 * g + 2]) * inv_l, __uint_as_float(o[8 * g + 3]) * inv_l);
            v.z = pack_bf16x2(__uint_as_float(o[8 * g + 4]) * inv_l, __uint_as_float(o[8 * g + 5]) * inv_l);
            v.w = pack_bf16x2(__uint_as_float(o[8 * g + 6]) * inv_l, __uint_as_float(o[8 * g + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + c + 8 * g) = v;
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    if (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) {
      for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// For every (batch, 128-row query tile): the range [x, y) of 128-key tiles that contain at least
// one key whose segment id lies within [min, max] of the query tile's ids.  One CTA per batch
// row; key-tile minima / maxima are staged in shared memory (up to 2048 tiles = 256K keys).
__global__ void seg_tile_ranges_kernel(const int* __restrict__ q_seg, const int* __restrict__ k_seg, int2* ranges,
                                       int T, int S) {
  __shared__ int kmin[2048], kmax[2048];
  const int b = blockIdx.x;
  const int n_kt = (S + 127) / 128, n_qt = (T + 127) / 128;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
  for (int t = warp; t < n_kt; t += n_warps) {
    int mn = INT_MAX, mx = INT_MIN;
    for (int i = lane; i < 128; i += 32) {
      const int c = t * 128 + i;
      if (c < S) {
        const int v = k_seg[static_cast<int64_t>(b) * S + c];
        mn = min(mn, v), mx = max(mx, v);
      }
    }
    for (int off = 16; off > 0; off >>= 1) {
      mn = min(mn, __shfl_xor_sync(0xffffffffu, mn, off));
      mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    }
    if (lane == 0) kmin[t] = mn, kmax[t] = mx;
  }
  __syncthreads();
  for (int t = warp; t < n_qt; t += n_warps) {
    int mn = INT_MAX, mx = INT_MIN;
    for (int i = lane; i < 128; i += 32) {
      const int r = t * 128 + i;
      if (r < T) {
        const int v = q_seg[static_cast<int64_t>(b) * T + r];
        mn = min(mn, v), mx = max(mx, v);
      }
    }
    for (int off = 16; off > 0; off >>= 1) {
      mn = min(mn, __shfl_xor_sync(0xffffffffu, mn, off));
      mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    }
    int first = INT_MAX, last = -1;
    for (int kt = lane; kt < n_kt; kt += 32) {
      if (kmax[kt] >= mn && kmin[kt] <= mx) first = min(first, kt), last = max(last, kt);
    }
    for (int off = 16; off > 0; off >>= 1) {
      first = min(first, __shfl_xor_sync(0xffffffffu, first, off));
      last = max(last, __shfl_xor_sync(0xffffffffu, last, off));
    }
    if (lane == 0) ranges[b * n_qt + t] = last >= 0 ? make_int2(first, last + 1) : make_int2(0, 0);
  }
}

template <int H, bool kGeneral>
static int launch_flash_fwd3(const void* q, const void* k, const void* v, FlashFwd3Params p, cudaStream_t stream) {
  CUtensorMap tq, tk, tv;
  if (make_bthd_map(&tq, q, p.B, p.T, p.N, H, 128)) return -2;
  if (make_bthd_map(&tk, k, p.B, p.S, p.Nkv, H, 128)) return -2;
  if (make_bthd_map(&tv, v, p.B, p.S, p.Nkv, H, 128)) return -2;
  auto kernel = flash_fwd3_kernel<H, kGeneral>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F3Smem<H>::kTotal) != cudaSuccess)
      return -3;
    // The in-kernel register redistribution only balances if the launch allocates exactly the
    // assumed count per thread; refuse to launch a build for which it does not.
    cudaFuncAttributes attr;
    if (cudaFuncGetAttributes(&attr, kernel) != cudaSuccess) return -3;
    if (attr.numRegs != kF3LaunchRegs) {
      fprintf(stderr, "axb flash fwd: built with %d registers per thread, the kernel assumes %d\n", attr.numRegs,
              kF3LaunchRegs);
      return -5;
    }
    configured = true;
  }
  dim3 grid((p.T + 255) / 256, p.N, p.B);
  kernel<<<grid, kF3Threads, F3Smem<H>::kTotal, stream>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace axb

// Writes, for every batch row and 128-row query tile, the range of 128-key tiles that can hold a
// key of one of the tile's segments (see seg_tile_ranges_kernel).  ranges: int32 [B, ceil(T/128), 2].
extern "C" int axb_seg_tile_ranges(const int* q_seg, const int* k_seg, int* ranges, int B, int T, int S,
                                   cudaStream_t stream) {
  if ((S + 127) / 128 > 2048) return -10;
  axb::seg_tile_ranges_kernel<<<B, 256, 0, stream>>>(q_seg, k_seg, reinterpret_cast<int2*>(ranges), T, S);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// q: [B, T, N, H], k/v: [B, S, Nkv, H], out: [B, T, N, H] (bf16, contiguous); lse: [B, N, T] fp32.
// causal: key s is visible to query t iff s <= t + (S - T).  window >= 0 additionally hides keys
// with s < t + (S - T) - window.  q_seg [B, T] / k_seg [B, S] int32 (both or neither): a key is
// visible only when the ids match; `ranges` (from axb_seg_tile_ranges) lets whole key tiles be
// skipped.  logit_cap > 0 replaces a scaled score z by cap * tanh(z / cap).
extern "C" int axb_flash_fwd_v3(const void* q, const void* k, const void* v, void* out, float* lse,
                                const int* q_seg, const int* k_seg, const int* ranges, int B, int T, int S, int N,
                                int Nkv, int H, float softmax_scale, int causal, int window, float logit_cap,
                                int* status, cudaStream_t stream) {
  using namespace axb;
  if (N % Nkv != 0 || (H != 64 && H != 128)) return -10;
  if ((q_seg == nullptr) != (k_seg == nullptr)) return -11;
  FlashFwd3Params p;
  p.out = out, p.lse = lse;
  p.q_seg = q_seg, p.k_seg = k_seg, p.ranges = reinterpret_cast<const int2*>(ranges);
  p.B = B, p.T = T, p.S = S, p.N = N, p.Nkv = Nkv, p.H = H;
  const float log2e = 1.4426950408889634f;
  if (logit_cap > 0.f) {
    p.sc = 1.f, p.cap_in = softmax_scale / logit_cap, p.cap_out = logit_cap * log2e;
  } else {
    p.sc = softmax_scale * log2e, p.cap_in = 0.f, p.cap_out = 0.f;
  }
  p.causal = causal;
  p.q_offset = S - T;
  p.window = window;
  p.status = status;
  const bool general = q_seg != nullptr || window >= 0 || logit_cap > 0.f;
  if (H == 128) {
    return general ? launch_flash_fwd3<128, true>(q, k, v, p, stream) : launch_flash_fwd3<128, false>(q, k, v, p, stream);
  }
  return general ? launch_flash_fwd3<64, true>(q, k, v, p, stream) : launch_flash_fwd3<64, false>(q, k, v, p, stream);
}
