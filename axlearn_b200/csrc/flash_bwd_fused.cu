// Flash attention backward as ONE kernel: five GEMMs and one exponential per (key tile, query
// tile) pair instead of the seven GEMMs and two exponentials of the dK/dV + dQ kernel pair in
// flash_bwd.cu.
//
// One CTA owns a 128-key tile of one (batch, kv head) and walks over the query tiles (of every
// query head of the group) that can see it.  Scores are computed TRANSPOSED, keys on the TMEM
// lanes and queries along the columns, so that
//   S^T  = K Q^T                       (TMEM, 128 columns)
//   dP^T = V dO^T                      (TMEM, 128 columns)
//   P^T  = exp2(S^T c - lse[q])        registers -> bf16 pairs written back over S^T: it is the
//                                      A operand (tensor memory) of   dV += P^T dO
//   dS^T = P^T (dP^T - delta[q])       registers -> bf16 -> one swizzled shared-memory tile that
//                                      serves both                    dK += dS^T Q   (K-major A)
//                                      and                            dQ_i = dS K    (MN-major A)
// dV and dK accumulate in TMEM over the whole walk.  dQ_i is a per-pair partial result: it lands
// in the columns dP^T occupied, four "drain" warps read it and add it into an fp32 accumulation
// buffer with 16-byte vector reductions (red.global.add.v4.f32), and a small post-pass scales
// and rounds that buffer to bf16.  The accumulation buffer is tile-permuted
// ([B, N, T/128][H/4][128 rows][4]) so that the 32 lanes of a drain warp (32 query rows) always
// hit 512 consecutive bytes.  The order of those reductions is not fixed, so dQ is not
// bit-reproducible from run to run; flash_bwd.cu stays available as the deterministic path.
//
// Warps (512 threads): 0 TMA producer, 1 MMA issuer, 2-3 idle (the control warpgroup gives most
// of its registers away), 4-11 exponential / dS (two warps per TMEM lane quarter, 64 query
// columns each), 12-15 dQ drain.
//
// Per pair the tensor pipe has 5 x 512 cycles of work and the exponential unit about 1024, so
// the schedule is arranged for the MMA queue never to run dry: while the dS of pair i is being
// formed the pipe runs dV_i and S^T_{i+1}; while the exponentials of pair i+1 run it works
// through dQ_i, dK_i and dP^T_{i+1}.
//
// Masks: causal, ragged ends, sliding window, segment ids and the tanh logit cap of the forward
// kernel (flash_fwd_v3.cu); query tiles outside a key tile's visible range are skipped.
//
// Reference: axlearn/common/flash_attention/gpu_attention.py:436-616 (two Pallas kernels).
#include "host_utils.cuh"
#include "sm100.cuh"

namespace axb {

int make_bthd_map(CUtensorMap* map, const void* base, int B, int L, int N, int H, int box_rows);

constexpr int kFbThreads = 512;
// Register budget: 512 threads launch with 128 registers each; setmaxnreg only redistributes that
// launch-time allocation (control 4 warps x 96, exponential / dS 8 warps x 168, drain 4 warps x 80).
static_assert(128 * 96 + 256 * 168 + 128 * 80 <= 512 * 128, "setmaxnreg split exceeds the launch allocation");
constexpr int kFbSub = 16384;  // [128 x 64] bf16

struct FlashBwdFusedParams {
  const float* lse2;   // [B, N, Tp]  lse * log2(e); +inf for rows >= T
  const float* delta;  // [B, N, Tp]  rowsum(dO * O); 0 for rows >= T
  float* dq_acc;       // [B, N, Tp/128][H/4][128][4] fp32, zeroed by the launcher
  void* dk;            // [B, S, Nkv, H]
  void* dv;            // [B, S, Nkv, H]
  const int* q_seg;    // [B, T] or null
  const int* k_seg;    // [B, S] or null
  const int2* ranges;  // [B, ceil(S/128)]: query tiles [x, y) that share a segment with the key tile
  int B, T, Tp, S, N, Nkv, H;
  float scale;         // softmax scale (applied to dK here, to dQ in the post-pass)
  float sc;            // multiplier of a (transformed) score before exp2
  float cap_in, cap_out;
  int causal, q_offset, window;
  int* status;
};

// delta = rowsum(dO * O) and lse2 = lse * log2(e), both padded to Tp rows per (batch, head).
// H / 8 lanes share a row (one 16-byte load of O and of dO each), so a warp covers 32 / (H / 8) rows
// per trip with full-width loads.  H / 8 must be a power of two not above 32.
__global__ void flash_bwd_prep_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                      const float* __restrict__ lse, float* __restrict__ lse2,
                                      float* __restrict__ delta, int B, int T, int Tp, int N, int H) {
  const int64_t rows = static_cast<int64_t>(B) * Tp * N;
  const int lane = threadIdx.x & 31;
  const int lpr = H / 8;                 // lanes per row
  const int rpw = 32 / lpr;              // rows per warp and trip
  const int sub = lane / lpr, col = lane % lpr;
  const int64_t warp = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  const int64_t warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t base = warp * rpw; base < rows; base += warps * rpw) {
    const int64_t r = base + sub;
    const bool live = r < rows;
    const int n = live ? static_cast<int>(r % N) : 0;
    const int64_t bt = live ? r / N : 0;
    const int t = static_cast<int>(bt % Tp);
    const int64_t b_ = bt / Tp;
    const int64_t dst = (b_ * N + n) * Tp + t;
    const bool real = live && t < T;
    float s = 0.f;
    if (real) {
      const int64_t src_row = (b_ * T + t) * N + n;
      const uint4 x = *(reinterpret_cast<const uint4*>(o + src_row * H) + col);
      const uint4 y = *(reinterpret_cast<const uint4*>(d_o + src_row * H) + col);
      const __nv_bfloat162* xa = reinterpret_cast<const __nv_bfloat162*>(&x);
      const __nv_bfloat162* ya = reinterpret_cast<const __nv_bfloat162*>(&y);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 xf = __bfloat1622float2(xa[j]), yf = __bfloat1622float2(ya[j]);
        s += xf.x * yf.x + xf.y * yf.y;
      }
    }
    // Sum over the lanes of the row (every lane takes part; the offsets stay inside the row's lanes).
    for (int off = lpr >> 1; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (live && col == 0) {
      if (!real) {
        lse2[dst] = INFINITY;
        delta[dst] = 0.f;
      } else {
        const float l = lse[(b_ * N + n) * T + t];
        // A row that saw no key has lse = -inf; +inf here makes its probabilities exactly zero.
        lse2[dst] = (l == -INFINITY) ? INFINITY : l * 1.4426950408889634f;
        delta[dst] = s;
      }
    }
  }
}

// dq[b, t, n, :] = bf16(scale * accumulation buffer); one thread per (row, 8 columns).
__global__ void flash_bwd_dq_post_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, int B, int T,
                                         int Tp, int N, int H, float scale) {
  const int chunks = H / 8;
  const int64_t total = static_cast<int64_t>(B) * N * Tp * chunks;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int r = i % 128;
    int64_t rest = i / 128;
    const int ch = rest % chunks;
    rest /= chunks;
    const int tile = rest % (Tp / 128);
    const int64_t bn = rest / (Tp / 128);
    const int t = tile * 128 + r;
    if (t >= T) continue;
    const int n = bn % N;
    const int64_t b = bn / N;
    const float4* src = reinterpret_cast<const float4*>(acc) + ((bn * (Tp / 128) + tile) * (H / 4) + 2 * ch) * 128 + r;
    const float4 lo = src[0], hi = src[128];
    uint4 o;
    o.x = pack_bf16x2(lo.x * scale, lo.y * scale);
    o.y = pack_bf16x2(lo.z * scale, lo.w * scale);
    o.z = pack_bf16x2(hi.x * scale, hi.y * scale);
    o.w = pack_bf16x2(hi.z * scale, hi.w * scale);
    *reinterpret_cast<uint4*>(dq + ((b * T + t) * N + n) * H + ch * 8) = o;
  }
}

template <int H>
struct FbSmem {
  static constexpr int kTile = (H / 64) * kFbSub;
  static constexpr int kK = 0;
  static constexpr int kV = kK + kTile;
  static constexpr int kQ = kV + kTile;            // 2 stages
  static constexpr int kDO = kQ + 2 * kTile;       // 2 stages
  static constexpr int kDS = kDO + 2 * kTile;      // [128 keys x 128 queries]
  static constexpr int kLse = kDS + 2 * kFbSub;    // 2 stages x (128 lse2 + 128 delta) floats
  static constexpr int kBar = kLse + 2048;
  static constexpr int kTotal = kBar + 256;
};

__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

__device__ __forceinline__ float tanh_approx_b(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 32 consecutive bf16 values (columns c .. c+31 of row `row_in_tile`) of a [128 x 128] swizzled
// tile made of two [128 x 64] sub-tiles.
__device__ __forceinline__ void fb_store_row_chunk(uint8_t* tile, int row_in_tile, int c, const float (&v)[32]) {
  uint8_t* row = tile + row_in_tile * 128;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    uint4 o;
    o.x = pack_bf16x2(v[8 * g + 0], v[8 * g + 1]);
    o.y = pack_bf16x2(v[8 * g + 2], v[8 * g + 3]);
    o.z = pack_bf16x2(v[8 * g + 4], v[8 * g + 5]);
    o.w = pack_bf16x2(v[8 * g + 6], v[8 * g + 7]);
    const int c16 = (c >> 3) + g;
    const int sub = c16 >> 3, chunk = (c16 & 7) ^ (row_in_tile & 7);
    *reinterpret_cast<uint4*>(row + sub * kFbSub + chunk * 16) = o;
  }
}

template <int H, bool kGeneral>
__global__ void __launch_bounds__(kFbThreads, 1)
flash_bwd_fused_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                       const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                       FlashBwdFusedParams p) {
  using L = FbSmem<H>;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBar);
  uint64_t* kv_full = bars + 0;
  uint64_t* q_full = bars + 1;    // [2]
  uint64_t* q_empty = bars + 3;   // [2]
  uint64_t* do_full = bars + 5;   // [2]
  uint64_t* do_empty = bars + 7;  // [2]
  uint64_t* s_full = bars + 9;
  uint64_t* dp_full = bars + 10;
  uint64_t* p_full = bars + 11;   // 8 arrivals
  uint64_t* ds_full = bars + 12;  // 8 arrivals
  uint64_t* ds_free = bars + 13;
  uint64_t* dq_full = bars + 14;
  uint64_t* dq_free = bars + 15;  // 4 arrivals
  uint64_t* acc_done = bars + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_tile = blockIdx.x, kv_head = blockIdx.y, batch = blockIdx.z;
  const int group = p.N / p.Nkv;
  const int s0 = kv_tile * 128;
  const int n_qt = p.Tp / 128;
  // Query tiles [i_lo, i_hi) that can see this key tile.
  int i_lo = 0, i_hi = (p.T + 127) / 128;
  if (p.causal) i_lo = max(0, s0 - p.q_offset) / 128;
  if (kGeneral) {
    if (p.window >= 0) i_hi = min(i_hi, max(0, s0 + 127 - p.q_offset + p.window) / 128 + 1);
    if (p.ranges != nullptr) {
      const int2 r = p.ranges[batch * ((p.S + 127) / 128) + kv_tile];
      i_lo = max(i_lo, r.x);
      i_hi = min(i_hi, r.y);
    }
  }
  const int tiles_per_head = max(0, i_hi - i_lo);
  const int n_iters = tiles_per_head * group;
  const bool aligned = (smem_u32(smem) & 1023u) == 0;
  if (!aligned && threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0, kStatusBadArgument);
  const bool run = aligned && n_iters > 0;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    tma_prefetch_desc(&tmap_do);
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
      mbar_init(&do_full[i], 1);
      mbar_init(&do_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(p_full, 8);
    mbar_init(ds_full, 8);
    mbar_init(ds_free, 1);
    mbar_init(dq_full, 1);
    mbar_init(dq_free, 4);
    mbar_init(acc_done, 1);
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
  const uint32_t tm_s = tmem_base, tm_dp = tmem_base + 128, tm_dv = tmem_base + 256, tm_dk = tmem_base + 256 + H;

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 96;");
    if (warp == 0) {
      // ---------------------------------------------------------------- TMA producer
      if (elect_one() && run) {
        mbar_arrive_expect_tx(kv_full, 2 * L::kTile);
#pragma unroll
        for (int j = 0; j < H / 64; ++j) {
          tma_load_4d(smem + L::kK + j * kFbSub, &tmap_k, kv_full, j * 64, kv_head, s0, batch);
          tma_load_4d(smem + L::kV + j * kFbSub, &tmap_v, kv_full, j * 64, kv_head, s0, batch);
        }
        for (int it = 0; it < n_iters; ++it) {
          const int head = kv_head * group + it / tiles_per_head;
          const int qt = i_lo + it % tiles_per_head;
          const int st = it & 1;
          const uint32_t ph = (it >> 1) & 1;
          if (!mbar_wait(&q_empty[st], ph ^ 1, p.status, kStatusWaitTimeoutProducer)) break;
          mbar_arrive_expect_tx(&q_full[st], L::kTile + 1024);
#pragma unroll
          for (int j = 0; j < H / 64; ++j)
            tma_load_4d(smem + L::kQ + st * L::kTile + j * kFbSub, &tmap_q, &q_full[st], j * 64, head, qt * 128,
                        batch);
          const int64_t row0 = (static_cast<int64_t>(batch) * p.N + head) * p.Tp + qt * 128;
          bulk_load_1d(smem + L::kLse + st * 1024, p.lse2 + row0, 512, &q_full[st]);
          bulk_load_1d(smem + L::kLse + st * 1024 + 512, p.delta + row0, 512, &q_full[st]);
          if (!mbar_wait(&do_empty[st], ph ^ 1, p.status, kStatusWaitTimeoutProducer)) break;
          mbar_arrive_expect_tx(&do_full[st], L::kTile);
#pragma unroll
          for (int j = 0; j < H / 64; ++j)
            tma_load_4d(smem + L::kDO + st * L::kTile + j * kFbSub, &tmap_do, &do_full[st], j * 64, head, qt * 128,
                        batch);
        }
      }
    } else if (warp == 1) {
      // ---------------------------------------------------------------- MMA issuer
      if (elect_one() && run) {
        constexpr uint32_t idesc_s = umma_idesc_f16(128, 128, 1, 1, 0, 0);  // [keys x queries]
        constexpr uint32_t idesc_ts = umma_idesc_f16(128, H, 1, 1, 0, 1);   // A K-major (or TMEM), B MN-major
        constexpr uint32_t idesc_mn = umma_idesc_f16(128, H, 1, 1, 1, 1);   // A and B MN-major
        const uint32_t k_addr = smem_u32(smem + L::kK), v_addr = smem_u32(smem + L::kV);
        const uint32_t ds_addr = smem_u32(smem + L::kDS);
        auto issue_s = [&](int st) {  // S^T = K Q^T
          const uint32_t q_addr = smem_u32(smem + L::kQ + st * L::kTile);
#pragma unroll
          for (int kk = 0; kk < H / 16; ++kk) {
            const uint32_t off = (kk >> 2) * kFbSub + (kk & 3) * 32;
            tc_mma_f16(tm_s, umma_smem_desc(k_addr + off, 16, 1024), umma_smem_desc(q_addr + off, 16, 1024), idesc_s,
                       kk > 0 ? 1u : 0u);
          }
          tc_commit(s_full);
        };
        auto issue_dp = [&](int st) {  // dP^T = V dO^T
          const uint32_t do_addr = smem_u32(smem + L::kDO + st * L::kTile);
#pragma unroll
          for (int kk = 0; kk < H / 16; ++kk) {
            const uint32_t off = (kk >> 2) * kFbSub + (kk & 3) * 32;
            tc_mma_f16(tm_dp, umma_smem_desc(v_addr + off, 16, 1024), umma_smem_desc(do_addr + off, 16, 1024), idesc_s,
                       kk > 0 ? 1u : 0u);
          }
          tc_commit(dp_full);
        };
        bool ok = mbar_wait(kv_full, 0, p.status, kStatusWaitTimeoutMma);
        if (ok) ok = mbar_wait(&q_full[0], 0, p.status, kStatusWaitTimeoutMma);
        if (ok) {
          tc_fence_after_sync();
          issue_s(0);
          ok = mbar_wait(&do_full[0], 0, p.status, kStatusWaitTimeoutMma);
        }
        if (ok) {
          tc_fence_after_sync();
          issue_dp(0);
        }
        for (int it = 0; it < n_iters && ok; ++it) {
          const int st = it & 1;
          const bool has_next = it + 1 < n_iters;
          const uint32_t q_addr = smem_u32(smem + L::kQ + st * L::kTile);
          const uint32_t do_addr = smem_u32(smem + L::kDO + st * L::kTile);
          // dV += P^T dO  (A = bf16 pairs in tensor memory: queries 0-63 at columns 0-31,
          // queries 64-127 at columns 64-95 of the S^T buffer).
          if (!mbar_wait(p_full, it & 1, p.status, kStatusWaitTimeoutMma)) break;
          tc_fence_after_sync();
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint32_t a_col = tm_s + (kk >> 2) * 64 + (kk & 3) * 8;
            tc_mma_f16_ts(tm_dv, a_col, umma_smem_desc(do_addr + kk * 2048, kFbSub, 1024), idesc_ts,
                          (it > 0 || kk > 0) ? 1u : 0u);
          }
          tc_commit(&do_empty[st]);
          if (has_next) {
            if (!mbar_wait(&q_full[st ^ 1], ((it + 1) >> 1) & 1, p.status, kStatusWaitTimeoutMma)) break;
            tc_fence_after_sync();
            issue_s(st ^ 1);
          }
          // dQ_i = dS K (fresh accumulator in the dP^T columns), dK += dS^T Q.
          if (!mbar_wait(ds_full, it & 1, p.status, kStatusWaitTimeoutMma)) break;
          tc_fence_after_sync();
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            tc_mma_f16(tm_dp, umma_smem_desc(ds_addr + kk * 2048, kFbSub, 1024),
                       umma_smem_desc(k_addr + kk * 2048, kFbSub, 1024), idesc_mn, kk > 0 ? 1u : 0u);
          }
          tc_commit(dq_full);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint32_t a_off = (kk >> 2) * kFbSub + (kk & 3) * 32;
            tc_mma_f16(tm_dk, umma_smem_desc(ds_addr + a_off, 16, 1024),
                       umma_smem_desc(q_addr + kk * 2048, kFbSub, 1024), idesc_ts, (it > 0 || kk > 0) ? 1u : 0u);
          }
          tc_commit(&q_empty[st]);
          tc_commit(ds_free);
          if (has_next) {
            if (!mbar_wait(dq_free, it & 1, p.status, kStatusWaitTimeoutMma)) break;
            if (!mbar_wait(&do_full[st ^ 1], ((it + 1) >> 1) & 1, p.status, kStatusWaitTimeoutMma)) break;
            tc_fence_after_sync();
            issue_dp(st ^ 1);
          } else {
            tc_commit(acc_done);
          }
        }
      }
    }
  } else if (warp < 12) {
    // ------------------------------------------------------------------ exponential / dS
    asm volatile("setmaxnreg.inc.sync.aligned.u32 168;");
    const int quarter = warp & 3;
    const int half = (warp - 4) >> 2;  // which 64 query columns
    const int r_in = quarter * 32 + lane;
    const int key = s0 + r_in;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t s_addr = tm_s + lane_base + half * 64;    // scores; P^T pairs go to its first 32 columns
    const uint32_t dp_addr = tm_dp + lane_base + half * 64;
    int kseg = 0;
    const int* qseg_row = nullptr;
    if (kGeneral && p.k_seg != nullptr) {
      kseg = key < p.S ? p.k_seg[static_cast<int64_t>(batch) * p.S + key] : -2;
      qseg_row = p.q_seg + static_cast<int64_t>(batch) * p.T;
    }
    bool ok = run;
    for (int it = 0; it < n_iters && ok; ++it) {
      const int qt = i_lo + it % tiles_per_head;
      const int st = it & 1;
      const int t0 = qt * 128;
      // Visible query columns of this key: c_min <= c <= c_max (tile-relative).
      int c_min = 0, c_max = 127;
      if (p.causal) c_min = key - p.q_offset - t0;
      if (kGeneral && p.window >= 0) c_max = key - p.q_offset + p.window - t0;
      if (key >= p.S) c_min = 1 << 20;
      const bool need_mask = c_min > half * 64 || c_max < half * 64 + 63;
      const float* lse_s = reinterpret_cast<const float*>(smem + L::kLse + st * 1024) + half * 64;
      const float* delta_s = lse_s + 128;
      if (!mbar_wait_warp(&q_full[st], (it >> 1) & 1, p.status, kStatusWaitTimeoutEpilogue)) { ok = false; break; }
      if (!mbar_wait_warp(s_full, it & 1, p.status, kStatusWaitTimeoutEpilogue)) { ok = false; break; }
      tc_fence_after_sync();
      // P^T as bf16 pairs: written to tensor memory for dV and kept in registers (32 instead of
      // 64 for fp32) as the factor of dS; under a logit cap the factor is P (1 - tanh^2), kept
      // the same way in a second array.
      uint32_t pk[32], pw[kGeneral ? 32 : 1];
      {
        uint32_t rs[2][32];
        tmem_ld_32x32(s_addr, rs[0]);
        tmem_ld_32x32(s_addr + 32, rs[1]);
        tmem_ld_wait();
        const bool capped = kGeneral && p.cap_out != 0.f;
#pragma unroll
        for (int c4 = 0; c4 < 16; ++c4) {
          const float4 l4 = *reinterpret_cast<const float4*>(lse_s + 4 * c4);
          const float ls[4] = {l4.x, l4.y, l4.z, l4.w};
          float e[4], ew[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int c = 4 * c4 + u;
            float val = __uint_as_float(rs[c >> 5][c & 31]);
            float w = 1.f;
            if (capped) {
              const float th = tanh_approx_b(val * p.cap_in);
              val = th * p.cap_out;
              w = 1.f - th * th;
            }
            float pr = ex2_approx(val * p.sc - ls[u]);
            if (need_mask) {
              const int cc = half * 64 + c;
              if (cc < c_min || cc > c_max) pr = 0.f;
            }
            if (kGeneral && qseg_row != nullptr) {
              const int t = t0 + half * 64 + c;
              const int qs = t < p.T ? __ldg(qseg_row + t) : -1;
              if (qs != kseg) pr = 0.f;
            }
            e[u] = pr;
            ew[u] = pr * w;
          }
          pk[2 * c4] = pack_bf16x2(e[0], e[1]);
          pk[2 * c4 + 1] = pack_bf16x2(e[2], e[3]);
          if (kGeneral) {
            pw[2 * c4] = capped ? pack_bf16x2(ew[0], ew[1]) : pk[2 * c4];
            pw[2 * c4 + 1] = capped ? pack_bf16x2(ew[2], ew[3]) : pk[2 * c4 + 1];
          }
          if (c4 == 7) {
            // The first 32 columns travel to tensor memory while the other 32 are computed.
            uint32_t lo[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) lo[i] = pk[i];
            tmem_st_32x16(s_addr, lo);
          }
        }
        uint32_t hi[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) hi[i] = pk[16 + i];
        tmem_st_32x16(s_addr + 16, hi);
        tmem_st_wait();
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
      // dS^T = P^T (dP^T - delta): needs dP^T of this pair and the shared-memory tile free.
      if (!mbar_wait_warp(dp_full, it & 1, p.status, kStatusWaitTimeoutEpilogue)) { ok = false; break; }
      tc_fence_after_sync();
      if (it > 0) {
        if (!mbar_wait_warp(ds_free, (it - 1) & 1, p.status, kStatusWaitTimeoutEpilogue)) { ok = false; break; }
      }
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        uint32_t rd[32];
        tmem_ld_32x32(dp_addr + ch * 32, rd);
        tmem_ld_wait();
        float dsv[32];
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4) {
          const float4 d4 = *reinterpret_cast<const float4*>(delta_s + ch * 32 + 4 * c4);
          const uint32_t f01 = kGeneral ? pw[ch * 16 + 2 * c4] : pk[ch * 16 + 2 * c4];
          const uint32_t f23 = kGeneral ? pw[ch * 16 + 2 * c4 + 1] : pk[ch * 16 + 2 * c4 + 1];
          dsv[4 * c4 + 0] = __uint_as_float(f01 << 16) * (__uint_as_float(rd[4 * c4 + 0]) - d4.x);
          dsv[4 * c4 + 1] = __uint_as_float(f01 & 0xffff0000u) * (__uint_as_float(rd[4 * c4 + 1]) - d4.y);
          dsv[4 * c4 + 2] = __uint_as_float(f23 << 16) * (__uint_as_float(rd[4 * c4 + 2]) - d4.z);
          dsv[4 * c4 + 3] = __uint_as_float(f23 & 0xffff0000u) * (__uint_as_float(rd[4 * c4 + 3]) - d4.w);
        }
        fb_store_row_chunk(smem + L::kDS, r_in, half * 64 + ch * 32, dsv);
      }
      fence_proxy_async();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
    }
    // Epilogue: lane = key; each half stores half of the columns of dK (scaled) and dV.
    if (ok) ok = mbar_wait_warp(acc_done, 0, p.status, kStatusWaitTimeoutEpilogue);
    if (ok || (aligned && n_iters == 0)) {
      // tcgen05.ld is warp-collective: every lane runs the loads, only lanes with a real key store.
      tc_fence_after_sync();
      const int64_t orow = ((static_cast<int64_t>(batch) * p.S + key) * p.Nkv + kv_head) * H;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        const uint32_t src = (which == 0 ? tm_dk : tm_dv) + lane_base;
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(which == 0 ? p.dk : p.dv) + orow;
        const float mul = which == 0 ? p.scale : 1.f;
#pragma unroll 1
        for (int c = half * (H / 2); c < (half + 1) * (H / 2); c += 32) {
          uint32_t r[32];
          if (n_iters > 0) {
            tmem_ld_32x32(src + c, r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = 0;
          }
          if (key < p.S) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r[8 * g + 0]) * mul, __uint_as_float(r[8 * g + 1]) * mul);
              o.y = pack_bf16x2(__uint_as_float(r[8 * g + 2]) * mul, __uint_as_float(r[8 * g + 3]) * mul);
              o.z = pack_bf16x2(__uint_as_float(r[8 * g + 4]) * mul, __uint_as_float(r[8 * g + 5]) * mul);
              o.w = pack_bf16x2(__uint_as_float(r[8 * g + 6]) * mul, __uint_as_float(r[8 * g + 7]) * mul);
              *reinterpret_cast<uint4*>(dst + c + 8 * g) = o;
            }
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ dQ drain
    asm volatile("setmaxnreg.dec.sync.aligned.u32 80;");
    const int quarter = warp & 3;
    const int r_in = quarter * 32 + lane;  // query row within the tile
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    bool ok = run;
    for (int it = 0; it < n_iters && ok; ++it) {
      const int head = kv_head * group + it / tiles_per_head;
      const int qt = i_lo + it % tiles_per_head;
      float* tile = p.dq_acc + ((static_cast<int64_t>(batch) * p.N + head) * n_qt + qt) * (H * 128) + r_in * 4;
      if (!mbar_wait_warp(dq_full, it & 1, p.status, kStatusWaitTimeoutEpilogue)) { ok = false; break; }
      tc_fence_after_sync();
#pragma unroll
      for (int c = 0; c < H; c += 32) {
        uint32_t r0[32];
        tmem_ld_32x32(tm_dp + lane_base + c, r0);
        tmem_ld_wait();
        if (c + 32 >= H) {
          // Everything is in registers: the MMA issuer may overwrite these columns.
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(dq_free);
        }
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          red_add_v4(tile + ((c >> 2) + g) * 512, __uint_as_float(r0[4 * g]), __uint_as_float(r0[4 * g + 1]),
                     __uint_as_float(r0[4 * g + 2]), __uint_as_float(r0[4 * g + 3]));
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

template <int H, bool kGeneral>
static int launch_flash_bwd_fused(const void* q, const void* k, const void* v, const void* d_o,
                                  FlashBwdFusedParams p, cudaStream_t stream) {
  CUtensorMap tq, tk, tv, tdo;
  if (make_bthd_map(&tq, q, p.B, p.T, p.N, H, 128)) return -2;
  if (make_bthd_map(&tk, k, p.B, p.S, p.Nkv, H, 128)) return -2;
  if (make_bthd_map(&tv, v, p.B, p.S, p.Nkv, H, 128)) return -2;
  if (make_bthd_map(&tdo, d_o, p.B, p.T, p.N, H, 128)) return -2;
  auto kernel = flash_bwd_fused_kernel<H, kGeneral>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FbSmem<H>::kTotal) != cudaSuccess)
      return -3;
    configured = true;
  }
  dim3 grid((p.S + 127) / 128, p.Nkv, p.B);
  kernel<<<grid, kFbThreads, FbSmem<H>::kTotal, stream>>>(tq, tk, tv, tdo, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace axb

// Number of fp32 elements of each of the three work buffers (lse2, delta, dq accumulation).
extern "C" int64_t axb_flash_bwd_fused_workspace(int B, int T, int N, int H, int which) {
  const int64_t tp = (static_cast<int64_t>(T) + 127) / 128 * 128;
  return which == 2 ? static_cast<int64_t>(B) * N * tp * H : static_cast<int64_t>(B) * N * tp;
}

// All tensors bf16 contiguous: q, dout, out, dq: [B, T, N, H]; k, v, dk, dv: [B, S, Nkv, H];
// lse: [B, N, T] fp32 from the forward.  lse2, delta, dq_acc: work buffers sized by
// axb_flash_bwd_fused_workspace (dq_acc is cleared here).  Masks as in axb_flash_fwd_v3; `ranges`
// is indexed by KEY tile (axb_seg_tile_ranges called with the key ids first).
extern "C" int axb_flash_bwd_fused(const void* q, const void* k, const void* v, const void* out, const void* dout,
                                   const float* lse, float* lse2, float* delta, float* dq_acc, void* dq, void* dk,
                                   void* dv, const int* q_seg, const int* k_seg, const int* ranges, int B, int T,
                                   int S, int N, int Nkv, int H, float softmax_scale, int causal, int window,
                                   float logit_cap, int* status, cudaStream_t stream) {
  using namespace axb;
  if (N % Nkv != 0 || (H != 64 && H != 128)) return -10;
  if ((q_seg == nullptr) != (k_seg == nullptr)) return -11;
  const int Tp = (T + 127) / 128 * 128;
  {
    const int64_t rows = static_cast<int64_t>(B) * Tp * N;
    int blocks = static_cast<int>((rows * 32 + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    flash_bwd_prep_kernel<<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(out),
                                                      static_cast<const __nv_bfloat16*>(dout), lse, lse2, delta, B, T,
                                                      Tp, N, H);
  }
  if (cudaMemsetAsync(dq_acc, 0, static_cast<size_t>(B) * N * Tp * H * sizeof(float), stream) != cudaSuccess) return -5;
  FlashBwdFusedParams p;
  p.lse2 = lse2, p.delta = delta, p.dq_acc = dq_acc, p.dk = dk, p.dv = dv;
  p.q_seg = q_seg, p.k_seg = k_seg, p.ranges = reinterpret_cast<const int2*>(ranges);
  p.B = B, p.T = T, p.Tp = Tp, p.S = S, p.N = N, p.Nkv = Nkv, p.H = H;
  p.scale = softmax_scale;
  const float log2e = 1.4426950408889634f;
  if (logit_cap > 0.f) {
    p.sc = 1.f, p.cap_in = softmax_scale / logit_cap, p.cap_out = logit_cap * log2e;
  } else {
    p.sc = softmax_scale * log2e, p.cap_in = 0.f, p.cap_out = 0.f;
  }
  p.causal = causal, p.q_offset = S - T, p.window = window, p.status = status;
  const bool general = q_seg != nullptr || window >= 0 || logit_cap > 0.f;
  int rc;
  if (H == 128) {
    rc = general ? launch_flash_bwd_fused<128, true>(q, k, v, dout, p, stream)
                 : launch_flash_bwd_fused<128, false>(q, k, v, dout, p, stream);
  } else {
    rc = general ? launch_flash_bwd_fused<64, true>(q, k, v, dout, p, stream)
                 : launch_flash_bwd_fused<64, false>(q, k, v, dout, p, stream);
  }
  if (rc != 0) return rc;
  {
    const int64_t total = static_cast<int64_t>(B) * N * Tp * (H / 8);
    int blocks = static_cast<int>((total + 255) / 256);
    if (blocks > 148 * 32) blocks = 148 * 32;
    flash_bwd_dq_post_kernel<<<blocks, 256, 0, stream>>>(dq_acc, static_cast<__nv_bfloat16*>(dq), B, T, Tp, N, H,
                                                         softmax_scale);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
