// Flash attention backward for sm_100a (bf16, head dim 64 or 128, causal or full, GQA).
//
// Three kernels, all deterministic (no atomics):
//   delta      delta[b,n,t] = sum_h dO * O                      (memory-bound pre-pass)
//   dK/dV      one CTA per 128-key tile of one (batch, kv head); loops over the query heads of
//              the group and their query tiles:  S = Q K^T, dP = dO V^T (TMEM) ->
//              P = exp2(S*c - lse), dS = P*(dP - delta)*scale (registers -> swizzled smem) ->
//              dV += P^T dO, dK += dS^T Q (TMEM accumulators, 128 key lanes x H columns)
//   dQ         one CTA per 128-query tile of one (batch, head); loops over key tiles:
//              S, dP as above -> dS -> dQ += dS K
// Every tile in shared memory is a row-major [128 x 64]-column sub-tile with the 128-byte
// swizzle; the same bytes serve as a K-major operand (rows index M/N) or as an MN-major operand
// (rows index the contraction), so Q, dO, K, P and dS are each staged once.
//
// The split into a dK/dV kernel and a dQ kernel mirrors the reference's Pallas backward
// (axlearn/common/flash_attention/gpu_attention.py:436-616), which reports the split to be
// faster than a fused kernel (:637-640).
#include "host_utils.cuh"
#include "sm100.cuh"

namespace axb {

int make_bthd_map(CUtensorMap* map, const void* base, int B, int L, int N, int H, int box_rows);

constexpr int kBwdThreads = 320;  // TMA producer, MMA issuer, 8 softmax / dS warps
constexpr int kSubTile = 16384;  // [128 x 64] bf16

struct FlashBwdParams {
  const float* lse;    // [B, N, T]
  const float* delta;  // [B, N, T]
  void* dq;            // [B, T, N, H]
  void* dk;            // [B, S, Nkv, H]
  void* dv;            // [B, S, Nkv, H]
  int B, T, S, N, Nkv, H;
  float scale, scale_log2;
  int causal, q_offset;
  int* status;
};

// delta = rowsum(dO * O); one warp per (b, t, n) row of H elements.
__global__ void flash_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                   float* __restrict__ delta, int B, int T, int N, int H) {
  const int64_t rows = static_cast<int64_t>(B) * T * N;
  const int lane = threadIdx.x & 31;
  for (int64_t r = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5; r < rows;
       r += (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5) {
    const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(o + r * H);
    const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(d_o + r * H);
    float s = 0.f;
    for (int i = lane; i < H / 2; i += 32) {
      const float2 x = __bfloat1622float2(a[i]), y = __bfloat1622float2(b[i]);
      s += x.x * y.x + x.y * y.y;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (lane == 0) {
      const int n = r % N;
      const int64_t bt = r / N;
      const int t = bt % T;
      const int64_t b_ = bt / T;
      delta[(b_ * N + n) * T + t] = s;
    }
  }
}

// Writes 32 consecutive bf16 values (columns c .. c+31 of row `row_in_tile`) of a [128 x 128]
// swizzled tile made of two [128 x 64] sub-tiles.
__device__ __forceinline__ void store_row_chunk(uint8_t* tile, int row_in_tile, int c, const float (&v)[32]) {
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
    *reinterpret_cast<uint4*>(row + sub * kSubTile + chunk * 16) = o;
  }
}

// ------------------------------------------------------------------------------ dK / dV
template <int H>
struct DkvSmem {
  static constexpr int kTile = (H / 64) * kSubTile;
  static constexpr int kK = 0;
  static constexpr int kV = kK + kTile;
  static constexpr int kQ = kV + kTile;
  static constexpr int kDO = kQ + kTile;
  static constexpr int kP = kDO + kTile;          // [128 q x 128 keys]
  static constexpr int kDS = kP + 2 * kSubTile;
  static constexpr int kBar = kDS + 2 * kSubTile;
  static constexpr int kTotal = kBar + 256 + 1024;
};

template <int H>
__global__ void __launch_bounds__(kBwdThreads, 1)
flash_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                      const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                      FlashBwdParams p) {
  using L = DkvSmem<H>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBar);
  uint64_t* kv_full = bars + 0;
  uint64_t* qdo_full = bars + 1;
  uint64_t* qdo_empty = bars + 2;
  uint64_t* sdp_full = bars + 3;
  uint64_t* pds_full = bars + 4;
  uint64_t* pds_free = bars + 5;
  uint64_t* acc_done = bars + 6;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_tile = blockIdx.x, kv_head = blockIdx.y, batch = blockIdx.z;
  const int group = p.N / p.Nkv;
  const int s0 = kv_tile * 128;
  const int q_tiles = (p.T + 127) / 128;
  // First query tile that can see this key tile under the causal mask.
  int first_q_tile = 0;
  if (p.causal) first_q_tile = max(0, (s0 - p.q_offset) / 128);
  const int tiles_per_head = max(0, q_tiles - first_q_tile);
  const int n_iters = tiles_per_head * group;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    tma_prefetch_desc(&tmap_do);
    mbar_init(kv_full, 1);
    mbar_init(qdo_full, 1);
    mbar_init(qdo_empty, 1);
    mbar_init(sdp_full, 1);
    mbar_init(pds_full, 8);
    mbar_init(pds_free, 1);
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

  if (warp == 0) {
    if (elect_one() && n_iters > 0) {
      mbar_arrive_expect_tx(kv_full, 2 * L::kTile);
#pragma unroll
      for (int j = 0; j < H / 64; ++j) {
        tma_load_4d(smem + L::kK + j * kSubTile, &tmap_k, kv_full, j * 64, kv_head, s0, batch);
        tma_load_4d(smem + L::kV + j * kSubTile, &tmap_v, kv_full, j * 64, kv_head, s0, batch);
      }
      for (int it = 0; it < n_iters; ++it) {
        const int head = kv_head * group + it / tiles_per_head;
        const int t0 = (first_q_tile + it % tiles_per_head) * 128;
        if (!mbar_wait(qdo_empty, (it & 1) ^ 1, p.status, kStatusWaitTimeoutProducer)) break;
        mbar_arrive_expect_tx(qdo_full, 2 * L::kTile);
#pragma unroll
        for (int j = 0; j < H / 64; ++j) {
          tma_load_4d(smem + L::kQ + j * kSubTile, &tmap_q, qdo_full, j * 64, head, t0, batch);
          tma_load_4d(smem + L::kDO + j * kSubTile, &tmap_do, qdo_full, j * 64, head, t0, batch);
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one() && n_iters > 0) {
      constexpr uint32_t idesc_s = umma_idesc_f16(128, 128, 1, 1, 0, 0);   // [q x keys]
      constexpr uint32_t idesc_g = umma_idesc_f16(128, H, 1, 1, 1, 1);     // [keys x H], A and B MN-major
      const uint32_t k_addr = smem_u32(smem + L::kK), v_addr = smem_u32(smem + L::kV);
      const uint32_t q_addr = smem_u32(smem + L::kQ), do_addr = smem_u32(smem + L::kDO);
      const uint32_t p_addr = smem_u32(smem + L::kP), ds_addr = smem_u32(smem + L::kDS);
      bool ok = mbar_wait(kv_full, 0, p.status, kStatusWaitTimeoutMma);
      for (int it = 0; it < n_iters && ok; ++it) {
        if (!mbar_wait(qdo_full, it & 1, p.status, kStatusWaitTimeoutMma)) break;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < H / 16; ++kk) {
          const uint32_t off = (kk >> 2) * kSubTile + (kk & 3) * 32;
          tc_mma_f16(tm_s, umma_smem_desc(q_addr + off, 16, 1024), umma_smem_desc(k_addr + off, 16, 1024),
                     idesc_s, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < H / 16; ++kk) {
          const uint32_t off = (kk >> 2) * kSubTile + (kk & 3) * 32;
          tc_mma_f16(tm_dp, umma_smem_desc(do_addr + off, 16, 1024), umma_smem_desc(v_addr + off, 16, 1024),
                     idesc_s, kk > 0 ? 1u : 0u);
        }
        tc_commit(sdp_full);
        if (!mbar_wait(pds_full, it & 1, p.status, kStatusWaitTimeoutMma)) break;
        tc_fence_after_sync();
        // Contraction over the 128 query rows: 8 steps of 16 rows (2048 B each).
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          tc_mma_f16(tm_dv, umma_smem_desc(p_addr + kk * 2048, kSubTile, 1024),
                     umma_smem_desc(do_addr + kk * 2048, kSubTile, 1024), idesc_g, (it > 0 || kk > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          tc_mma_f16(tm_dk, umma_smem_desc(ds_addr + kk * 2048, kSubTile, 1024),
                     umma_smem_desc(q_addr + kk * 2048, kSubTile, 1024), idesc_g, (it > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(qdo_empty);
        tc_commit(pds_free);
        if (it == n_iters - 1) tc_commit(acc_done);
      }
    }
  } else {
    // Two warps per TMEM lane quarter: each takes one half (64 columns) of the score tile.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r_in = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    bool ok = true;
    for (int it = 0; it < n_iters && ok; ++it) {
      const int head = kv_head * group + it / tiles_per_head;
      const int t0 = (first_q_tile + it % tiles_per_head) * 128;
      const int row = t0 + r_in;
      const int row_pos = row + p.q_offset;
      float lse_l2 = INFINITY, delta = 0.f;
      if (row < p.T) {
        const int64_t idx = (static_cast<int64_t>(batch) * p.N + head) * p.T + row;
        lse_l2 = p.lse[idx] * 1.4426950408889634f;
        delta = p.delta[idx];
      }
      if (!mbar_wait(sdp_full, it & 1, p.status, kStatusWaitTimeoutEpilogue)) { ok = false; break; }
      tc_fence_after_sync();
      if (it > 0) {
        if (!mbar_wait(pds_free, (it - 1) & 1, p.status, kStatusWaitTimeoutEpilogue)) { ok = false; break; }
      }
      const bool need_mask = (p.causal && s0 + 127 > t0 + p.q_offset) || (s0 + 128 > p.S);
      {
        // 64 score columns and 64 dP columns per TMEM round trip.
        const int c = half * 64;
        uint32_t rs[2][32], rd[2][32];
        tmem_ld_32x32(tm_s + lane_base + c, rs[0]);
        tmem_ld_32x32(tm_s + lane_base + c + 32, rs[1]);
        tmem_ld_32x32(tm_dp + lane_base + c, rd[0]);
        tmem_ld_32x32(tm_dp + lane_base + c + 32, rd[1]);
        tmem_ld_wait();
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
          float pv[32], dsv[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float e = exp2f(__uint_as_float(rs[h2][j]) * p.scale_log2 - lse_l2);
            if (need_mask) {
              const int col = s0 + c + h2 * 32 + j;
              if (col >= p.S || (p.causal && col > row_pos)) e = 0.f;
            }
            pv[j] = e;
            dsv[j] = e * (__uint_as_float(rd[h2][j]) - delta) * p.scale;
          }
          store_row_chunk(smem + L::kP, r_in, c + h2 * 32, pv);
          store_row_chunk(smem + L::kDS, r_in, c + h2 * 32, dsv);
        }
      }
      fence_proxy_async();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
    }
    // Epilogue: lane = key index within the tile.
    if (ok && n_iters > 0) ok = mbar_wait(acc_done, 0, p.status, kStatusWaitTimeoutEpilogue);
    if (ok) {
      tc_fence_after_sync();
      const int key = s0 + r_in;
      __nv_bfloat16* dk_row = reinterpret_cast<__nv_bfloat16*>(p.dk) +
                              ((static_cast<int64_t>(batch) * p.S + key) * p.Nkv + kv_head) * H;
      __nv_bfloat16* dv_row = reinterpret_cast<__nv_bfloat16*>(p.dv) +
                              ((static_cast<int64_t>(batch) * p.S + key) * p.Nkv + kv_head) * H;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        const uint32_t src = (which == 0 ? tm_dk : tm_dv) + lane_base;
        __nv_bfloat16* dst = which == 0 ? dk_row : dv_row;
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
              o.x = pack_bf16x2(__uint_as_float(r[8 * g + 0]), __uint_as_float(r[8 * g + 1]));
              o.y = pack_bf16x2(__uint_as_float(r[8 * g + 2]), __uint_as_float(r[8 * g + 3]));
              o.z = pack_bf16x2(__uint_as_float(r[8 * g + 4]), __uint_as_float(r[8 * g + 5]));
              o.w = pack_bf16x2(__uint_as_float(r[8 * g + 6]), __uint_as_float(r[8 * g + 7]));
              *reinterpret_cast<uint4*>(dst + c + 8 * g) = o;
            }
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

// ------------------------------------------------------------------------------ dQ
template <int H>
struct DqSmem {
  static constexpr int kTile = (H / 64) * kSubTile;
  static constexpr int kQ = 0;
  static constexpr int kDO = kQ + kTile;
  static constexpr int kK = kDO + kTile;           // 2 stages
  static constexpr int kV = kK + 2 * kTile;        // 2 stages
  static constexpr int kDS = kV + 2 * kTile;       // [128 q x 128 keys]
  static constexpr int kBar = kDS + 2 * kSubTile;
  static constexpr int kTotal = kBar + 256 + 1024;
};

template <int H>
__global__ void __launch_bounds__(kBwdThreads, 1)
flash_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                    FlashBwdParams p) {
  using L = DqSmem<H>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBar);
  uint64_t* qdo_full = bars + 0;
  uint64_t* kv_full = bars + 1;    // [2]
  uint64_t* kv_empty = bars + 3;   // [2]
  uint64_t* sdp_full = bars + 5;
  uint64_t* ds_full = bars + 6;
  uint64_t* ds_free = bars + 7;
  uint64_t* acc_done = bars + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_tile = gridDim.x - 1 - blockIdx.x;
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / (p.N / p.Nkv);
  const int t0 = q_tile * 128;
  int kv_len = p.S;
  if (p.causal) kv_len = min(p.S, t0 + 128 + p.q_offset);
  const int n_tiles = max(0, (kv_len + 127) / 128);

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    tma_prefetch_desc(&tmap_do);
    mbar_init(qdo_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    mbar_init(sdp_full, 1);
    mbar_init(ds_full, 8);
    mbar_init(ds_free, 1);
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
  const uint32_t tm_s = tmem_base, tm_dp = tmem_base + 128, tm_dq = tmem_base + 256;

  if (warp == 0) {
    if (elect_one() && n_tiles > 0) {
      mbar_arrive_expect_tx(qdo_full, 2 * L::kTile);
#pragma unroll
      for (int j = 0; j < H / 64; ++j) {
        tma_load_4d(smem + L::kQ + j * kSubTile, &tmap_q, qdo_full, j * 64, head, t0, batch);
        tma_load_4d(smem + L::kDO + j * kSubTile, &tmap_do, qdo_full, j * 64, head, t0, batch);
      }
      for (int it = 0; it < n_tiles; ++it) {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(&kv_empty[st], ph ^ 1, p.status, kStatusWaitTimeoutProducer)) break;
        mbar_arrive_expect_tx(&kv_full[st], 2 * L::kTile);
#pragma unroll
        for (int j = 0; j < H / 64; ++j) {
          tma_load_4d(smem + L::kK + st * L::kTile + j * kSubTile, &tmap_k, &kv_full[st], j * 64, kv_head,
                      it * 128, batch);
          tma_load_4d(smem + L::kV + st * L::kTile + j * kSubTile, &tmap_v, &kv_full[st], j * 64, kv_head,
                      it * 128, batch);
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one() && n_tiles > 0) {
      constexpr uint32_t idesc_s = umma_idesc_f16(128, 128, 1, 1, 0, 0);
      constexpr uint32_t idesc_dq = umma_idesc_f16(128, H, 1, 1, 0, 1);  // A = dS K-major, B = K MN-major
      const uint32_t q_addr = smem_u32(smem + L::kQ), do_addr = smem_u32(smem + L::kDO);
      const uint32_t ds_addr = smem_u32(smem + L::kDS);
      bool ok = mbar_wait(qdo_full, 0, p.status, kStatusWaitTimeoutMma);
      for (int it = 0; it < n_tiles && ok; ++it) {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(&kv_full[st], ph, p.status, kStatusWaitTimeoutMma)) break;
        tc_fence_after_sync();
        const uint32_t k_addr = smem_u32(smem + L::kK + st * L::kTile);
        const uint32_t v_addr = smem_u32(smem + L::kV + st * L::kTile);
#pragma unroll
        for (int kk = 0; kk < H / 16; ++kk) {
          const uint32_t off = (kk >> 2) * kSubTile + (kk & 3) * 32;
          tc_mma_f16(tm_s, umma_smem_desc(q_addr + off, 16, 1024), umma_smem_desc(k_addr + off, 16, 1024),
                     idesc_s, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < H / 16; ++kk) {
          const uint32_t off = (kk >> 2) * kSubTile + (kk & 3) * 32;
          tc_mma_f16(tm_dp, umma_smem_desc(do_addr + off, 16, 1024), umma_smem_desc(v_addr + off, 16, 1024),
                     idesc_s, kk > 0 ? 1u : 0u);
        }
        tc_commit(sdp_full);
        if (!mbar_wait(ds_full, it & 1, p.status, kStatusWaitTimeoutMma)) break;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t a_off = (kk >> 2) * kSubTile + (kk & 3) * 32;
          tc_mma_f16(tm_dq, umma_smem_desc(ds_addr + a_off, 16, 1024),
                     umma_smem_desc(k_addr + kk * 2048, kSubTile, 1024), idesc_dq, (it > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(&kv_empty[st]);
        tc_commit(ds_free);
        if (it == n_tiles - 1) tc_commit(acc_done);
      }
    }
  } else {
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r_in = quarter * 32 + lane;
    const int row = t0 + r_in;
    const int row_pos = row + p.q_offset;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    float lse_l2 = INFINITY, delta = 0.f;
    if (row < p.T) {
      const int64_t idx = (static_cast<int64_t>(batch) * p.N + head) * p.T + row;
      lse_l2 = p.lse[idx] * 1.4426950408889634f;
      delta = p.delta[idx];
    }
    bool ok = true;
    for (int it = 0; it < n_tiles && ok; ++it) {
      const int s0 = it * 128;
      if (!mbar_wait(sdp_full, it & 1, p.status, kStatusWaitTimeoutEpilogue)) { ok = false; break; }
      tc_fence_after_sync();
      if (it > 0) {
        if (!mbar_wait(ds_free, (it - 1) & 1, p.status, kStatusWaitTimeoutEpilogue)) { ok = false; break; }
      }
      const bool need_mask = (p.causal && s0 + 127 > t0 + p.q_offset) || (s0 + 128 > p.S);
      {
        const int c = half * 64;
        uint32_t rs[2][32], rd[2][32];
        tmem_ld_32x32(tm_s + lane_base + c, rs[0]);
        tmem_ld_32x32(tm_s + lane_base + c + 32, rs[1]);
        tmem_ld_32x32(tm_dp + lane_base + c, rd[0]);
        tmem_ld_32x32(tm_dp + lane_base + c + 32, rd[1]);
        tmem_ld_wait();
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
          float dsv[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float e = exp2f(__uint_as_float(rs[h2][j]) * p.scale_log2 - lse_l2);
            if (need_mask) {
              const int col = s0 + c + h2 * 32 + j;
              if (col >= p.S || (p.causal && col > row_pos)) e = 0.f;
            }
            dsv[j] = e * (__uint_as_float(rd[h2][j]) - delta) * p.scale;
          }
          store_row_chunk(smem + L::kDS, r_in, c + h2 * 32, dsv);
        }
      }
      fence_proxy_async();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
    }
    if (ok && n_tiles > 0) ok = mbar_wait(acc_done, 0, p.status, kStatusWaitTimeoutEpilogue);
    if (ok) {
      tc_fence_after_sync();
      __nv_bfloat16* dq_row = reinterpret_cast<__nv_bfloat16*>(p.dq) +
                              ((static_cast<int64_t>(batch) * p.T + row) * p.N + head) * H;
#pragma unroll 1
      for (int c = half * (H / 2); c < (half + 1) * (H / 2); c += 32) {
        uint32_t r[32];
        if (n_tiles > 0) {
          tmem_ld_32x32(tm_dq + lane_base + c, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0;
        }
        if (row < p.T) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r[8 * g + 0]), __uint_as_float(r[8 * g + 1]));
            o.y = pack_bf16x2(__uint_as_float(r[8 * g + 2]), __uint_as_float(r[8 * g + 3]));
            o.z = pack_bf16x2(__uint_as_float(r[8 * g + 4]), __uint_as_float(r[8 * g + 5]));
            o.w = pack_bf16x2(__uint_as_float(r[8 * g + 6]), __uint_as_float(r[8 * g + 7]));
            *reinterpret_cast<uint4*>(dq_row + c + 8 * g) = o;
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

template <int H>
static int launch_flash_bwd(const void* q, const void* k, const void* v, const void* d_o,
                            FlashBwdParams p, cudaStream_t stream) {
  CUtensorMap tq, tk, tv, tdo;
  if (make_bthd_map(&tq, q, p.B, p.T, p.N, H, 128)) return -2;
  if (make_bthd_map(&tk, k, p.B, p.S, p.Nkv, H, 128)) return -2;
  if (make_bthd_map(&tv, v, p.B, p.S, p.Nkv, H, 128)) return -2;
  if (make_bthd_map(&tdo, d_o, p.B, p.T, p.N, H, 128)) return -2;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(flash_bwd_dkdv_kernel<H>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             DkvSmem<H>::kTotal) != cudaSuccess)
      return -3;
    if (cudaFuncSetAttribute(flash_bwd_dq_kernel<H>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             DqSmem<H>::kTotal) != cudaSuccess)
      return -3;
    configured = true;
  }
  dim3 grid_kv((p.S + 127) / 128, p.Nkv, p.B);
  flash_bwd_dkdv_kernel<H><<<grid_kv, kBwdThreads, DkvSmem<H>::kTotal, stream>>>(tq, tk, tv, tdo, p);
  dim3 grid_q((p.T + 127) / 128, p.N, p.B);
  flash_bwd_dq_kernel<H><<<grid_q, kBwdThreads, DqSmem<H>::kTotal, stream>>>(tq, tk, tv, tdo, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace axb

// All tensors bf16 contiguous: q, dout, out, dq: [B, T, N, H]; k, v, dk, dv: [B, S, Nkv, H];
// lse, delta (workspace, written here): [B, N, T] fp32.
extern "C" int axb_flash_bwd(const void* q, const void* k, const void* v, const void* out,
                             const void* dout, const float* lse, float* delta, void* dq, void* dk,
                             void* dv, int B, int T, int S, int N, int Nkv, int H,
                             float softmax_scale, int causal, int* status, cudaStream_t stream) {
  using namespace axb;
  if (N % Nkv != 0 || (H != 64 && H != 128)) return -10;
  const int64_t rows = static_cast<int64_t>(B) * T * N;
  int blocks = static_cast<int>((rows * 32 + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  flash_delta_kernel<<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(out),
                                                 static_cast<const __nv_bfloat16*>(dout), delta, B, T, N, H);
  FlashBwdParams p;
  p.lse = lse, p.delta = delta, p.dq = dq, p.dk = dk, p.dv = dv;
  p.B = B, p.T = T, p.S = S, p.N = N, p.Nkv = Nkv, p.H = H;
  p.scale = softmax_scale;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.causal = causal;
  p.q_offset = S - T;
  p.status = status;
  if (H == 128) return launch_flash_bwd<128>(q, k, v, dout, p, stream);
  return launch_flash_bwd<64>(q, k, v, dout, p, stream);
}
