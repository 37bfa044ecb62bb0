// bf16 GEMM for sm_100a: C[M,N] = A[M,K] * B[K,N] with fp32 accumulation in tensor memory.
//
// Structure (one persistent CTA per SM, 192 threads):
//   warp 0      TMA producer: streams 128xK64 A tiles and K64xBN B tiles through a ring of
//               shared-memory stages (128-byte swizzle), one mbarrier pair per stage;
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma (128 x BN x 16) per K step into
//               one of two TMEM accumulators, and tcgen05.commit to release stages / publish
//               the accumulator;
//   warps 2-5   epilogue: tcgen05.ld the finished accumulator (each thread owns one row),
//               convert, store to global; overlaps the next tile's main loop thanks to the
//               double-buffered accumulator.
//
// Either operand may be K-major (contraction dim contiguous) or MN-major (the M or N dim
// contiguous), so forward (x*W), data-gradient (dy*W^T) and weight-gradient (x^T*dy) GEMMs all
// read their operands in place; no transposed copies exist anywhere.
//
// Reference behaviour being replaced: every jnp.einsum of the dense layers lowers to a cuBLAS
// GEMM in the reference (axlearn/common/layers.py:715-770, axlearn/common/attention.py:536-562,
// 864-1060).
#include <stdlib.h>
#include <string.h>

#include "gemm_fused.cuh"
#include "host_utils.cuh"
#include "sm100.cuh"

namespace axb {

constexpr int kBlockM = 128;
constexpr int kBlockK = 64;
constexpr int kNumThreads = 192;
constexpr int kGroupM = 8;

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int kABytes = kBlockM * kBlockK * 2;
  static constexpr int kBBytes = BN * kBlockK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarrierBytes = 1024;
  static constexpr int kTotal = STAGES * kStageBytes + kBarrierBytes + 1024;  // +align slack
};

struct GemmParams {
  int M, N, K;
  void* C;
  int64_t ldc;
  int* status;
  int accumulate;  // C += A*B (read-modify-write in the epilogue)
  // Split-K (skinny problems): `split_k` CTAs share one output tile, each over a slice of the
  // k-blocks; fp32 partials go to `ws [split_k, M, N]` and the CTA that arrives last on
  // `counters[tile]` sums them into C (and leaves the counter at zero for the next launch).
  int split_k;
  float* ws;
  int* counters;
  // Grouped problems (mixture-of-experts), rows sorted by group and every group padded to whole
  // blocks of `group_block_rows` rows (a multiple of 128).  Mode 1: the rows of block b use B
  // matrix number `group_index[b]` (-1 = unused block, skipped); the B tensor map stacks the groups along its outer dim, `b_group_rows`
  // apart.  Mode 2: one output [M, N] per group g (`c_group_stride` elements apart), contracting
  // rows [group_index[g], group_index[g + 1]) of the (MN-major) operands; an empty group's
  // output is zero.
  int group_mode;
  int num_groups;
  const int* group_index;
  int b_group_rows;
  int64_t c_group_stride;
  int group_block_rows;
};

constexpr int kFusedThreads = kNumThreads + 32;  // + one copy warp per CTA

template <int BN, int STAGES, bool A_MN, bool B_MN, typename OutT, bool FUSED>
__global__ void __launch_bounds__(FUSED ? kFusedThreads : kNumThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a,
                 const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_b_local, GemmParams p,
                 const __grid_constant__ FusedParams f) {
  using S = GemmSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment is required by the 128B swizzle pattern.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* bar_base = smem + STAGES * S::kStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(bar_base);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_blocks = (p.M + kBlockM - 1) / kBlockM;
  const int n_blocks = (p.N + BN - 1) / BN;
  const int num_tiles = m_blocks * n_blocks;
  const int num_kb = (p.K + kBlockK - 1) / kBlockK;
  const int split = (!FUSED && p.split_k > 1) ? p.split_k : 1;
  const int gmode = FUSED ? 0 : p.group_mode;
  // item = (k slice or group, tile); the slices / groups of a tile run as separate items.
  const int num_items = num_tiles * (gmode == 2 ? p.num_groups : split);
  // k-block range of an item.
  auto kb_range = [&](int ks, int& kb_lo, int& kb_hi) {
    if (gmode == 2) {
      kb_lo = p.group_index[ks] / kBlockK;
      kb_hi = p.group_index[ks + 1] / kBlockK;
    } else {
      kb_lo = ks * num_kb / split;
      kb_hi = (ks + 1) * num_kb / split;
    }
  };

  // Fused all-gather: two barriers and two chunk buffers behind the pipeline's own.
  uint64_t* copy_full = reinterpret_cast<uint64_t*>(bar_base + 256);
  uint8_t* copy_bufs = bar_base + S::kBarrierBytes;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if constexpr (FUSED) {
      tma_prefetch_desc(&tmap_b_local);
      for (int b = 0; b < kCopyBufs; ++b) mbar_init(&copy_full[b], 1);
    }
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 4);  // one arrival per epilogue warp
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

  const bool copy_on = FUSED && (f.ag[0].world > 1 || f.ag[1].world > 1);  // carries gathers
  const bool ag_on = FUSED && f.ag_consume && f.ag[0].world > 1;           // ... one of its own B
  const int cta = static_cast<int>(blockIdx.x);
  const int num_ctas = static_cast<int>(gridDim.x);
  // Rows [own_lo, own_hi) of the split dim are this rank's own slab: tiles inside it are read
  // straight from the shard (`tmap_b_local`), without waiting for any copy.
  const int own_lo = ag_on ? f.ag[0].rank * f.ag_shard_extent : 0;
  const int own_hi = own_lo + (ag_on ? f.ag_shard_extent : 0);
  // Rotation that makes every rank start on the first tile fully inside its own slab.
  const int n_rot = (ag_on && !f.ag_along_k) ? ((own_lo + BN - 1) / BN) % n_blocks : 0;
  const int kb_rot = (ag_on && f.ag_along_k) ? ((own_lo + kBlockK - 1) / kBlockK) % num_kb : 0;

  auto tile_coords = [&](int t, int& m_blk, int& n_blk) {
    const int per_group = kGroupM * n_blocks;
    const int g = t / per_group;
    const int first_m = g * kGroupM;
    const int gsize = min(m_blocks - first_m, kGroupM);
    const int r = t % per_group;
    m_blk = first_m + r % gsize;
    n_blk = r / gsize;
    if (FUSED && n_rot) n_blk = (n_blk + n_rot) % n_blocks;
  };

  if (warp == 6) {
    // ------------------------------------------------------------------ copy warp (fused only)
    if constexpr (FUSED) {
      if (copy_on && elect_one()) {
        int64_t seq = 0;
        bool ok = true;
        for (int j = 0; j < 2 && ok; ++j)
          if (f.ag[j].world > 1) ok = ag_copy_warp(copy_bufs, copy_full, f.ag[j], seq, p.status);
      }
    }
  } else if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      uint32_t slab_ready = 0;  // bit r: slab r of the gathered operand has landed
      auto need_slab = [&](int r) -> bool {
        if (slab_ready >> r & 1u) return true;
        if (!wait_flag(&f.ag[0].flags[r], f.ag[0].epoch, p.status)) return false;
        // Later TMA reads (async proxy) must observe the copy CTAs' writes.
        asm volatile("fence.proxy.async;" ::: "memory");
        slab_ready |= 1u << r;
        return true;
      };
      for (int t = cta; t < num_items && ok; t += num_ctas) {
        int m_blk, n_blk;
        const int ks = t / num_tiles;
        tile_coords(t - ks * num_tiles, m_blk, n_blk);
        int kb_lo, kb_hi;
        kb_range(ks, kb_lo, kb_hi);
        int b_off = 0;  // grouped mode 1: outer-dim offset of this row block's B matrix
        if (gmode == 1) {
          const int g = p.group_index[m_blk / (p.group_block_rows / kBlockM)];
          if (g < 0) continue;
          b_off = g * p.b_group_rows;
        }
        const int m0 = m_blk * kBlockM, n0 = n_blk * BN;
        bool local = false;  // read this B tile from the own shard
        if (FUSED && ag_on && !f.ag_along_k) {
          const int last = min(n0 + BN, p.N) - 1;
          local = n0 >= own_lo && last < own_hi;
          for (int r = n0 / f.ag_shard_extent; !local && r <= last / f.ag_shard_extent && ok; ++r)
            ok = need_slab(r);
          if (!ok) break;
        }
        for (int kbi = kb_lo; kbi < kb_hi; ++kbi) {
          const int kb = FUSED ? (kbi + kb_rot) % num_kb : kbi;
          if (FUSED && ag_on && f.ag_along_k) {
            const int k_lo = kb * kBlockK, k_hi = min(k_lo + kBlockK, p.K) - 1;
            local = k_lo >= own_lo && k_hi < own_hi;
            for (int r = k_lo / f.ag_shard_extent; !local && r <= k_hi / f.ag_shard_extent && ok; ++r)
              ok = need_slab(r);
            if (!ok) break;
          }
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, kStatusWaitTimeoutProducer)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * S::kStageBytes;
          uint8_t* sb = sa + S::kABytes;
          mbar_arrive_expect_tx(&full_bar[stage], S::kStageBytes);
          const int k0 = kb * kBlockK;
          if constexpr (!A_MN) {
            tma_load_2d(sa, &tmap_a, &full_bar[stage], k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < kBlockM / 64; ++j)
              tma_load_2d(sa + j * 8192, &tmap_a, &full_bar[stage], m0 + j * 64, k0);
          }
          if (FUSED && local) {
            // B_MN: slabs split K (rows of the stored [K, N]); otherwise they split N.
            if constexpr (!B_MN) {
              tma_load_2d(sb, &tmap_b_local, &full_bar[stage], k0, n0 - own_lo);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_2d(sb + j * 8192, &tmap_b_local, &full_bar[stage], n0 + j * 64, k0 - own_lo);
            }
          } else if constexpr (!B_MN) {
            tma_load_2d(sb, &tmap_b, &full_bar[stage], k0, n0 + b_off);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * 8192, &tmap_b, &full_bar[stage], n0 + j * 64, k0 + b_off);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_f16(kBlockM, BN, 1, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = cta; t < num_items && ok; t += num_ctas) {
        const int ks = t / num_tiles;
        if (gmode == 1) {
          int m_blk, n_blk;
          tile_coords(t - ks * num_tiles, m_blk, n_blk);
          if (p.group_index[m_blk / (p.group_block_rows / kBlockM)] < 0) continue;
        }
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, p.status, kStatusWaitTimeoutMma)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        int kb_lo, kb_hi;
        kb_range(ks, kb_lo, kb_hi);
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, p.status, kStatusWaitTimeoutMma)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * S::kStageBytes);
          const uint32_t sb = sa + S::kABytes;
#pragma unroll
          for (int k = 0; k < kBlockK / 16; ++k) {
            // K-major: 16 K elements = 32 B inside the 128 B swizzle row.
            // MN-major: 16 K rows of 128 B = 2048 B.
            const uint64_t da = A_MN ? umma_smem_desc(sa + k * 2048, 8192, 1024)
                                     : umma_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? umma_smem_desc(sb + k * 2048, 8192, 1024)
                                     : umma_smem_desc(sb + k * 32, 16, 1024);
            tc_mma_f16(d_tmem, da, db, idesc, (kb > kb_lo || k > 0) ? 1u : 0u);
          }
          tc_commit(&empty_bar[stage]);  // stage reusable once these MMAs retire
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) tc_commit(&tmem_full[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, +32) are accessible to this warp
    int acc = 0;
    uint32_t acc_phase = 0;
    OutT* C = reinterpret_cast<OutT*>(p.C);
    for (int t = cta; t < num_items; t += num_ctas) {
      int m_blk, n_blk;
      const int ks = t / num_tiles;
      const int tile = t - ks * num_tiles;
      tile_coords(tile, m_blk, n_blk);
      if (gmode == 1 && p.group_index[m_blk / (p.group_block_rows / kBlockM)] < 0) continue;
      if (!mbar_wait(&tmem_full[acc], acc_phase, p.status, kStatusWaitTimeoutEpilogue)) break;
      tc_fence_after_sync();
      const int row = m_blk * kBlockM + quarter * 32 + lane;
      const int n0 = n_blk * BN;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      OutT* crow = C + static_cast<int64_t>(row) * p.ldc + n0;
      bool empty_group = false;  // grouped mode 2: nothing was accumulated, the result is zero
      if (gmode == 2) {
        crow += static_cast<int64_t>(ks) * p.c_group_stride;
        empty_group = p.group_index[ks] / kBlockK == p.group_index[ks + 1] / kBlockK;
      }
      if (split > 1) {
        // Split-K: park the fp32 partial, then the last of the tile's `split` CTAs reduces.
        // (N is a multiple of 32 here, so a 32-column chunk is entirely inside or outside.)
        float* wrow = p.ws + (static_cast<int64_t>(ks) * p.M + row) * p.N + n0;
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c, r);
          tmem_ld_wait();
          if (c + 32 >= BN) {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[acc]);
          }
          if (row < p.M && n0 + c < p.N) {
#pragma unroll
            for (int v = 0; v < 8; ++v)
              __stcg(reinterpret_cast<uint4*>(wrow + c + 4 * v),
                     make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]));
          }
        }
        __threadfence();
        int* last_flag = reinterpret_cast<int*>(bar_base + 512);
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 2 && lane == 0) {
          const int prev = atomicAdd(&p.counters[tile], 1);
          if (prev == split - 1) p.counters[tile] = 0;
          *last_flag = prev == split - 1;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const bool is_last = *last_flag != 0;
        if (is_last) {
          __threadfence();
          // The 128 epilogue threads sum the tile's partials with coalesced 16-byte accesses,
          // two vectors per thread and round so that 2 * split loads are in flight at once.
          const int m0 = m_blk * kBlockM;
          const int rows_valid = min(kBlockM, p.M - m0);
          const int vec_per_row = min(BN, p.N - n0) / 4;
          const int total_vec = rows_valid * vec_per_row;
          const int et = (warp - 2) * 32 + lane;
          const int64_t slice = static_cast<int64_t>(p.M) * p.N;
          for (int idx = et; idx < total_vec; idx += 256) {
            float4 part[2][8];
            int64_t off[2];
            bool on[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const int i = idx + u * 128;
              on[u] = i < total_vec;
              const int r = on[u] ? i / vec_per_row : 0;
              const int c4 = on[u] ? i - r * vec_per_row : 0;
              off[u] = static_cast<int64_t>(m0 + r) * p.N + n0 + c4 * 4;
#pragma unroll
              for (int sidx = 0; sidx < 8; ++sidx) {
                part[u][sidx] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (on[u] && sidx < split)
                  part[u][sidx] = __ldcg(reinterpret_cast<const float4*>(p.ws + sidx * slice + off[u]));
              }
            }
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              if (!on[u]) continue;
              float4 sum = part[u][0];
#pragma unroll
              for (int sidx = 1; sidx < 8; ++sidx) {
                sum.x += part[u][sidx].x;
                sum.y += part[u][sidx].y;
                sum.z += part[u][sidx].z;
                sum.w += part[u][sidx].w;
              }
              const int i = idx + u * 128;
              const int r = i / vec_per_row;
              const int c4 = i - r * vec_per_row;
              OutT* dst = C + static_cast<int64_t>(m0 + r) * p.ldc + n0 + c4 * 4;
              if constexpr (sizeof(OutT) == 2) {
                if (p.accumulate) {
                  const uint2 old = *reinterpret_cast<const uint2*>(dst);
                  sum.x += __uint_as_float(old.x << 16);
                  sum.y += __uint_as_float(old.x & 0xffff0000u);
                  sum.z += __uint_as_float(old.y << 16);
                  sum.w += __uint_as_float(old.y & 0xffff0000u);
                }
                *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16x2(sum.x, sum.y), pack_bf16x2(sum.z, sum.w));
              } else {
                if (p.accumulate) {
                  const float4 old = *reinterpret_cast<const float4*>(dst);
                  sum.x += old.x;
                  sum.y += old.y;
                  sum.z += old.z;
                  sum.w += old.w;
                }
                *reinterpret_cast<float4*>(dst) = sum;
              }
            }
          }
        }
        // `last_flag` is rewritten by the next item: everyone must have read it first.
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
        continue;
      }
      const int n_dst = (FUSED && f.rs_world > 1 && f.rs_mode == 1) ? f.rs_world : 1;
      if (FUSED && f.rs_world > 1 && f.rs_mode == 0 && row < p.M) {
        // Reduce-scatter epilogue: this row goes to its owner's staging slot for this rank
        // (a store to peer memory over NVLink when the owner is another GPU).
        const int owner = row / f.rs_rows_per_rank;
        const int local_row = row - owner * f.rs_rows_per_rank;
        crow = reinterpret_cast<OutT*>(f.rs_dst[owner]) +
               (static_cast<int64_t>(f.rs_rank) * f.rs_rows_per_rank + local_row) * p.ldc + n0;
      }
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c, r);
        tmem_ld_wait();
        if (empty_group) {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        if (c + 32 >= BN) {
          // All of this warp's reads of the accumulator are done: hand it back early.
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tmem_empty[acc]);
        }
        if (row < p.M) {
          if constexpr (sizeof(OutT) == 2) {
            if (n0 + c + 32 <= p.N && !p.accumulate) {
              uint4 o[4];
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                o[v].x = pack_bf16x2(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
                o[v].y = pack_bf16x2(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
                o[v].z = pack_bf16x2(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
                o[v].w = pack_bf16x2(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
              }
              for (int d = 0; d < n_dst; ++d) {
                OutT* cr = crow;
                if (FUSED && n_dst > 1)
                  cr = reinterpret_cast<OutT*>(f.rs_dst[d]) +
                       (static_cast<int64_t>(f.rs_rank) * p.M + row) * p.ldc + n0;
#pragma unroll
                for (int v = 0; v < 4; ++v) *reinterpret_cast<uint4*>(cr + c + 8 * v) = o[v];
              }
            } else {
              for (int j = 0; j < 32; ++j) {
                if (n0 + c + j < p.N) {
                  float v = __uint_as_float(r[j]);
                  if (p.accumulate) v += __bfloat162float(reinterpret_cast<__nv_bfloat16*>(crow)[c + j]);
                  reinterpret_cast<__nv_bfloat16*>(crow)[c + j] = __float2bfloat16(v);
                }
              }
            }
          } else {
            if (n0 + c + 32 <= p.N && !p.accumulate) {
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                uint4 o = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
                *reinterpret_cast<uint4*>(reinterpret_cast<float*>(crow) + c + 4 * v) = o;
              }
            } else {
              for (int j = 0; j < 32; ++j) {
                if (n0 + c + j < p.N) {
                  float v = __uint_as_float(r[j]);
                  float* dst = reinterpret_cast<float*>(crow) + c + j;
                  *dst = p.accumulate ? (*dst + v) : v;
                }
              }
            }
          }
        }
      }
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    // Stores to peer memory are posted: make each writer's rows visible system-wide before the
    // kernel can complete, so the flag raised by the next launch cannot overtake them.
    if (FUSED && f.rs_world > 1) __threadfence_system();
    if (FUSED && f.rs_world > 1 && f.rs_mode == 1) {
      // All four epilogue warps of this CTA are past their fences; the last CTA raises the flags.
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (warp == 2 && lane == 0) {
        if (atomicAdd(f.rs_counter, 1) == static_cast<int>(gridDim.x) - 1) {
          *f.rs_counter = 0;
          __threadfence_system();
          const int epoch = *reinterpret_cast<const volatile int*>(f.rs_epoch_ptr);
          for (int r = 0; r < f.rs_world; ++r)
            st_release_sys(f.rs_flags[r] + f.rs_site * f.rs_world + f.rs_rank, epoch);
        }
      }
    }
  }

  // ---------------------------------------------------------------------- tear-down
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    if (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) {
      // A wait gave up: let copies that may still be in flight land before the CTA exits.
      for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int BN, int STAGES, bool A_MN, bool B_MN, typename OutT, bool FUSED = false>
static int launch_gemm(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda,
                       int64_t ldb, int64_t ldc, int accumulate, int* status, int max_ctas,
                       cudaStream_t stream, const FusedParams* fused = nullptr, int split_k = 1,
                       float* ws = nullptr, int* counters = nullptr, int group_mode = 0,
                       int num_groups = 1, const int* group_index = nullptr,
                       int64_t c_group_stride = 0, int group_block_rows = kBlockM) {
  // Grouped mode 1 stacks the groups' B matrices along the outer dim of one tensor map.
  const uint64_t b_stack = group_mode == 1 ? static_cast<uint64_t>(num_groups) : 1;
  CUtensorMap ta, tb;
  int rc;
  if (!A_MN) {
    uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
    uint64_t strides[1] = {static_cast<uint64_t>(lda) * 2};
    uint32_t box[2] = {kBlockK, kBlockM};
    rc = make_tensor_map(&ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, dims, strides, box,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  } else {
    uint64_t dims[2] = {static_cast<uint64_t>(M), static_cast<uint64_t>(K)};
    uint64_t strides[1] = {static_cast<uint64_t>(lda) * 2};
    uint32_t box[2] = {64, kBlockK};
    rc = make_tensor_map(&ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, dims, strides, box,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  }
  if (rc != 0) return rc;
  if (!B_MN) {
    uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N) * b_stack};
    uint64_t strides[1] = {static_cast<uint64_t>(ldb) * 2};
    uint32_t box[2] = {kBlockK, BN};
    rc = make_tensor_map(&tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, dims, strides, box,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  } else {
    uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(K) * b_stack};
    uint64_t strides[1] = {static_cast<uint64_t>(ldb) * 2};
    uint32_t box[2] = {64, kBlockK};
    rc = make_tensor_map(&tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, dims, strides, box,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  }
  if (rc != 0) return rc;
  using S = GemmSmem<BN, STAGES>;
  FusedParams fp;
  memset(&fp, 0, sizeof(fp));
  if (FUSED && fused != nullptr) fp = *fused;
  // The own shard as a tensor of its own (consume mode): same row pitch, one slab of rows.
  CUtensorMap tl = tb;
  if (FUSED && fp.ag[0].world > 1 && fp.ag_consume) {
    const void* own = fp.ag[0].src[fp.ag[0].rank];
    const uint64_t ext = static_cast<uint64_t>(fp.ag_shard_extent);
    uint64_t strides[1] = {static_cast<uint64_t>(ldb) * 2};
    if (!B_MN) {
      uint64_t dims[2] = {static_cast<uint64_t>(K), ext};
      uint32_t box[2] = {kBlockK, BN};
      rc = make_tensor_map(&tl, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, own, dims, strides, box,
                           CU_TENSOR_MAP_SWIZZLE_128B);
    } else {
      uint64_t dims[2] = {static_cast<uint64_t>(N), ext};
      uint32_t box[2] = {64, kBlockK};
      rc = make_tensor_map(&tl, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, own, dims, strides, box,
                           CU_TENSOR_MAP_SWIZZLE_128B);
    }
    if (rc != 0) return rc;
  }
  constexpr int kSmem = S::kTotal + (FUSED ? kCopyBufs * static_cast<int>(kCopyChunk) : 0);
  auto kernel = gemm_bf16_kernel<BN, STAGES, A_MN, B_MN, OutT, FUSED>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (e != cudaSuccess) {
      fprintf(stderr, "axb gemm: cudaFuncSetAttribute: %s\n", cudaGetErrorString(e));
      return -3;
    }
    configured = true;
  }
  const int m_blocks = (M + kBlockM - 1) / kBlockM;
  const int n_blocks = (N + BN - 1) / BN;
  int grid = m_blocks * n_blocks * (group_mode == 2 ? num_groups : (split_k > 1 ? split_k : 1));
  int cap = max_ctas > 0 && max_ctas < sm_count() ? max_ctas : sm_count();
  // All CTAs must be co-resident (one per SM): tiles may wait on flags that every CTA's copy
  // warp contributes to.
  if (grid > cap) grid = cap;
  if (grid < 1) return -12;
  GemmParams p{M, N, K, C, ldc, status, accumulate, split_k, ws, counters,
               group_mode, num_groups, group_index, B_MN ? K : N, c_group_stride, group_block_rows};
  kernel<<<grid, FUSED ? kFusedThreads : kNumThreads, kSmem, stream>>>(ta, tb, tl, p, fp);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    fprintf(stderr, "axb gemm: launch failed: %s\n", cudaGetErrorString(e));
    return -4;
  }
  return 0;
}

// AXB_GEMM_SKINNY selects the treatment of skinny problems (one row block): 0 = the general tiles,
// 1 = 64-column tiles, 2 (default) = 64-column tiles and split-K.
static int skinny_mode() {
  static int mode = -1;
  if (mode < 0) {
    const char* e = getenv("AXB_GEMM_SKINNY");
    mode = (e != nullptr && e[0] >= '0' && e[0] <= '2') ? e[0] - '0' : 2;
  }
  return mode;
}

template <bool A_MN, bool B_MN, typename OutT>
static int dispatch_bn(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda,
                       int64_t ldb, int64_t ldc, int accumulate, int* status, int max_ctas,
                       cudaStream_t stream) {
  // 128x256 tiles when they fill the machine, 128x128 otherwise (more CTAs for small problems),
  // and 128x64 for skinny decode-time GEMMs (M <= 128), which are weight-streaming problems: the
  // more CTAs pull weight columns concurrently, the closer they get to the HBM rate.
  const int m_blocks = (M + kBlockM - 1) / kBlockM;
  const int tiles256 = m_blocks * ((N + 255) / 256);
  if (m_blocks == 1 && (N + 127) / 128 < sm_count() / 2 && skinny_mode() >= 1)
    return launch_gemm<64, 8, A_MN, B_MN, OutT>(A, B, C, M, N, K, lda, ldb, ldc, accumulate, status,
                                                max_ctas, stream);
  if (N >= 256 && tiles256 >= sm_count() / 2)
    return launch_gemm<256, 4, A_MN, B_MN, OutT>(A, B, C, M, N, K, lda, ldb, ldc, accumulate,
                                                  status, max_ctas, stream);
  return launch_gemm<128, 6, A_MN, B_MN, OutT>(A, B, C, M, N, K, lda, ldb, ldc, accumulate, status,
                                                max_ctas, stream);
}

// Split-K plan for a skinny problem (one row block): how many CTAs share an output tile so that
// the weight stream is pulled by (nearly) every SM.  1 = no split.
static int splitk_plan(int M, int N, int K) {
  if (M > kBlockM || (N % 32) != 0 || skinny_mode() < 2) return 1;
  const int tiles = (N + 63) / 64;
  const int num_kb = (K + kBlockK - 1) / kBlockK;
  if ((N + 127) / 128 >= sm_count() / 2) return 1;
  int split = sm_count() / tiles;
  if (split > num_kb / 4) split = num_kb / 4;  // at least four k-blocks per slice
  if (split > 8) split = 8;
  // The hand-over (fence, counter, reduction by the last CTA) costs about as much as two dozen
  // k-blocks of streaming: split only when it takes more than that off every CTA's loop.
  if (split < 2 || num_kb - num_kb / split < 24) return 1;
  return split;
}

}  // namespace axb

extern "C" int axb_gemm_splitk_plan(int M, int N, int K) { return axb::splitk_plan(M, N, K); }

// Skinny GEMM (M <= 128, N a multiple of 32) with split-K: `ws` holds split * M * N floats and
// `counters` ceil(N / 64) ints that are zero on entry (the kernel leaves them zero).  The caller
// owns both and must not share them between launches that may overlap in time.
extern "C" int axb_gemm_bf16_splitk(const void* A, const void* B, void* C, int M, int N, int K,
                                    int64_t lda, int64_t ldb, int64_t ldc, int a_mn_major,
                                    int b_mn_major, int out_fp32, int accumulate, int split,
                                    void* ws, void* counters, int* status, int max_ctas,
                                    cudaStream_t stream) {
  using namespace axb;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(B) & 15) || (reinterpret_cast<uintptr_t>(C) & 15) ||
      (ldc % (out_fp32 ? 4 : 8)) || (reinterpret_cast<uintptr_t>(ws) & 15))
    return -10;
  if (M > kBlockM || (N % 32) || split < 2 || split > (K + kBlockK - 1) / kBlockK || ws == nullptr ||
      counters == nullptr)
    return -15;
#define AXB_SPLITK_CASE(AM, BM)                                                                    \
  if (a_mn_major == (AM ? 1 : 0) && b_mn_major == (BM ? 1 : 0)) {                                  \
    if (out_fp32)                                                                                  \
      return launch_gemm<64, 8, AM, BM, float>(A, B, C, M, N, K, lda, ldb, ldc, accumulate,       \
                                               status, max_ctas, stream, nullptr, split,          \
                                               static_cast<float*>(ws), static_cast<int*>(counters)); \
    return launch_gemm<64, 8, AM, BM, __nv_bfloat16>(A, B, C, M, N, K, lda, ldb, ldc, accumulate,  \
                                                     status, max_ctas, stream, nullptr, split,     \
                                                     static_cast<float*>(ws), static_cast<int*>(counters)); \
  }
  AXB_SPLITK_CASE(false, false)
  AXB_SPLITK_CASE(false, true)
  AXB_SPLITK_CASE(true, false)
  AXB_SPLITK_CASE(true, true)
#undef AXB_SPLITK_CASE
  return -11;
}

// AXB200_GEMM=1cta keeps every problem on the single-CTA kernels (for comparisons).
static bool cta_pairs_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("AXB200_GEMM");
    on = (e != nullptr && strcmp(e, "1cta") == 0) ? 0 : 1;
  }
  return on != 0;
}

extern "C" int axb_gemm_bf16_grouped_2cta(const void* A, const void* B, void* C, int M, int N, int K,
                                          int64_t lda, int64_t ldb, int64_t ldc, int a_mn_major,
                                          int b_mn_major, int mode, int num_groups,
                                          const int* group_index, int64_t c_group_stride,
                                          int block_rows, int* status, int max_ctas, cudaStream_t stream);

// Grouped GEMMs for mixture-of-experts layers whose token rows are sorted by expert, each expert's
// run padded to a whole number of `block_rows`-row blocks (a multiple of 128; multiples of 256 run
// on CTA pairs).
//   mode 1: C[M, N] = A[M, K] * B[g(m)]  with B stacked [G, K, N] (b_mn_major = 1) or [G, N, K]
//           (b_mn_major = 0) and `group_index[M / block_rows]` = the group of each row block (-1 =
//           unused block: its rows of C are not written).  With b_mn_major = 1, K must be a multiple
//           of 64.
//   mode 2: C[g] [M, N] = sum over rows r in [group_index[g], group_index[g + 1]) of
//           A[r, :M]^T * B[r, :N]  (both operands stored row-major over the token rows, i.e.
//           a_mn_major = b_mn_major = 1; K = total rows); offsets are multiples of `block_rows`.
extern "C" int axb_gemm_bf16_grouped(const void* A, const void* B, void* C, int M, int N, int K,
                                     int64_t lda, int64_t ldb, int64_t ldc, int a_mn_major,
                                     int b_mn_major, int out_fp32, int mode, int num_groups,
                                     const int* group_index, int64_t c_group_stride, int block_rows,
                                     int* status, int max_ctas, cudaStream_t stream) {
  using namespace axb;
  if (M <= 0 || N <= 0 || K <= 0 || num_groups <= 0) return 0;
  if (block_rows < kBlockM || (block_rows % kBlockM) != 0) return -16;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(B) & 15) || (reinterpret_cast<uintptr_t>(C) & 15) ||
      (ldc % (out_fp32 ? 4 : 8)) || group_index == nullptr)
    return -10;
  if (mode == 1 && (a_mn_major || (M % kBlockM) || (b_mn_major && (K % kBlockK)))) return -16;
  if (mode == 2 && (!a_mn_major || !b_mn_major || (c_group_stride % 8))) return -16;
  if (mode != 1 && mode != 2) return -16;
  if (cta_pairs_enabled() && !out_fp32) {
    const int rc = axb_gemm_bf16_grouped_2cta(A, B, C, M, N, K, lda, ldb, ldc, a_mn_major, b_mn_major, mode,
                                              num_groups, group_index, c_group_stride, block_rows, status,
                                              max_ctas, stream);
    if (rc != -20) return rc;
  }
#define AXB_GROUPED_CASE(AM, BM, T)                                                                \
  if (a_mn_major == (AM ? 1 : 0) && b_mn_major == (BM ? 1 : 0) && out_fp32 == (sizeof(T) == 4)) { \
    if (N >= 256)                                                                                  \
      return launch_gemm<256, 4, AM, BM, T>(A, B, C, M, N, K, lda, ldb, ldc, 0, status, max_ctas,  \
                                            stream, nullptr, 1, nullptr, nullptr, mode,           \
                                            num_groups, group_index, c_group_stride, block_rows);  \
    return launch_gemm<128, 6, AM, BM, T>(A, B, C, M, N, K, lda, ldb, ldc, 0, status, max_ctas,    \
                                          stream, nullptr, 1, nullptr, nullptr, mode, num_groups, \
                                          group_index, c_group_stride, block_rows);                \
  }
  AXB_GROUPED_CASE(false, false, __nv_bfloat16)
  AXB_GROUPED_CASE(false, true, __nv_bfloat16)
  AXB_GROUPED_CASE(true, true, __nv_bfloat16)
  AXB_GROUPED_CASE(true, true, float)
#undef AXB_GROUPED_CASE
  return -11;
}

// Fused compute+collective GEMM (bf16 out). `fused` points to a host copy of axb::FusedParams
// (see the struct for the all-gather-of-B and reduce-scatter-of-C contracts). With
// ag_world > 1, B must be the local full-size buffer `fused->ag_dst`.
extern "C" int axb_gemm_bf16_fused_2cta(const void* A, const void* B, void* C, int M, int N, int K,
                                        int64_t lda, int64_t ldb, int64_t ldc, int a_mn_major,
                                        int b_mn_major, int* status, int max_ctas, const void* fused,
                                        cudaStream_t stream);


extern "C" int axb_gemm_bf16_fused(const void* A, const void* B, void* C, int M, int N, int K,
                                   int64_t lda, int64_t ldb, int64_t ldc, int a_mn_major,
                                   int b_mn_major, int* status, int max_ctas,
                                   const void* fused, cudaStream_t stream) {
  using namespace axb;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const FusedParams* fp = static_cast<const FusedParams*>(fused);
  if ((lda % 8) || (ldb % 8) || (ldc % 8) || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(B) & 15))
    return -10;
  for (int j = 0; j < 2; ++j) {
    const GatherJob& g = fp->ag[j];
    if (g.world > 1 && (g.world > kMaxPeers || (g.shard_bytes % 16) || g.rank < 0 || g.rank >= g.world))
      return -13;
  }
  if (fp->ag_consume && fp->ag[0].world > 1 && fp->ag_shard_extent < 1) return -13;
  if (fp->rs_world > 1 && fp->rs_mode == 0 &&
      (fp->rs_world > kMaxPeers || fp->rs_rows_per_rank * fp->rs_world != M))
    return -14;
  if (fp->rs_world > 1 && fp->rs_mode == 1 &&
      (fp->rs_world > kMaxPeers || (N % 32) || fp->rs_counter == nullptr || fp->rs_epoch_ptr == nullptr))
    return -14;
  if (cta_pairs_enabled()) {
    // Large problems run on CTA pairs; -20 means "not one of mine".
    const int rc2 = axb_gemm_bf16_fused_2cta(A, B, C, M, N, K, lda, ldb, ldc, a_mn_major, b_mn_major, status,
                                             max_ctas, fused, stream);
    if (rc2 != -20) return rc2;
  }
#define AXB_FUSED_CASE(AM, BM)                                                                     \
  if (a_mn_major == (AM ? 1 : 0) && b_mn_major == (BM ? 1 : 0)) {                                  \
    if (M <= kBlockM && fp->ag[0].world <= 1 && fp->ag[1].world <= 1)                              \
      return launch_gemm<64, 8, AM, BM, __nv_bfloat16, true>(A, B, C, M, N, K, lda, ldb, ldc, 0,   \
                                                             status, max_ctas, stream, fp);        \
    return launch_gemm<256, 4, AM, BM, __nv_bfloat16, true>(A, B, C, M, N, K, lda, ldb, ldc, 0,    \
                                                            status, max_ctas, stream, fp);         \
  }
  AXB_FUSED_CASE(false, false)
  AXB_FUSED_CASE(false, true)
  AXB_FUSED_CASE(true, false)
  AXB_FUSED_CASE(true, true)
#undef AXB_FUSED_CASE
  return -11;
}

// C[M,N] (bf16 or fp32, row-major with leading dim ldc) = A * B (+ C when accumulate).
//   a_mn_major = 0: A is [M, K] row-major (lda = row pitch);  1: A is stored [K, M] row-major.
//   b_mn_major = 0: B is stored [N, K] row-major (ldb);        1: B is [K, N] row-major.
// Requirements: all pointers 16-byte aligned; lda, ldb multiples of 8 elements; for a vector
// store epilogue ldc a multiple of 8 (bf16) or 4 (fp32).  Returns 0 on a successful launch.
extern "C" int axb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K,
                             int64_t lda, int64_t ldb, int64_t ldc, int a_mn_major, int b_mn_major,
                             int out_fp32, int accumulate, int* status, int max_ctas,
                             cudaStream_t stream) {
  using namespace axb;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(B) & 15) || (reinterpret_cast<uintptr_t>(C) & 15) ||
      (ldc % (out_fp32 ? 4 : 8))) {
    return -10;
  }
#define AXB_GEMM_CASE(AM, BM)                                                                    \
  if (a_mn_major == (AM ? 1 : 0) && b_mn_major == (BM ? 1 : 0)) {                                \
    if (out_fp32)                                                                                \
      return dispatch_bn<AM, BM, float>(A, B, C, M, N, K, lda, ldb, ldc, accumulate, status,     \
                                        max_ctas, stream);                                       \
    return dispatch_bn<AM, BM, __nv_bfloat16>(A, B, C, M, N, K, lda, ldb, ldc, accumulate,       \
                                              status, max_ctas, stream);                         \
  }
  AXB_GEMM_CASE(false, false)
  AXB_GEMM_CASE(false, true)
  AXB_GEMM_CASE(true, false)
  AXB_GEMM_CASE(true, true)
#undef AXB_GEMM_CASE
  return -11;
}
