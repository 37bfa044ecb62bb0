// bf16 GEMM on CTA pairs for sm_100a: C[M,N] = A[M,K] * B[K,N], fp32 accumulation in tensor memory.
//
// Two CTAs on neighbouring SMs (a cluster of 2) share one 256 x 256 output tile:
//   * each CTA stages ITS OWN half of the operands -- 128 rows of A and 128 columns of B per
//     64-deep k-block -- with its own TMA loads (no load is shared between CTAs);
//   * one thread of the pair's first CTA issues tcgen05.mma.cta_group::2 (256 x 256 x 16), which
//     reads A from each CTA's own shared memory and B from both, and accumulates 128 rows x 256
//     fp32 columns in each CTA's tensor memory;
//   * both CTAs drain their half of the accumulator.
// Per MMA each SM reads 128 x 16 of A and 128 x 16 of B from shared memory instead of 128 x 16 and
// 256 x 16: a third less shared-memory traffic and 32 KB instead of 48 KB per stage, which pays
// for a six-stage ring and a staging buffer for the epilogue.
//
// Warps (192 threads per CTA): 0 = TMA producer, 1 = MMA issuer (first CTA only) and tensor-memory
// owner, 2-5 = epilogue.  The epilogue converts 32 rows x 128 bytes per warp into a 128-byte
// swizzled shared-memory tile and writes it with one TMA store (full 128-byte lines, clipped at
// the matrix edge by the hardware) while the pair already computes the next tile into the second
// accumulator.  With `accumulate` the store is a TMA reduction (add) into C.
//
// Barriers: `full` (first CTA only) counts the bytes of both CTAs' loads; `empty` and
// `tmem_full` exist in both CTAs and are signalled by the issuer with one commit each;
// `tmem_empty` (first CTA) collects the eight epilogue warps of the pair.  Every wait is bounded;
// a CTA that gives up still reaches the cluster barrier of the tear-down, so its partner never
// waits for it unboundedly there.
#include <stdlib.h>
#include <string.h>

#include "gemm_fused.cuh"
#include "host_utils.cuh"
#include "sm100.cuh"

namespace axb {

constexpr int k2RowsPerCta = 128;
constexpr int k2TileM = 256;
constexpr int k2TileN = 256;
constexpr int k2HalfN = 128;
constexpr int k2BlockK = 64;
constexpr int k2Threads = 192;
constexpr int k2FusedThreads = k2Threads + 32;  // + one copy warp per CTA

// The fused variants give one stage of the ring to the copy warp's two chunk buffers.
template <bool FUSED>
struct Gemm2Smem {
  static constexpr int kStages = FUSED ? 5 : 6;
  static constexpr int kABytes = k2RowsPerCta * k2BlockK * 2;
  static constexpr int kBBytes = k2HalfN * k2BlockK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;  // 32 KB
  static constexpr int kRingBytes = kStages * kStageBytes;
  static constexpr int kStagingPerWarp = 2 * 4096;  // two 32-row x 128-byte tiles
  static constexpr int kStagingBytes = 4 * kStagingPerWarp;
  static constexpr int kCopyBytes = FUSED ? kCopyBufs * static_cast<int>(kCopyChunk) : 0;
  static constexpr int kBarrierBytes = 1024;
  static constexpr int kTotal = kRingBytes + kStagingBytes + kCopyBytes + kBarrierBytes + 1024;  // + align slack
};
static_assert(Gemm2Smem<false>::kTotal <= 227 * 1024 && Gemm2Smem<true>::kTotal <= 227 * 1024, "shared memory budget");

// One store map per owner of the reduce-scatter: its staging buffer seen as a
// [world * rows_per_rank, N] matrix.
struct PeerMaps {
  CUtensorMap m[kMaxPeers];
};

struct Gemm2Params {
  int M, N, K;
  int accumulate;
  int* status;
  int group_m;  // row blocks per rasterisation group
  // Grouped problems (mixture-of-experts; plain kernel only), rows sorted by group and every group
  // padded to whole blocks of `group_block_rows` rows (a multiple of 256).  Mode 1: the rows of
  // block b use B matrix number `group_index[b]` (-1 = unused block, skipped); the B tensor map
  // stacks the groups along its outer dim, `b_group_rows` apart.  Mode 2: one output [M, N] per
  // group g (third coordinate of the C map), contracting rows [group_index[g], group_index[g + 1])
  // of the MN-major operands; an empty group's output is zero.
  int group_mode;
  int num_groups;
  const int* group_index;
  int b_group_rows;
  int group_block_rows;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_addr), "r"(rank));
  return out;
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// TMA load into this CTA's shared memory whose bytes are counted on a barrier that may live in
// the partner CTA (`bar_cluster_addr` is a cluster-wide address).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
      "{%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// Arrives on the barrier at `bar_cluster_addr` (either CTA of the pair) when all MMAs issued so far
// by this thread have completed.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
               : "memory");
}

__device__ __forceinline__ void tc_mma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, const void* smem_src, int c0, int c1) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(smem_u32(smem_src)), "r"(c0), "r"(c1)
               : "memory");
}

__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* smem_src, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}

// FUSED adds what the single-CTA fused kernel has (same `FusedParams` contract): a copy warp that
// carries parameter gathers, consumption of a gathered B behind per-slab flags (every CTA of the
// pair waits for the slabs ITS half of B touches), and a reduce-scatter epilogue whose TMA stores
// go to the row owner's staging buffer (peer memory over NVLink: plain stores, full lines).
template <bool A_MN, bool B_MN, typename OutT, bool FUSED>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(FUSED ? k2FusedThreads : k2Threads, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ CUtensorMap tmap_c, Gemm2Params p,
                  const __grid_constant__ CUtensorMap tmap_b_local, const __grid_constant__ FusedParams f,
                  const __grid_constant__ PeerMaps rs_maps) {
  using S = Gemm2Smem<FUSED>;
  constexpr int k2Stages = S::kStages;
  extern __shared__ uint8_t smem_raw[];
  // The dynamic shared-memory window starts at the same offset in both CTAs, so rounding up to
  // 1024 bytes (required by the 128-byte swizzle) gives the same layout in both.
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  uint8_t* staging = smem + S::kRingBytes;
  uint8_t* copy_bufs = staging + S::kStagingBytes;
  uint8_t* bar_base = copy_bufs + S::kCopyBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(bar_base);
  uint64_t* empty_bar = full_bar + k2Stages;
  uint64_t* tmem_full = empty_bar + k2Stages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  uint64_t* copy_full = reinterpret_cast<uint64_t*>(bar_base + 512);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = static_cast<int>(blockIdx.x >> 1);
  const int num_pairs = static_cast<int>(gridDim.x >> 1);
  const int m_blocks = (p.M + k2TileM - 1) / k2TileM;
  const int n_blocks = (p.N + k2TileN - 1) / k2TileN;
  const int num_tiles = m_blocks * n_blocks;
  const int num_kb = (p.K + k2BlockK - 1) / k2BlockK;
  const int gmode = FUSED ? 0 : p.group_mode;
  // item = (group, tile) in grouped mode 2, a tile otherwise.
  const int num_items = num_tiles * (gmode == 2 ? p.num_groups : 1);
  auto kb_range = [&](int g, int& kb_lo, int& kb_hi) {
    if (gmode == 2) {
      kb_lo = p.group_index[g] / k2BlockK;
      kb_hi = p.group_index[g + 1] / k2BlockK;
    } else {
      kb_lo = 0;
      kb_hi = num_kb;
    }
  };
  // Grouped mode 1: the group of a 256-row tile (every block of the index covers whole tiles).
  auto tile_group = [&](int m_blk) { return p.group_index[m_blk / (p.group_block_rows / k2TileM)]; };

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    tma_prefetch_desc(&tmap_c);
    if constexpr (FUSED) {
      tma_prefetch_desc(&tmap_b_local);
      for (int b = 0; b < kCopyBufs; ++b) mbar_init(&copy_full[b], 1);
    }
    for (int s = 0; s < k2Stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 8);  // four epilogue warps in each CTA of the pair
    }
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anyone signals across the pair
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const bool copy_on = FUSED && (f.ag[0].world > 1 || f.ag[1].world > 1);  // carries gathers
  const bool ag_on = FUSED && f.ag_consume && f.ag[0].world > 1;           // ... one of its own B
  // Rows [own_lo, own_hi) of the split dim are this rank's own slab: tiles inside it are read
  // straight from the shard (`tmap_b_local`), without waiting for any copy.
  const int own_lo = ag_on ? f.ag[0].rank * f.ag_shard_extent : 0;
  const int own_hi = own_lo + (ag_on ? f.ag_shard_extent : 0);
  // Rotation that makes every rank start on the first tile fully inside its own slab.
  const int n_rot = (ag_on && !f.ag_along_k) ? ((own_lo + k2TileN - 1) / k2TileN) % n_blocks : 0;
  const int kb_rot = (ag_on && f.ag_along_k) ? ((own_lo + k2BlockK - 1) / k2BlockK) % num_kb : 0;

  auto tile_coords = [&](int t, int& m_blk, int& n_blk) {
    const int per_group = p.group_m * n_blocks;
    const int g = t / per_group;
    const int first_m = g * p.group_m;
    const int gsize = min(m_blocks - first_m, p.group_m);
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
    // ------------------------------------------------------------------ producer (both CTAs)
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
      for (int t = pair; t < num_items && ok; t += num_pairs) {
        int m_blk, n_blk;
        const int grp = t / num_tiles;
        tile_coords(t - grp * num_tiles, m_blk, n_blk);
        int kb_lo, kb_hi;
        kb_range(grp, kb_lo, kb_hi);
        int b_off = 0;  // grouped mode 1: outer-dim offset of this tile's B matrix
        if (gmode == 1) {
          const int g = tile_group(m_blk);
          if (g < 0) continue;
          b_off = g * p.b_group_rows;
        }
        const int m0 = m_blk * k2TileM + static_cast<int>(rank) * k2RowsPerCta;
        const int n0 = n_blk * k2TileN + static_cast<int>(rank) * k2HalfN;
        bool local = false;  // read this CTA's half of the B tile from the own shard
        if (FUSED && ag_on && !f.ag_along_k && n0 < p.N) {
          const int last = min(n0 + k2HalfN, p.N) - 1;
          local = n0 >= own_lo && last < own_hi;
          for (int r = n0 / f.ag_shard_extent; !local && r <= last / f.ag_shard_extent && ok; ++r) ok = need_slab(r);
          if (!ok) break;
        }
        for (int kbi = kb_lo; kbi < kb_hi; ++kbi) {
          const int kb = FUSED ? (kbi + kb_rot) % num_kb : kbi;
          if (FUSED && ag_on && f.ag_along_k) {
            const int k_lo = kb * k2BlockK, k_hi = min(k_lo + k2BlockK, p.K) - 1;
            local = k_lo >= own_lo && k_hi < own_hi;
            for (int r = k_lo / f.ag_shard_extent; !local && r <= k_hi / f.ag_shard_extent && ok; ++r) ok = need_slab(r);
            if (!ok) break;
          }
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, kStatusWaitTimeoutProducer)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * S::kStageBytes;
          uint8_t* sb = sa + S::kABytes;
          // The first CTA's barrier counts the bytes of both CTAs.
          if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * S::kStageBytes);
          const uint32_t bar = map_to_cta(smem_u32(&full_bar[stage]), 0);
          const int k0 = kb * k2BlockK;
          if constexpr (!A_MN) {
            tma_load_2d_pair(sa, &tmap_a, bar, k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < k2RowsPerCta / 64; ++j) tma_load_2d_pair(sa + j * 8192, &tmap_a, bar, m0 + j * 64, k0);
          }
          if (FUSED && local) {
            // B_MN: slabs split K (rows of the stored [K, N]); otherwise they split N.
            if constexpr (!B_MN) {
              tma_load_2d_pair(sb, &tmap_b_local, bar, k0, n0 - own_lo);
            } else {
#pragma unroll
              for (int j = 0; j < k2HalfN / 64; ++j)
                tma_load_2d_pair(sb + j * 8192, &tmap_b_local, bar, n0 + j * 64, k0 - own_lo);
            }
          } else if constexpr (!B_MN) {
            tma_load_2d_pair(sb, &tmap_b, bar, k0, n0 + b_off);
          } else {
#pragma unroll
            for (int j = 0; j < k2HalfN / 64; ++j)
              tma_load_2d_pair(sb + j * 8192, &tmap_b, bar, n0 + j * 64, k0 + b_off);
          }
          if (++stage == k2Stages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (first CTA)
    if (leader && elect_one()) {
      constexpr uint32_t idesc = umma_idesc_f16(k2TileM, k2TileN, 1, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = pair; t < num_items && ok; t += num_pairs) {
        const int grp = t / num_tiles;
        if (gmode == 1) {
          int m_blk, n_blk;
          tile_coords(t - grp * num_tiles, m_blk, n_blk);
          if (tile_group(m_blk) < 0) continue;
        }
        int kb_lo, kb_hi;
        kb_range(grp, kb_lo, kb_hi);
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, p.status, kStatusWaitTimeoutMma)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * k2TileN;
        for (int kb = kb_lo; kb < kb_hi; ++kb) {  // the producer's k order (rotated or not) is irrelevant here
          if (!mbar_wait(&full_bar[stage], phase, p.status, kStatusWaitTimeoutMma)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * S::kStageBytes);
          const uint32_t sb = sa + S::kABytes;
#pragma unroll
          for (int k = 0; k < k2BlockK / 16; ++k) {
            const uint64_t da = A_MN ? umma_smem_desc(sa + k * 2048, 8192, 1024) : umma_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? umma_smem_desc(sb + k * 2048, 8192, 1024) : umma_smem_desc(sb + k * 32, 16, 1024);
            tc_mma_f16_pair(d_tmem, da, db, idesc, (kb > kb_lo || k > 0) ? 1u : 0u);
          }
          // The stage is free in BOTH CTAs once these MMAs retire.
          const uint32_t eb = smem_u32(&empty_bar[stage]);
          tc_commit_pair(eb);
          tc_commit_pair(map_to_cta(eb, 1));
          if (++stage == k2Stages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) {
          const uint32_t fb = smem_u32(&tmem_full[acc]);
          tc_commit_pair(fb);
          tc_commit_pair(map_to_cta(fb, 1));
        }
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (both CTAs)
    constexpr int kChunkCols = 128 / static_cast<int>(sizeof(OutT));  // 128 bytes of output per row
    constexpr int kChunks = k2TileN / kChunkCols;
    const int quarter = warp & 3;  // tensor-memory lanes [32 * quarter, +32) belong to this warp
    uint8_t* my_staging = staging + quarter * S::kStagingPerWarp;
    const uint32_t empty_addr = map_to_cta(smem_u32(&tmem_empty[0]), 0);
    int acc = 0;
    uint32_t acc_phase = 0;
    uint32_t store_seq = 0;
    for (int t = pair; t < num_items; t += num_pairs) {
      int m_blk, n_blk;
      const int grp = t / num_tiles;
      tile_coords(t - grp * num_tiles, m_blk, n_blk);
      if (gmode == 1 && tile_group(m_blk) < 0) continue;
      // Grouped mode 2: nothing was accumulated for an empty group, its result is zero.
      const bool empty_group = gmode == 2 && p.group_index[grp] / k2BlockK == p.group_index[grp + 1] / k2BlockK;
      if (!mbar_wait_warp_relaxed(&tmem_full[acc], acc_phase, p.status, kStatusWaitTimeoutEpilogue)) break;
      tc_fence_after_sync();
      const int row0 = m_blk * k2TileM + static_cast<int>(rank) * k2RowsPerCta + quarter * 32;
      const int n0 = n_blk * k2TileN;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * k2TileN;
      // Reduce-scatter: these 32 rows go to their owner's staging slot for this rank (the host
      // checks that a 32-row block never straddles two owners).
      const CUtensorMap* out_map = &tmap_c;
      int out_row = row0;
      // rs_mode 1 (all-reduce push): the tile goes to slot `rs_rank` of EVERY peer's staging.
      const int n_dst = (FUSED && f.rs_world > 1 && f.rs_mode == 1) ? f.rs_world : 1;
      if (FUSED && f.rs_world > 1 && row0 < p.M) {
        if (f.rs_mode == 1) {
          out_row = f.rs_rank * p.M + row0;
        } else {
          const int owner = row0 / f.rs_rows_per_rank;
          out_map = &rs_maps.m[owner];
          out_row = f.rs_rank * f.rs_rows_per_rank + (row0 - owner * f.rs_rows_per_rank);
        }
      }
#pragma unroll 1
      for (int ch = 0; ch < kChunks; ++ch) {
        uint32_t r[32];
        uint4 o[8];
        if constexpr (sizeof(OutT) == 2) {
          uint32_t r2[32];
          tmem_ld_32x32(taddr + ch * 64, r);
          tmem_ld_32x32(taddr + ch * 64 + 32, r2);
          tmem_ld_wait();
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            o[v].x = pack_bf16x2(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
            o[v].y = pack_bf16x2(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
            o[v].z = pack_bf16x2(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
            o[v].w = pack_bf16x2(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
            o[4 + v].x = pack_bf16x2(__uint_as_float(r2[8 * v + 0]), __uint_as_float(r2[8 * v + 1]));
            o[4 + v].y = pack_bf16x2(__uint_as_float(r2[8 * v + 2]), __uint_as_float(r2[8 * v + 3]));
            o[4 + v].z = pack_bf16x2(__uint_as_float(r2[8 * v + 4]), __uint_as_float(r2[8 * v + 5]));
            o[4 + v].w = pack_bf16x2(__uint_as_float(r2[8 * v + 6]), __uint_as_float(r2[8 * v + 7]));
          }
        } else {
          tmem_ld_32x32(taddr + ch * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int v = 0; v < 8; ++v) o[v] = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
        }
        if (empty_group) {
#pragma unroll
          for (int v = 0; v < 8; ++v) o[v] = make_uint4(0u, 0u, 0u, 0u);
        }
        if (ch == kChunks - 1) {
          // All of this warp's reads of the accumulator are done: hand it back early.
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(empty_addr + acc * 8);
        }
        // The staging tile about to be written was read by the TMA store issued two chunks ago.
        if (lane == 0) tma_store_wait_read<1>();
        __syncwarp();
        uint8_t* tile = my_staging + (store_seq & 1) * 4096;
        // 128-byte swizzle: 16-byte unit j of row `lane` lives at unit j ^ (lane & 7).
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<uint4*>(tile + lane * 128 + ((j ^ (lane & 7)) << 4)) = o[j];
        fence_proxy_async();
        __syncwarp();
        if (lane == 0 && row0 < p.M && n0 + ch * kChunkCols < p.N) {
          if (n_dst > 1) {
            for (int d = 0; d < n_dst; ++d) tma_store_2d(&rs_maps.m[d], tile, n0 + ch * kChunkCols, out_row);
          } else if (gmode == 2) {
            tma_store_3d(out_map, tile, n0 + ch * kChunkCols, out_row, grp);
          } else if (p.accumulate) {
            tma_reduce_add_2d(out_map, tile, n0 + ch * kChunkCols, out_row);
          } else {
            tma_store_2d(out_map, tile, n0 + ch * kChunkCols, out_row);
          }
        }
        if (lane == 0) tma_store_commit();
        ++store_seq;
      }
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    if (lane == 0) {
      tma_store_wait<0>();
      // Stores to peer memory: visible system-wide before the kernel can complete, so the flag
      // raised by the next launch cannot overtake them.
      if (FUSED && f.rs_world > 1) __threadfence_system();
    }
    __syncwarp();
    if (FUSED && f.rs_world > 1 && f.rs_mode == 1) {
      // All four epilogue warps of this CTA are past their fences; the last CTA of the grid raises
      // this rank's flag on every peer.
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (warp == 2 && lane == 0) {
        if (atomicAdd(f.rs_counter, 1) == static_cast<int>(gridDim.x) - 1) {
          *f.rs_counter = 0;
          __threadfence_system();
          const int epoch = *reinterpret_cast<const volatile int*>(f.rs_epoch_ptr);
          for (int r = 0; r < f.rs_world; ++r) st_release_sys(f.rs_flags[r] + f.rs_site * f.rs_world + f.rs_rank, epoch);
        }
      }
    }
  }

  // ---------------------------------------------------------------------- tear-down
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1 && p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) {
    // A wait gave up: let copies that may still be in flight land before the CTAs exit.
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  // Neither CTA may exit (or free tensor memory) while its partner can still touch it.
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

// Tiles are visited in groups of `group_m` row blocks x all column blocks (row block fastest): a
// wave of 74 pairs then covers about 8 x 9 tiles, and the group's rows of A are reused by the next
// wave.  Measured DRAM reads on the Fuji shapes (ncu, one launch): 16384 x 4096 x 4096: 215 / 322 /
// 343 / 624 MB for groups of 4 / 8 / 16 / 32; 16384 x 4096 x 11008: 2.81 / 2.24 / 2.43 / 3.65 GB (a
// wave's operand panels, (8 + 9) x 256 x K x 2 bytes, no longer fit the L2 at this K); times within
// 2 % of each other up to 16 and worse beyond.  Eight is the choice; AXB_GEMM2_GROUP_M overrides it.
static int raster_group_m(int M, int N, int K) {
  static int forced = -1;
  if (forced < 0) {
    const char* e = getenv("AXB_GEMM2_GROUP_M");
    forced = e != nullptr ? atoi(e) : 0;
  }
  (void)M;
  (void)N;
  (void)K;
  return forced > 0 ? forced : 8;
}

template <bool A_MN, bool B_MN, typename OutT, bool FUSED = false>
static int launch_gemm2(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb,
                        int64_t ldc, int accumulate, int* status, int max_ctas, cudaStream_t stream,
                        const FusedParams* fused = nullptr, int group_mode = 0, int num_groups = 1,
                        const int* group_index = nullptr, int64_t c_group_stride = 0, int group_block_rows = k2TileM) {
  CUtensorMap ta, tb, tc;
  // Grouped mode 1 stacks the groups' B matrices along the outer dim of one tensor map.
  const uint64_t b_stack = group_mode == 1 ? static_cast<uint64_t>(num_groups) : 1;
  int rc;
  {
    uint64_t dims[2] = {static_cast<uint64_t>(A_MN ? M : K), static_cast<uint64_t>(A_MN ? K : M)};
    uint64_t strides[1] = {static_cast<uint64_t>(lda) * 2};
    uint32_t box[2] = {64, static_cast<uint32_t>(A_MN ? k2BlockK : k2RowsPerCta)};
    rc = make_tensor_map(&ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != 0) return rc;
  }
  const uint32_t b_box[2] = {64, static_cast<uint32_t>(B_MN ? k2BlockK : k2HalfN)};
  {
    uint64_t dims[2] = {static_cast<uint64_t>(B_MN ? N : K), b_stack * static_cast<uint64_t>(B_MN ? K : N)};
    uint64_t strides[1] = {static_cast<uint64_t>(ldb) * 2};
    rc = make_tensor_map(&tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, dims, strides, b_box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != 0) return rc;
  }
  const CUtensorMapDataType c_type = sizeof(OutT) == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  const uint32_t c_box[2] = {static_cast<uint32_t>(128 / sizeof(OutT)), 32};
  const uint64_t c_strides[1] = {static_cast<uint64_t>(ldc) * sizeof(OutT)};
  FusedParams fp;
  memset(&fp, 0, sizeof(fp));
  if (FUSED && fused != nullptr) fp = *fused;
  const bool scatter = FUSED && fp.rs_world > 1;
  if (group_mode == 2) {
    // One [M, N] output per group: the group is the third coordinate, so rows past M are clipped
    // instead of running into the next group's matrix.
    uint64_t dims[3] = {static_cast<uint64_t>(N), static_cast<uint64_t>(M), static_cast<uint64_t>(num_groups)};
    uint64_t strides[2] = {c_strides[0], static_cast<uint64_t>(c_group_stride) * sizeof(OutT)};
    uint32_t box[3] = {c_box[0], c_box[1], 1};
    rc = make_tensor_map(&tc, c_type, 3, C, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != 0) return rc;
  } else if (!scatter) {
    uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(M)};
    rc = make_tensor_map(&tc, c_type, 2, C, dims, c_strides, c_box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != 0) return rc;
  }
  // The own shard as a tensor of its own (consume mode): same row pitch, one slab of rows.
  CUtensorMap tl = tb;
  if (FUSED && fp.ag[0].world > 1 && fp.ag_consume) {
    const void* own = fp.ag[0].src[fp.ag[0].rank];
    uint64_t dims[2] = {static_cast<uint64_t>(B_MN ? N : K), static_cast<uint64_t>(fp.ag_shard_extent)};
    uint64_t strides[1] = {static_cast<uint64_t>(ldb) * 2};
    rc = make_tensor_map(&tl, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, own, dims, strides, b_box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != 0) return rc;
  }
  static PeerMaps no_maps;  // zero-initialised; unused unless scattering
  PeerMaps maps = no_maps;
  if (scatter) {
    for (int r = 0; r < fp.rs_world; ++r) {
      const uint64_t slot_rows = fp.rs_mode == 1 ? static_cast<uint64_t>(M) : static_cast<uint64_t>(fp.rs_rows_per_rank);
      uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(fp.rs_world) * slot_rows};
      rc = make_tensor_map(&maps.m[r], c_type, 2, fp.rs_dst[r], dims, c_strides, c_box, CU_TENSOR_MAP_SWIZZLE_128B);
      if (rc != 0) return rc;
    }
    tc = maps.m[fp.rs_rank];
  }
  using S = Gemm2Smem<FUSED>;
  auto kernel = gemm2_bf16_kernel<A_MN, B_MN, OutT, FUSED>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal);
    if (e != cudaSuccess) {
      fprintf(stderr, "axb gemm2: cudaFuncSetAttribute: %s\n", cudaGetErrorString(e));
      return -3;
    }
    configured = true;
  }
  const int tiles = ((M + k2TileM - 1) / k2TileM) * ((N + k2TileN - 1) / k2TileN) * (group_mode == 2 ? num_groups : 1);
  int pairs = sm_count() / 2;
  if (max_ctas > 0 && max_ctas / 2 < pairs) pairs = max_ctas / 2;
  if (tiles < pairs) pairs = tiles;
  if (pairs < 1) return -12;
  // Grouped mode 1: sixteen row blocks per rasterisation group, so that a wave mostly stays inside
  // one group's B matrix (measured at 32768 pairs, 8 groups, 4096 -> 14336: 3.07 / 2.85 / 2.78 ms for
  // 4 / 8 / 16).
  const int raster = group_mode == 1 && getenv("AXB_GEMM2_GROUP_M") == nullptr ? 16 : raster_group_m(M, N, K);
  Gemm2Params p{M,          N,          K,           accumulate,     status,          raster,
                group_mode, num_groups, group_index, B_MN ? K : N, group_block_rows};
  kernel<<<2 * pairs, FUSED ? k2FusedThreads : k2Threads, S::kTotal, stream>>>(ta, tb, tc, p, tl, fp, maps);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    fprintf(stderr, "axb gemm2: launch failed: %s\n", cudaGetErrorString(e));
    return -4;
  }
  return 0;
}

}  // namespace axb

// Same contract as axb_gemm_bf16 (row-major C with leading dim ldc; operands K-major or MN-major).
// Returns -20 for problems this kernel does not take (the caller then uses the single-CTA kernel).
extern "C" int axb_gemm_bf16_2cta(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda,
                                  int64_t ldb, int64_t ldc, int a_mn_major, int b_mn_major, int out_fp32,
                                  int accumulate, int* status, int max_ctas, cudaStream_t stream) {
  using namespace axb;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) ||
      (reinterpret_cast<uintptr_t>(C) & 15) || (ldc % (out_fp32 ? 4 : 8)))
    return -10;
  if (M < k2TileM || N < k2TileN) return -20;
#define AXB_GEMM2_CASE(AM, BM)                                                                                   \
  if (a_mn_major == (AM ? 1 : 0) && b_mn_major == (BM ? 1 : 0)) {                                                \
    if (out_fp32)                                                                                                \
      return launch_gemm2<AM, BM, float>(A, B, C, M, N, K, lda, ldb, ldc, accumulate, status, max_ctas, stream); \
    return launch_gemm2<AM, BM, __nv_bfloat16>(A, B, C, M, N, K, lda, ldb, ldc, accumulate, status, max_ctas,    \
                                               stream);                                                          \
  }
  AXB_GEMM2_CASE(false, false)
  AXB_GEMM2_CASE(false, true)
  AXB_GEMM2_CASE(true, false)
  AXB_GEMM2_CASE(true, true)
#undef AXB_GEMM2_CASE
  return -11;
}

// Grouped form on CTA pairs (same contract as axb_gemm_bf16_grouped, bf16 output).  `block_rows`
// is the padding unit of the row groups: every group starts on a multiple of it, and mode 1's
// `group_index` has one entry per block.  Returns -20 for what this kernel does not take.
extern "C" int axb_gemm_bf16_grouped_2cta(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda,
                                          int64_t ldb, int64_t ldc, int a_mn_major, int b_mn_major, int mode,
                                          int num_groups, const int* group_index, int64_t c_group_stride,
                                          int block_rows, int* status, int max_ctas, cudaStream_t stream) {
  using namespace axb;
  if (block_rows < k2TileM || (block_rows % k2TileM) != 0 || M < k2TileM || N < k2TileN) return -20;
  if (mode == 1 && (a_mn_major || (M % block_rows) != 0)) return -20;
  if (mode == 2 && (!a_mn_major || !b_mn_major)) return -20;
#define AXB_GROUPED2_CASE(AM, BM)                                                                              \
  if (a_mn_major == (AM ? 1 : 0) && b_mn_major == (BM ? 1 : 0))                                                \
    return launch_gemm2<AM, BM, __nv_bfloat16>(A, B, C, M, N, K, lda, ldb, ldc, 0, status, max_ctas, stream,   \
                                               nullptr, mode, num_groups, group_index, c_group_stride, block_rows);
  AXB_GROUPED2_CASE(false, false)
  AXB_GROUPED2_CASE(false, true)
  AXB_GROUPED2_CASE(true, true)
#undef AXB_GROUPED2_CASE
  return -11;
}

// Fused compute+collective form on CTA pairs; same arguments as axb_gemm_bf16_fused.  Returns -20
// when the problem is not one this kernel takes (small problems, the all-reduce-push epilogue,
// owner slabs that are no multiple of 32 rows): the caller then uses the single-CTA kernel.
extern "C" int axb_gemm_bf16_fused_2cta(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda,
                                        int64_t ldb, int64_t ldc, int a_mn_major, int b_mn_major, int* status,
                                        int max_ctas, const void* fused, cudaStream_t stream) {
  using namespace axb;
  const FusedParams* fp = static_cast<const FusedParams*>(fused);
  if (M < 2 * k2TileM || N < k2TileN || ((M + k2TileM - 1) / k2TileM) * ((N + k2TileN - 1) / k2TileN) < 64) return -20;
  if (fp->rs_world > 1 && fp->rs_mode == 0 && (fp->rs_rows_per_rank % 32) != 0) return -20;
  if (fp->rs_world > 1 && fp->rs_mode == 1 && ((M % 32) != 0 || fp->rs_counter == nullptr || fp->rs_epoch_ptr == nullptr))
    return -20;
  if (fp->rs_world <= 1 && (reinterpret_cast<uintptr_t>(C) & 15)) return -10;
#define AXB_FUSED2_CASE(AM, BM)                                                                                  \
  if (a_mn_major == (AM ? 1 : 0) && b_mn_major == (BM ? 1 : 0))                                                  \
    return launch_gemm2<AM, BM, __nv_bfloat16, true>(A, B, C, M, N, K, lda, ldb, ldc, 0, status, max_ctas, stream, fp);
  AXB_FUSED2_CASE(false, false)
  AXB_FUSED2_CASE(false, true)
  AXB_FUSED2_CASE(true, false)
  AXB_FUSED2_CASE(true, true)
#undef AXB_FUSED2_CASE
  return -11;
}
