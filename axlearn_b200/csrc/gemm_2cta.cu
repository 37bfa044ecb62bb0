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

#include "host_utils.cuh"
#include "sm100.cuh"

namespace axb {

constexpr int k2RowsPerCta = 128;
constexpr int k2TileM = 256;
constexpr int k2TileN = 256;
constexpr int k2HalfN = 128;
constexpr int k2BlockK = 64;
constexpr int k2Stages = 6;
constexpr int k2Threads = 192;
constexpr int k2GroupM = 8;

struct Gemm2Smem {
  static constexpr int kABytes = k2RowsPerCta * k2BlockK * 2;
  static constexpr int kBBytes = k2HalfN * k2BlockK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;  // 32 KB
  static constexpr int kRingBytes = k2Stages * kStageBytes;
  static constexpr int kStagingPerWarp = 2 * 4096;  // two 32-row x 128-byte tiles
  static constexpr int kStagingBytes = 4 * kStagingPerWarp;
  static constexpr int kBarrierBytes = 1024;
  static constexpr int kTotal = kRingBytes + kStagingBytes + kBarrierBytes + 1024;  // + align slack
};
static_assert(Gemm2Smem::kTotal <= 227 * 1024, "shared memory budget");

struct Gemm2Params {
  int M, N, K;
  int accumulate;
  int* status;
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

template <bool A_MN, bool B_MN, typename OutT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(k2Threads, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ CUtensorMap tmap_c, Gemm2Params p) {
  using S = Gemm2Smem;
  extern __shared__ uint8_t smem_raw[];
  // The dynamic shared-memory window starts at the same offset in both CTAs, so rounding up to
  // 1024 bytes (required by the 128-byte swizzle) gives the same layout in both.
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);
  uint8_t* staging = smem + S::kRingBytes;
  uint8_t* bar_base = staging + S::kStagingBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(bar_base);
  uint64_t* empty_bar = full_bar + k2Stages;
  uint64_t* tmem_full = empty_bar + k2Stages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

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

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    tma_prefetch_desc(&tmap_c);
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

  auto tile_coords = [&](int t, int& m_blk, int& n_blk) {
    const int per_group = k2GroupM * n_blocks;
    const int g = t / per_group;
    const int first_m = g * k2GroupM;
    const int gsize = min(m_blocks - first_m, k2GroupM);
    const int r = t % per_group;
    m_blk = first_m + r % gsize;
    n_blk = r / gsize;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (both CTAs)
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        int m_blk, n_blk;
        tile_coords(t, m_blk, n_blk);
        const int m0 = m_blk * k2TileM + static_cast<int>(rank) * k2RowsPerCta;
        const int n0 = n_blk * k2TileN + static_cast<int>(rank) * k2HalfN;
        for (int kb = 0; kb < num_kb; ++kb) {
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
          if constexpr (!B_MN) {
            tma_load_2d_pair(sb, &tmap_b, bar, k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < k2HalfN / 64; ++j) tma_load_2d_pair(sb + j * 8192, &tmap_b, bar, n0 + j * 64, k0);
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
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, p.status, kStatusWaitTimeoutMma)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * k2TileN;
        for (int kb = 0; kb < num_kb; ++kb) {
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
            tc_mma_f16_pair(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
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
    for (int t = pair; t < num_tiles; t += num_pairs) {
      int m_blk, n_blk;
      tile_coords(t, m_blk, n_blk);
      if (!mbar_wait_warp(&tmem_full[acc], acc_phase, p.status, kStatusWaitTimeoutEpilogue)) break;
      tc_fence_after_sync();
      const int row0 = m_blk * k2TileM + static_cast<int>(rank) * k2RowsPerCta + quarter * 32;
      const int n0 = n_blk * k2TileN;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * k2TileN;
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
          if (p.accumulate)
            tma_reduce_add_2d(&tmap_c, tile, n0 + ch * kChunkCols, row0);
          else
            tma_store_2d(&tmap_c, tile, n0 + ch * kChunkCols, row0);
        }
        if (lane == 0) tma_store_commit();
        ++store_seq;
      }
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    if (lane == 0) tma_store_wait<0>();
    __syncwarp();
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

template <bool A_MN, bool B_MN, typename OutT>
static int launch_gemm2(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb,
                        int64_t ldc, int accumulate, int* status, int max_ctas, cudaStream_t stream) {
  CUtensorMap ta, tb, tc;
  int rc;
  {
    uint64_t dims[2] = {static_cast<uint64_t>(A_MN ? M : K), static_cast<uint64_t>(A_MN ? K : M)};
    uint64_t strides[1] = {static_cast<uint64_t>(lda) * 2};
    uint32_t box[2] = {64, static_cast<uint32_t>(A_MN ? k2BlockK : k2RowsPerCta)};
    rc = make_tensor_map(&ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != 0) return rc;
  }
  {
    uint64_t dims[2] = {static_cast<uint64_t>(B_MN ? N : K), static_cast<uint64_t>(B_MN ? K : N)};
    uint64_t strides[1] = {static_cast<uint64_t>(ldb) * 2};
    uint32_t box[2] = {64, static_cast<uint32_t>(B_MN ? k2BlockK : k2HalfN)};
    rc = make_tensor_map(&tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != 0) return rc;
  }
  {
    uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(M)};
    uint64_t strides[1] = {static_cast<uint64_t>(ldc) * sizeof(OutT)};
    uint32_t box[2] = {static_cast<uint32_t>(128 / sizeof(OutT)), 32};
    rc = make_tensor_map(&tc, sizeof(OutT) == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                         C, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != 0) return rc;
  }
  auto kernel = gemm2_bf16_kernel<A_MN, B_MN, OutT>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Gemm2Smem::kTotal);
    if (e != cudaSuccess) {
      fprintf(stderr, "axb gemm2: cudaFuncSetAttribute: %s\n", cudaGetErrorString(e));
      return -3;
    }
    configured = true;
  }
  const int tiles = ((M + k2TileM - 1) / k2TileM) * ((N + k2TileN - 1) / k2TileN);
  int pairs = sm_count() / 2;
  if (max_ctas > 0 && max_ctas / 2 < pairs) pairs = max_ctas / 2;
  if (tiles < pairs) pairs = tiles;
  if (pairs < 1) return -12;
  Gemm2Params p{M, N, K, accumulate, status};
  kernel<<<2 * pairs, k2Threads, Gemm2Smem::kTotal, stream>>>(ta, tb, tc, p);
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
