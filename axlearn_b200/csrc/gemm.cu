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
};

template <int BN, int STAGES, bool A_MN, bool B_MN, typename OutT>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a,
                 const __grid_constant__ CUtensorMap tmap_b, GemmParams p) {
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

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
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

  auto tile_coords = [&](int t, int& m_blk, int& n_blk) {
    const int per_group = kGroupM * n_blocks;
    const int g = t / per_group;
    const int first_m = g * kGroupM;
    const int gsize = min(m_blocks - first_m, kGroupM);
    const int r = t % per_group;
    m_blk = first_m + r % gsize;
    n_blk = r / gsize;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int m_blk, n_blk;
        tile_coords(t, m_blk, n_blk);
        const int m0 = m_blk * kBlockM, n0 = n_blk * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
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
          if constexpr (!B_MN) {
            tma_load_2d(sb, &tmap_b, &full_bar[stage], k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * 8192, &tmap_b, &full_bar[stage], n0 + j * 64, k0);
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
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, p.status, kStatusWaitTimeoutMma)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
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
            tc_mma_f16(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
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
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      int m_blk, n_blk;
      tile_coords(t, m_blk, n_blk);
      if (!mbar_wait(&tmem_full[acc], acc_phase, p.status, kStatusWaitTimeoutEpilogue)) break;
      tc_fence_after_sync();
      const int row = m_blk * kBlockM + quarter * 32 + lane;
      const int n0 = n_blk * BN;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      OutT* crow = C + static_cast<int64_t>(row) * p.ldc + n0;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c, r);
        tmem_ld_wait();
        if (c + 32 >= BN) {
          // All of this warp's reads of the accumulator are done: hand it back early.
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tmem_empty[acc]);
        }
        if (row < p.M) {
          if constexpr (sizeof(OutT) == 2) {
            if (n0 + c + 32 <= p.N && !p.accumulate) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint4 o;
                o.x = pack_bf16x2(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
                o.y = pack_bf16x2(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
                o.z = pack_bf16x2(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
                o.w = pack_bf16x2(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
                *reinterpret_cast<uint4*>(crow + c + 8 * v) = o;
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

template <int BN, int STAGES, bool A_MN, bool B_MN, typename OutT>
static int launch_gemm(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda,
                       int64_t ldb, int64_t ldc, int accumulate, int* status, int max_ctas,
                       cudaStream_t stream) {
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
    uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N)};
    uint64_t strides[1] = {static_cast<uint64_t>(ldb) * 2};
    uint32_t box[2] = {kBlockK, BN};
    rc = make_tensor_map(&tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, dims, strides, box,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  } else {
    uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(K)};
    uint64_t strides[1] = {static_cast<uint64_t>(ldb) * 2};
    uint32_t box[2] = {64, kBlockK};
    rc = make_tensor_map(&tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, dims, strides, box,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  }
  if (rc != 0) return rc;
  using S = GemmSmem<BN, STAGES>;
  auto kernel = gemm_bf16_kernel<BN, STAGES, A_MN, B_MN, OutT>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e =
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal);
    if (e != cudaSuccess) {
      fprintf(stderr, "axb gemm: cudaFuncSetAttribute: %s\n", cudaGetErrorString(e));
      return -3;
    }
    configured = true;
  }
  const int m_blocks = (M + kBlockM - 1) / kBlockM;
  const int n_blocks = (N + BN - 1) / BN;
  int grid = m_blocks * n_blocks;
  int cap = max_ctas > 0 ? max_ctas : sm_count();
  if (grid > cap) grid = cap;
  GemmParams p{M, N, K, C, ldc, status, accumulate};
  kernel<<<grid, kNumThreads, S::kTotal, stream>>>(ta, tb, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    fprintf(stderr, "axb gemm: launch failed: %s\n", cudaGetErrorString(e));
    return -4;
  }
  return 0;
}

template <bool A_MN, bool B_MN, typename OutT>
static int dispatch_bn(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda,
                       int64_t ldb, int64_t ldc, int accumulate, int* status, int max_ctas,
                       cudaStream_t stream) {
  // 128x256 tiles when they fill the machine, 128x128 otherwise (more CTAs for small problems).
  const int m_blocks = (M + kBlockM - 1) / kBlockM;
  const int tiles256 = m_blocks * ((N + 255) / 256);
  if (N >= 256 && tiles256 >= sm_count() / 2)
    return launch_gemm<256, 4, A_MN, B_MN, OutT>(A, B, C, M, N, K, lda, ldb, ldc, accumulate,
                                                  status, max_ctas, stream);
  return launch_gemm<128, 6, A_MN, B_MN, OutT>(A, B, C, M, N, K, lda, ldb, ldc, accumulate, status,
                                                max_ctas, stream);
}

}  // namespace axb

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
