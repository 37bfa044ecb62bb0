// Block-scaled fp8 GEMM for sm_100a, and the quantisers that feed it.
//
//   C[M, N] = sum over 128-wide K blocks kb of
//             (A[:, kb] * B[:, kb]^T) * sA[m / ga, kb] * sB[n / 128, kb]
//
// A [M, K] and B [N, K] hold e4m3 or e5m2 bytes, K contiguous ("K-major"); sA has one fp32 scale
// per row and K block (ga = 1, the 1x128 activation recipe) or per 128 rows and K block
// (ga = 128); sB has one scale per 128x128 block (the weight recipe).  K and N are multiples
// of 128.
//
// Each K block is one group of four tcgen05.mma.kind::f8f6f4 (128x256x32) into a tensor-memory
// buffer with fp32 accumulation *within* the block; the scaling and the accumulation *across*
// blocks happen in fp32 registers of the four accumulator warps, which read every finished
// block with tcgen05.ld while the tensor core already works on the next block in the other
// buffer.  This is the "promote every 128 K" scheme that block scaling needs, with the tensor
// memory ring turning the promotion into a pipeline stage instead of a stall.
//
// Warp roles (320 threads, persistent over output tiles): warp 0 TMA producer (4 stages of
// 128x128 A + 256x128 B bytes, 128-byte swizzle), warp 1 MMA issuer, warps 2-9 accumulate /
// scale / store (thread = one output row x 128 columns, fp32 accumulators in registers).
//
// Quantisers: `quantize_rows` (1x128 blocks along the contiguous dim), `quantize_blocks`
// (128x128 blocks, optionally writing the transposed matrix) produce the byte matrices and
// scale tables in the layouts above; scale = amax / max_normal (448 for e4m3, 57344 for e5m2).
//
// Reference behaviour being replaced: the reference's fp8 path quantises per tensor inside
// `quantized_dot_general` and calls XLA's cuBLASLt fp8 GEMM
// (axlearn/common/quantized_dot_general/layers.py:1-400).
#include <cuda_fp8.h>
#include <string.h>

#include "host_utils.cuh"
#include "sm100.cuh"

namespace axb {

constexpr int kF8BM = 128, kF8BN = 256, kF8BK = 128;
constexpr int kF8Stages = 4;
constexpr int kF8AccBufs = 2;  // tensor-memory accumulator ring (2 x 256 columns = all of TMEM)
constexpr int kF8Threads = 320;  // producer, MMA issuer, 8 accumulator warps
constexpr int kF8StageBytes = kF8BM * kF8BK + kF8BN * kF8BK;  // 32 KB
constexpr int kF8Smem = kF8Stages * kF8StageBytes + 1024 + 1024;

struct Fp8GemmParams {
  int M, N, K;
  void* C;
  int64_t ldc;
  const float* sa;   // [ceil(M / a_gran), K / 128]
  const float* sb;   // [N / 128, K / 128]
  int a_gran;        // 1 or 128
  int* status;
};

template <typename OutT>
__global__ void __launch_bounds__(kF8Threads, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                Fp8GemmParams p, uint32_t idesc) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* bar_base = smem + kF8Stages * kF8StageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(bar_base);
  uint64_t* empty_bar = full_bar + kF8Stages;
  uint64_t* acc_full = empty_bar + kF8Stages;
  uint64_t* acc_empty = acc_full + kF8AccBufs;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + kF8AccBufs);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_blocks = (p.M + kF8BM - 1) / kF8BM;
  const int n_blocks = (p.N + kF8BN - 1) / kF8BN;
  const int num_tiles = m_blocks * n_blocks;
  const int num_kb = p.K / kF8BK;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    for (int s = 0; s < kF8Stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < kF8AccBufs; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 8);
    }
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kF8AccBufs * kF8BN);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // N-fastest tile order: consecutive CTAs share the A row panel through L2.
  auto tile_coords = [&](int t, int& m_blk, int& n_blk) {
    m_blk = t / n_blocks;
    n_blk = t % n_blocks;
  };

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int m_blk, n_blk;
        tile_coords(t, m_blk, n_blk);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, kStatusWaitTimeoutProducer)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * kF8StageBytes;
          uint8_t* sb = sa + kF8BM * kF8BK;
          mbar_arrive_expect_tx(&full_bar[stage], kF8StageBytes);
          tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * kF8BK, m_blk * kF8BM);
          tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * kF8BK, n_blk * kF8BN);
          if (++stage == kF8Stages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t it = 0;  // K blocks issued so far: buffer = it % kF8AccBufs
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int buf = it % kF8AccBufs;
          if (!mbar_wait(&acc_empty[buf], ((it / kF8AccBufs) & 1) ^ 1, p.status, kStatusWaitTimeoutMma) ||
              !mbar_wait(&full_bar[stage], phase, p.status, kStatusWaitTimeoutMma)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * kF8StageBytes);
          const uint32_t sb = sa + kF8BM * kF8BK;
          const uint32_t d_tmem = tmem_base + buf * kF8BN;
#pragma unroll
          for (int k = 0; k < kF8BK / 32; ++k) {
            // 32 fp8 elements = 32 B inside the 128 B swizzle row.
            tc_mma_f8(d_tmem, umma_smem_desc(sa + k * 32, 16, 1024), umma_smem_desc(sb + k * 32, 16, 1024),
                      idesc, k > 0 ? 1u : 0u);
          }
          tc_commit(&empty_bar[stage]);
          tc_commit(&acc_full[buf]);
          if (++stage == kF8Stages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else {
    // Warp w owns TMEM lanes [32 * (w & 3), +32) (the hardware's lane partition) and one half of
    // the tile's columns: 64 fp32 accumulators per thread.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    constexpr int kCols = kF8BN / 2;
    uint32_t it = 0;
    OutT* C = reinterpret_cast<OutT*>(p.C);
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int m_blk, n_blk;
      tile_coords(t, m_blk, n_blk);
      const int row = m_blk * kF8BM + quarter * 32 + lane;
      const int srow = min(row, p.M - 1) / p.a_gran;
      const float* sa_row = p.sa + static_cast<int64_t>(srow) * num_kb;
      // One weight scale per 128 columns: this warp's half of the 256-wide tile is one block.
      const int sb_blk = min(n_blk * 2 + half, p.N / 128 - 1);
      const float* sb_row = p.sb + static_cast<int64_t>(sb_blk) * num_kb;
      float acc[kCols];
#pragma unroll
      for (int j = 0; j < kCols; ++j) acc[j] = 0.f;
      float scale_next = sa_row[0] * sb_row[0];
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int buf = it % kF8AccBufs;
        const float scale = scale_next;
        if (kb + 1 < num_kb) scale_next = sa_row[kb + 1] * sb_row[kb + 1];
        if (!mbar_wait(&acc_full[buf], (it / kF8AccBufs) & 1, p.status, kStatusWaitTimeoutEpilogue)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t taddr =
            tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * kF8BN + half * kCols;
#pragma unroll
        for (int c = 0; c < kCols; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c, r);
          tmem_ld_wait();
          if (c + 32 == kCols) {
            // This warp's part of the buffer is in registers: hand it back to the tensor core.
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[c + j] = fmaf(__uint_as_float(r[j]), scale, acc[c + j]);
        }
      }
      if (ok && row < p.M && n_blk * kF8BN + half * kCols < p.N) {
        OutT* crow = C + static_cast<int64_t>(row) * p.ldc + n_blk * kF8BN + half * kCols;
        if constexpr (sizeof(OutT) == 2) {
#pragma unroll
          for (int v = 0; v < kCols / 8; ++v) {
            uint4 o;
            o.x = pack_bf16x2(acc[8 * v + 0], acc[8 * v + 1]);
            o.y = pack_bf16x2(acc[8 * v + 2], acc[8 * v + 3]);
            o.z = pack_bf16x2(acc[8 * v + 4], acc[8 * v + 5]);
            o.w = pack_bf16x2(acc[8 * v + 6], acc[8 * v + 7]);
            *reinterpret_cast<uint4*>(crow + 8 * v) = o;
          }
        } else {
#pragma unroll
          for (int v = 0; v < kCols / 4; ++v)
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(crow) + 4 * v) =
                make_float4(acc[4 * v], acc[4 * v + 1], acc[4 * v + 2], acc[4 * v + 3]);
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
    tmem_dealloc(tmem_base, kF8AccBufs * kF8BN);
  }
}

// ------------------------------------------------------------------------------ quantisers
template <bool E5M2>
__device__ __forceinline__ uint8_t to_fp8(float v) {
  if constexpr (E5M2) {
    return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E5M2));
  } else {
    return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
  }
}

// One warp per (row, 128-column block): amax over the block, scale = amax / max_normal, bytes out.
template <bool E5M2>
__global__ void quantize_rows_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, uint8_t* __restrict__ q,
                                     int64_t ldq, float* __restrict__ scales, int64_t rows, int cols) {
  const float max_normal = E5M2 ? 57344.f : 448.f;
  const int blocks = cols / 128;
  const int lane = threadIdx.x & 31;
  const int64_t warp = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t w = warp; w < rows * blocks; w += nwarps) {
    const int64_t r = w / blocks;
    const int b = static_cast<int>(w % blocks);
    const uint2 raw = *reinterpret_cast<const uint2*>(x + r * ldx + b * 128 + lane * 4);
    const float2 f0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 f1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    float amax = fmaxf(fmaxf(fabsf(f0.x), fabsf(f0.y)), fmaxf(fabsf(f1.x), fabsf(f1.y)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = amax > 0.f ? amax / max_normal : 1.f;
    const float inv = 1.f / scale;
    uint32_t packed = to_fp8<E5M2>(f0.x * inv) | (to_fp8<E5M2>(f0.y * inv) << 8) |
                      (to_fp8<E5M2>(f1.x * inv) << 16) | (to_fp8<E5M2>(f1.y * inv) << 24);
    *reinterpret_cast<uint32_t*>(q + r * ldq + b * 128 + lane * 4) = packed;
    if (lane == 0) scales[r * blocks + b] = scale;
  }
}

// One CTA (256 threads) per 128x128 block of x [R, C]; writes q in the same layout, or the
// transposed matrix q^T [C, R] when `transpose`; scales[rb, cb] (or [cb, rb] when transposed).
template <bool E5M2>
__global__ void quantize_blocks_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, uint8_t* __restrict__ q,
                                       int64_t ldq, float* __restrict__ scales, int rows, int cols, int transpose) {
  __shared__ __nv_bfloat16 tile[128][130];
  __shared__ float red[8];
  const float max_normal = E5M2 ? 57344.f : 448.f;
  const int rb = blockIdx.y, cb = blockIdx.x;
  const int tid = threadIdx.x;
  float amax = 0.f;
  for (int i = tid; i < 128 * 128; i += 256) {
    const int r = i >> 7, c = i & 127;
    const int gr = rb * 128 + r, gc = cb * 128 + c;
    const __nv_bfloat16 raw = (gr < rows && gc < cols) ? x[static_cast<int64_t>(gr) * ldx + gc] : __float2bfloat16(0.f);
    tile[r][c] = raw;
    amax = fmaxf(amax, fabsf(__bfloat162float(raw)));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((tid & 31) == 0) red[tid >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) amax = fmaxf(amax, red[w]);
  const float scale = amax > 0.f ? amax / max_normal : 1.f;
  const float inv = 1.f / scale;
  for (int i = tid; i < 128 * 128; i += 256) {
    const int a = i >> 7, b = i & 127;  // output-row-in-block, output-col-in-block
    if (!transpose) {
      const int gr = rb * 128 + a, gc = cb * 128 + b;
      if (gr < rows && gc < cols) q[static_cast<int64_t>(gr) * ldq + gc] = to_fp8<E5M2>(__bfloat162float(tile[a][b]) * inv);
    } else {
      const int gr = cb * 128 + a, gc = rb * 128 + b;  // position in q^T
      if (gr < cols && gc < rows) q[static_cast<int64_t>(gr) * ldq + gc] = to_fp8<E5M2>(__bfloat162float(tile[b][a]) * inv);
    }
  }
  if (tid == 0) {
    if (!transpose)
      scales[static_cast<int64_t>(rb) * gridDim.x + cb] = scale;
    else
      scales[static_cast<int64_t>(cb) * gridDim.y + rb] = scale;
  }
}

}  // namespace axb

// fmt: 0 = e4m3, 1 = e5m2.  out_fp32: C is fp32 instead of bf16.  Returns 0, or -10 for shapes the
// kernel does not cover (K or N not a multiple of 128, unaligned pointers / pitches).
extern "C" int axb_gemm_fp8(const void* A, const void* B, void* C, const float* sa, const float* sb, int M, int N,
                            int K, int64_t lda, int64_t ldb, int64_t ldc, int a_fmt, int b_fmt, int a_gran,
                            int out_fp32, int* status, int max_ctas, cudaStream_t stream) {
  using namespace axb;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K % 128) || (N % 128) || (lda % 16) || (ldb % 16) || (ldc % 8) || (a_gran != 1 && a_gran != 128) ||
      (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -10;
  CUtensorMap ta, tb;
  {
    uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
    uint64_t strides[1] = {static_cast<uint64_t>(lda)};
    uint32_t box[2] = {kF8BK, kF8BM};
    int rc = make_tensor_map(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, A, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != 0) return rc;
  }
  {
    uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N)};
    uint64_t strides[1] = {static_cast<uint64_t>(ldb)};
    uint32_t box[2] = {kF8BK, kF8BN};
    int rc = make_tensor_map(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, B, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != 0) return rc;
  }
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_fp8_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kF8Smem) !=
            cudaSuccess ||
        cudaFuncSetAttribute(gemm_fp8_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, kF8Smem) !=
            cudaSuccess)
      return -3;
    configured = true;
  }
  const int tiles = ((M + kF8BM - 1) / kF8BM) * ((N + kF8BN - 1) / kF8BN);
  int cap = max_ctas > 0 && max_ctas < sm_count() ? max_ctas : sm_count();
  const int grid = tiles < cap ? tiles : cap;
  Fp8GemmParams p{M, N, K, C, ldc, sa, sb, a_gran, status};
  const uint32_t idesc = umma_idesc_f8(kF8BM, kF8BN, a_fmt, b_fmt);
  if (out_fp32)
    gemm_fp8_kernel<float><<<grid, kF8Threads, kF8Smem, stream>>>(ta, tb, p, idesc);
  else
    gemm_fp8_kernel<__nv_bfloat16><<<grid, kF8Threads, kF8Smem, stream>>>(ta, tb, p, idesc);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// x [rows, cols] bf16 (pitch ldx) -> q bytes (pitch ldq) + scales [rows, cols / 128]; cols % 128 == 0.
extern "C" int axb_quantize_rows(const void* x, int64_t ldx, void* q, int64_t ldq, float* scales, int64_t rows,
                                 int cols, int e5m2, cudaStream_t stream) {
  if (cols % 128 || (ldx % 4) || (ldq % 4)) return -10;
  if (rows <= 0) return 0;
  const int64_t warps = rows * (cols / 128);
  int64_t ctas = (warps * 32 + 255) / 256;
  if (ctas > 148 * 16) ctas = 148 * 16;
  if (e5m2)
    axb::quantize_rows_kernel<true><<<static_cast<int>(ctas), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(x), ldx, static_cast<uint8_t*>(q), ldq, scales, rows, cols);
  else
    axb::quantize_rows_kernel<false><<<static_cast<int>(ctas), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(x), ldx, static_cast<uint8_t*>(q), ldq, scales, rows, cols);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// x [rows, cols] bf16 -> 128x128-block-scaled bytes; transpose = 1 writes q^T [cols, rows] and the
// scale table transposed with it.  Scale table: [ceil(rows/128), ceil(cols/128)] (or transposed).
extern "C" int axb_quantize_blocks(const void* x, int64_t ldx, void* q, int64_t ldq, float* scales, int rows,
                                   int cols, int transpose, int e5m2, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  dim3 grid((cols + 127) / 128, (rows + 127) / 128);
  if (e5m2)
    axb::quantize_blocks_kernel<true><<<grid, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(x), ldx, static_cast<uint8_t*>(q), ldq, scales, rows, cols, transpose);
  else
    axb::quantize_blocks_kernel<false><<<grid, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(x), ldx, static_cast<uint8_t*>(q), ldq, scales, rows, cols, transpose);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
