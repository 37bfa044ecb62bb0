// Flash attention forward for sm_100a (bf16, head dim 64 or 128, causal or full, GQA).
//
// One CTA computes a 128-row query tile of one (batch, head) and walks the key/value sequence
// in tiles of 128 keys:
//   warp 0      TMA producer: Q once; K and V tiles through two-stage rings.
//   warp 1      MMA issuer:   S_j = Q K_j^T into one of two TMEM buffers (so S_{j+1} is computed
//               while the softmax of tile j runs), then O += P_j V_j with P read from shared
//               memory and O accumulated in TMEM.
//   warps 2-5   softmax: each thread owns one query row; reads S from TMEM, applies scale /
//               causal / length masks, keeps a running reference maximum and row sum, writes
//               P (bf16) into a 128B-swizzled shared tile, and rescales O in TMEM only when the
//               row maximum grew by more than 2^8 (the reference max is otherwise kept, which
//               bounds P by 256 and is exact after the final division).
// Output: O / rowsum in bf16, and lse = m*ln2 + log(rowsum) per row for the backward pass.
//
// Reference kernels being replaced: axlearn/common/flash_attention/gpu_attention.py:114-243
// (Pallas-Triton forward) and the cuDNN call at :792-926.
#include "host_utils.cuh"
#include "sm100.cuh"

namespace axb {

constexpr int kFaBlockM = 128;
constexpr int kFaBlockN = 128;
constexpr int kFaThreads = 192;

struct FlashFwdParams {
  void* out;      // [B, T, N, H] bf16
  float* lse;     // [B, N, T]
  int B, T, S, N, Nkv, H;
  float scale_log2;  // softmax_scale * log2(e)
  int causal;
  int q_offset;   // key position of query row 0 is q_offset (S - T for suffix queries)
  int* status;
};

template <int H>
struct FaSmem {
  static constexpr int kSub = 16384;              // one [128 x 64] bf16 sub-tile
  static constexpr int kTile = (H / 64) * kSub;   // a [128 x H] tile
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + kTile;           // 2 stages
  static constexpr int kV = kK + 2 * kTile;       // 2 stages
  static constexpr int kP = kV + 2 * kTile;       // [128 x 128] bf16 = 2 sub-tiles
  static constexpr int kBar = kP + 2 * kSub;
  static constexpr int kTotal = kBar + 256 + 1024;
};

template <int H>
__global__ void __launch_bounds__(kFaThreads, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, FlashFwdParams p) {
  using L = FaSmem<H>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBar);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* k_empty = bars + 3;   // [2]
  uint64_t* v_full = bars + 5;    // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;    // [2]
  uint64_t* s_empty = bars + 11;  // [2]
  uint64_t* p_full = bars + 13;
  uint64_t* p_empty = bars + 14;
  uint64_t* pv_done = bars + 15;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_tile = gridDim.x - 1 - blockIdx.x;  // heavy (late) causal tiles first
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / (p.N / p.Nkv);
  const int t0 = q_tile * kFaBlockM;
  // Number of key tiles this query tile attends to.
  int kv_len = p.S;
  if (p.causal) kv_len = min(p.S, t0 + kFaBlockM + p.q_offset);
  const int n_tiles = (kv_len + kFaBlockN - 1) / kFaBlockN;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 4);
    }
    mbar_init(p_full, 4);
    mbar_init(p_empty, 1);
    mbar_init(pv_done, 1);
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
  const uint32_t tmem_o = tmem_base + 256;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one() && n_tiles > 0) {
      mbar_arrive_expect_tx(q_full, L::kTile);
#pragma unroll
      for (int j = 0; j < H / 64; ++j)
        tma_load_4d(smem + L::kQ + j * L::kSub, &tmap_q, q_full, j * 64, head, t0, batch);
      for (int it = 0; it < n_tiles; ++it) {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        const int s0 = it * kFaBlockN;
        if (!mbar_wait(&k_empty[st], ph ^ 1, p.status, kStatusWaitTimeoutProducer)) break;
        mbar_arrive_expect_tx(&k_full[st], L::kTile);
#pragma unroll
        for (int j = 0; j < H / 64; ++j)
          tma_load_4d(smem + L::kK + st * L::kTile + j * L::kSub, &tmap_k, &k_full[st], j * 64,
                      kv_head, s0, batch);
        if (!mbar_wait(&v_empty[st], ph ^ 1, p.status, kStatusWaitTimeoutProducer)) break;
        mbar_arrive_expect_tx(&v_full[st], L::kTile);
#pragma unroll
        for (int j = 0; j < H / 64; ++j)
          tma_load_4d(smem + L::kV + st * L::kTile + j * L::kSub, &tmap_v, &v_full[st], j * 64,
                      kv_head, s0, batch);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one() && n_tiles > 0) {
      constexpr uint32_t idesc_qk = umma_idesc_f16(128, kFaBlockN, 1, 1, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_f16(128, H, 1, 1, 0, 1);
      const uint32_t q_addr = smem_u32(smem + L::kQ);
      const uint32_t p_addr = smem_u32(smem + L::kP);
      bool ok = mbar_wait(q_full, 0, p.status, kStatusWaitTimeoutMma);
      auto issue_qk = [&](int it) -> bool {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(&k_full[st], ph, p.status, kStatusWaitTimeoutMma)) return false;
        if (!mbar_wait(&s_empty[st], ph ^ 1, p.status, kStatusWaitTimeoutMma)) return false;
        tc_fence_after_sync();
        const uint32_t k_addr = smem_u32(smem + L::kK + st * L::kTile);
#pragma unroll
        for (int kk = 0; kk < H / 16; ++kk) {
          const uint32_t off = (kk >> 2) * L::kSub + (kk & 3) * 32;
          tc_mma_f16(tmem_base + st * 128, umma_smem_desc(q_addr + off, 16, 1024),
                     umma_smem_desc(k_addr + off, 16, 1024), idesc_qk, kk > 0 ? 1u : 0u);
        }
        tc_commit(&k_empty[st]);
        tc_commit(&s_full[st]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int it = 0; it < n_tiles && ok; ++it) {
        if (it + 1 < n_tiles) {
          ok = issue_qk(it + 1);
          if (!ok) break;
        }
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(p_full, it & 1, p.status, kStatusWaitTimeoutMma)) { ok = false; break; }
        if (!mbar_wait(&v_full[st], ph, p.status, kStatusWaitTimeoutMma)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t v_addr = smem_u32(smem + L::kV + st * L::kTile);
#pragma unroll
        for (int kk = 0; kk < kFaBlockN / 16; ++kk) {
          const uint32_t a_off = (kk >> 2) * L::kSub + (kk & 3) * 32;
          tc_mma_f16(tmem_o, umma_smem_desc(p_addr + a_off, 16, 1024),
                     umma_smem_desc(v_addr + kk * 2048, L::kSub, 1024), idesc_pv,
                     (it > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(&v_empty[st]);
        tc_commit(p_empty);
        tc_commit(pv_done);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax / epilogue
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const int row = t0 + row_in_tile;                 // query index
    const int row_pos = row + p.q_offset;             // its key-space position (causal limit)
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    float m_ref = -INFINITY, l_sum = 0.f;
    uint8_t* p_row = smem + L::kP + row_in_tile * 128;
    bool ok = true;
    for (int it = 0; it < n_tiles && ok; ++it) {
      const int st = it & 1;
      const uint32_t ph = (it >> 1) & 1;
      if (!mbar_wait(&s_full[st], ph, p.status, kStatusWaitTimeoutEpilogue)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t s_addr = tmem_base + lane_base + st * 128;
      const int s0 = it * kFaBlockN;
      const bool need_mask = (p.causal && s0 + kFaBlockN - 1 > t0 + p.q_offset) || (s0 + kFaBlockN > p.S);
      // Pass 1: tile maximum of the scaled, masked scores (log2 domain).
      float tmax = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < kFaBlockN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32(s_addr + c, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float v = __uint_as_float(r[j]) * p.scale_log2;
          if (need_mask) {
            const int col = s0 + c + j;
            if (col >= p.S || (p.causal && col > row_pos)) v = -INFINITY;
          }
          tmax = fmaxf(tmax, v);
        }
      }
      // Reference-maximum update with slack: rescale only if the max grew by > 8 (log2).
      float alpha = 1.f;
      bool rescale = false;
      if (tmax > m_ref + 8.f) {
        if (m_ref != -INFINITY) {
          alpha = exp2f(m_ref - tmax);
          rescale = true;
        }
        m_ref = tmax;
      }
      const bool any_rescale = __any_sync(0xffffffffu, rescale);
      if (it > 0) {
        // P buffer and O are owned by the previous PV MMA until it retires.
        if (!mbar_wait(pv_done, (it - 1) & 1, p.status, kStatusWaitTimeoutEpilogue)) { ok = false; break; }
        tc_fence_after_sync();
      }
      if (any_rescale) {
        const uint32_t o_addr = tmem_o + lane_base;
#pragma unroll 1
        for (int c = 0; c < H; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32(o_addr + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * alpha);
          tmem_st_32x32(o_addr + c, r);
        }
        tmem_st_wait();
        l_sum *= alpha;
      }
      // Pass 2: probabilities -> bf16 -> swizzled shared tile; row sum.
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
#pragma unroll 1
      for (int c = 0; c < kFaBlockN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32(s_addr + c, r);
        tmem_ld_wait();
        float pv[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float v = __uint_as_float(r[j]) * p.scale_log2;
          if (need_mask) {
            const int col = s0 + c + j;
            if (col >= p.S || (p.causal && col > row_pos)) v = -INFINITY;
          }
          const float e = exp2f(v - m_use);
          pv[j] = e;
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 o;
          o.x = pack_bf16x2(pv[8 * g + 0], pv[8 * g + 1]);
          o.y = pack_bf16x2(pv[8 * g + 2], pv[8 * g + 3]);
          o.z = pack_bf16x2(pv[8 * g + 4], pv[8 * g + 5]);
          o.w = pack_bf16x2(pv[8 * g + 6], pv[8 * g + 7]);
          // Row sum of what the tensor core will actually see (bf16-rounded probabilities).
          const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&o);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 f = __bfloat1622float2(h2[q]);
            l_sum += f.x + f.y;
          }
          const int c16 = (c >> 3) + g;  // 16-byte chunk index within the 128-key row
          const int sub = c16 >> 3, chunk = (c16 & 7) ^ (row_in_tile & 7);
          *reinterpret_cast<uint4*>(p_row + sub * L::kSub + chunk * 16) = o;
        }
      }
      // Publish P to the async proxy (tensor core reads) and release this S buffer.
      fence_proxy_async();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(p_full);
        mbar_arrive(&s_empty[st]);
      }
    }
    // Epilogue: O / l -> bf16; lse.
    if (ok && n_tiles > 0) {
      ok = mbar_wait(pv_done, (n_tiles - 1) & 1, p.status, kStatusWaitTimeoutEpilogue);
      tc_fence_after_sync();
    }
    if (ok) {
      const float inv_l = l_sum > 0.f ? 1.f / l_sum : 0.f;
      __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) +
                            ((static_cast<int64_t>(batch) * p.T + row) * p.N + head) * H;
#pragma unroll 1
      for (int c = 0; c < H; c += 32) {
        uint32_t r[32];
        if (n_tiles > 0) {
          tmem_ld_32x32(tmem_o + lane_base + c, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0;
        }
        if (row < p.T) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r[8 * g + 0]) * inv_l, __uint_as_float(r[8 * g + 1]) * inv_l);
            o.y = pack_bf16x2(__uint_as_float(r[8 * g + 2]) * inv_l, __uint_as_float(r[8 * g + 3]) * inv_l);
            o.z = pack_bf16x2(__uint_as_float(r[8 * g + 4]) * inv_l, __uint_as_float(r[8 * g + 5]) * inv_l);
            o.w = pack_bf16x2(__uint_as_float(r[8 * g + 6]) * inv_l, __uint_as_float(r[8 * g + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + c + 8 * g) = o;
          }
        }
      }
      if (row < p.T) {
        const float lse = (l_sum > 0.f) ? (m_ref * 0.6931471805599453f + logf(l_sum)) : -INFINITY;
        p.lse[(static_cast<int64_t>(batch) * p.N + head) * p.T + row] = lse;
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

// 4-D map over a [B, L, N, H] bf16 tensor: dims (innermost first) {H, N, L, B}; box = one
// [128 rows x 64 cols] sub-tile of a single (batch, head).
int make_bthd_map(CUtensorMap* map, const void* base, int B, int L, int N, int H, int box_rows) {
  uint64_t dims[4] = {static_cast<uint64_t>(H), static_cast<uint64_t>(N), static_cast<uint64_t>(L),
                      static_cast<uint64_t>(B)};
  uint64_t strides[3] = {static_cast<uint64_t>(H) * 2, static_cast<uint64_t>(N) * H * 2,
                         static_cast<uint64_t>(L) * N * H * 2};
  uint32_t box[4] = {64, 1, static_cast<uint32_t>(box_rows), 1};
  return make_tensor_map(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, base, dims, strides, box,
                         CU_TENSOR_MAP_SWIZZLE_128B);
}

template <int H>
static int launch_flash_fwd(const void* q, const void* k, const void* v, FlashFwdParams p,
                            cudaStream_t stream) {
  CUtensorMap tq, tk, tv;
  if (make_bthd_map(&tq, q, p.B, p.T, p.N, H, kFaBlockM)) return -2;
  if (make_bthd_map(&tk, k, p.B, p.S, p.Nkv, H, kFaBlockN)) return -2;
  if (make_bthd_map(&tv, v, p.B, p.S, p.Nkv, H, kFaBlockN)) return -2;
  auto kernel = flash_fwd_kernel<H>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             FaSmem<H>::kTotal) != cudaSuccess)
      return -3;
    configured = true;
  }
  dim3 grid((p.T + kFaBlockM - 1) / kFaBlockM, p.N, p.B);
  kernel<<<grid, kFaThreads, FaSmem<H>::kTotal, stream>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace axb

// q: [B, T, N, H], k/v: [B, S, Nkv, H], out: [B, T, N, H] (bf16, contiguous); lse: [B, N, T] fp32.
// causal: key position s is visible to query t iff s <= t + (S - T).
extern "C" int axb_flash_fwd(const void* q, const void* k, const void* v, void* out, float* lse,
                             int B, int T, int S, int N, int Nkv, int H, float softmax_scale,
                             int causal, int* status, cudaStream_t stream) {
  using namespace axb;
  if (N % Nkv != 0 || (H != 64 && H != 128)) return -10;
  FlashFwdParams p;
  p.out = out;
  p.lse = lse;
  p.B = B, p.T = T, p.S = S, p.N = N, p.Nkv = Nkv, p.H = H;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.causal = causal;
  p.q_offset = S - T;
  p.status = status;
  if (H == 128) return launch_flash_fwd<128>(q, k, v, p, stream);
  return launch_flash_fwd<64>(q, k, v, p, stream);
}
