// Flash attention forward, second generation: two 128-row query tiles per CTA and softmax
// probabilities kept in tensor memory.
//
// Per CTA (320 threads): 256 query rows of one (batch, head) as tiles A and B.
//   warp 0        TMA producer (Q_A, Q_B once; K/V tiles through two-stage rings)
//   warp 1        MMA issuer. For each key tile j, per query tile X in {A, B}:
//                   O_X += P_X(j) V_j      (A operand = P_X read from TMEM, B = V tile in smem)
//                   S_X  = Q_X K_{j+1}^T   (overwrites the TMEM columns P_X(j) lived in; the
//                                           tensor pipe executes one thread's MMAs in order)
//                 so while the softmax of tile A runs, the tensor core works for tile B.
//   warps 2-5     softmax for tile A, warps 6-9 for tile B: one thread per query row; the whole
//                 128-wide score row is read into registers with one TMEM wait, reduced,
//                 exponentiated, rounded to bf16 and stored back into the first 64 columns of the
//                 S buffer as packed pairs (the layout tcgen05.mma expects for a 16-bit A operand
//                 in TMEM: lane = row, each 32-bit column = two consecutive K elements).
// TMEM map (512 columns): S_A/P_A 0..127, S_B/P_B 128..255, O_A 256.., O_B 384...
// O is rescaled only when a row maximum grows by more than 2^8 (see flash_fwd.cu).
//
// Reference kernels being replaced: axlearn/common/flash_attention/gpu_attention.py:114-243 and
// the cuDNN call at :792-926.
#include "host_utils.cuh"
#include "sm100.cuh"

namespace axb {

int make_bthd_map(CUtensorMap* map, const void* base, int B, int L, int N, int H, int box_rows);

constexpr int kF2Threads = 320;

struct FlashFwd2Params {
  void* out;
  float* lse;
  int B, T, S, N, Nkv, H;
  float scale_log2;
  int causal, q_offset;
  int* status;
};

template <int H>
struct F2Smem {
  static constexpr int kSub = 16384;
  static constexpr int kTile = (H / 64) * kSub;
  static constexpr int kQ = 0;                    // two tiles
  static constexpr int kK = kQ + 2 * kTile;       // two stages
  static constexpr int kV = kK + 2 * kTile;       // two stages
  static constexpr int kBar = kV + 2 * kTile;
  static constexpr int kTotal = kBar + 256 + 1024;
};

template <int H>
__global__ void __launch_bounds__(kF2Threads, 1)
flash_fwd2_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                  const __grid_constant__ CUtensorMap tmap_v, FlashFwd2Params p) {
  using L = F2Smem<H>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBar);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* k_empty = bars + 3;   // [2]
  uint64_t* v_full = bars + 5;    // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;    // [2] per query tile
  uint64_t* p_full = bars + 11;   // [2] per query tile
  uint64_t* pv_done = bars + 13;  // [2] per query tile
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pair = gridDim.x - 1 - blockIdx.x;
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / (p.N / p.Nkv);
  const int t0 = pair * 256;
  // Key tiles needed by each query tile.
  int n_tiles[2];
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    const int tx = t0 + x * 128;
    int kv_len = p.S;
    if (p.causal) kv_len = min(p.S, tx + 128 + p.q_offset);
    n_tiles[x] = (tx < p.T && kv_len > 0) ? (kv_len + 127) / 128 : 0;
  }
  const int n_max = max(n_tiles[0], n_tiles[1]);

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
      mbar_init(&p_full[i], 4);
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

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one() && n_max > 0) {
      mbar_arrive_expect_tx(q_full, 2 * L::kTile);
#pragma unroll
      for (int x = 0; x < 2; ++x)
#pragma unroll
        for (int j = 0; j < H / 64; ++j)
          tma_load_4d(smem + L::kQ + x * L::kTile + j * L::kSub, &tmap_q, q_full, j * 64, head,
                      t0 + x * 128, batch);
      for (int it = 0; it < n_max; ++it) {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(&k_empty[st], ph ^ 1, p.status, kStatusWaitTimeoutProducer)) break;
        mbar_arrive_expect_tx(&k_full[st], L::kTile);
#pragma unroll
        for (int j = 0; j < H / 64; ++j)
          tma_load_4d(smem + L::kK + st * L::kTile + j * L::kSub, &tmap_k, &k_full[st], j * 64, kv_head,
                      it * 128, batch);
        if (!mbar_wait(&v_empty[st], ph ^ 1, p.status, kStatusWaitTimeoutProducer)) break;
        mbar_arrive_expect_tx(&v_full[st], L::kTile);
#pragma unroll
        for (int j = 0; j < H / 64; ++j)
          tma_load_4d(smem + L::kV + st * L::kTile + j * L::kSub, &tmap_v, &v_full[st], j * 64, kv_head,
                      it * 128, batch);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one() && n_max > 0) {
      constexpr uint32_t idesc_qk = umma_idesc_f16(128, 128, 1, 1, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_f16(128, H, 1, 1, 0, 1);
      bool ok = mbar_wait(q_full, 0, p.status, kStatusWaitTimeoutMma);
      auto issue_qk = [&](int x, int it) {
        const uint32_t q_addr = smem_u32(smem + L::kQ + x * L::kTile);
        const uint32_t k_addr = smem_u32(smem + L::kK + (it & 1) * L::kTile);
#pragma unroll
        for (int kk = 0; kk < H / 16; ++kk) {
          const uint32_t off = (kk >> 2) * L::kSub + (kk & 3) * 32;
          tc_mma_f16(tmem_base + x * 128, umma_smem_desc(q_addr + off, 16, 1024),
                     umma_smem_desc(k_addr + off, 16, 1024), idesc_qk, kk > 0 ? 1u : 0u);
        }
        tc_commit(&s_full[x]);
      };
      auto issue_pv = [&](int x, int it) {
        const uint32_t v_addr = smem_u32(smem + L::kV + (it & 1) * L::kTile);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          // 16 keys per step: 8 TMEM columns of packed bf16 pairs; 16 V rows = 2048 B.
          tc_mma_f16_ts(tmem_base + 256 + x * 128, tmem_base + x * 128 + kk * 8,
                        umma_smem_desc(v_addr + kk * 2048, L::kSub, 1024), idesc_pv,
                        (it > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(&pv_done[x]);
      };
      // Prologue: scores of key tile 0 for both query tiles.
      if (ok) ok = mbar_wait(&k_full[0], 0, p.status, kStatusWaitTimeoutMma);
      if (ok) {
        tc_fence_after_sync();
        for (int x = 0; x < 2; ++x)
          if (n_tiles[x] > 0) issue_qk(x, 0);
        tc_commit(&k_empty[0]);
      }
      for (int it = 0; it < n_max && ok; ++it) {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        const bool has_next = it + 1 < n_max;
        if (!mbar_wait(&v_full[st], ph, p.status, kStatusWaitTimeoutMma)) break;
        if (has_next) {
          if (!mbar_wait(&k_full[st ^ 1], ((it + 1) >> 1) & 1, p.status, kStatusWaitTimeoutMma)) break;
        }
        for (int x = 0; x < 2 && ok; ++x) {
          if (it < n_tiles[x]) {
            if (!mbar_wait(&p_full[x], it & 1, p.status, kStatusWaitTimeoutMma)) {
              ok = false;
              break;
            }
            tc_fence_after_sync();
            issue_pv(x, it);
            if (it + 1 < n_tiles[x]) issue_qk(x, it + 1);
          }
        }
        if (!ok) break;
        tc_commit(&v_empty[st]);
        if (has_next) tc_commit(&k_empty[st ^ 1]);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax / epilogue
    const int x = (warp - 2) >> 2;       // query tile of this warpgroup
    const int quarter = warp & 3;         // TMEM lane quarter accessible to this warp
    const int r_in = quarter * 32 + lane;
    const int row = t0 + x * 128 + r_in;
    const int row_pos = row + p.q_offset;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_base + x * 128;
    const uint32_t o_addr = tmem_base + lane_base + 256 + x * 128;
    const int nt = n_tiles[x];
    float m_ref = -INFINITY, l_sum = 0.f;
    bool ok = true;
    for (int it = 0; it < nt && ok; ++it) {
      if (!mbar_wait(&s_full[x], it & 1, p.status, kStatusWaitTimeoutEpilogue)) { ok = false; break; }
      tc_fence_after_sync();
      uint32_t r0[32], r1[32], r2[32], r3[32];
      tmem_ld_32x32(s_addr, r0);
      tmem_ld_32x32(s_addr + 32, r1);
      tmem_ld_32x32(s_addr + 64, r2);
      tmem_ld_32x32(s_addr + 96, r3);
      tmem_ld_wait();
      const int s0 = it * 128;
      const int tile_t0 = t0 + x * 128;
      const bool need_mask = (p.causal && s0 + 127 > tile_t0 + p.q_offset) || (s0 + 128 > p.S);
      if (need_mask) {
        const uint32_t ninf = __float_as_uint(-INFINITY);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int c = s0 + j;
          if (c >= p.S || (p.causal && c > row_pos)) r0[j] = ninf;
          if (c + 32 >= p.S || (p.causal && c + 32 > row_pos)) r1[j] = ninf;
          if (c + 64 >= p.S || (p.causal && c + 64 > row_pos)) r2[j] = ninf;
          if (c + 96 >= p.S || (p.causal && c + 96 > row_pos)) r3[j] = ninf;
        }
      }
      float tmax = -INFINITY;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        tmax = fmaxf(tmax, fmaxf(fmaxf(__uint_as_float(r0[j]), __uint_as_float(r1[j])),
                                 fmaxf(__uint_as_float(r2[j]), __uint_as_float(r3[j]))));
      }
      tmax *= p.scale_log2;  // scale > 0, so max commutes with scaling
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
        // s_full for this tile was committed after the previous P*V of this query tile, so O
        // is quiescent here.
#pragma unroll 1
        for (int c = 0; c < H; c += 32) {
          uint32_t o[32];
          tmem_ld_32x32(o_addr + c, o);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
          tmem_st_32x32(o_addr + c, o);
        }
        l_sum *= alpha;
      }
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
      // Probabilities rounded to bf16 and packed two per register: q[j] = (p[2j], p[2j+1]).
      uint32_t q0[32], q1[32];
      float l_part = 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const uint32_t a = pack_bf16x2(exp2f(__uint_as_float(r0[2 * j]) * p.scale_log2 - m_use),
                                       exp2f(__uint_as_float(r0[2 * j + 1]) * p.scale_log2 - m_use));
        const uint32_t b = pack_bf16x2(exp2f(__uint_as_float(r1[2 * j]) * p.scale_log2 - m_use),
                                       exp2f(__uint_as_float(r1[2 * j + 1]) * p.scale_log2 - m_use));
        const uint32_t c = pack_bf16x2(exp2f(__uint_as_float(r2[2 * j]) * p.scale_log2 - m_use),
                                       exp2f(__uint_as_float(r2[2 * j + 1]) * p.scale_log2 - m_use));
        const uint32_t d = pack_bf16x2(exp2f(__uint_as_float(r3[2 * j]) * p.scale_log2 - m_use),
                                       exp2f(__uint_as_float(r3[2 * j + 1]) * p.scale_log2 - m_use));
        q0[j] = a, q0[16 + j] = b, q1[j] = c, q1[16 + j] = d;
        const float2 fa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a));
        const float2 fb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b));
        const float2 fc = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&c));
        const float2 fd = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&d));
        l_part += (fa.x + fa.y) + (fb.x + fb.y) + (fc.x + fc.y) + (fd.x + fd.y);
      }
      l_sum += l_part;
      tmem_st_32x32(s_addr, q0);
      tmem_st_32x32(s_addr + 32, q1);
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[x]);
    }
    if (ok && nt > 0) {
      ok = mbar_wait(&pv_done[x], (nt - 1) & 1, p.status, kStatusWaitTimeoutEpilogue);
      tc_fence_after_sync();
    }
    if (ok && row < p.T) {
      // Rows of a tile that lies entirely beyond T are skipped (nt == 0 and row >= T).
      const float inv_l = l_sum > 0.f ? 1.f / l_sum : 0.f;
      __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) +
                            ((static_cast<int64_t>(batch) * p.T + row) * p.N + head) * H;
      p.lse[(static_cast<int64_t>(batch) * p.N + head) * p.T + row] =
          (l_sum > 0.f) ? (m_ref * 0.6931471805599453f + logf(l_sum)) : -INFINITY;
      if (nt == 0) {
        for (int c = 0; c < H; c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(0, 0, 0, 0);
      }
    }
    if (ok && nt > 0) {
      const float inv_l = l_sum > 0.f ? 1.f / l_sum : 0.f;
      __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) +
                            ((static_cast<int64_t>(batch) * p.T + row) * p.N + head) * H;
#pragma unroll 1
      for (int c = 0; c < H; c += 32) {
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

template <int H>
static int launch_flash_fwd2(const void* q, const void* k, const void* v, FlashFwd2Params p, cudaStream_t stream) {
  CUtensorMap tq, tk, tv;
  if (make_bthd_map(&tq, q, p.B, p.T, p.N, H, 128)) return -2;
  if (make_bthd_map(&tk, k, p.B, p.S, p.Nkv, H, 128)) return -2;
  if (make_bthd_map(&tv, v, p.B, p.S, p.Nkv, H, 128)) return -2;
  auto kernel = flash_fwd2_kernel<H>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F2Smem<H>::kTotal) != cudaSuccess)
      return -3;
    configured = true;
  }
  dim3 grid((p.T + 255) / 256, p.N, p.B);
  kernel<<<grid, kF2Threads, F2Smem<H>::kTotal, stream>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace axb

// Same contract as axb_flash_fwd (flash_fwd.cu).
extern "C" int axb_flash_fwd_v2(const void* q, const void* k, const void* v, void* out, float* lse, int B, int T,
                                int S, int N, int Nkv, int H, float softmax_scale, int causal, int* status,
                                cudaStream_t stream) {
  using namespace axb;
  if (N % Nkv != 0 || (H != 64 && H != 128)) return -10;
  FlashFwd2Params p;
  p.out = out, p.lse = lse;
  p.B = B, p.T = T, p.S = S, p.N = N, p.Nkv = Nkv, p.H = H;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.causal = causal;
  p.q_offset = S - T;
  p.status = status;
  if (H == 128) return launch_flash_fwd2<128>(q, k, v, p, stream);
  return launch_flash_fwd2<64>(q, k, v, p, stream);
}
