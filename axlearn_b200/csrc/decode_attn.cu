// Decode-time attention over a paged KV cache, and the fused RoPE + cache append that feeds it.
//
// One new token per sequence attends to everything cached for that sequence.  The work is a
// matrix-vector product per (sequence, KV head): every cached K and V byte is read exactly once
// and nothing is reused, so the kernel is built to keep HBM busy rather than the tensor cores:
//
//   grid = (KV splits, KV heads x query-head groups, sequences), 128 threads.
//   A warp walks the sequence's pages; 8 lanes share one key (16 dims = two 16-byte loads each),
//   so a warp covers 4 keys per step and one 16-token page in 4 steps, with the loads of the
//   whole page issued before the first use.  Scores are reduced over the 8 lanes with three
//   shuffles, the softmax is kept online per lane group, and each lane accumulates its 16 dims
//   of P*V.  Warps (and lane groups) merge through shared memory; KV splits write partial
//   (max, sum, out) triples that `decode_combine_kernel` merges.
//
// Cache layout: pool [num_pages, page_size, Nkv, H] for K and for V (H = 128), page table
// [B, max_pages] of pool page ids, `lengths[b]` = number of valid tokens (the new token
// included).  A dense cache is the same thing with an identity page table.
//
// `rope_append_kernel` takes the fused QKV projection of the new token(s), rotates q and k
// (interleaved pairs, position = lengths[b] - 1), writes the rotated q out and stores k / v
// into their page slot -- the cache append is not a separate pass.
//
// Reference behaviour being replaced: `PagedKVCache.extend_step` + reference attention over
// gathered pages (axlearn/common/kv_cache/paged_kv_cache.py:22-150) and the Pallas paged
// attention kernel the reference uses on GPU (axlearn/common/flash_attention/gpu_paged_attention.py).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

namespace axb {

constexpr int kHeadDim = 128;
constexpr int kDecodeThreads = 128;

struct DecodeParams {
  const __nv_bfloat16* q;     // [B, Nq, H]
  const __nv_bfloat16* k_pool;
  const __nv_bfloat16* v_pool;
  const int* page_table;      // [B, max_pages]
  const int* lengths;         // [B]
  float* part_out;            // [B, Nq, splits, H]
  float* part_ml;             // [B, Nq, splits, 2]
  __nv_bfloat16* out;         // [B, Nq, H]
  int num_q_heads, num_kv_heads, page_size, max_pages, splits;
  float scale_log2;           // softmax scale * log2(e)
};

__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

// GT query heads of one KV head per CTA (GT = 1, 2 or 4).
// One query head per CTA (GT == 1) fits 64 registers without spills: eight CTAs per SM instead of
// six, i.e. 1184 resident CTAs, so that a 32 x 32-head batch is one wave instead of 1.15.
template <int GT>
__global__ void __launch_bounds__(kDecodeThreads, GT == 1 ? 8 : 1)
decode_attn_kernel(DecodeParams p) {
  const int split = blockIdx.x;
  const int groups_per_kv = (p.num_q_heads / p.num_kv_heads) / GT;
  const int kvh = blockIdx.y / groups_per_kv;
  const int qh0 = kvh * (p.num_q_heads / p.num_kv_heads) + (blockIdx.y % groups_per_kv) * GT;
  const int b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kq = lane >> 3;   // key slot within a step (0..3)
  const int dc = lane & 7;    // dim chunk: dims [16*dc, 16*dc + 16)
  const int len = p.lengths[b];
  const int num_pages = (len + p.page_size - 1) / p.page_size;
  // Pages [pg_lo, pg_hi) belong to this split.
  const int per_split = (num_pages + p.splits - 1) / p.splits;
  const int pg_lo = split * per_split;
  const int pg_hi = min(num_pages, pg_lo + per_split);

  float q[GT][16];
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    const uint4* qp = reinterpret_cast<const uint4*>(
        p.q + (static_cast<int64_t>(b) * p.num_q_heads + qh0 + g) * kHeadDim + dc * 16);
    unpack8(qp[0], q[g]);
    unpack8(qp[1], q[g] + 8);
  }
  float m[GT], l[GT], acc[GT][16];
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int d = 0; d < 16; ++d) acc[g][d] = 0.f;
  }

  const int64_t row_stride = static_cast<int64_t>(p.num_kv_heads) * kHeadDim;  // one token
  const int steps_per_page = p.page_size / 4;
  for (int pg = pg_lo + warp; pg < pg_hi; pg += kDecodeThreads / 32) {
    const int page = p.page_table[static_cast<int64_t>(b) * p.max_pages + pg];
    const int64_t base = (static_cast<int64_t>(page) * p.page_size) * row_stride + kvh * kHeadDim + dc * 16;
    const int tok0 = pg * p.page_size;
    for (int st = 0; st < steps_per_page; ++st) {
      const int t = st * 4 + kq;
      const bool valid = tok0 + t < len;
      uint4 k0 = make_uint4(0, 0, 0, 0), k1 = k0, v0 = k0, v1 = k0;
      if (valid) {
        const uint4* kp = reinterpret_cast<const uint4*>(p.k_pool + base + t * row_stride);
        const uint4* vp = reinterpret_cast<const uint4*>(p.v_pool + base + t * row_stride);
        k0 = __ldg(kp);
        k1 = __ldg(kp + 1);
        v0 = __ldg(vp);
        v1 = __ldg(vp + 1);
      }
      float kf[16], vf[16];
      unpack8(k0, kf);
      unpack8(k1, kf + 8);
      unpack8(v0, vf);
      unpack8(v1, vf + 8);
#pragma unroll
      for (int g = 0; g < GT; ++g) {
        float s = 0.f;
#pragma unroll
        for (int d = 0; d < 16; ++d) s += q[g][d] * kf[d];
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        s = valid ? s * p.scale_log2 : -INFINITY;
        const float m_new = fmaxf(m[g], s);
        // exp2(-inf - -inf) would be NaN: a lane group that has seen no valid key keeps zeros.
        const float corr = (m_new == -INFINITY) ? 1.f : exp2f(m[g] - m_new);
        const float pr = (m_new == -INFINITY) ? 0.f : exp2f(s - m_new);
        l[g] = l[g] * corr + pr;
#pragma unroll
        for (int d = 0; d < 16; ++d) acc[g][d] = acc[g][d] * corr + pr * vf[d];
        m[g] = m_new;
      }
    }
  }

  // Merge the 4 key slots of each warp (lanes with equal dc), then the 4 warps via shared memory.
  __shared__ float s_m[4][GT], s_l[4][GT];
  __shared__ float s_acc[4][GT][kHeadDim];
#pragma unroll
  for (int g = 0; g < GT; ++g) {
#pragma unroll
    for (int off = 8; off <= 16; off <<= 1) {
      const float m_o = __shfl_xor_sync(0xffffffffu, m[g], off);
      const float l_o = __shfl_xor_sync(0xffffffffu, l[g], off);
      const float m_new = fmaxf(m[g], m_o);
      const float c_self = (m_new == -INFINITY) ? 1.f : exp2f(m[g] - m_new);
      const float c_oth = (m_new == -INFINITY) ? 1.f : exp2f(m_o - m_new);
      l[g] = l[g] * c_self + l_o * c_oth;
#pragma unroll
      for (int d = 0; d < 16; ++d) {
        const float a_o = __shfl_xor_sync(0xffffffffu, acc[g][d], off);
        acc[g][d] = acc[g][d] * c_self + a_o * c_oth;
      }
      m[g] = m_new;
    }
    if (kq == 0) {
#pragma unroll
      for (int d = 0; d < 16; ++d) s_acc[warp][g][dc * 16 + d] = acc[g][d];
      if (dc == 0) {
        s_m[warp][g] = m[g];
        s_l[warp][g] = l[g];
      }
    }
  }
  __syncthreads();
  // Thread d owns output dim d.
  const int d = threadIdx.x;
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, s_m[w][g]);
    float ll = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float c = (mm == -INFINITY) ? 0.f : exp2f(s_m[w][g] - mm);
      ll += s_l[w][g] * c;
      o += s_acc[w][g][d] * c;
    }
    const int64_t row = (static_cast<int64_t>(b) * p.num_q_heads + qh0 + g) * p.splits + split;
    if (p.splits == 1) {
      p.out[(static_cast<int64_t>(b) * p.num_q_heads + qh0 + g) * kHeadDim + d] =
          __float2bfloat16(ll > 0.f ? o / ll : 0.f);
    } else {
      p.part_out[row * kHeadDim + d] = o;
      if (d == 0) {
        p.part_ml[row * 2] = mm;
        p.part_ml[row * 2 + 1] = ll;
      }
    }
  }
}

// Row-contiguous variant for caches with a multiple of four KV heads: a warp reads ONE token
// across FOUR neighbouring KV heads per load (8 lanes x 32 bytes per head = 1 KB contiguous in
// the pool, where the per-head kernel above reads four 256-byte pieces 1 KB or more apart), so
// every DRAM burst it opens is used in full.  Lane group `hl` (8 lanes) owns KV head 4 * hg + hl
// and all GT query heads attending to it; nothing is merged across lane groups, only across the
// four warps (which split the pages).  GT = query heads per KV head (2 or 4; the launcher keeps
// GT = 1 on the per-head kernel, which is as fast or faster there).
template <int GT>
__global__ void __launch_bounds__(kDecodeThreads)
decode_attn_rows_kernel(DecodeParams p) {
  const int split = blockIdx.x;
  const int hg = blockIdx.y;  // group of four KV heads
  const int b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hl = lane >> 3;   // KV head within the group
  const int dc = lane & 7;    // dim chunk: dims [16*dc, 16*dc + 16)
  const int kvh = hg * 4 + hl;
  const int qh0 = kvh * GT;
  const int len = p.lengths[b];
  const int num_pages = (len + p.page_size - 1) / p.page_size;
  const int per_split = (num_pages + p.splits - 1) / p.splits;
  const int pg_lo = split * per_split;
  const int pg_hi = min(num_pages, pg_lo + per_split);

  float q[GT][16];
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    const uint4* qp = reinterpret_cast<const uint4*>(
        p.q + (static_cast<int64_t>(b) * p.num_q_heads + qh0 + g) * kHeadDim + dc * 16);
    unpack8(qp[0], q[g]);
    unpack8(qp[1], q[g] + 8);
  }
  float m[GT], l[GT], acc[GT][16];
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int d = 0; d < 16; ++d) acc[g][d] = 0.f;
  }

  const int64_t row_stride = static_cast<int64_t>(p.num_kv_heads) * kHeadDim;  // one token
  constexpr int kPageStride = kDecodeThreads / 32;
  constexpr int kBatch = GT >= 4 ? 2 : 4;  // tokens whose loads are in flight together
  const int* table_row = p.page_table + static_cast<int64_t>(b) * p.max_pages;
  int page = (pg_lo + warp < pg_hi) ? __ldg(table_row + pg_lo + warp) : 0;
  for (int pg = pg_lo + warp; pg < pg_hi; pg += kPageStride) {
    // The next page's id is requested before this page's rows (it is a dependent load).
    const int next_page = (pg + kPageStride < pg_hi) ? __ldg(table_row + pg + kPageStride) : 0;
    const int64_t base = (static_cast<int64_t>(page) * p.page_size) * row_stride + kvh * kHeadDim + dc * 16;
    const int tok0 = pg * p.page_size;
    for (int t0 = 0; t0 < p.page_size; t0 += kBatch) {
      uint4 kk[kBatch][2], vv[kBatch][2];
      bool ok[kBatch];
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        const int t = t0 + u;
        ok[u] = t < p.page_size && tok0 + t < len;
        kk[u][0] = kk[u][1] = vv[u][0] = vv[u][1] = make_uint4(0, 0, 0, 0);
        if (ok[u]) {
          const uint4* kp = reinterpret_cast<const uint4*>(p.k_pool + base + t * row_stride);
          const uint4* vp = reinterpret_cast<const uint4*>(p.v_pool + base + t * row_stride);
          kk[u][0] = __ldg(kp);
          kk[u][1] = __ldg(kp + 1);
          vv[u][0] = __ldg(vp);
          vv[u][1] = __ldg(vp + 1);
        }
      }
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        if (t0 + u >= p.page_size) break;
        float kf[16], vf[16];
        unpack8(kk[u][0], kf);
        unpack8(kk[u][1], kf + 8);
        unpack8(vv[u][0], vf);
        unpack8(vv[u][1], vf + 8);
#pragma unroll
        for (int g = 0; g < GT; ++g) {
          float s = 0.f;
#pragma unroll
          for (int d = 0; d < 16; ++d) s += q[g][d] * kf[d];
          s += __shfl_xor_sync(0xffffffffu, s, 1);
          s += __shfl_xor_sync(0xffffffffu, s, 2);
          s += __shfl_xor_sync(0xffffffffu, s, 4);
          s = ok[u] ? s * p.scale_log2 : -INFINITY;
          const float m_new = fmaxf(m[g], s);
          const float corr = (m_new == -INFINITY) ? 1.f : exp2f(m[g] - m_new);
          const float pr = (m_new == -INFINITY) ? 0.f : exp2f(s - m_new);
          l[g] = l[g] * corr + pr;
#pragma unroll
          for (int d = 0; d < 16; ++d) acc[g][d] = acc[g][d] * corr + pr * vf[d];
          m[g] = m_new;
        }
      }
    }
    page = next_page;
  }

  // Merge the four warps' partial results per (KV head of the group, query head).
  __shared__ float s_m[4][4][GT], s_l[4][4][GT];
  __shared__ float s_acc[4][4][GT][kHeadDim];
#pragma unroll
  for (int g = 0; g < GT; ++g) {
#pragma unroll
    for (int d = 0; d < 16; ++d) s_acc[warp][hl][g][dc * 16 + d] = acc[g][d];
    if (dc == 0) {
      s_m[warp][hl][g] = m[g];
      s_l[warp][hl][g] = l[g];
    }
  }
  __syncthreads();
  // Thread (warp w, lane) finishes KV head w of the group: lane owns dims [4 * lane, 4 * lane + 4).
  const int oh = warp;
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, s_m[w][oh][g]);
    float ll = 0.f, o[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float c = (mm == -INFINITY) ? 0.f : exp2f(s_m[w][oh][g] - mm);
      ll += s_l[w][oh][g] * c;
#pragma unroll
      for (int e = 0; e < 4; ++e) o[e] += s_acc[w][oh][g][lane * 4 + e] * c;
    }
    const int qh = (hg * 4 + oh) * GT + g;
    const int64_t row = (static_cast<int64_t>(b) * p.num_q_heads + qh) * p.splits + split;
    if (p.splits == 1) {
      __nv_bfloat16* dst = p.out + (static_cast<int64_t>(b) * p.num_q_heads + qh) * kHeadDim + lane * 4;
#pragma unroll
      for (int e = 0; e < 4; ++e) dst[e] = __float2bfloat16(ll > 0.f ? o[e] / ll : 0.f);
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) p.part_out[row * kHeadDim + lane * 4 + e] = o[e];
      if (lane == 0) {
        p.part_ml[row * 2] = mm;
        p.part_ml[row * 2 + 1] = ll;
      }
    }
  }
}

__global__ void __launch_bounds__(kHeadDim)
decode_combine_kernel(const float* __restrict__ part_out, const float* __restrict__ part_ml,
                      __nv_bfloat16* __restrict__ out, int splits) {
  const int64_t row = blockIdx.x;  // b * Nq + head
  const int d = threadIdx.x;
  float mm = -INFINITY;
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, part_ml[(row * splits + s) * 2]);
  float ll = 0.f, o = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = part_ml[(row * splits + s) * 2];
    const float c = (mm == -INFINITY) ? 0.f : exp2f(ms - mm);
    ll += part_ml[(row * splits + s) * 2 + 1] * c;
    o += part_out[(row * splits + s) * kHeadDim + d] * c;
  }
  out[row * kHeadDim + d] = __float2bfloat16(ll > 0.f ? o / ll : 0.f);
}

// qkv: [B, (Nq + 2 Nkv) * H] (q heads, then k heads, then v heads).  One CTA per (b, head);
// thread i rotates the pair (2i, 2i+1).
__global__ void __launch_bounds__(kHeadDim / 2)
rope_append_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q_out,
                   __nv_bfloat16* __restrict__ k_pool, __nv_bfloat16* __restrict__ v_pool,
                   const int* __restrict__ page_table, const int* __restrict__ lengths, int num_q_heads,
                   int num_kv_heads, int page_size, int max_pages, float log2_theta, int apply_rope) {
  const int b = blockIdx.y;
  const int head = blockIdx.x;  // 0..Nq+2Nkv-1
  const int i = threadIdx.x;
  const int total_heads = num_q_heads + 2 * num_kv_heads;
  const int pos = lengths[b] - 1;
  const __nv_bfloat162 x =
      reinterpret_cast<const __nv_bfloat162*>(qkv + (static_cast<int64_t>(b) * total_heads + head) * kHeadDim)[i];
  float2 f = __bfloat1622float2(x);
  const bool is_v = head >= num_q_heads + num_kv_heads;
  if (!is_v && apply_rope) {
    // inv_freq = theta^(-2i/H)
    const float inv = exp2f(-log2_theta * (2.f * i) / kHeadDim);
    float sn, cs;
    sincosf(static_cast<float>(pos) * inv, &sn, &cs);
    f = make_float2(f.x * cs - f.y * sn, f.y * cs + f.x * sn);
  }
  const __nv_bfloat162 y = __floats2bfloat162_rn(f.x, f.y);
  if (head < num_q_heads) {
    reinterpret_cast<__nv_bfloat162*>(q_out + (static_cast<int64_t>(b) * num_q_heads + head) * kHeadDim)[i] = y;
    return;
  }
  const int kvh = is_v ? head - num_q_heads - num_kv_heads : head - num_q_heads;
  const int page = page_table[static_cast<int64_t>(b) * max_pages + pos / page_size];
  const int64_t slot = static_cast<int64_t>(page) * page_size + pos % page_size;
  __nv_bfloat16* dst = (is_v ? v_pool : k_pool) + (slot * num_kv_heads + kvh) * kHeadDim;
  reinterpret_cast<__nv_bfloat162*>(dst)[i] = y;
}

}  // namespace axb

// Scratch needed by axb_decode_attn for `splits > 1`: floats.
extern "C" int64_t axb_decode_attn_scratch_floats(int B, int num_q_heads, int splits) {
  return static_cast<int64_t>(B) * num_q_heads * splits * (axb::kHeadDim + 2);
}

// Returns 0 on success, -10 for unsupported shapes (H != 128, page_size % 4, group size).
extern "C" int axb_decode_attn(const void* q, const void* k_pool, const void* v_pool, const int* page_table,
                               const int* lengths, void* out, float* scratch, int B, int num_q_heads,
                               int num_kv_heads, int head_dim, int page_size, int max_pages, int splits,
                               float softmax_scale, cudaStream_t stream) {
  using namespace axb;
  if (head_dim != kHeadDim || page_size % 4 || num_q_heads % num_kv_heads || splits < 1) return -10;
  if (B <= 0) return 0;
  const int g = num_q_heads / num_kv_heads;
  DecodeParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_pool = static_cast<const __nv_bfloat16*>(k_pool);
  p.v_pool = static_cast<const __nv_bfloat16*>(v_pool);
  p.page_table = page_table;
  p.lengths = lengths;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.part_out = scratch;
  p.part_ml = scratch == nullptr ? nullptr
                                 : scratch + static_cast<int64_t>(B) * num_q_heads * splits * kHeadDim;
  if (splits > 1 && scratch == nullptr) return -10;
  p.num_q_heads = num_q_heads;
  p.num_kv_heads = num_kv_heads;
  p.page_size = page_size;
  p.max_pages = max_pages;
  p.splits = splits;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  // AXB_DECODE_ATTN=head keeps the per-head kernel for every shape (for comparisons).
  // head1 / head2 additionally cap the query heads per CTA at 1 / 2.
  static int rows_ok = -1, gt_cap = 4;
  if (rows_ok < 0) {
    const char* e = getenv("AXB_DECODE_ATTN");
    if (e != nullptr && strcmp(e, "head1") == 0) gt_cap = 1;
    if (e != nullptr && strcmp(e, "head2") == 0) gt_cap = 2;
    rows_ok = (e != nullptr && strncmp(e, "head", 4) == 0) ? 0 : 1;
  }
  // Measured (2048 cached tokens, 32 query heads, bytes of K and V counted once):
  //   * four query heads per KV head, 8 KV heads: the row-contiguous kernel reaches 2250 GB/s at
  //     batch 64 and 1845 at batch 16 against 2073 / 1579 for one query head per CTA (which re-reads
  //     K and V through the L2 four times); at batch 4 the latter wins (1057 against 840) because
  //     the row kernel has too few CTAs to cover the machine;
  //   * two query heads per KV head (16 KV heads, batch 64): one query head per CTA 3870, row kernel
  //     3531 -- eight resident CTAs per SM at 64 registers beat two at 221;
  //   * one query head per KV head: the per-head kernel throughout.
  const bool few_row_ctas = static_cast<int64_t>(B) * (num_kv_heads / 4) <= 8;
  if (rows_ok && num_kv_heads % 4 == 0 && g == 4 && !few_row_ctas) {
    dim3 rgrid(splits, num_kv_heads / 4, B);
    decode_attn_rows_kernel<4><<<rgrid, kDecodeThreads, 0, stream>>>(p);
    if (splits > 1)
      decode_combine_kernel<<<B * num_q_heads, kHeadDim, 0, stream>>>(p.part_out, p.part_ml, p.out, splits);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
  }
  int gt = (g % 4 == 0) ? 4 : (g % 2 == 0) ? 2 : 1;
  if (rows_ok && (g == 2 || (g == 4 && num_kv_heads % 4 == 0))) gt = 1;
  if (gt > gt_cap) gt = gt_cap;
  dim3 grid(splits, num_kv_heads * (g / gt), B);
  if (gt == 4)
    decode_attn_kernel<4><<<grid, kDecodeThreads, 0, stream>>>(p);
  else if (gt == 2)
    decode_attn_kernel<2><<<grid, kDecodeThreads, 0, stream>>>(p);
  else
    decode_attn_kernel<1><<<grid, kDecodeThreads, 0, stream>>>(p);
  if (splits > 1)
    decode_combine_kernel<<<B * num_q_heads, kHeadDim, 0, stream>>>(p.part_out, p.part_ml, p.out, splits);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int axb_rope_append_paged(const void* qkv, void* q_out, void* k_pool, void* v_pool,
                                     const int* page_table, const int* lengths, int B, int num_q_heads,
                                     int num_kv_heads, int head_dim, int page_size, int max_pages,
                                     float theta, int apply_rope, cudaStream_t stream) {
  using namespace axb;
  if (head_dim != kHeadDim) return -10;
  if (B <= 0) return 0;
  dim3 grid(num_q_heads + 2 * num_kv_heads, B);
  rope_append_kernel<<<grid, kHeadDim / 2, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(qkv), static_cast<__nv_bfloat16*>(q_out),
      static_cast<__nv_bfloat16*>(k_pool), static_cast<__nv_bfloat16*>(v_pool), page_table, lengths,
      num_q_heads, num_kv_heads, page_size, max_pages, log2f(theta), apply_rope);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

namespace axb {

// out[r, c] = silu(gu[r, c]) * gu[r, F + c] for gu = [rows, 2F] (gate | up packed by one GEMM).
__global__ void swiglu_packed_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                                     int64_t rows, int F) {
  const int64_t total = rows * (F / 2);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / (F / 2);
    const int c = static_cast<int>(i % (F / 2)) * 2;
    const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gu + r * 2 * F + c));
    const float2 u = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gu + r * 2 * F + F + c));
    const float a = g.x / (1.f + __expf(-g.x)) * u.x;
    const float b = g.y / (1.f + __expf(-g.y)) * u.y;
    *reinterpret_cast<__nv_bfloat162*>(out + r * F + c) = __floats2bfloat162_rn(a, b);
  }
}

}  // namespace axb

extern "C" int axb_swiglu_packed(const void* gu, void* out, int64_t rows, int F, cudaStream_t stream) {
  if (F % 2) return -10;
  const int64_t total = rows * (F / 2);
  if (total <= 0) return 0;
  int64_t ctas = (total + 255) / 256;
  if (ctas > 148 * 8) ctas = 148 * 8;
  axb::swiglu_packed_kernel<<<static_cast<int>(ctas), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<__nv_bfloat16*>(out), rows, F);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
