// Memory-bound kernels of the transformer block and the optimizer: RMSNorm fwd/bwd, SwiGLU
// fwd/bwd, rotary embedding, fused softmax-cross-entropy (+gradient in place), AdamW with
// fp32 masters and a bf16 shadow, and a deterministic sum of squares for global-norm clipping.
//
// All of them stream their operands once with 16-byte accesses and keep reductions in fp32.
// In the reference these are XLA loop/reduce fusions generated from axlearn/common/layers.py:
// 374-417 (RMSNorm), axlearn/common/attention.py:1301-1349 (RoPE), :3354-3370 (SwiGLU),
// axlearn/common/loss.py:234-327 (cross entropy) and axlearn/common/optimizers.py:741-856,
// 1149-1184 (AdamW chain, global-norm clip).
#include "no_alloc.h"
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace axb {

using bf16 = __nv_bfloat16;

// Eight bf16 values moved as ONE 16-byte access: the copy operations are written out, because a
// member-wise copy of the four bf16 pairs compiles to four 4-byte accesses (four times the
// load / store instructions and cache sectors touched per warp).
struct alignas(16) Bf16x8 {
  __nv_bfloat162 v[4];
  Bf16x8() = default;
  __device__ __forceinline__ Bf16x8(const Bf16x8& o) { *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(o.v); }
  __device__ __forceinline__ Bf16x8& operator=(const Bf16x8& o) {
    *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(o.v);
    return *this;
  }
};

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}

// Block-wide sum; every thread gets the result. `red` holds >= 32 floats.
__device__ __forceinline__ float block_sum(float x, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  x = warp_sum(x);
  __syncthreads();
  if (lane == 0) red[warp] = x;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  return warp_sum(t);
}

__device__ __forceinline__ float block_max(float x, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  x = warp_max(x);
  __syncthreads();
  if (lane == 0) red[warp] = x;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : -INFINITY;
  return warp_max(t);
}

// ------------------------------------------------------------------------------ RMSNorm
// One CTA per row (grid-stride). D % 8 == 0. rstd[row] is kept for the backward pass.
// If `residual` is given, computes s = x + residual first, writes s to `sum_out` and
// normalises s (the pre-norm residual add of a transformer block fused in).
__global__ void rmsnorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ residual,
                                   const bf16* __restrict__ scale, bf16* __restrict__ y,
                                   bf16* __restrict__ sum_out, float* __restrict__ rstd_out,
                                   int64_t rows, int D, float eps) {
  __shared__ float red[32];
  const int nvec = D / 8;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const Bf16x8* xr = reinterpret_cast<const Bf16x8*>(x + row * D);
    const Bf16x8* rr = residual ? reinterpret_cast<const Bf16x8*>(residual + row * D) : nullptr;
    Bf16x8* sr = sum_out ? reinterpret_cast<Bf16x8*>(sum_out + row * D) : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      Bf16x8 a = xr[i];
      if (rr) {
        Bf16x8 b = rr[i];
#pragma unroll
        for (int j = 0; j < 4; ++j) a.v[j] = __hadd2(a.v[j], b.v[j]);
        sr[i] = a;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(a.v[j]);
        ss += f.x * f.x + f.y * f.y;
      }
    }
    ss = block_sum(ss, red);
    const float rstd = rsqrtf(ss / D + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
    const Bf16x8* src = sr ? reinterpret_cast<const Bf16x8*>(sr) : xr;
    const Bf16x8* sc = reinterpret_cast<const Bf16x8*>(scale);
    Bf16x8* yr = reinterpret_cast<Bf16x8*>(y + row * D);
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      Bf16x8 a = src[i], s = sc[i], o;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(a.v[j]);
        float2 g = __bfloat1622float2(s.v[j]);
        // Match the unfused definition: normalise, round to bf16, then scale.
        __nv_bfloat162 n = __floats2bfloat162_rn(f.x * rstd, f.y * rstd);
        float2 nf = __bfloat1622float2(n);
        o.v[j] = __floats2bfloat162_rn(nf.x * g.x, nf.y * g.y);
      }
      yr[i] = o;
    }
  }
}

// dx = rstd * (g - xhat * mean(g * xhat)), g = dy * scale, xhat = x * rstd.
// dscale partials: each CTA accumulates sum over its rows of dy * xhat into
// partial[blockIdx.x, :] (fp32); a second kernel reduces over CTAs in a fixed order.
// If `dres` is given, it is added to dx (gradient arriving through the residual branch).
__global__ void rmsnorm_bwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ scale,
                                   const float* __restrict__ rstd_in, const bf16* __restrict__ dy,
                                   const bf16* __restrict__ dres, bf16* __restrict__ dx,
                                   float* __restrict__ partial, int64_t rows, int D) {
  __shared__ float red[32];
  extern __shared__ float dscale_acc[];  // [D]
  for (int i = threadIdx.x; i < D; i += blockDim.x) dscale_acc[i] = 0.f;
  const int nvec = D / 8;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const Bf16x8* xr = reinterpret_cast<const Bf16x8*>(x + row * D);
    const Bf16x8* gr = reinterpret_cast<const Bf16x8*>(dy + row * D);
    const Bf16x8* sc = reinterpret_cast<const Bf16x8*>(scale);
    const float rstd = rstd_in[row];
    float dot = 0.f;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      Bf16x8 a = xr[i], g = gr[i], s = sc[i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 xf = __bfloat1622float2(a.v[j]), gf = __bfloat1622float2(g.v[j]),
               sf = __bfloat1622float2(s.v[j]);
        dot += gf.x * sf.x * xf.x * rstd + gf.y * sf.y * xf.y * rstd;
      }
    }
    dot = block_sum(dot, red) / D;
    const Bf16x8* rr = dres ? reinterpret_cast<const Bf16x8*>(dres + row * D) : nullptr;
    Bf16x8* dxr = reinterpret_cast<Bf16x8*>(dx + row * D);
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      Bf16x8 a = xr[i], g = gr[i], s = sc[i], o;
      Bf16x8 r;
      if (rr) r = rr[i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 xf = __bfloat1622float2(a.v[j]), gf = __bfloat1622float2(g.v[j]),
               sf = __bfloat1622float2(s.v[j]);
        const float xh0 = xf.x * rstd, xh1 = xf.y * rstd;
        float d0 = rstd * (gf.x * sf.x - xh0 * dot);
        float d1 = rstd * (gf.y * sf.y - xh1 * dot);
        if (rr) {
          float2 rf = __bfloat1622float2(r.v[j]);
          d0 += rf.x;
          d1 += rf.y;
        }
        o.v[j] = __floats2bfloat162_rn(d0, d1);
        // Each thread owns fixed columns, so these shared-memory updates do not race.
        dscale_acc[i * 8 + 2 * j] += gf.x * xh0;
        dscale_acc[i * 8 + 2 * j + 1] += gf.y * xh1;
      }
      dxr[i] = o;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < D; i += blockDim.x)
    partial[static_cast<int64_t>(blockIdx.x) * D + i] = dscale_acc[i];
}

// ------------------------------------------------------------------------------ RMSNorm, one warp per row
// The row (D = 256 * VPL elements) lives in registers: every lane issues all of its 16-byte loads
// up front and the statistics need only warp shuffles, so a CTA of eight warps keeps eight rows
// (tens of KB) in flight with no block-wide barrier per row.  Same arithmetic as the kernels above.
// Keeps the compiler from hoisting the next group's loads above this group's stores (which would
// hold several more vectors per lane live than the register file has room for).
#define AXB_SCHED_FENCE() asm volatile("" ::: "memory")

// A 16-byte read-only load that the compiler neither merges with an identical earlier load nor
// moves: each use re-reads (from L1) instead of keeping the vector in registers between loops.
__device__ __forceinline__ Bf16x8 ld_again(const Bf16x8* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return *reinterpret_cast<Bf16x8*>(&v);
}

// WPR warps share a row (each a contiguous 256 * VPL-element part); wide rows are split so that a
// lane holds at most eight vectors and three CTAs fit an SM (more rows, hence bytes, in flight).
template <int VPL, int WPR>
__global__ void __launch_bounds__(256, 3)
rmsnorm_fwd_warp_kernel(const bf16* __restrict__ x, const bf16* __restrict__ residual,
                        const bf16* __restrict__ scale, bf16* __restrict__ y, bf16* __restrict__ sum_out,
                        float* __restrict__ rstd_out, int64_t rows, float eps) {
  constexpr int P = VPL * 256;
  constexpr int D = P * WPR;
  constexpr int kRowsPerCta = 8 / WPR;
  __shared__ float ss_part[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int part = warp % WPR, slot = warp / WPR;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kRowsPerCta;
  const Bf16x8* sc = reinterpret_cast<const Bf16x8*>(scale + part * P);
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * kRowsPerCta + slot; row < rows; row += stride) {
    const Bf16x8* xr = reinterpret_cast<const Bf16x8*>(x + row * D + part * P);
    Bf16x8 a[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) a[i] = xr[i * 32 + lane];
    if (residual != nullptr) {
      const Bf16x8* rr = reinterpret_cast<const Bf16x8*>(residual + row * D + part * P);
      Bf16x8* sr = reinterpret_cast<Bf16x8*>(sum_out + row * D + part * P);
      Bf16x8 b[VPL];
#pragma unroll
      for (int i = 0; i < VPL; ++i) b[i] = rr[i * 32 + lane];
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
#pragma unroll
        for (int j = 0; j < 4; ++j) a[i].v[j] = __hadd2(a[i].v[j], b[i].v[j]);
        sr[i * 32 + lane] = a[i];
      }
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(a[i].v[j]);
        ss += f.x * f.x + f.y * f.y;
      }
    }
    ss = warp_sum(ss);
    if constexpr (WPR > 1) {
      if (lane == 0) ss_part[warp] = ss;
      asm volatile("bar.sync %0, %1;" ::"r"(1 + slot), "r"(32 * WPR) : "memory");
      ss = 0.f;
#pragma unroll
      for (int w = 0; w < WPR; ++w) ss += ss_part[slot * WPR + w];
      asm volatile("bar.sync %0, %1;" ::"r"(1 + slot), "r"(32 * WPR) : "memory");
    }
    const float rstd = rsqrtf(ss / D + eps);
    if (lane == 0 && part == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
    Bf16x8* yr = reinterpret_cast<Bf16x8*>(y + row * D + part * P);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const Bf16x8 s = sc[i * 32 + lane];
      Bf16x8 o;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(a[i].v[j]);
        const float2 g = __bfloat1622float2(s.v[j]);
        // Match the unfused definition: normalise, round to bf16, then scale.
        const float2 nf = __bfloat1622float2(__floats2bfloat162_rn(f.x * rstd, f.y * rstd));
        o.v[j] = __floats2bfloat162_rn(nf.x * g.x, nf.y * g.y);
      }
      yr[i * 32 + lane] = o;
    }
  }
}

// Backward, WPR warps per row (each owns a contiguous 256 * VPL-element part of it; two warps
// for the widest rows, whose halves would not fit one lane's registers).  The per-column sums for
// dscale are kept per warp in shared memory (each lane owns its columns, so nothing races), summed
// over the CTA's warps in a fixed order at the end and written to partial[blockIdx.x, :].  Shared
// layout of a warp's part: float4 slot ((i * 2 + h) * 32 + lane) holds its columns
// (i * 32 + lane) * 8 + h * 4 .. + 3 (conflict-free for a warp).
template <int VPL, int WPR, int NW>
__global__ void __launch_bounds__(NW * 32, 1)
rmsnorm_bwd_warp_kernel(const bf16* __restrict__ x, const bf16* __restrict__ scale, const float* __restrict__ rstd_in,
                        const bf16* __restrict__ dy, const bf16* __restrict__ dres, bf16* __restrict__ dx,
                        float* __restrict__ partial, int64_t rows) {
  constexpr int P = VPL * 256;  // elements per warp
  constexpr int D = P * WPR;
  constexpr int kRowsPerCta = NW / WPR;
  extern __shared__ float4 acc_all[];  // [NW warps][P / 4]
  __shared__ float dot_part[NW];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int part = warp % WPR, slot = warp / WPR;
  float4* acc = acc_all + warp * (P / 4);
  for (int i = lane; i < P / 4; i += 32) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  __syncwarp();
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kRowsPerCta;
  const Bf16x8* sc = reinterpret_cast<const Bf16x8*>(scale + part * P);
  // Every warp of a row makes the same number of trips, so the pair barrier below always matches.
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * kRowsPerCta + slot; row < rows; row += stride) {
    const Bf16x8* xr = reinterpret_cast<const Bf16x8*>(x + row * D + part * P);
    const Bf16x8* gr = reinterpret_cast<const Bf16x8*>(dy + row * D + part * P);
    // Everything the row needs from global memory is requested up front (x, dy and, when
    // present, the residual branch's gradient): one exposed round trip per row instead of one
    // per use.
    const Bf16x8* rr = dres != nullptr ? reinterpret_cast<const Bf16x8*>(dres + row * D + part * P) : nullptr;
    Bf16x8 a[VPL], g[VPL], r[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      a[i] = xr[i * 32 + lane];
      g[i] = gr[i * 32 + lane];
      if (rr != nullptr) r[i] = rr[i * 32 + lane];
    }
    const float rstd = rstd_in[row];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const Bf16x8 s = ld_again(sc + i * 32 + lane);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 xf = __bfloat1622float2(a[i].v[j]), gf = __bfloat1622float2(g[i].v[j]),
                     sf = __bfloat1622float2(s.v[j]);
        dot += gf.x * sf.x * xf.x * rstd + gf.y * sf.y * xf.y * rstd;
      }
    }
    dot = warp_sum(dot);
    if constexpr (WPR > 1) {
      // Exchange the parts' sums between the warps of this row (a named barrier per row slot).
      if (lane == 0) dot_part[warp] = dot;
      asm volatile("bar.sync %0, %1;" ::"r"(1 + slot), "r"(32 * WPR) : "memory");
      dot = 0.f;
#pragma unroll
      for (int w = 0; w < WPR; ++w) dot += dot_part[slot * WPR + w];
      asm volatile("bar.sync %0, %1;" ::"r"(1 + slot), "r"(32 * WPR) : "memory");  // before the next row overwrites
    }
    dot /= D;
    Bf16x8* dxr = reinterpret_cast<Bf16x8*>(dx + row * D + part * P);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const Bf16x8 s = ld_again(sc + i * 32 + lane);
      Bf16x8 o;
      float ds[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 xf = __bfloat1622float2(a[i].v[j]), gf = __bfloat1622float2(g[i].v[j]),
                     sf = __bfloat1622float2(s.v[j]);
        const float xh0 = xf.x * rstd, xh1 = xf.y * rstd;
        float d0 = rstd * (gf.x * sf.x - xh0 * dot);
        float d1 = rstd * (gf.y * sf.y - xh1 * dot);
        if (rr != nullptr) {
          const float2 rf = __bfloat1622float2(r[i].v[j]);
          d0 += rf.x;
          d1 += rf.y;
        }
        o.v[j] = __floats2bfloat162_rn(d0, d1);
        ds[2 * j] = gf.x * xh0;
        ds[2 * j + 1] = gf.y * xh1;
      }
      dxr[i * 32 + lane] = o;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float4 v = acc[(i * 2 + h) * 32 + lane];
        v.x += ds[4 * h];
        v.y += ds[4 * h + 1];
        v.z += ds[4 * h + 2];
        v.w += ds[4 * h + 3];
        acc[(i * 2 + h) * 32 + lane] = v;
      }
    }
  }
  __syncthreads();
  // Column c of part q: cc = c - q * P = (i * 32 + l) * 8 + h * 4 + e  <->  float index
  // ((i * 2 + h) * 32 + l) * 4 + e of every warp with warp % WPR == q.
  const float* flat = reinterpret_cast<const float*>(acc_all);
  for (int c = threadIdx.x; c < D; c += NW * 32) {
    const int q = c / P, cc = c - q * P;
    const int vec = cc >> 3, h = (cc >> 2) & 1, e = cc & 3;
    const int i = vec >> 5, l = vec & 31;
    const int idx = ((i * 2 + h) * 32 + l) * 4 + e;
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < kRowsPerCta; ++w) sum += flat[(w * WPR + q) * P + idx];
    partial[static_cast<int64_t>(blockIdx.x) * D + c] = sum;
  }
}

__global__ void reduce_partials_kernel(const float* __restrict__ partial, bf16* __restrict__ out_bf16,
                                       float* __restrict__ out_f32, int nparts, int D) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= D) return;
  float s = 0.f;
  for (int p = 0; p < nparts; ++p) s += partial[static_cast<int64_t>(p) * D + i];
  if (out_bf16) out_bf16[i] = __float2bfloat16(s);
  if (out_f32) out_f32[i] = s;
}

// ------------------------------------------------------------------------------ SwiGLU
__global__ void swiglu_fwd_kernel(const bf16* __restrict__ gate, const bf16* __restrict__ up,
                                  bf16* __restrict__ out, int64_t nvec) {
  const Bf16x8* g8 = reinterpret_cast<const Bf16x8*>(gate);
  const Bf16x8* u8 = reinterpret_cast<const Bf16x8*>(up);
  Bf16x8* o8 = reinterpret_cast<Bf16x8*>(out);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    Bf16x8 g = g8[i], u = u8[i], o;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 gf = __bfloat1622float2(g.v[j]), uf = __bfloat1622float2(u.v[j]);
      const float s0 = gf.x / (1.f + __expf(-gf.x)), s1 = gf.y / (1.f + __expf(-gf.y));
      // silu is rounded to bf16 before the product, as in the unfused computation.
      float2 sr = __bfloat1622float2(__floats2bfloat162_rn(s0, s1));
      o.v[j] = __floats2bfloat162_rn(sr.x * uf.x, sr.y * uf.y);
    }
    o8[i] = o;
  }
}

__global__ void swiglu_bwd_kernel(const bf16* __restrict__ gate, const bf16* __restrict__ up,
                                  const bf16* __restrict__ dout, bf16* __restrict__ dgate,
                                  bf16* __restrict__ dup, int64_t nvec) {
  const Bf16x8* g8 = reinterpret_cast<const Bf16x8*>(gate);
  const Bf16x8* u8 = reinterpret_cast<const Bf16x8*>(up);
  const Bf16x8* d8 = reinterpret_cast<const Bf16x8*>(dout);
  Bf16x8* dg8 = reinterpret_cast<Bf16x8*>(dgate);
  Bf16x8* du8 = reinterpret_cast<Bf16x8*>(dup);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    Bf16x8 g = g8[i], u = u8[i], d = d8[i], dg, du;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 gf = __bfloat1622float2(g.v[j]), uf = __bfloat1622float2(u.v[j]),
             df = __bfloat1622float2(d.v[j]);
      const float sg0 = 1.f / (1.f + __expf(-gf.x)), sg1 = 1.f / (1.f + __expf(-gf.y));
      const float silu0 = gf.x * sg0, silu1 = gf.y * sg1;
      du.v[j] = __floats2bfloat162_rn(df.x * silu0, df.y * silu1);
      dg.v[j] = __floats2bfloat162_rn(df.x * uf.x * sg0 * (1.f + gf.x * (1.f - sg0)),
                                      df.y * uf.y * sg1 * (1.f + gf.y * (1.f - sg1)));
    }
    dg8[i] = dg;
    du8[i] = du;
  }
}

// ------------------------------------------------------------------------------ RoPE
// x: [B, T, N, H] contiguous, interleaved pairs (x[2i], x[2i+1]); angle = pos[t] * theta^(-2i/H).
// sign = +1 forward, -1 backward (rotation by the negative angle). In-place safe.
//
// The angles depend on (t, i) only, so a first tiny kernel fills a [T, H/2] table of (sin, cos)
// -- T * H/2 evaluations instead of B * T * N * H/2 -- and the main kernel is a pure streaming
// pass: 16-byte loads of x, the table row from L2, 16-byte stores.
__global__ void rope_table_kernel(const int64_t* __restrict__ pos, float2* __restrict__ table, int T, int hp,
                                  int H, float log2_theta) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= T * hp) return;
  const int i = idx % hp, t = idx / hp;
  const float inv_freq = exp2f(-(2.f * i / H) * log2_theta);
  float s, c;
  sincosf(static_cast<float>(pos[t]) * inv_freq, &s, &c);
  table[idx] = make_float2(s, c);
}

// One block handles `rows` (batch, position) rows of [N heads x H]; within a row a thread owns one
// 16-byte vector position of the head (`pv`) and every `lanes`-th head, so the sines and cosines
// of its four pairs are loaded once and reused over N / lanes heads, no index needs a division
// beyond the row's position, and a thread keeps several independent 16-byte loads in flight.
template <int kHeadsInFlight>
__global__ void rope_apply_kernel(const Bf16x8* __restrict__ x, Bf16x8* __restrict__ y,
                                  const float2* __restrict__ table, int64_t num_rows, int T, int N, int hp,
                                  float sign, int lanes, int rows) {
  const int vec_per_head = hp / 4;  // 4 pairs (8 elements) per 16-byte vector
  const int per_row = vec_per_head * lanes;
  const int r_in = threadIdx.x / per_row, j = threadIdx.x - r_in * per_row;
  const int pv = j % vec_per_head, n0 = j / vec_per_head;
  if (r_in >= rows) return;
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * rows + r_in; row < num_rows;
       row += static_cast<int64_t>(gridDim.x) * rows) {
    const int t = static_cast<int>(row % T);
    const float4* tab = reinterpret_cast<const float4*>(table + static_cast<int64_t>(t) * hp + pv * 4);
    const float4 sc0 = __ldg(tab), sc1 = __ldg(tab + 1);  // (s0, c0, s1, c1), (s2, c2, s3, c3)
    const float sn[4] = {sc0.x * sign, sc0.z * sign, sc1.x * sign, sc1.z * sign};
    const float cs[4] = {sc0.y, sc0.w, sc1.y, sc1.w};
    const int64_t base = row * (static_cast<int64_t>(N) * vec_per_head) + pv;
    for (int n = n0; n < N; n += lanes * kHeadsInFlight) {
      Bf16x8 v[kHeadsInFlight];
#pragma unroll
      for (int u = 0; u < kHeadsInFlight; ++u) {
        const int nn = n + u * lanes;
        if (nn < N) v[u] = x[base + static_cast<int64_t>(nn) * vec_per_head];
      }
#pragma unroll
      for (int u = 0; u < kHeadsInFlight; ++u) {
        const int nn = n + u * lanes;
        if (nn >= N) continue;
        Bf16x8 o;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = __bfloat1622float2(v[u].v[q]);
          o.v[q] = __floats2bfloat162_rn(f.x * cs[q] - f.y * sn[q], f.y * cs[q] + f.x * sn[q]);
        }
        y[base + static_cast<int64_t>(nn) * vec_per_head] = o;
      }
    }
  }
}

// Fallback without a table (H/2 not a multiple of 4, or no scratch given).
__global__ void rope_kernel(const bf16* __restrict__ x, bf16* __restrict__ y,
                            const int64_t* __restrict__ pos, int64_t B, int T, int N, int H,
                            float log2_theta, float sign) {
  const int hp = H / 2;  // pairs per head
  const int64_t total = B * T * static_cast<int64_t>(N) * hp;
  for (int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int i = idx % hp;
    const int64_t bt = idx / (static_cast<int64_t>(hp) * N);
    const int t = bt % T;
    const float inv_freq = exp2f(-(2.f * i / H) * log2_theta);
    float s, c;
    sincosf(static_cast<float>(pos[t]) * inv_freq, &s, &c);
    s *= sign;
    const __nv_bfloat162 v = reinterpret_cast<const __nv_bfloat162*>(x)[idx];
    const float2 f = __bfloat1622float2(v);
    reinterpret_cast<__nv_bfloat162*>(y)[idx] =
        __floats2bfloat162_rn(f.x * c - f.y * s, f.y * c + f.x * s);
  }
}

// ------------------------------------------------------------------------------ cross entropy
// One CTA per row of logits [n, V] (bf16 or fp32 via template). The row is staged in shared
// memory as fp32 when it fits, so global memory is read once and the gradient is written once
// (in place, in the logits buffer).  Per-row outputs (masked by live) are reduced by the caller
// in a fixed order, which keeps the loss bit-reproducible.
//   ce_out[r]  = live * (lse - logit[target]);  z_out[r] = live * lse^2
//   correct[r] = live * (argmax == target)
//   dlogits    = live * inv_denom * ((1 + 2*z_scale*lse) * softmax - onehot)
template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<bf16>(bf16 v) {
  return __bfloat162float(v);
}
template <>
__device__ __forceinline__ float to_f<float>(float v) {
  return v;
}
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ bf16 from_f<bf16>(float v) {
  return __float2bfloat16(v);
}
template <>
__device__ __forceinline__ float from_f<float>(float v) {
  return v;
}

template <typename T, bool STAGE>
__global__ void ce_fwd_bwd_kernel(T* __restrict__ logits, const int64_t* __restrict__ targets,
                                  const uint8_t* __restrict__ live, float* __restrict__ ce_out,
                                  float* __restrict__ z_out, float* __restrict__ correct_out,
                                  const float* __restrict__ inv_denom_ptr, float z_scale, int64_t n,
                                  int V, int write_grad) {
  __shared__ float red[32];
  __shared__ int red_idx[32];
  extern __shared__ float row_cache[];  // [V] when STAGE
  const float inv_denom = *inv_denom_ptr;
  for (int64_t row = blockIdx.x; row < n; row += gridDim.x) {
    T* lr = logits + row * V;
    // Pass 1: max and argmax (first index wins on ties, like argmax).
    float m = -INFINITY;
    int mi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float v = to_f<T>(lr[i]);
      if (STAGE) row_cache[i] = v;
      if (v > m) {
        m = v;
        mi = i;
      }
    }
    // Block arg-max.
    {
      const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, m, o);
        const int oi = __shfl_xor_sync(0xffffffffu, mi, o);
        if (om > m || (om == m && oi < mi)) {
          m = om;
          mi = oi;
        }
      }
      __syncthreads();
      if (lane == 0) {
        red[warp] = m;
        red_idx[warp] = mi;
      }
      __syncthreads();
      m = (lane < nw) ? red[lane] : -INFINITY;
      mi = (lane < nw) ? red_idx[lane] : 0x7fffffff;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, m, o);
        const int oi = __shfl_xor_sync(0xffffffffu, mi, o);
        if (om > m || (om == m && oi < mi)) {
          m = om;
          mi = oi;
        }
      }
    }
    // Pass 2: sum of exp.
    float se = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float v = STAGE ? row_cache[i] : to_f<T>(lr[i]);
      se += __expf(v - m);
    }
    se = block_sum(se, red);
    const float lse = m + logf(se);
    const int64_t tgt_raw = targets[row];
    const bool is_live = live[row] != 0;
    const int tgt = static_cast<int>(tgt_raw < 0 ? 0 : (tgt_raw >= V ? V - 1 : tgt_raw));
    if (threadIdx.x == 0) {
      const float picked = STAGE ? row_cache[tgt] : to_f<T>(lr[tgt]);
      ce_out[row] = is_live ? (lse - picked) : 0.f;
      z_out[row] = is_live ? lse * lse : 0.f;
      correct_out[row] = (is_live && mi == tgt) ? 1.f : 0.f;
    }
    if (write_grad) {
      const float g = is_live ? inv_denom : 0.f;
      const float coef = g * (1.f + 2.f * z_scale * lse);
      for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = STAGE ? row_cache[i] : to_f<T>(lr[i]);
        float d = coef * __expf(v - lse);
        if (i == tgt) d -= g;
        lr[i] = from_f<T>(d);
      }
    }
    __syncthreads();
  }
}

// bf16 rows with V % 8 == 0: the same three passes with 16-byte accesses, the row staged in shared
// memory as bf16 (V * 2 bytes, so three CTAs of 512 threads fit on an SM for V = 32768) and the
// gradient written back with 16-byte stores.  Ties in the arg-max resolve to the lowest index.
__global__ void __launch_bounds__(512)
ce_fwd_bwd_bf16_vec_kernel(bf16* __restrict__ logits, const int64_t* __restrict__ targets,
                           const uint8_t* __restrict__ live, float* __restrict__ ce_out,
                           float* __restrict__ z_out, float* __restrict__ correct_out,
                           const float* __restrict__ inv_denom_ptr, float z_scale, int64_t n, int V,
                           int write_grad) {
  __shared__ float red[32];
  __shared__ int red_idx[32];
  extern __shared__ __align__(16) unsigned char ce_smem[];
  Bf16x8* cache = reinterpret_cast<Bf16x8*>(ce_smem);
  const int nvec = V / 8;
  const float inv_denom = *inv_denom_ptr;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int64_t row = blockIdx.x; row < n; row += gridDim.x) {
    Bf16x8* lr = reinterpret_cast<Bf16x8*>(logits + row * V);
    float m = -INFINITY;
    int mi = 0x7fffffff;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      const Bf16x8 v = lr[i];
      cache[i] = v;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(v.v[j]);
        if (f.x > m) {
          m = f.x;
          mi = i * 8 + 2 * j;
        }
        if (f.y > m) {
          m = f.y;
          mi = i * 8 + 2 * j + 1;
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o);
      const int oi = __shfl_xor_sync(0xffffffffu, mi, o);
      if (om > m || (om == m && oi < mi)) {
        m = om;
        mi = oi;
      }
    }
    __syncthreads();
    if (lane == 0) {
      red[warp] = m;
      red_idx[warp] = mi;
    }
    __syncthreads();
    m = (lane < nw) ? red[lane] : -INFINITY;
    mi = (lane < nw) ? red_idx[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o);
      const int oi = __shfl_xor_sync(0xffffffffu, mi, o);
      if (om > m || (om == m && oi < mi)) {
        m = om;
        mi = oi;
      }
    }
    const int64_t tgt_raw = targets[row];
    const bool is_live = live[row] != 0;
    const int tgt = static_cast<int>(tgt_raw < 0 ? 0 : (tgt_raw >= V ? V - 1 : tgt_raw));
    // The target's logit is read before the staged row is overwritten below (every thread's own
    // copy: the value is the same and nobody has to wait for a broadcast).
    const float picked = __bfloat162float(reinterpret_cast<const bf16*>(cache)[tgt]);
    __syncthreads();
    // Each exponential is evaluated ONCE: exp(x - max) feeds the sum and, rounded to bf16, replaces
    // the staged logit; the gradient pass then only scales it by coef / sum.  (Two exponentials
    // per element made the special-function unit as busy as the memory system.)
    float se = 0.f;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      const Bf16x8 v = cache[i];
      Bf16x8 e;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(v.v[j]);
        const float e0 = __expf(f.x - m), e1 = __expf(f.y - m);
        se += e0 + e1;
        e.v[j] = __floats2bfloat162_rn(e0, e1);
      }
      if (write_grad) cache[i] = e;
    }
    se = block_sum(se, red);
    const float lse = m + logf(se);
    if (threadIdx.x == 0) {
      ce_out[row] = is_live ? (lse - picked) : 0.f;
      z_out[row] = is_live ? lse * lse : 0.f;
      correct_out[row] = (is_live && mi == tgt) ? 1.f : 0.f;
    }
    if (write_grad) {
      const float g = is_live ? inv_denom : 0.f;
      const float coef = g * (1.f + 2.f * z_scale * lse) / se;   // exp(x - lse) = exp(x - max) / sum
      for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
        const Bf16x8 v = cache[i];
        Bf16x8 o;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(v.v[j]);
          float d0 = coef * f.x, d1 = coef * f.y;
          if (i * 8 + 2 * j == tgt) d0 -= g;
          if (i * 8 + 2 * j + 1 == tgt) d1 -= g;
          o.v[j] = __floats2bfloat162_rn(d0, d1);
        }
        lr[i] = o;
      }
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------------------ AdamW
// p (fp32 master), m, v fp32; g bf16 or fp32; optional bf16 shadow written with the new p.
//   g' = g * grad_scale[0];  m = b1 m + (1-b1) g';  v = b2 v + (1-b2) g'^2
//   p -= lr * (m / bc1) / (sqrt(v / bc2) + eps) + wd * p
template <typename G>
__global__ void adamw_kernel(float* __restrict__ p, const G* __restrict__ g, float* __restrict__ m,
                             float* __restrict__ v, bf16* __restrict__ shadow,
                             const float* __restrict__ grad_scale, int64_t n, float lr, float wd,
                             float b1, float b2, float eps, float bc1, float bc2) {
  const float gs = grad_scale ? *grad_scale : 1.f;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x * 4;
  for (int64_t i = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) * 4; i < n;
       i += stride) {
    if (i + 4 <= n) {
      float4 pf = *reinterpret_cast<float4*>(p + i);
      float4 mf = *reinterpret_cast<float4*>(m + i);
      float4 vf = *reinterpret_cast<float4*>(v + i);
      float gg[4];
      if constexpr (sizeof(G) == 2) {
        const uint2 raw = *reinterpret_cast<const uint2*>(g + i);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        gg[0] = a.x, gg[1] = a.y, gg[2] = b.x, gg[3] = b.y;
      } else {
        const float4 a = *reinterpret_cast<const float4*>(g + i);
        gg[0] = a.x, gg[1] = a.y, gg[2] = a.z, gg[3] = a.w;
      }
      float* pp = &pf.x;
      float* mm = &mf.x;
      float* vv = &vf.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float gj = gg[j] * gs;
        mm[j] = b1 * mm[j] + (1.f - b1) * gj;
        vv[j] = b2 * vv[j] + (1.f - b2) * gj * gj;
        const float upd = lr * (mm[j] / bc1) / (sqrtf(vv[j] / bc2) + eps) + wd * pp[j];
        pp[j] -= upd;
      }
      *reinterpret_cast<float4*>(p + i) = pf;
      *reinterpret_cast<float4*>(m + i) = mf;
      *reinterpret_cast<float4*>(v + i) = vf;
      if (shadow) {
        uint2 o;
        *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(pf.x, pf.y);
        *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(pf.z, pf.w);
        *reinterpret_cast<uint2*>(shadow + i) = o;
      }
    } else {
      for (int64_t k = i; k < n; ++k) {
        float gj;
        if constexpr (sizeof(G) == 2) gj = __bfloat162float(g[k]) * gs;
        else gj = g[k] * gs;
        const float mk = b1 * m[k] + (1.f - b1) * gj;
        const float vk = b2 * v[k] + (1.f - b2) * gj * gj;
        const float pk = p[k] - (lr * (mk / bc1) / (sqrtf(vk / bc2) + eps) + wd * p[k]);
        m[k] = mk, v[k] = vk, p[k] = pk;
        if (shadow) shadow[k] = __float2bfloat16(pk);
      }
    }
  }
}

// ------------------------------------------------------------------------------ sum of squares
// partial[blockIdx.x] = sum over this block's grid-stride share of x^2 (fixed assignment, so
// the result is reproducible); the caller adds the partials in index order.
__global__ void sumsq_f32_kernel(const float* __restrict__ x, int64_t n, float* __restrict__ partial) {
  __shared__ float red[32];
  float s = 0.f;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const float v = x[i];
    s += v * v;
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}

__global__ void sumsq_bf16_kernel(const bf16* __restrict__ x, int64_t n, float* __restrict__ partial) {
  __shared__ float red[32];
  float s = 0.f;
  const int64_t nvec = n / 8;
  const Bf16x8* x8 = reinterpret_cast<const Bf16x8*>(x);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const Bf16x8 a = x8[i];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(a.v[j]);
      s += f.x * f.x + f.y * f.y;
    }
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    for (int64_t k = nvec * 8; k < n; ++k) {
      const float f = __bfloat162float(x[k]);
      s += f * f;
    }
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}

__global__ void sum_partials_kernel(const float* __restrict__ partial, int n, float* __restrict__ out,
                                    float weight, int accumulate) {
  // Single thread, fixed order: n is a few hundred.
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    float s = 0.f;
    for (int i = 0; i < n; ++i) s += partial[i];
    s *= weight;
    *out = accumulate ? (*out + s) : s;
  }
}

static inline int grid_for(int64_t work, int threads, int max_blocks) {
  int64_t b = (work + threads - 1) / threads;
  if (b < 1) b = 1;
  return static_cast<int>(b < max_blocks ? b : max_blocks);
}

}  // namespace axb

using namespace axb;

extern "C" int axb_rmsnorm_fwd(const void* x, const void* residual, const void* scale, void* y,
                               void* sum_out, float* rstd, int64_t rows, int D, float eps,
                               cudaStream_t stream) {
  if (D % 8) return -10;
  const int threads = D >= 2048 ? 256 : 128;
  const int grid = static_cast<int>(rows < 148 * 8 ? rows : 148 * 8);
  rmsnorm_fwd_kernel<<<grid, threads, 0, stream>>>(
      static_cast<const bf16*>(x), static_cast<const bf16*>(residual),
      static_cast<const bf16*>(scale), static_cast<bf16*>(y), static_cast<bf16*>(sum_out), rstd,
      rows, D, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Number of CTAs (= rows of the fp32 `partial` workspace [ctas, D]) the backward will use.
extern "C" int axb_rmsnorm_bwd_ctas(int64_t rows) {
  // The allocation-free variant (no_alloc.cu) sizes its built-in workspace with the same constant
  // and promises bit-equal results, which needs the same grid: keep both on the one definition.
  return static_cast<int>(rows < AXB_NOALLOC_RMSNORM_MAX_CTAS ? rows : AXB_NOALLOC_RMSNORM_MAX_CTAS);
}

extern "C" int axb_rmsnorm_bwd(const void* x, const void* scale, const float* rstd, const void* dy,
                               const void* dres, void* dx, float* partial, void* dscale_bf16,
                               float* dscale_f32, int64_t rows, int D, cudaStream_t stream) {
  if (D % 8 || D * 4 > 200 * 1024) return -10;
  const int grid = axb_rmsnorm_bwd_ctas(rows);
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(rmsnorm_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    configured = true;
  }
  rmsnorm_bwd_kernel<<<grid, 256, D * sizeof(float), stream>>>(
      static_cast<const bf16*>(x), static_cast<const bf16*>(scale), rstd,
      static_cast<const bf16*>(dy), static_cast<const bf16*>(dres), static_cast<bf16*>(dx), partial,
      rows, D);
  reduce_partials_kernel<<<(D + 255) / 256, 256, 0, stream>>>(
      partial, static_cast<bf16*>(dscale_bf16), dscale_f32, grid, D);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

template <int VPL, int WPR>
static int launch_rmsnorm_fwd_warp(const void* x, const void* residual, const void* scale, void* y, void* sum_out,
                                   float* rstd, int64_t rows, float eps, cudaStream_t stream) {
  const int64_t want = (rows + 8 / WPR - 1) / (8 / WPR);
  const int grid = static_cast<int>(want < 148 * 3 ? want : 148 * 3);
  rmsnorm_fwd_warp_kernel<VPL, WPR><<<grid, 256, 0, stream>>>(
      static_cast<const bf16*>(x), static_cast<const bf16*>(residual), static_cast<const bf16*>(scale),
      static_cast<bf16*>(y), static_cast<bf16*>(sum_out), rstd, rows, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

template <int VPL, int WPR, int NW>
static int launch_rmsnorm_bwd_warp(const void* x, const void* scale, const float* rstd, const void* dy,
                                   const void* dres, void* dx, float* partial, int cap, int64_t rows,
                                   cudaStream_t stream) {
  constexpr int kSmem = NW * VPL * 256 * static_cast<int>(sizeof(float));
  const int64_t want = (rows + NW / WPR - 1) / (NW / WPR);
  const int grid = static_cast<int>(want < cap ? want : cap);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(rmsnorm_bwd_warp_kernel<VPL, WPR, NW>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) !=
        cudaSuccess)
      return -3;
    configured = true;
  }
  rmsnorm_bwd_warp_kernel<VPL, WPR, NW><<<grid, NW * 32, kSmem, stream>>>(
      static_cast<const bf16*>(x), static_cast<const bf16*>(scale), rstd, static_cast<const bf16*>(dy),
      static_cast<const bf16*>(dres), static_cast<bf16*>(dx), partial, rows);
  return cudaGetLastError() == cudaSuccess ? grid : -4;
}

// 1 when the warp-per-row kernels take this width (rows of 512, 1024, 2048 or 4096 elements).
extern "C" int axb_rmsnorm_fast_supported(int D) { return (D == 512 || D == 1024 || D == 2048 || D == 4096) ? 1 : 0; }

// Same contract as axb_rmsnorm_fwd, on the warp-per-row kernel (D must be a supported width).
extern "C" int axb_rmsnorm_fwd_fast(const void* x, const void* residual, const void* scale, void* y, void* sum_out,
                                    float* rstd, int64_t rows, int D, float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (residual != nullptr && sum_out == nullptr) return -10;
  switch (D) {
    case 512: return launch_rmsnorm_fwd_warp<2, 1>(x, residual, scale, y, sum_out, rstd, rows, eps, stream);
    case 1024: return launch_rmsnorm_fwd_warp<4, 1>(x, residual, scale, y, sum_out, rstd, rows, eps, stream);
    case 2048: return launch_rmsnorm_fwd_warp<8, 1>(x, residual, scale, y, sum_out, rstd, rows, eps, stream);
    case 4096: return launch_rmsnorm_fwd_warp<8, 2>(x, residual, scale, y, sum_out, rstd, rows, eps, stream);
    default: return -10;
  }
}

// Same contract as axb_rmsnorm_bwd (`partial` has axb_rmsnorm_bwd_ctas(rows) rows), on the
// warp-per-row kernel.  The order of the dscale summation differs from axb_rmsnorm_bwd, so the two
// agree to rounding, not bit for bit.
extern "C" int axb_rmsnorm_bwd_fast(const void* x, const void* scale, const float* rstd, const void* dy,
                                    const void* dres, void* dx, float* partial, void* dscale_bf16, float* dscale_f32,
                                    int64_t rows, int D, cudaStream_t stream) {
  if (rows <= 0) {
    if (dscale_bf16 != nullptr) cudaMemsetAsync(dscale_bf16, 0, D * sizeof(bf16), stream);
    if (dscale_f32 != nullptr) cudaMemsetAsync(dscale_f32, 0, D * sizeof(float), stream);
    return 0;
  }
  const int cap = axb_rmsnorm_bwd_ctas(rows) < 148 ? axb_rmsnorm_bwd_ctas(rows) : 148;
  int grid;  // the launcher returns the number of CTAs (= rows of `partial`) it used
  switch (D) {
    case 512: grid = launch_rmsnorm_bwd_warp<2, 1, 8>(x, scale, rstd, dy, dres, dx, partial, cap, rows, stream); break;
    case 1024: grid = launch_rmsnorm_bwd_warp<4, 1, 8>(x, scale, rstd, dy, dres, dx, partial, cap, rows, stream); break;
    case 2048: grid = launch_rmsnorm_bwd_warp<4, 2, 16>(x, scale, rstd, dy, dres, dx, partial, cap, rows, stream); break;
    case 4096: grid = launch_rmsnorm_bwd_warp<4, 4, 16>(x, scale, rstd, dy, dres, dx, partial, cap, rows, stream); break;
    default: return -10;
  }
  if (grid < 0) return grid;
  reduce_partials_kernel<<<(D + 255) / 256, 256, 0, stream>>>(partial, static_cast<bf16*>(dscale_bf16), dscale_f32,
                                                              grid, D);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int axb_swiglu_fwd(const void* gate, const void* up, void* out, int64_t n,
                              cudaStream_t stream) {
  if (n % 8) return -10;
  swiglu_fwd_kernel<<<grid_for(n / 8, 256, 148 * 16), 256, 0, stream>>>(
      static_cast<const bf16*>(gate), static_cast<const bf16*>(up), static_cast<bf16*>(out), n / 8);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int axb_swiglu_bwd(const void* gate, const void* up, const void* dout, void* dgate,
                              void* dup, int64_t n, cudaStream_t stream) {
  if (n % 8) return -10;
  swiglu_bwd_kernel<<<grid_for(n / 8, 256, 148 * 16), 256, 0, stream>>>(
      static_cast<const bf16*>(gate), static_cast<const bf16*>(up), static_cast<const bf16*>(dout),
      static_cast<bf16*>(dgate), static_cast<bf16*>(dup), n / 8);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// `table`: optional scratch of T * H floats (sin/cos pairs); with it (and H % 8 == 0) the
// table-driven streaming kernel runs, otherwise every element evaluates its own angle.
extern "C" int axb_rope(const void* x, void* y, const int64_t* positions, int64_t B, int T, int N,
                        int H, float theta, int backward, float* table, cudaStream_t stream) {
  if (H % 2) return -10;
  const int hp = H / 2;
  const int64_t total = B * T * static_cast<int64_t>(N) * hp;
  if (total <= 0) return 0;
  if (table != nullptr && hp % 4 == 0 && hp / 4 <= 256 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(y) & 15) == 0) {
    rope_table_kernel<<<(T * hp + 255) / 256, 256, 0, stream>>>(positions, reinterpret_cast<float2*>(table), T, hp,
                                                                H, log2f(theta));
    // 64 threads' worth of (vector position, head lane) per row where the head allows it.
    const int vec_per_head = hp / 4;
    int lanes = 64 / vec_per_head;
    if (lanes < 1) lanes = 1;
    if (lanes > N) lanes = N;
    int rows = 256 / (vec_per_head * lanes);
    if (rows < 1) rows = 1;
    const int64_t num_rows = B * static_cast<int64_t>(T);
    const int threads = rows * vec_per_head * lanes;
    int64_t blocks = (num_rows + rows - 1) / rows;
    if (blocks > 148 * 16) blocks = 148 * 16;
    rope_apply_kernel<4><<<static_cast<int>(blocks), threads, 0, stream>>>(
        static_cast<const Bf16x8*>(x), static_cast<Bf16x8*>(y), reinterpret_cast<const float2*>(table), num_rows, T,
        N, hp, backward ? -1.f : 1.f, lanes, rows);
  } else {
    rope_kernel<<<grid_for(total, 256, 148 * 16), 256, 0, stream>>>(
        static_cast<const bf16*>(x), static_cast<bf16*>(y), positions, B, T, N, H, log2f(theta),
        backward ? -1.f : 1.f);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int axb_ce_fwd_bwd(void* logits, int is_fp32, const int64_t* targets,
                              const uint8_t* live, float* ce_out, float* z_out, float* correct_out,
                              const float* inv_denom, float z_scale, int64_t n, int V,
                              int write_grad, cudaStream_t stream) {
  if (!is_fp32 && V % 8 == 0 && static_cast<size_t>(V) * 2 <= 72 * 1024 &&
      (reinterpret_cast<uintptr_t>(logits) & 15) == 0) {
    static bool vec_configured = false;
    if (!vec_configured) {
      cudaFuncSetAttribute(ce_fwd_bwd_bf16_vec_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024);
      vec_configured = true;
    }
    const int vgrid = static_cast<int>(n < 148 * 3 ? n : 148 * 3);
    ce_fwd_bwd_bf16_vec_kernel<<<vgrid, 512, static_cast<size_t>(V) * 2, stream>>>(
        static_cast<bf16*>(logits), targets, live, ce_out, z_out, correct_out, inv_denom, z_scale, n, V, write_grad);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
  }
  const int grid = static_cast<int>(n < 148 * 4 ? n : 148 * 4);
  const size_t cache = static_cast<size_t>(V) * sizeof(float);
  const bool stage = cache <= 200 * 1024;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(ce_fwd_bwd_kernel<bf16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    cudaFuncSetAttribute(ce_fwd_bwd_kernel<float, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    configured = true;
  }
#define AXB_CE(T, ST)                                                                             \
  ce_fwd_bwd_kernel<T, ST><<<grid, 512, ST ? cache : 0, stream>>>(                                \
      static_cast<T*>(logits), targets, live, ce_out, z_out, correct_out, inv_denom, z_scale, n, V, \
      write_grad)
  if (is_fp32) {
    if (stage) AXB_CE(float, true); else AXB_CE(float, false);
  } else {
    if (stage) AXB_CE(bf16, true); else AXB_CE(bf16, false);
  }
#undef AXB_CE
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int axb_adamw(float* p, const void* g, int g_is_bf16, float* m, float* v, void* shadow,
                         const float* grad_scale, int64_t n, float lr, float wd, float b1, float b2,
                         float eps, float bc1, float bc2, cudaStream_t stream) {
  const int grid = grid_for((n + 3) / 4, 256, 148 * 8);
  if (g_is_bf16)
    adamw_kernel<bf16><<<grid, 256, 0, stream>>>(p, static_cast<const bf16*>(g), m, v,
                                                 static_cast<bf16*>(shadow), grad_scale, n, lr, wd,
                                                 b1, b2, eps, bc1, bc2);
  else
    adamw_kernel<float><<<grid, 256, 0, stream>>>(p, static_cast<const float*>(g), m, v,
                                                  static_cast<bf16*>(shadow), grad_scale, n, lr, wd,
                                                  b1, b2, eps, bc1, bc2);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// The CUDA runtime's current device as seen by this library (diagnostic: it must equal the
// framework's current device, or launches would land on the wrong GPU).
extern "C" int axb_current_device() {
  int dev = -1;
  cudaGetDevice(&dev);
  return dev;
}

// out (+)= weight * sum(x^2). `partial` is an fp32 workspace of axb_sumsq_ctas() entries.
extern "C" int axb_sumsq_ctas() { return 148 * 4; }

extern "C" int axb_sumsq(const void* x, int is_bf16, int64_t n, float* partial, float* out,
                         float weight, int accumulate, cudaStream_t stream) {
  const int grid = grid_for(is_bf16 ? (n + 7) / 8 : n, 512, axb_sumsq_ctas());
  if (is_bf16)
    sumsq_bf16_kernel<<<grid, 512, 0, stream>>>(static_cast<const bf16*>(x), n, partial);
  else
    sumsq_f32_kernel<<<grid, 512, 0, stream>>>(static_cast<const float*>(x), n, partial);
  sum_partials_kernel<<<1, 32, 0, stream>>>(partial, grid, out, weight, accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
