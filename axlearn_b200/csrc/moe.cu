// Token movement for mixture-of-experts layers: rows of [tokens, M] activations are gathered into
// per-expert buffers ("dispatch") and expert outputs are summed back per token with the gate
// weights ("combine").  Routing is index-based: for every (token, choice) `dest` holds the row of
// the expert buffer (or -1 when the assignment was dropped), and `inv` is its inverse (expert-buffer
// row -> token, -1 for an unfilled slot).
//
//   gather_rows    out[r] = scale[r] * src[idx[r]]   (zero row where idx[r] < 0): dispatch forward,
//                  and the backward of combine with scale = gate weight;
//   combine_rows   out[t] = sum_k w[t,k] * y[dest[t,k]]: combine forward, and the backward of
//                  dispatch with w = 1;
//   row_dots       out[t,k] = <a[t], y[dest[t,k]]>: gradient of the gate weights.
//
// All three are pure bandwidth: each CTA handles rows with 16-byte loads/stores, fp32 math.
// The reference expresses the same thing as einsums against one-hot [tokens, E, C] tensors
// (axlearn/common/mixture_of_experts.py:676-725, 1050-1098).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace axb {

struct alignas(16) Bf8 {
  __nv_bfloat162 v[4];
};

__global__ void gather_rows_kernel(const Bf8* __restrict__ src, const int* __restrict__ idx,
                                   const float* __restrict__ scale, Bf8* __restrict__ out, int64_t rows, int mvec) {
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const int s = idx[r];
    const float sc = (scale != nullptr && s >= 0) ? scale[r] : 1.f;
    for (int c = threadIdx.x; c < mvec; c += blockDim.x) {
      Bf8 o;
      if (s < 0) {
#pragma unroll
        for (int j = 0; j < 4; ++j) o.v[j] = __floats2bfloat162_rn(0.f, 0.f);
      } else {
        o = src[static_cast<int64_t>(s) * mvec + c];
        if (scale != nullptr) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(o.v[j]);
            o.v[j] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
          }
        }
      }
      out[r * mvec + c] = o;
    }
  }
}

__global__ void combine_rows_kernel(const Bf8* __restrict__ y, const int* __restrict__ dest,
                                    const float* __restrict__ w, Bf8* __restrict__ out, int64_t tokens, int k,
                                    int mvec) {
  for (int64_t t = blockIdx.x; t < tokens; t += gridDim.x) {
    for (int c = threadIdx.x; c < mvec; c += blockDim.x) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int kk = 0; kk < k; ++kk) {
        const int d = dest[t * k + kk];
        if (d < 0) continue;
        const float wk = w != nullptr ? w[t * k + kk] : 1.f;
        const Bf8 a = y[static_cast<int64_t>(d) * mvec + c];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(a.v[j]);
          acc[2 * j] += wk * f.x;
          acc[2 * j + 1] += wk * f.y;
        }
      }
      Bf8 o;
#pragma unroll
      for (int j = 0; j < 4; ++j) o.v[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      out[t * mvec + c] = o;
    }
  }
}

// One warp per (token, choice).
__global__ void row_dots_kernel(const Bf8* __restrict__ a, const Bf8* __restrict__ y, const int* __restrict__ dest,
                                float* __restrict__ out, int64_t pairs, int k, int mvec) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t p = warp; p < pairs; p += nwarps) {
    const int d = dest[p];
    float s = 0.f;
    if (d >= 0) {
      const int64_t t = p / k;
      for (int c = lane; c < mvec; c += 32) {
        const Bf8 u = a[t * mvec + c];
        const Bf8 v = y[static_cast<int64_t>(d) * mvec + c];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(u.v[j]);
          const float2 g = __bfloat1622float2(v.v[j]);
          s += f.x * g.x + f.y * g.y;
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) out[p] = s;
  }
}

static int row_grid(int64_t rows) {
  const int64_t cap = 148 * 16;
  return static_cast<int>(rows < cap ? (rows > 0 ? rows : 1) : cap);
}

}  // namespace axb

// m (the row length in bf16 elements) must be a multiple of 8; pointers 16-byte aligned.
extern "C" int axb_moe_gather_rows(const void* src, const int* idx, const float* scale, void* out, int64_t rows,
                                   int m, cudaStream_t stream) {
  if (m % 8) return -10;
  if (rows <= 0) return 0;
  axb::gather_rows_kernel<<<axb::row_grid(rows), 256, 0, stream>>>(
      static_cast<const axb::Bf8*>(src), idx, scale, static_cast<axb::Bf8*>(out), rows, m / 8);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int axb_moe_combine_rows(const void* y, const int* dest, const float* w, void* out, int64_t tokens,
                                    int k, int m, cudaStream_t stream) {
  if (m % 8) return -10;
  if (tokens <= 0) return 0;
  axb::combine_rows_kernel<<<axb::row_grid(tokens), 256, 0, stream>>>(
      static_cast<const axb::Bf8*>(y), dest, w, static_cast<axb::Bf8*>(out), tokens, k, m / 8);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int axb_moe_row_dots(const void* a, const void* y, const int* dest, float* out, int64_t tokens, int k,
                                int m, cudaStream_t stream) {
  if (m % 8) return -10;
  const int64_t pairs = tokens * k;
  if (pairs <= 0) return 0;
  const int64_t ctas = (pairs * 32 + 255) / 256;
  axb::row_dots_kernel<<<static_cast<int>(ctas < 148 * 16 ? ctas : 148 * 16), 256, 0, stream>>>(
      static_cast<const axb::Bf8*>(a), static_cast<const axb::Bf8*>(y), dest, out, pairs, k, m / 8);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
