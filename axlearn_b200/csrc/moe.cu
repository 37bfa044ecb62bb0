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
// Expert-parallel variants (`*_peer`): the expert buffer is spread over the GPUs that own the
// experts and addressed through peer pointers, so dispatch *stores rows straight into the owner's
// memory* and combine *loads rows straight from it* over NVLink -- the all-to-all is fused into
// the token gather / weighted sum instead of being a separate collective plus a local copy.  A
// flat row d = e * slots + slot (expert e, slot within this rank's share of e) lives on rank
// e / experts_per_rank at row ((e % experts_per_rank) * world + this_rank) * slots + slot.
// Hand-shakes (flags) are separate tiny kernels in peer_sync.cu.
//
// All of them are pure bandwidth: each CTA handles rows with 16-byte loads/stores, fp32 math.
// The reference expresses the same thing as einsums against one-hot [tokens, E, C] tensors
// (axlearn/common/mixture_of_experts.py:676-725, 1050-1098).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace axb {

// Eight bf16 values moved as ONE 16-byte access (a member-wise copy of the four pairs compiles to
// four 4-byte accesses).
struct alignas(16) Bf8 {
  __nv_bfloat162 v[4];
  Bf8() = default;
  __device__ __forceinline__ Bf8(const Bf8& o) { *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(o.v); }
  __device__ __forceinline__ Bf8& operator=(const Bf8& o) {
    *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(o.v);
    return *this;
  }
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

struct PeerMap {
  void* base[8];
  int slots;             // rows per (expert, source rank)
  int experts_per_rank;
  int world;
  int rank;
};

__device__ __forceinline__ int64_t peer_row(const PeerMap& pm, int64_t d, int& owner) {
  const int e = static_cast<int>(d / pm.slots);
  const int slot = static_cast<int>(d - static_cast<int64_t>(e) * pm.slots);
  owner = e / pm.experts_per_rank;
  const int el = e - owner * pm.experts_per_rank;
  return (static_cast<int64_t>(el) * pm.world + pm.rank) * pm.slots + slot;
}

__global__ void push_rows_kernel(const Bf8* __restrict__ src, const int* __restrict__ idx,
                                 const float* __restrict__ scale, const __grid_constant__ PeerMap pm,
                                 int64_t rows, int mvec) {
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const int s = idx[r];
    const float sc = (scale != nullptr && s >= 0) ? scale[r] : 1.f;
    int owner;
    const int64_t row = peer_row(pm, r, owner);
    Bf8* out = static_cast<Bf8*>(pm.base[owner]) + row * mvec;
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
      out[c] = o;
    }
  }
  // Peer stores are posted: make them visible system-wide before this kernel completes, so
  // that the flag raised by the next launch cannot overtake them.
  __threadfence_system();
}

__global__ void pull_combine_kernel(const __grid_constant__ PeerMap pm, const int* __restrict__ dest,
                                    const float* __restrict__ w, Bf8* __restrict__ out, int64_t tokens,
                                    int k, int mvec) {
  for (int64_t t = blockIdx.x; t < tokens; t += gridDim.x) {
    for (int c = threadIdx.x; c < mvec; c += blockDim.x) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int kk = 0; kk < k; ++kk) {
        const int d = dest[t * k + kk];
        if (d < 0) continue;
        const float wk = w != nullptr ? w[t * k + kk] : 1.f;
        int owner;
        const int64_t row = peer_row(pm, d, owner);
        const Bf8 a = static_cast<const Bf8*>(pm.base[owner])[row * mvec + c];
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

__global__ void pull_row_dots_kernel(const Bf8* __restrict__ a, const __grid_constant__ PeerMap pm,
                                     const int* __restrict__ dest, float* __restrict__ out, int64_t pairs,
                                     int k, int mvec) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  const int64_t nwarps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t p = warp; p < pairs; p += nwarps) {
    const int d = dest[p];
    float s = 0.f;
    if (d >= 0) {
      const int64_t t = p / k;
      int owner;
      const int64_t row = peer_row(pm, d, owner);
      const Bf8* y = static_cast<const Bf8*>(pm.base[owner]) + row * mvec;
      for (int c = lane; c < mvec; c += 32) {
        const Bf8 u = a[t * mvec + c];
        const Bf8 v = y[c];
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

static int fill_peer_map(PeerMap& pm, const void* const* bases, int world, int rank, int slots,
                         int experts_per_rank) {
  if (world < 1 || world > 8 || rank < 0 || rank >= world || slots < 1 || experts_per_rank < 1) return -10;
  for (int i = 0; i < 8; ++i) pm.base[i] = i < world ? const_cast<void*>(bases[i]) : nullptr;
  pm.slots = slots;
  pm.experts_per_rank = experts_per_rank;
  pm.world = world;
  pm.rank = rank;
  return 0;
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

// Expert-parallel dispatch: row r of this rank's [num_experts * slots, m] dispatch output is
// written into the memory of the rank that owns its expert.  `bases` is a host array of the
// `world` ranks' buffer addresses (own included), each [experts_per_rank, world, slots, m].
extern "C" int axb_moe_push_rows(const void* src, const int* idx, const float* scale, const void* const* bases,
                                 int world, int rank, int slots, int experts_per_rank, int64_t rows, int m,
                                 cudaStream_t stream) {
  if (m % 8) return -10;
  if (rows <= 0) return 0;
  axb::PeerMap pm;
  if (int rc = axb::fill_peer_map(pm, bases, world, rank, slots, experts_per_rank)) return rc;
  if (rows != static_cast<int64_t>(world) * experts_per_rank * slots) return -10;
  axb::push_rows_kernel<<<axb::row_grid(rows), 256, 0, stream>>>(static_cast<const axb::Bf8*>(src), idx, scale, pm,
                                                               rows, m / 8);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Expert-parallel combine: out[t] = sum_k w[t,k] * (row dest[t,k] of the owners' output buffers).
extern "C" int axb_moe_pull_combine(const void* const* bases, int world, int rank, int slots, int experts_per_rank,
                                    const int* dest, const float* w, void* out, int64_t tokens, int k, int m,
                                    cudaStream_t stream) {
  if (m % 8) return -10;
  if (tokens <= 0) return 0;
  axb::PeerMap pm;
  if (int rc = axb::fill_peer_map(pm, bases, world, rank, slots, experts_per_rank)) return rc;
  axb::pull_combine_kernel<<<axb::row_grid(tokens), 256, 0, stream>>>(pm, dest, w, static_cast<axb::Bf8*>(out),
                                                                    tokens, k, m / 8);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int axb_moe_pull_row_dots(const void* a, const void* const* bases, int world, int rank, int slots,
                                     int experts_per_rank, const int* dest, float* out, int64_t tokens, int k,
                                     int m, cudaStream_t stream) {
  if (m % 8) return -10;
  const int64_t pairs = tokens * k;
  if (pairs <= 0) return 0;
  axb::PeerMap pm;
  if (int rc = axb::fill_peer_map(pm, bases, world, rank, slots, experts_per_rank)) return rc;
  const int64_t ctas = (pairs * 32 + 255) / 256;
  axb::pull_row_dots_kernel<<<static_cast<int>(ctas < 148 * 16 ? ctas : 148 * 16), 256, 0, stream>>>(
      static_cast<const axb::Bf8*>(a), pm, dest, out, pairs, k, m / 8);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
