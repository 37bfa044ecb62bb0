// Cross-GPU signalling and the reduction half of the fused reduce-scatter.
//
//   axb_signal_peers    one thread per peer stores `value` (release, system scope) into
//                       flags[slot] of that peer's flag array, after a system-wide fence that
//                       orders this stream's earlier stores to peer memory before the flag.
//   axb_wait_flags      waits (bounded) until `count` local flags all equal `value`; on timeout
//                       records a code in the status word and returns (the stream continues).
//   axb_reduce_slots    out[i] = sum_r staging[r][i] in fp32 and fixed slot order (so the result
//                       is bit-reproducible), written as bf16; optionally accumulates the sum
//                       of squares of the result into per-CTA partials for global-norm clipping.
//
// Waiting kernels never wait on a kernel that might not be resident: flags are written by
// kernels of *other* GPUs (or, in single-GPU tests, by an earlier launch on the same stream).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace axb {

__global__ void signal_peers_kernel(int* const* peer_flags, int world, int slot, int value) {
  const int r = threadIdx.x;
  if (r < world) {
    __threadfence_system();
    asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(peer_flags[r] + slot), "r"(value) : "memory");
  }
}

__global__ void wait_flags_kernel(const int* flags, int count, int value, int* status) {
  const int i = threadIdx.x;
  if (i < count) {
    bool ok = false;
    for (uint32_t it = 0; it < (1u << 22); ++it) {
      int v;
      asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(flags + i) : "memory");
      if (v == value) {
        ok = true;
        break;
      }
      __nanosleep(200);
    }
    if (!ok && status != nullptr) atomicCAS(status, 0, 4);
  }
}

struct alignas(16) V8 {
  __nv_bfloat162 v[4];
};

__global__ void reduce_slots_kernel(const __nv_bfloat16* __restrict__ staging, __nv_bfloat16* __restrict__ out,
                                    int slots, int64_t n, float* __restrict__ sumsq_partial) {
  __shared__ float red[32];
  const int64_t nvec = n / 8;
  float ss = 0.f;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int r = 0; r < slots; ++r) {
      const V8 a = reinterpret_cast<const V8*>(staging + r * n)[i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(a.v[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    V8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      o.v[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      const float2 f = __bfloat1622float2(o.v[j]);
      ss += f.x * f.x + f.y * f.y;
    }
    reinterpret_cast<V8*>(out)[i] = o;
  }
  if (sumsq_partial != nullptr) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    if (warp == 0) {
      float t = lane < nw ? red[lane] : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
      if (lane == 0) sumsq_partial[blockIdx.x] = t;
    }
  }
}

}  // namespace axb

extern "C" int axb_signal_peers(int* const* peer_flags_dev, int world, int slot, int value, cudaStream_t stream) {
  if (world > 32) return -10;
  axb::signal_peers_kernel<<<1, 32, 0, stream>>>(peer_flags_dev, world, slot, value);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int axb_wait_flags(const int* flags, int count, int value, int* status, cudaStream_t stream) {
  if (count > 1024) return -10;
  axb::wait_flags_kernel<<<1, ((count + 31) / 32) * 32, 0, stream>>>(flags, count, value, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Number of CTAs (= entries of `sumsq_partial`) used for a tensor of n elements.
extern "C" int axb_reduce_slots_ctas(int64_t n) {
  int64_t b = (n / 8 + 255) / 256;
  if (b < 1) b = 1;
  return static_cast<int>(b < 16 * 4 ? b : 16 * 4);
}

// n must be a multiple of 8. Uses few CTAs on purpose: it runs beside the backward GEMMs.
extern "C" int axb_reduce_slots(const void* staging, void* out, int slots, int64_t n, float* sumsq_partial,
                                cudaStream_t stream) {
  if (n % 8) return -10;
  axb::reduce_slots_kernel<<<axb_reduce_slots_ctas(n), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(staging), static_cast<__nv_bfloat16*>(out), slots, n, sumsq_partial);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
