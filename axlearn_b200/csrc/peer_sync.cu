// Cross-GPU signalling and the reduction half of the fused reduce-scatter.
//
//   axb_signal_peers    one thread per peer stores `value` (release, system scope) into
//                       flags[slot] of that peer's flag array, after a system-wide fence that
//                       orders this stream's earlier stores to peer memory before the flag.
//   axb_wait_flags      waits (bounded) until `count` local flags all equal `value`; on timeout
//                       records a code in the status word and returns (the stream continues).
//   axb_reduce_slots    out[i] (+)= sum_r staging[r][i] in fp32 and fixed slot order (so the result
//                       is bit-reproducible), written as bf16; optionally accumulates the sum
//                       of squares of the result into per-CTA partials for global-norm clipping.
//
//   axb_multimem_allreduce   the reduction half of an in-switch (NVLS) all-reduce: this rank's slice
//                       of a multicast-bound symmetric buffer is read with multimem.ld_reduce
//                       (the NVSwitch sums all ranks' copies, fp32 accumulation) and the sums are
//                       written back to every rank's copy with multimem.st.  The callers order
//                       it between two flag barriers (signal + wait above).
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

// Eight bf16 values moved as ONE 16-byte access (a member-wise copy of the four pairs compiles to
// four 4-byte accesses).
struct alignas(16) V8 {
  __nv_bfloat162 v[4];
  V8() = default;
  __device__ __forceinline__ V8(const V8& o) { *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(o.v); }
  __device__ __forceinline__ V8& operator=(const V8& o) {
    *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(o.v);
    return *this;
  }
};

__global__ void reduce_slots_kernel(const __nv_bfloat16* __restrict__ staging, __nv_bfloat16* __restrict__ out,
                                    int slots, int64_t n, float* __restrict__ sumsq_partial, int accumulate) {
  __shared__ float red[32];
  const int64_t nvec = n / 8;
  float ss = 0.f;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    if (accumulate) {
      const V8 a = reinterpret_cast<const V8*>(out)[i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(a.v[j]);
        acc[2 * j] = f.x;
        acc[2 * j + 1] = f.y;
      }
    }
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

// One 16-byte vector (eight bf16) per thread and trip.  `mc` is the multicast address of the buffer;
// vectors [first, first + count) are this rank's share.
__global__ void multimem_allreduce_kernel(uint64_t mc, int64_t first, int64_t count) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < count;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const uint64_t addr = mc + static_cast<uint64_t>(first + i) * 16;
    uint32_t a, b, c, d;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(a), "=r"(b), "=r"(c), "=r"(d)
                 : "l"(addr)
                 : "memory");
    asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(addr), "r"(a), "r"(b),
                 "r"(c), "r"(d)
                 : "memory");
  }
  // The stores travel through the switch to every peer: ordered before this kernel can complete,
  // so the flag raised by the next launch cannot overtake them.
  __threadfence_system();
}

}  // namespace axb

// Reduces vectors [rank * nvec / world, (rank + 1) * nvec / world) of a buffer of `nvec` 16-byte
// vectors (bf16) bound to the multicast address `mc_ptr`, in place on every rank.
extern "C" int axb_multimem_allreduce(uint64_t mc_ptr, int64_t nvec, int world, int rank, cudaStream_t stream) {
  if (mc_ptr == 0 || (mc_ptr & 15) || world < 1 || rank < 0 || rank >= world) return -10;
  const int64_t first = nvec * rank / world, last = nvec * (rank + 1) / world;
  const int64_t count = last - first;
  if (count <= 0) return 0;
  int64_t ctas = (count + 255) / 256;
  if (ctas > 296) ctas = 296;
  axb::multimem_allreduce_kernel<<<static_cast<int>(ctas), 256, 0, stream>>>(mc_ptr, first, count);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

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
                                int accumulate, cudaStream_t stream) {
  if (n % 8) return -10;
  axb::reduce_slots_kernel<<<axb_reduce_slots_ctas(n), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(staging), static_cast<__nv_bfloat16*>(out), slots, n, sumsq_partial,
      accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// ---------------------------------------------------------------------------------------------
// One-shot all-reduce for small, latency-bound messages (tensor-parallel decode).
//
//   axb_allreduce_push    copies this rank's partial vector into slot `rank` of every peer's
//                         staging buffer (plain peer stores), and the last CTA to finish raises
//                         flag [site * world + rank] on every peer to the current epoch;
//   axb_allreduce_finish  every CTA waits (bounded) until the `world` local flags of the site
//                         equal the epoch, then writes out = (residual +) sum of the slots for
//                         its share of the vector.
//
// The epoch lives in device memory (`epoch_ptr`) so that both launches can sit in a captured
// CUDA graph and still see a new value every replay; the caller bumps it once per step.
// Staging and flags are per call site, so a rank that runs ahead never overwrites data that a
// slower peer has not reduced yet (see DecodeEngine in axlearn_b200/inference).
namespace axb {

__global__ void allreduce_push_kernel(const uint4* __restrict__ src, uint4* const* peer_staging,
                                      int* const* peer_flags, int* done_counter, const int* epoch_ptr,
                                      int world, int rank, int site, int64_t nvec) {
  for (int r = 0; r < world; ++r) {
    uint4* dst = peer_staging[r] + static_cast<int64_t>(rank) * nvec;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)
      dst[i] = src[i];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(done_counter, 1) == static_cast<int>(gridDim.x) - 1) {
      *done_counter = 0;
      __threadfence_system();
      const int epoch = *epoch_ptr;
      for (int r = 0; r < world; ++r)
        asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(peer_flags[r] + site * world + rank), "r"(epoch)
                     : "memory");
    }
  }
}

__global__ void allreduce_finish_kernel(const __nv_bfloat16* staging,
                                        const __nv_bfloat16* __restrict__ residual,
                                        __nv_bfloat16* __restrict__ out, const int* flags, const int* epoch_ptr,
                                        int world, int site, int64_t n, int* status) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < world) {
    const int epoch = *epoch_ptr;
    bool ok = false;
    for (uint32_t it = 0; it < (1u << 22); ++it) {
      int v;
      asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(flags + site * world + threadIdx.x) : "memory");
      if (v == epoch) {
        ok = true;
        break;
      }
      __nanosleep(100);
    }
    if (!ok) {
      s_ok = 0;
      if (status != nullptr) atomicCAS(status, 0, 4);
    }
  }
  __syncthreads();
  if (!s_ok) return;
  const int64_t nvec = n / 8;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float acc[8];
    if (residual != nullptr) {
      const V8 a = reinterpret_cast<const V8*>(residual)[i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(a.v[j]);
        acc[2 * j] = f.x;
        acc[2 * j + 1] = f.y;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    }
    for (int r = 0; r < world; ++r) {
      // Written by peers while this kernel may already be resident: L2-coherent loads.
      const uint4 u = __ldcg(reinterpret_cast<const uint4*>(staging + r * n) + i);
      const __nv_bfloat162* av = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(av[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    V8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) o.v[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    reinterpret_cast<V8*>(out)[i] = o;
  }
}

}  // namespace axb

// n (elements, bf16) must be a multiple of 8; `peer_staging_dev[r]` points at rank r's staging
// buffer [world, n] for this site; `peer_flags_dev[r]` at rank r's flag array [sites, world].
extern "C" int axb_allreduce_push(const void* src, void* const* peer_staging_dev, int* const* peer_flags_dev,
                                  int* done_counter, const int* epoch_ptr, int world, int rank, int site,
                                  int64_t n, cudaStream_t stream) {
  if (n % 8 || world > 32) return -10;
  const int64_t nvec = n / 8;
  // Decode-sized messages stay on a few CTAs (launch latency matters, not bandwidth); large
  // activations (tensor-parallel training) get enough CTAs to fill the memory system.
  int ctas = static_cast<int>((nvec + 255) / 256);
  const int cap = nvec > (1 << 20) ? 592 : 32;
  if (ctas > cap) ctas = cap;
  axb::allreduce_push_kernel<<<ctas, 256, 0, stream>>>(
      static_cast<const uint4*>(src), reinterpret_cast<uint4* const*>(peer_staging_dev), peer_flags_dev,
      done_counter, epoch_ptr, world, rank, site, nvec);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int axb_allreduce_finish(const void* staging, const void* residual, void* out, const int* flags,
                                    const int* epoch_ptr, int world, int site, int64_t n, int* status,
                                    cudaStream_t stream) {
  if (n % 8 || world > 32) return -10;
  const int64_t nvec = n / 8;
  int ctas = static_cast<int>((nvec + 255) / 256);
  const int cap = nvec > (1 << 20) ? 592 : 32;
  if (ctas > cap) ctas = cap;
  axb::allreduce_finish_kernel<<<ctas, 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(staging), static_cast<const __nv_bfloat16*>(residual),
      static_cast<__nv_bfloat16*>(out), flags, epoch_ptr, world, site, n, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
