// Allocation-free RMSNorm backward: see no_alloc.h for the contract and for who needs it.
//
// The math and the summation order are those of axb_rmsnorm_bwd() in elementwise.cu (per-CTA
// partial sums of dscale over a fixed set of rows, then a reduction over CTAs in index order),
// so both entry points return identical bits.  The only difference is where the partial sums
// live: here in `g_partials`, a device array owned by the library.
#include "no_alloc.h"

#include <cuda_bf16.h>
#include <stdio.h>

namespace {

using bf16 = __nv_bfloat16;

// Eight bf16 values moved as ONE 16-byte access: the copy operations are written out, because a
// member-wise copy of the four bf16 pairs compiles to four 4-byte accesses (four times the
// load / store instructions and cache sectors touched per warp).
struct alignas(16) Vec8 {
  __nv_bfloat162 v[4];
  Vec8() = default;
  __device__ __forceinline__ Vec8(const Vec8& o) { *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(o.v); }
  __device__ __forceinline__ Vec8& operator=(const Vec8& o) {
    *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(o.v);
    return *this;
  }
};

// The library-owned workspace: [AXB_NOALLOC_RMSNORM_MAX_CTAS][AXB_NOALLOC_RMSNORM_MAX_D] fp32.
// In host code this name is only a handle for cudaGetSymbolAddress(); it is not a device
// pointer and must never be passed to a kernel directly.
static __device__ __align__(256) float g_partials[AXB_NOALLOC_RMSNORM_MAX_CTAS * AXB_NOALLOC_RMSNORM_MAX_D];

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

__device__ __forceinline__ float block_sum(float x, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  x = warp_sum(x);
  __syncthreads();
  if (lane == 0) red[warp] = x;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  return warp_sum(t);
}

__global__ void rmsnorm_bwd_noalloc_kernel(const bf16* __restrict__ x, const bf16* __restrict__ scale,
                                           const float* __restrict__ rstd_in, const bf16* __restrict__ dy,
                                           const bf16* __restrict__ dres, bf16* __restrict__ dx,
                                           float* __restrict__ partial, int64_t rows, int D) {
  __shared__ float red[32];
  extern __shared__ float dscale_acc[];
  for (int i = threadIdx.x; i < D; i += blockDim.x) dscale_acc[i] = 0.f;
  const int nvec = D / 8;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const Vec8* xr = reinterpret_cast<const Vec8*>(x + row * D);
    const Vec8* gr = reinterpret_cast<const Vec8*>(dy + row * D);
    const Vec8* sc = reinterpret_cast<const Vec8*>(scale);
    const float rstd = rstd_in[row];
    float dot = 0.f;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      Vec8 a = xr[i], g = gr[i], s = sc[i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 xf = __bfloat1622float2(a.v[j]), gf = __bfloat1622float2(g.v[j]), sf = __bfloat1622float2(s.v[j]);
        dot += gf.x * sf.x * xf.x * rstd + gf.y * sf.y * xf.y * rstd;
      }
    }
    dot = block_sum(dot, red) / D;
    const Vec8* rr = dres ? reinterpret_cast<const Vec8*>(dres + row * D) : nullptr;
    Vec8* dxr = reinterpret_cast<Vec8*>(dx + row * D);
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      Vec8 a = xr[i], g = gr[i], s = sc[i], o, r;
      if (rr) r = rr[i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 xf = __bfloat1622float2(a.v[j]), gf = __bfloat1622float2(g.v[j]), sf = __bfloat1622float2(s.v[j]);
        const float xh0 = xf.x * rstd, xh1 = xf.y * rstd;
        float d0 = rstd * (gf.x * sf.x - xh0 * dot);
        float d1 = rstd * (gf.y * sf.y - xh1 * dot);
        if (rr) {
          float2 rf = __bfloat1622float2(r.v[j]);
          d0 += rf.x;
          d1 += rf.y;
        }
        o.v[j] = __floats2bfloat162_rn(d0, d1);
        dscale_acc[i * 8 + 2 * j] += gf.x * xh0;
        dscale_acc[i * 8 + 2 * j + 1] += gf.y * xh1;
      }
      dxr[i] = o;
    }
  }
  __syncthreads();
  // Row blockIdx.x of the workspace is written in full here, before the reduction reads it.
  for (int i = threadIdx.x; i < D; i += blockDim.x)
    partial[static_cast<int64_t>(blockIdx.x) * D + i] = dscale_acc[i];
}

__global__ void reduce_noalloc_kernel(const float* __restrict__ partial, bf16* __restrict__ out_bf16,
                                      float* __restrict__ out_f32, int nparts, int D) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= D) return;
  float s = 0.f;
  for (int p = 0; p < nparts; ++p) s += partial[static_cast<int64_t>(p) * D + i];
  if (out_bf16) out_bf16[i] = __float2bfloat16(s);
  if (out_f32) out_f32[i] = s;
}

constexpr int kMaxDevices = 64;
float* g_partials_addr[kMaxDevices] = {nullptr};
bool g_kernel_configured[kMaxDevices] = {false};

// Resolves (once per device) the device address of g_partials for the current device.
float* workspace_for_current_device(int* device_out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  *device_out = dev;
  if (g_partials_addr[dev] == nullptr) {
    float* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_partials);
    if (e != cudaSuccess || ptr == nullptr) {
      fprintf(stderr, "axb_rmsnorm_bwd_noalloc: cudaGetSymbolAddress failed on device %d: %s\n", dev,
              cudaGetErrorString(e));
      return nullptr;
    }
    g_partials_addr[dev] = ptr;
  }
  return g_partials_addr[dev];
}

}  // namespace

extern "C" int axb_rmsnorm_bwd_noalloc(const void* x, const void* scale, const float* rstd, const void* dy,
                                       const void* dres, void* dx, void* dscale_bf16, float* dscale_f32,
                                       int64_t rows, int D, cudaStream_t stream) {
  if (D <= 0 || D % 8) return -10;
  if (D > AXB_NOALLOC_RMSNORM_MAX_D) {
    fprintf(stderr,
            "axb_rmsnorm_bwd_noalloc: D = %d exceeds the built-in workspace (max D = %d); use "
            "axb_rmsnorm_bwd with a caller-provided workspace instead\n",
            D, AXB_NOALLOC_RMSNORM_MAX_D);
    return -20;
  }
  int dev = 0;
  float* partial = workspace_for_current_device(&dev);
  if (partial == nullptr) return -21;
  if (!g_kernel_configured[dev]) {
    if (cudaFuncSetAttribute(rmsnorm_bwd_noalloc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             AXB_NOALLOC_RMSNORM_MAX_D * static_cast<int>(sizeof(float))) != cudaSuccess)
      return -4;
    g_kernel_configured[dev] = true;
  }
  // Same grid rule as axb_rmsnorm_bwd_ctas() (one shared constant), so the summation order, and
  // with it the result, match the regular entry point bit for bit.
  const int grid = static_cast<int>(rows < AXB_NOALLOC_RMSNORM_MAX_CTAS ? rows : AXB_NOALLOC_RMSNORM_MAX_CTAS);
  if (grid <= 0) {
    // No rows: the gradient of the scale is exactly zero.
    if (dscale_bf16 != nullptr && cudaMemsetAsync(dscale_bf16, 0, D * sizeof(bf16), stream) != cudaSuccess) return -4;
    if (dscale_f32 != nullptr && cudaMemsetAsync(dscale_f32, 0, D * sizeof(float), stream) != cudaSuccess) return -4;
    return 0;
  }
  rmsnorm_bwd_noalloc_kernel<<<grid, 256, D * sizeof(float), stream>>>(
      static_cast<const bf16*>(x), static_cast<const bf16*>(scale), rstd, static_cast<const bf16*>(dy),
      static_cast<const bf16*>(dres), static_cast<bf16*>(dx), partial, rows, D);
  reduce_noalloc_kernel<<<(D + 255) / 256, 256, 0, stream>>>(partial, static_cast<bf16*>(dscale_bf16), dscale_f32,
                                                             grid, D);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
