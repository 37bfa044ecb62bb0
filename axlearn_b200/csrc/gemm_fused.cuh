// Pieces shared by the fused compute+collective GEMM kernels: the argument blocks that describe a
// parameter all-gather riding along with a GEMM and a reduce-scatter out of its epilogue, bounded
// flag waits on peer-visible memory, and the copy warp that moves peer slabs with bulk copies.
#pragma once

#include "sm100.cuh"

namespace axb {

constexpr int kMaxPeers = 8;

// Extra arguments of the fused compute+collective variants (FUSED = true).
//
// All-gather of FSDP weights inside the GEMM (a `GatherJob`).  Every rank stores a contiguous
// row-slab of the weight (`shard_bytes` bytes).  One extra warp in every CTA of this kernel pulls
// its share of each rank's slab from `src[r]` (peers in ring order, the own slab last) into this
// GPU's full-size buffer `dst` (slab r at byte offset r * shard_bytes) with bulk asynchronous
// copies, and `epoch` is published in `flags[r]` when slab r is complete.  Two uses:
//   carried         the gathered weight is NOT this GEMM's operand (it is the operand of a later
//                   launch, typically the same matrix of the next layer): the copy simply rides
//                   along and is complete, by stream order, when this kernel ends;
//   ag_consume = 1  B is `ag[0].dst` itself: tiles inside the own slab are read straight from the
//                   shard, other tiles wait (bounded) for the flags of the slabs they touch, and
//                   every rank starts on its own slab (`ag_shard_extent` rows per slab).
//                   `ag_along_k` says whether the slab rows are B's contraction dim (B stored
//                   [K, N]) or its N dim (B stored [N, K]).
//
// Reduce-scatter of C (weight gradients) out of the epilogue: row m of C belongs to rank
// m / rs_rows_per_rank and is stored into that rank's staging buffer at slot `rs_rank`
// (`rs_dst[owner] + (rs_rank * rs_rows_per_rank + m % rs_rows_per_rank) * ldc`), i.e. every
// rank ends up holding one partial per peer, which it later reduces in a fixed order.
// With rs_mode = 1 the same epilogue implements the first half of a small-message all-reduce
// (tensor-parallel decode): rows go to every peer and the kernel itself raises the flags.
struct GatherJob {
  const void* src[kMaxPeers];  // every rank's slab (peer pointers; the own shard at [rank])
  void* dst;                   // this GPU's full-size buffer
  int* flags;                  // [world], this GPU's memory: epoch once slab r is complete
  int* cnt;                    // [world], zero-initialised arrival counters of the copy warps
  int64_t shard_bytes;
  int world, rank, epoch, reserved;
};

struct FusedParams {
  // Up to two gathers per launch; with ag_consume, ag[0] is the gather of this GEMM's B.
  GatherJob ag[2];
  int ag_consume, ag_along_k;
  int ag_shard_extent;  // consume mode: rows of the split dim (K or N) per slab
  int reserved;
  // reduce-scatter of C
  void* rs_dst[kMaxPeers];
  int rs_world, rs_rank, rs_rows_per_rank;
  // rs_mode 1 ("all-reduce push"): every row is stored into slot `rs_rank` of EVERY peer's
  // staging buffer [rs_world, M, N], and the last CTA to finish raises flag
  // [rs_site * rs_world + rs_rank] = *rs_epoch_ptr in every peer's flag array.
  int rs_mode, rs_site;
  int* rs_counter;             // zero-initialised arrival counter of the CTAs (this GPU)
  const int* rs_epoch_ptr;     // device memory, so that captured graphs see a new epoch each replay
  int* rs_flags[kMaxPeers];
};

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded wait until *flag == epoch. Returns false (and records a status) on timeout.
__device__ __forceinline__ bool wait_flag(const int* flag, int epoch, int* status) {
  for (uint32_t i = 0; i < (1u << 24); ++i) {
    if (ld_acquire_sys(flag) == epoch) return true;
    __nanosleep(64);
  }
  if (status != nullptr) atomicCAS(status, 0, kStatusWaitTimeoutPeer);
  return false;
}

// Bulk (non-tensor) asynchronous copies used by the copy warps of the fused all-gather.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(
                   reinterpret_cast<uint64_t>(gdst)),
               "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}

constexpr int kCopyBufs = 2;
constexpr uint32_t kCopyChunk = 16384;

// Copy warp of the fused all-gather (one per CTA, one elected thread): CTA c moves chunks
// c, c + G, ... of every slab (peers in ring order, the own slab last) into the local full-size
// buffer with bulk asynchronous copies staged through two shared-memory buffers, and the last
// CTA to finish a slab publishes its flag.  No SM is taken away from the GEMM: the copies ride
// on the otherwise idle bulk-copy path of every CTA.
__device__ inline bool ag_copy_warp(uint8_t* bufs, uint64_t* copy_full, const GatherJob& f, int64_t& seq, int* status) {
  const int c = blockIdx.x, num_c = gridDim.x;
  const int64_t shard_bytes = f.shard_bytes;
  const int64_t chunks_per_shard = (shard_bytes + kCopyChunk - 1) / kCopyChunk;
  const int64_t mine = c < chunks_per_shard ? (chunks_per_shard - c + num_c - 1) / num_c : 0;  // per slab
  const int64_t total = mine * f.world;
  auto locate = [&](int64_t n, const uint8_t*& src, uint8_t*& dst, uint32_t& bytes) {
    const int s = static_cast<int>(n / mine);
    const int r = (f.rank + 1 + s) % f.world;  // peers first, own slab last
    const int64_t off = (c + (n % mine) * num_c) * static_cast<int64_t>(kCopyChunk);
    const int64_t left = shard_bytes - off;
    bytes = left < static_cast<int64_t>(kCopyChunk) ? static_cast<uint32_t>(left) : kCopyChunk;
    src = static_cast<const uint8_t*>(f.src[r]) + off;
    dst = static_cast<uint8_t*>(f.dst) + r * shard_bytes + off;
  };
  auto issue_load = [&](int64_t n) {
    const uint8_t* src;
    uint8_t* dst;
    uint32_t bytes;
    locate(n, src, dst, bytes);
    const int b = static_cast<int>((seq + n) % kCopyBufs);
    mbar_arrive_expect_tx(&copy_full[b], bytes);
    bulk_load(bufs + b * kCopyChunk, src, bytes, &copy_full[b]);
  };
  bool ok = true;
  tma_store_wait_read<0>();  // a previous job's last stores may still be reading the buffers
  if (total > 0) issue_load(0);
  for (int64_t n = 0; n < total && ok; ++n) {
    if (n + 1 < total) {
      // Buffer (n+1) % 2 was read by store n-1: wait until that read is over, then refill it.
      tma_store_wait_read<0>();
      issue_load(n + 1);
    }
    const int b = static_cast<int>((seq + n) % kCopyBufs);
    const uint32_t ph = static_cast<uint32_t>(((seq + n) / kCopyBufs) & 1);
    if (!mbar_wait(&copy_full[b], ph, status, kStatusWaitTimeoutProducer)) {
      ok = false;
      break;
    }
    const uint8_t* src;
    uint8_t* dst;
    uint32_t bytes;
    locate(n, src, dst, bytes);
    bulk_store(dst, bufs + b * kCopyChunk, bytes);
    tma_store_commit();
    if ((n + 1) % mine == 0) {
      // Slab done for this CTA: its stores must be complete before the arrival is counted.
      const int r = (f.rank + 1 + static_cast<int>(n / mine)) % f.world;
      tma_store_wait<0>();
      __threadfence();
      if (atomicAdd(&f.cnt[r], 1) == num_c - 1) {
        f.cnt[r] = 0;
        __threadfence();
        st_release_sys(&f.flags[r], f.epoch);
      }
    }
  }
  if (ok && mine == 0) {
    // Nothing to copy (more CTAs than chunks): still count this CTA's arrival for every slab.
    for (int s = 0; s < f.world; ++s) {
      const int r = (f.rank + 1 + s) % f.world;
      if (atomicAdd(&f.cnt[r], 1) == num_c - 1) {
        f.cnt[r] = 0;
        __threadfence();
        st_release_sys(&f.flags[r], f.epoch);
      }
    }
  }
  tma_store_wait<0>();
  seq += total;
  return ok;
}

}  // namespace axb
