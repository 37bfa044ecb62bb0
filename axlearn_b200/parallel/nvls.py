"""In-switch (NVLS) all-reduce with ``multimem`` instructions.

Every rank owns a symmetric bf16 buffer that is also bound to an NVLink multicast object.  An
all-reduce is: write the input into the own buffer; barrier (flags over peer memory); each rank
reduces ITS slice of the buffer with ``multimem.ld_reduce`` -- the NVSwitch reads every rank's copy
and returns the fp32-accumulated sum -- and writes the sums to every rank's copy with
``multimem.st``; barrier.  Each GPU sends and receives ``numel / world`` elements per direction
instead of the ``(world - 1) / world * numel`` of a ring (``csrc/peer_sync.cu``
``axb_multimem_allreduce``).

Multicast binding is opt-in (``AXB200_NVLS=1`` in the environment before the first symmetric
allocation of the process): a rank that exits while its memory is bound to a multicast object
raises NVLink faults on its peers, so fault-tolerant (supervised, restartable) jobs leave it off.
"""

from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

from axlearn_b200.parallel import symm


def enabled() -> bool:
    return os.environ.get("AXB200_NVLS", "0") == "1"


class MultimemAllReduce:
    """All-reduce (sum) of bf16 tensors of up to ``numel`` elements over ``group``."""

    def __init__(self, numel: int, *, group=None, device=None):
        if not enabled():
            raise RuntimeError("NVLS is opt-in: set AXB200_NVLS=1 before the first symmetric allocation")
        if numel % 8:
            raise ValueError("numel must be a multiple of 8")
        self.numel = numel
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.buffer, self._sym = symm.symmetric_empty_like_sharded((numel,), torch.bfloat16, group, device)
        self.multicast_ptr = self._sym.multicast_ptr
        if not self.multicast_ptr:
            raise RuntimeError("the symmetric allocation has no multicast address (NVLS unavailable on this system)")
        # Two barriers per call, each with its own flag row: [2, world].
        self.flags, self._flags_sym = symm.symmetric_empty_like_sharded((2, self.world), torch.int32, group, device)
        self.flags.zero_()
        self._flag_ptrs = symm.device_pointer_array(self._flags_sym.peer_ptrs, device)
        self._flags_sym.barrier()
        self.epoch = 0

    def _barrier(self, which: int) -> None:
        from axlearn_b200.ops import cuda_ops, fused_comm

        del cuda_ops
        # Raise flag [which][rank] on every peer, then wait for the whole row locally.
        fused_comm.signal_peers(self._flag_ptrs, self.world, which * self.world + self.rank, self.epoch)
        fused_comm.wait_flags(self.flags[which], self.world, self.epoch)

    def all_reduce(self, x: torch.Tensor, *, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Sum of ``x`` over the group.  Every rank must call with the same number of elements."""
        from axlearn_b200.ops import cuda_ops

        n = x.numel()
        if n > self.numel or n % 8 or x.dtype != torch.bfloat16:
            raise ValueError(f"unsupported all-reduce input: {tuple(x.shape)} {x.dtype}")
        self.epoch += 1
        self.buffer[:n].copy_(x.reshape(-1))
        self._barrier(0)            # every rank's input is in place
        rc = cuda_ops.lib().axb_multimem_allreduce(self.multicast_ptr, n // 8, self.world, self.rank,
                                                   cuda_ops._stream())  # pylint: disable=protected-access
        cuda_ops._check(rc, "axb_multimem_allreduce")  # pylint: disable=protected-access
        self._barrier(1)            # every slice has been reduced and broadcast
        result = self.buffer[:n].view(x.shape)
        if out is None:
            return result.clone()
        out.copy_(result)
        return out
