"""Symmetric (peer-mapped) device memory for the fused compute+collective kernels.

A symmetric allocation exists at the same size on every rank of a group and is mapped into
every peer's address space over NVLink, so a kernel on rank A can load from / store to rank
B's copy through an ordinary pointer.  Allocation and the address exchange go through
``torch.distributed._symmetric_memory`` (CUDA VMM handles exchanged over the process group);
the kernels in ``axlearn_b200/csrc`` only ever see raw peer pointers.

``SymmetricBuffer`` wraps one allocation; ``find`` maps any tensor that lives inside a
symmetric allocation to the corresponding peer addresses (same offset on every rank).
In single-process tests ``FakePeers`` stands in: "peers" are just other local tensors.
"""

from __future__ import annotations

import bisect
import os
from typing import Optional, Sequence

import torch
import torch.distributed as dist

_registry: list[tuple[int, int, "SymmetricBuffer"]] = []  # (start, end, buffer), sorted by start


class SymmetricBuffer:
    """One symmetric allocation of ``numel`` elements of ``dtype`` on every rank of ``group``."""

    def __init__(self, numel: int, dtype: torch.dtype, group, device: torch.device):
        # The kernels use unicast peer pointers only.  Without this switch the rendezvous also
        # binds every allocation to an NVLink multicast object, which buys nothing here and turns
        # a rank that exits abruptly (watchdog or supervisor kill) into NVLink faults on its peers.
        # AXB200_NVLS=1 opts in to the binding (parallel/nvls.py: in-switch reductions).
        if os.environ.get("AXB200_NVLS", "0") == "1":
            os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "0"
        else:
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group
        try:  # Needed by some versions before the first rendezvous on a group.
            symm_mem.enable_symm_mem_for_group(group.group_name)
        except Exception:  # pylint: disable=broad-except
            pass
        self.tensor = symm_mem.empty(numel, dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(self.tensor, group=group)
        self.rank = self.handle.rank
        self.world = self.handle.world_size
        self.peer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.multicast_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        self.nbytes = numel * self.tensor.element_size()
        start = self.tensor.data_ptr()
        bisect.insort(_registry, (start, start + self.nbytes, self), key=lambda e: e[0])

    def peer_addresses(self, t: torch.Tensor) -> list[int]:
        """Addresses of the peers' copies of ``t`` (a view into this buffer)."""
        off = t.data_ptr() - self.tensor.data_ptr()
        if off < 0 or off >= self.nbytes:
            raise ValueError("tensor does not live in this symmetric buffer")
        return [p + off for p in self.peer_ptrs]

    def barrier(self) -> None:
        self.handle.barrier()


def find(t: torch.Tensor) -> Optional[SymmetricBuffer]:
    ptr = t.data_ptr()
    for start, end, buf in _registry:  # few buffers exist: a scan is enough
        if start <= ptr < end:
            return buf
    return None


def symmetric_empty_like_sharded(shape: Sequence[int], dtype: torch.dtype, group, device) -> tuple[torch.Tensor, SymmetricBuffer]:
    numel = 1
    for s in shape:
        numel *= s
    buf = SymmetricBuffer(numel, dtype, group, device)
    return buf.tensor.view(*shape), buf


def device_pointer_array(ptrs: Sequence[int], device) -> torch.Tensor:
    """A device int64 tensor holding raw pointers (for kernels that take ``T* const*``)."""
    return torch.tensor(list(ptrs), dtype=torch.int64, device=device)
