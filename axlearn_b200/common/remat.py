"""Selective rematerialisation: what a replayed layer keeps between its first pass and its replay.

The reference expresses remat policies as ``jax.checkpoint`` policies over tensors tagged with
``checkpoint_name`` (axlearn/common/utils.py:163-328: ``save_only_these_names``,
``save_and_offload_only_these_names_regex``, ``dots_saveable``, ``offload_dots_saveable``;
axlearn/common/base_layer.py:783-797 ``_remat_name``; the default Fuji policy keeps
``.*([qkvo]_proj|context)``, axlearn/common/attention.py:4574-4653) and lets XLA drop the
recomputation of everything that a saved tensor makes unnecessary.

An eager runtime has no graph to prune, so the saving is done where the time goes: by the
expensive operators themselves.  A layer that is replayed in backward (``Repeat`` with a
``remat_spec``, or any layer whose wrapped methods run under ``remat_call``) opens a
``LayerStash``.  During the first (no-grad) pass the stash *records*: a projection GEMM or the
attention kernel that runs inside ``tagged(owner, names)`` asks the policy about
``"{OwnerClass}.{name}"`` and, if every name of the scope may be kept, stores its output (for
attention: the context and the log-sum-exp the backward kernel needs) on the device or, for
names the policy offloads, in pinned host memory.  During the replay the same operators find
their stored outputs and skip their forward kernels; their backward passes never needed the
forward result of a GEMM, and the attention backward gets the context and log-sum-exp it was
going to recompute.  Everything untagged (norms, RoPE, activation functions) is recomputed.

Only operators whose saved output is *sufficient* take part, so a policy can never change a
gradient: it only decides how much is recomputed.
"""

from __future__ import annotations

import contextlib
import dataclasses
import re
import threading
from typing import Any, Callable, Optional, Sequence, Union

import torch

SAVE, OFFLOAD = "save", "offload"


# ------------------------------------------------------------------------------------------
# Policies: callables ``name -> None | "save" | "offload"``.
# ------------------------------------------------------------------------------------------


@dataclasses.dataclass(frozen=True)
class RematPolicy:
    """Decides per tagged name.  ``dots`` extends the decision to every projection GEMM, tagged or
    not (the reference's ``dots_saveable`` family)."""

    save_pattern: Optional[str] = None
    offload_pattern: Optional[str] = None
    dots: Optional[str] = None  # None, "save" or "offload"
    offload_dst: str = "pinned_host"

    def __call__(self, name: str) -> Optional[str]:
        if self.offload_pattern is not None and re.fullmatch(self.offload_pattern, name):
            return OFFLOAD
        if self.save_pattern is not None and re.fullmatch(self.save_pattern, name):
            return SAVE
        return None

    @property
    def pattern(self) -> Optional[str]:
        return self.save_pattern

    def keeps_anything(self) -> bool:
        return self.save_pattern is not None or self.offload_pattern is not None or self.dots is not None


def save_only_these_names(*names: str) -> RematPolicy:
    return RematPolicy(save_pattern="|".join(re.escape(n) for n in names) if names else None)


def save_only_these_names_regex(pattern: str) -> RematPolicy:
    return RematPolicy(save_pattern=pattern)


def save_and_offload_only_these_names_regex(
    *,
    names_which_can_be_saved: Optional[str] = None,
    names_which_can_be_offloaded: Optional[str] = None,
    offload_src: str = "device",
    offload_dst: str = "pinned_host",
) -> RematPolicy:
    del offload_src
    return RematPolicy(save_pattern=names_which_can_be_saved, offload_pattern=names_which_can_be_offloaded,
                       offload_dst=offload_dst)


def dots_saveable() -> RematPolicy:
    """Keep the output of every projection GEMM."""
    return RematPolicy(dots=SAVE)


def offload_dots_saveable(offload_src: str = "device", offload_dst: str = "pinned_host") -> RematPolicy:
    """Keep the output of every projection GEMM in pinned host memory."""
    del offload_src
    return RematPolicy(dots=OFFLOAD, offload_dst=offload_dst)


def as_policy(policy: Any) -> Optional[RematPolicy]:
    """The selective policy behind a ``RematSpec.policy`` value, or None when the policy keeps
    nothing (full rematerialisation) or is not understood."""
    from axlearn_b200.common.config import InstantiableConfig, maybe_instantiate

    if isinstance(policy, InstantiableConfig):
        policy = maybe_instantiate(policy)
    if isinstance(policy, RematPolicy):
        return policy if policy.keeps_anything() else None
    pattern = getattr(policy, "pattern", None)
    if isinstance(pattern, str):
        return RematPolicy(save_pattern=pattern)
    return None


# ------------------------------------------------------------------------------------------
# Pinned staging buffers (cudaHostAlloc is slow: buffers are pooled by shape and dtype).
# ------------------------------------------------------------------------------------------

_pinned_pool: dict[tuple, list[torch.Tensor]] = {}
_pool_lock = threading.Lock()


def _take_pinned(shape: torch.Size, dtype: torch.dtype) -> torch.Tensor:
    key = (tuple(shape), dtype)
    with _pool_lock:
        free = _pinned_pool.get(key)
        if free:
            return free.pop()
    return torch.empty(shape, dtype=dtype, pin_memory=torch.cuda.is_available())


def _give_pinned(t: torch.Tensor) -> None:
    with _pool_lock:
        _pinned_pool.setdefault((tuple(t.shape), t.dtype), []).append(t)


_offload_streams: dict[int, "torch.cuda.Stream"] = {}


def _offload_stream(device: torch.device):
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _offload_streams:
        _offload_streams[idx] = torch.cuda.Stream(device=device)
    return _offload_streams[idx]


class _Kept:
    """One stored tensor: on the device, or in pinned host memory with the copy events."""

    def __init__(self, t: torch.Tensor, where: str):
        self.where = where
        self.device = t.device
        self._dev: Optional[torch.Tensor] = None
        self._host: Optional[torch.Tensor] = None
        self._event = None
        if where == OFFLOAD and t.is_cuda:
            self._host = _take_pinned(t.shape, t.dtype)
            side = _offload_stream(t.device)
            side.wait_stream(torch.cuda.current_stream(t.device))
            with torch.cuda.stream(side):
                self._host.copy_(t, non_blocking=True)
                self._event = torch.cuda.Event()
                self._event.record(side)
            t.record_stream(side)
        elif where == OFFLOAD:
            self._host = t.detach().clone()
        else:
            self._dev = t.detach()

    def prefetch(self) -> None:
        """Starts the copy back to the device (no-op for tensors that never left it)."""
        if self._dev is not None or self._host is None:
            return
        if self.device.type == "cuda":
            side = _offload_stream(self.device)
            with torch.cuda.stream(side):
                if self._event is not None:
                    side.wait_event(self._event)
                self._dev = torch.empty(self._host.shape, dtype=self._host.dtype, device=self.device)
                self._dev.copy_(self._host, non_blocking=True)
                self._event = torch.cuda.Event()
                self._event.record(side)
        else:
            self._dev = self._host

    def get(self) -> torch.Tensor:
        self.prefetch()
        if self._event is not None and self.device.type == "cuda":
            torch.cuda.current_stream(self.device).wait_event(self._event)
            self._event = None
        return self._dev

    def release(self) -> None:
        if self._host is not None and self._host.is_pinned():
            _give_pinned(self._host)
        self._host = self._dev = None


class LayerStash:
    """Outputs kept for one call of a replayed layer."""

    def __init__(self, policy: RematPolicy):
        self.policy = policy
        self.mode = "record"
        self._kept: dict[tuple, tuple[_Kept, ...]] = {}
        self._counts: dict[tuple, int] = {}
        self.bytes_kept = 0
        self.forwards_skipped = 0

    def start(self, mode: str) -> None:
        self.mode = mode
        self._counts = {}
        if mode == "replay":
            for entry in self._kept.values():
                for k in entry:
                    k.prefetch()

    def _next_key(self, names: tuple) -> tuple:
        n = self._counts.get(names, 0)
        self._counts[names] = n + 1
        return names + (n,)

    def decide(self, names: tuple, *, is_dot: bool) -> Optional[str]:
        """What to do with the output of an operator that runs under ``names``."""
        if names:
            verdicts = [self.policy(n) for n in names]
            if all(v is not None for v in verdicts):
                return OFFLOAD if any(v == OFFLOAD for v in verdicts) else SAVE
        if is_dot and self.policy.dots is not None:
            return self.policy.dots
        return None

    def record(self, names: tuple, where: str, tensors: Sequence[torch.Tensor]) -> None:
        key = self._next_key(names)
        self._kept[key] = tuple(_Kept(t, where) for t in tensors)
        self.bytes_kept += sum(t.numel() * t.element_size() for t in tensors)

    def replay(self, names: tuple) -> Optional[tuple[torch.Tensor, ...]]:
        key = self._next_key(names)
        entry = self._kept.get(key)
        if entry is None:
            return None
        self.forwards_skipped += 1
        return tuple(k.get() for k in entry)

    def clear(self) -> None:
        for entry in self._kept.values():
            for k in entry:
                k.release()
        self._kept.clear()


# ------------------------------------------------------------------------------------------
# Thread-local state: the active stash and the names of the enclosing tagged scope.
# ------------------------------------------------------------------------------------------


class _Local(threading.local):
    stash: Optional[LayerStash] = None
    names: tuple = ()


_local = _Local()


@contextlib.contextmanager
def recording(stash: Optional[LayerStash]):
    prev = _local.stash
    if stash is not None:
        stash.start("record")
    _local.stash = stash
    try:
        yield stash
    finally:
        _local.stash = prev


@contextlib.contextmanager
def replaying(stash: Optional[LayerStash]):
    prev = _local.stash
    if stash is not None:
        stash.start("replay")
    _local.stash = stash
    try:
        yield stash
    finally:
        _local.stash = prev


@contextlib.contextmanager
def tagged(owner: Any, names: Union[str, Sequence[str]]):
    """Operators that run inside produce the tensors the reference tags ``"{Class}.{name}"``."""
    if _local.stash is None:
        yield
        return
    if isinstance(names, str):
        names = (names,)
    cls = type(owner).__name__
    prev = _local.names
    _local.names = tuple(f"{cls}.{n}" for n in names)
    try:
        yield
    finally:
        _local.names = prev


def active() -> Optional[LayerStash]:
    return _local.stash


def operator_outputs(
    compute: Callable[[], tuple[torch.Tensor, ...]],
    *,
    is_dot: bool,
    can_skip: bool = True,
) -> tuple[tuple[torch.Tensor, ...], bool]:
    """Runs ``compute`` unless the active stash already holds this operator's outputs.

    Returns ``(outputs, replayed)``.  In record mode the outputs are stored when the policy says
    so; in replay mode stored outputs are returned without calling ``compute`` (``can_skip=False``
    forces the call, for operators whose forward has a side effect that is still needed, e.g. a
    GEMM that carries a parameter gather).
    """
    stash = _local.stash
    if stash is None:
        return compute(), False
    names = _local.names
    where = stash.decide(names, is_dot=is_dot)
    if where is None:
        return compute(), False
    if stash.mode == "record":
        outs = compute()
        stash.record(names, where, outs)
        return outs, False
    kept = stash.replay(names)
    if kept is None or not can_skip:
        return compute(), False
    return kept, True
