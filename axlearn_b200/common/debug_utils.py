"""Run-time checks for debugging numerics (the role of the reference's ``checkify`` wrappers,
axlearn/common/debug_utils.py:40-114, which turn NaN / division / index errors inside jitted
code into Python exceptions).

Eager PyTorch needs no functionalisation for that: with ``check_module_outputs()`` active, every
wrapped module call has its tensor outputs tested and the FIRST module that produces a NaN or an
infinity raises ``FloatingPointError`` naming its path.  Each test synchronises with the GPU, so
this is a debugging mode, not something to train under.  ``guard_index`` is the bounds-checked
accessor for gather-style indexing.
"""

from __future__ import annotations

import contextlib
import threading
from typing import Any, Iterable, Optional

import torch


class _State(threading.local):
    def __init__(self):
        self.checks: Optional[frozenset] = None


_state = _State()
NAN, INF = "nan", "inf"


@contextlib.contextmanager
def check_module_outputs(errors: Iterable[str] = (NAN, INF)):
    """Within the block, module outputs are tested for the given kinds of non-finite values."""
    prev, _state.checks = _state.checks, frozenset(errors)
    try:
        yield
    finally:
        _state.checks = prev


def active_checks() -> Optional[frozenset]:
    return _state.checks


def _tensors(tree: Any):
    if isinstance(tree, torch.Tensor):
        yield tree
    elif isinstance(tree, dict):
        for v in tree.values():
            yield from _tensors(v)
    elif isinstance(tree, (list, tuple)):
        for v in tree:
            yield from _tensors(v)
    elif hasattr(tree, "__dataclass_fields__"):
        for name in tree.__dataclass_fields__:
            yield from _tensors(getattr(tree, name))


def check_outputs(outputs: Any, *, where: str) -> None:
    """Raises ``FloatingPointError`` if a floating-point tensor in ``outputs`` violates the active
    checks (no-op outside ``check_module_outputs``)."""
    checks = _state.checks
    if not checks:
        return
    for t in _tensors(outputs):
        if not t.is_floating_point() or t.numel() == 0:
            continue
        d = t.detach()
        if NAN in checks and bool(torch.isnan(d).any()):
            raise FloatingPointError(f"NaN in an output of {where} (shape {tuple(t.shape)}, dtype {t.dtype})")
        if INF in checks and bool(torch.isinf(d).any()):
            raise FloatingPointError(f"infinity in an output of {where} (shape {tuple(t.shape)}, dtype {t.dtype})")


def guard_index(index: torch.Tensor, size: int, *, what: str = "index") -> torch.Tensor:
    """Returns ``index`` after checking ``0 <= index < size`` for every element (a gather with an
    out-of-range index is undefined behaviour on the GPU; this is the accessor to use while
    hunting one).  Synchronises."""
    if index.numel():
        lo, hi = int(index.min()), int(index.max())
        if lo < 0 or hi >= size:
            raise IndexError(f"{what}: values span [{lo}, {hi}] but the indexed dimension has size {size}")
    return index
