"""Attention bias algebra.

Biases are small objects describing *why* a logit is masked (causal, sliding window,
segment ids, an explicit tensor) rather than materialised ``[B, N, T, S]`` tensors.  The
fused attention kernels consume the structured forms directly (causal block skipping,
segment-id comparison in registers); only ``TensorAttentionBias`` forces the generic path.

Parity targets in the reference (axlearn/common/attention_bias.py): ``NEG_INF`` (:48),
``BaseAttentionBias`` (:54), ``CompositeAttentionBias`` (:216), ``split`` (:321),
``TensorAttentionBias`` (:350), ``BoolAttentionBias`` (:400), ``SegmentIdAttentionBias``
(:434), ``MaskFnAttentionBias`` (:502), ``CausalAttentionBias`` (:663),
``SlidingWindowAttentionBias`` (:685), ``ZeroAttentionBias`` (:725), mask combinators
(:745-827) and bias builders (:830-901).
"""

from __future__ import annotations

import dataclasses
from typing import Callable, Optional, Sequence, Type, TypeVar, Union

import torch

Tensor = torch.Tensor
NEG_INF = -0.7 * float(torch.finfo(torch.float32).max)

MaskFn = Callable[[Tensor, Tensor], Tensor]
B = TypeVar("B", bound="BaseAttentionBias")


@dataclasses.dataclass
class BaseAttentionBias:
    """An additive bias on attention logits of (broadcast) shape ``[batch, heads, T, S]``."""

    dtype: Optional[torch.dtype] = dataclasses.field(default=None, kw_only=True)

    def value(self) -> Optional[Tensor]:
        """The additive bias tensor (4-D, broadcastable) or None when empty."""
        v = self._value()
        if v is None:
            return None
        if v.dim() == 3:
            v = v[:, None]
        elif v.dim() == 2:
            v = v[None, None]
        if v.dim() != 4:
            raise ValueError(f"bias must be 2/3/4-D, got {tuple(v.shape)}")
        return v if self.dtype is None else v.to(self.dtype)

    def _value(self) -> Optional[Tensor]:
        raise NotImplementedError(type(self))

    def has_value(self) -> bool:
        return self._value() is not None

    def bool_value(self) -> Optional[Tensor]:
        v = self.value()
        return None if v is None else v > NEG_INF / 2

    def __add__(self, other: "BaseAttentionBias") -> "CompositeAttentionBias":
        return CompositeAttentionBias([self, other])

    def astype(self, dtype: torch.dtype) -> "BaseAttentionBias":
        return dataclasses.replace(self, dtype=dtype)

    def bias_and_residual(self, cls: Type[B]) -> tuple[Optional[B], "BaseAttentionBias"]:
        """Splits into (part of type ``cls``, everything else)."""
        if isinstance(self, cls):
            return self, ZeroAttentionBias()
        return None, self

    @classmethod
    def from_sequence(cls, biases: Sequence["BaseAttentionBias"]) -> Optional["BaseAttentionBias"]:
        biases = [b for b in biases if b is not None]
        if not biases:
            return None
        if len(biases) == 1:
            return biases[0]
        return CompositeAttentionBias(list(biases))


@dataclasses.dataclass
class ZeroAttentionBias(BaseAttentionBias):
    def _value(self):
        return None


@dataclasses.dataclass
class CompositeAttentionBias(BaseAttentionBias):
    """Sum of several biases; nested composites are flattened lazily."""

    biases: Sequence[BaseAttentionBias] = ()

    def _flat(self) -> list[BaseAttentionBias]:
        out: list[BaseAttentionBias] = []
        for b in self.biases:
            if isinstance(b, CompositeAttentionBias):
                out.extend(b._flat())
            elif b is not None and not isinstance(b, ZeroAttentionBias):
                out.append(b)
        return out

    def _value(self):
        vals = [b.value() for b in self._flat()]
        vals = [v for v in vals if v is not None]
        if not vals:
            return None
        total = vals[0]
        for v in vals[1:]:
            total = total + v
        # Keep masked entries from overflowing to -inf when several masks stack.
        return total.clamp_min(NEG_INF)

    def bias_and_residual(self, cls):
        hits = [b for b in self._flat() if isinstance(b, cls)]
        rest = [b for b in self._flat() if not isinstance(b, cls)]
        hit = None
        if hits:
            hit = hits[0]
            for extra in hits[1:]:
                merged = hit._merge(extra) if hasattr(hit, "_merge") else None
                if merged is None:
                    rest.append(extra)
                else:
                    hit = merged
        residual = CompositeAttentionBias(rest) if rest else ZeroAttentionBias()
        return hit, residual

    def __add__(self, other):
        return CompositeAttentionBias(list(self.biases) + [other])


def split(bias: BaseAttentionBias, *cls: Type[BaseAttentionBias]) -> list[BaseAttentionBias]:
    """``[part_of_cls0, part_of_cls1, ..., residual]``; missing parts are ZeroAttentionBias."""
    out = []
    for c in cls:
        hit, bias = bias.bias_and_residual(c)
        out.append(hit if hit is not None else ZeroAttentionBias())
    out.append(bias)
    return out


@dataclasses.dataclass
class TensorAttentionBias(BaseAttentionBias):
    """An explicit float bias tensor ``[B|1, N|1, T, S]``."""

    _tensor: Optional[Tensor] = None

    @classmethod
    def from_tensor(cls, t: Tensor) -> "TensorAttentionBias":
        if t.dim() not in (3, 4):
            raise ValueError(f"bias tensor must be 3/4-D, got {tuple(t.shape)}")
        return cls(_tensor=t)

    def _value(self):
        return self._tensor


@dataclasses.dataclass
class BoolAttentionBias(BaseAttentionBias):
    """Bias defined by a boolean "may attend" tensor."""

    def _bool_value(self) -> Optional[Tensor]:
        raise NotImplementedError(type(self))

    def bool_value(self):
        v = self._bool_value()
        if v is None:
            return None
        if v.dim() == 3:
            v = v[:, None]
        elif v.dim() == 2:
            v = v[None, None]
        return v

    def _value(self):
        b = self._bool_value()
        return None if b is None else bool_to_bias(b)


@dataclasses.dataclass
class BoolTensorAttentionBias(BoolAttentionBias):
    _tensor: Optional[Tensor] = None

    @classmethod
    def from_tensor(cls, t: Tensor) -> "BoolTensorAttentionBias":
        if t.dtype != torch.bool:
            raise ValueError("BoolTensorAttentionBias needs a bool tensor")
        return cls(_tensor=t)

    def _bool_value(self):
        return self._tensor


@dataclasses.dataclass
class SegmentIdAttentionBias(BoolAttentionBias):
    """Tokens attend only within their own segment. ``segment_ids``: ``[B, T]`` ints."""

    segment_ids: Optional[Tensor] = None

    def _bool_value(self):
        s = self.segment_ids
        return (s[:, :, None] == s[:, None, :])[:, None]


@dataclasses.dataclass
class MaskFnAttentionBias(BoolAttentionBias):
    """Mask given by ``mask(query_position, key_position) -> bool`` evaluated on broadcast
    position grids.  ``target_positions`` ([B, T] or [T]) default to ``arange(T)``; during
    decoding they are the absolute step indices."""

    mask: Optional[MaskFn] = None
    shape: Optional[tuple[int, int]] = None  # (T, S)
    target_positions: Optional[Tensor] = None
    source_positions: Optional[Tensor] = None

    def _bool_value(self):
        t, s = self.shape
        dev = None
        for p in (self.target_positions, self.source_positions):
            if p is not None:
                dev = p.device
        tp = self.target_positions if self.target_positions is not None else torch.arange(t, device=dev)
        sp = self.source_positions if self.source_positions is not None else torch.arange(s, device=dev)
        if tp.dim() == 1:
            tp = tp[None]
        if sp.dim() == 1:
            sp = sp[None]
        return self.mask(tp[:, :, None], sp[:, None, :])[:, None]

    def _merge(self, other: "MaskFnAttentionBias") -> Optional["MaskFnAttentionBias"]:
        if (
            self.shape != other.shape
            or self.target_positions is not other.target_positions
            or self.source_positions is not other.source_positions
        ):
            return None
        return dataclasses.replace(self, mask=and_masks(self.mask, other.mask))


def causal_mask(query_position: Tensor, key_position: Tensor) -> Tensor:
    return query_position >= key_position


@dataclasses.dataclass
class _SlidingWindowMask:
    """``mask(q, k) = q - window <= k <= q`` as a picklable callable."""

    window: int

    def __call__(self, q: Tensor, k: Tensor) -> Tensor:
        return (k <= q) & (k >= q - self.window)

    __config_value__ = True


def sliding_window_causal_mask(sliding_window_size: int) -> MaskFn:
    return _SlidingWindowMask(sliding_window_size)


@dataclasses.dataclass
class _AndMask:
    a: MaskFn
    b: MaskFn

    def __call__(self, q, k):
        return self.a(q, k) & self.b(q, k)


@dataclasses.dataclass
class _OrMask:
    a: MaskFn
    b: MaskFn

    def __call__(self, q, k):
        return self.a(q, k) | self.b(q, k)


def and_masks(*fns: Optional[MaskFn]) -> Optional[MaskFn]:
    fns = [f for f in fns if f is not None]
    if not fns:
        return None
    out = fns[0]
    for f in fns[1:]:
        out = _AndMask(out, f)
    return out


def or_masks(*fns: Optional[MaskFn]) -> Optional[MaskFn]:
    fns = [f for f in fns if f is not None]
    if not fns:
        return None
    out = fns[0]
    for f in fns[1:]:
        out = _OrMask(out, f)
    return out


@dataclasses.dataclass
class CausalAttentionBias(MaskFnAttentionBias):
    mask: Optional[MaskFn] = causal_mask


@dataclasses.dataclass
class SlidingWindowAttentionBias(MaskFnAttentionBias):
    sliding_window_size: Optional[int] = None

    def __post_init__(self):
        if self.mask is None and self.sliding_window_size is not None:
            self.mask = sliding_window_causal_mask(self.sliding_window_size)


@dataclasses.dataclass
class LeftRightWindowAttentionBias(MaskFnAttentionBias):
    left_size: int = 0
    right_size: int = 0

    def __post_init__(self):
        if self.mask is None:
            l, r = self.left_size, self.right_size
            self.mask = lambda q, k: (k >= q - l) & (k <= q + r)


# ------------------------------------------------------------------------------------------
# Builders.
# ------------------------------------------------------------------------------------------


def bool_to_bias(mask: Tensor) -> Tensor:
    """``True`` -> 0, ``False`` -> NEG_INF (fp32)."""
    if mask.dtype != torch.bool:
        raise ValueError("mask must be bool")
    return torch.where(mask, 0.0, NEG_INF).to(torch.float32)


def make_causal_biases(seq_len: int, device=None) -> Tensor:
    """``[T, T]`` with NEG_INF above the diagonal."""
    pos = torch.arange(seq_len, device=device)
    return bool_to_bias(causal_mask(pos[:, None], pos[None, :]))


def make_sliding_window_causal_biases(seq_len: int, sliding_window: int, device=None) -> Tensor:
    pos = torch.arange(seq_len, device=device)
    return bool_to_bias(sliding_window_causal_mask(sliding_window)(pos[:, None], pos[None, :]))


def make_segment_mask(*, source_segments: Tensor, target_segments: Tensor) -> Tensor:
    """``[B, 1, T, S]`` additive bias blocking attention across segments."""
    same = target_segments[:, :, None] == source_segments[:, None, :]
    return bool_to_bias(same)[:, None]


def as_attention_bias(bias: Union[None, Tensor, BaseAttentionBias]) -> BaseAttentionBias:
    if bias is None:
        return ZeroAttentionBias()
    if isinstance(bias, BaseAttentionBias):
        return bias
    if bias.dtype == torch.bool:
        return BoolTensorAttentionBias.from_tensor(bias)
    return TensorAttentionBias.from_tensor(bias)
