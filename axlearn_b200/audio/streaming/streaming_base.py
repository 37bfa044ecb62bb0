"""Base class and helpers for streaming layers (reference:
axlearn/audio/streaming/streaming_base.py:14-140).

A streaming layer offers ``init_states`` / ``extend_step`` beside ``forward``, and describes itself
through three quantities that depend on its CONFIG alone, so that a stack can be planned before
anything is instantiated:

* ``in_stride``: inputs consumed per output (a stride-2 convolution: 2; a transposed one: 1);
* ``out_stride``: outputs produced per input (a stride-2 transposed convolution: 2);
* ``segment_pad``: padding frames needed between packed segments so that nothing leaks across a
  boundary (a convolution: ``max(left, right)`` padding; attention: 0, ``segment_ids`` do it).

Each is declared with ``@config_method`` and can be asked of the class with a config
(``Layer.in_stride(cfg)``) or of an instance (``layer.in_stride()``).
"""

from __future__ import annotations

import functools
import math
from typing import Any, Callable, Sequence


class config_method:  # pylint: disable=invalid-name
    """Descriptor for ``fn(cls, cfg)``: ``Class.name(cfg)`` or ``instance.name()`` (the instance's
    own config is passed)."""

    def __init__(self, fn: Callable[[type, Any], Any]):
        self._fn = fn
        functools.update_wrapper(self, fn)

    def __get__(self, obj, owner):
        if obj is None:
            return functools.partial(self._fn, owner)
        return functools.partial(self._fn, owner, obj.config)


class StreamingBase:
    """Mix-in for streaming layers.  Subclasses implement ``init_states`` and ``extend_step``."""

    @config_method
    def in_stride(cls, cfg) -> int:  # pylint: disable=no-self-argument
        del cfg
        return 1

    @config_method
    def out_stride(cls, cfg) -> int:  # pylint: disable=no-self-argument
        del cfg
        return 1

    @config_method
    def segment_pad(cls, cfg) -> int:  # pylint: disable=no-self-argument
        del cfg
        return 0

    def init_states(self, *, batch_size: int, dtype=None, **kwargs) -> Any:
        raise NotImplementedError(type(self))

    def extend_step(self, *, cached_states: Any, input_data: Any, is_prefill: bool = False) -> tuple[Any, Any]:
        """Returns ``(updated_states, output)``; ``output`` has the structure of ``forward``'s."""
        raise NotImplementedError(type(self))


def _ask(cfg_or_layer: Any, name: str) -> int:
    klass = getattr(cfg_or_layer, "klass", None)
    if klass is not None:                               # a config
        return getattr(klass, name)(cfg_or_layer) if hasattr(klass, name) else getattr(StreamingBase, name)(cfg_or_layer)
    return getattr(cfg_or_layer, name)() if hasattr(cfg_or_layer, name) else getattr(StreamingBase, name)(None)


def compute_encoder_segment_pad(layers: Sequence[Any]) -> int:
    """Segment padding of sequential down-sampling layers (configs or instances), in INPUT frames:
    ``max(S1, S2 * I1, S3 * I1 * I2, ...)``."""
    segment_pad, cum_stride = 0, 1
    for layer in layers:
        segment_pad = max(segment_pad, _ask(layer, "segment_pad") * cum_stride)
        cum_stride *= _ask(layer, "in_stride")
    return segment_pad


def compute_decoder_segment_pad(layers: Sequence[Any]) -> int:
    """Segment padding of sequential up-sampling layers: ``max(S1, ceil(S2 / O1), ceil(S3 / (O1 O2)), ...)``."""
    segment_pad, cum_out_stride = 0, 1
    for layer in layers:
        segment_pad = max(segment_pad, math.ceil(_ask(layer, "segment_pad") / cum_out_stride))
        cum_out_stride *= _ask(layer, "out_stride")
    return segment_pad


def next_segment_pos(current_len: int, *, segment_pad: int = 0, stride: int = 1) -> tuple[int, int]:
    """The smallest start position for the next packed segment that is a multiple of ``stride``
    (so the segment is processed exactly as if it began a batch row) and at least ``segment_pad``
    past ``current_len``; also returns the padding actually inserted."""
    next_pos = math.ceil((current_len + segment_pad) / stride) * stride
    return next_pos, next_pos - current_len
