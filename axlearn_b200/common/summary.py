"""Typed summaries: images, audio and deferred callbacks.

Counterpart of axlearn/common/summary.py (``Summary`` :14, ``ImageSummary`` :43, ``AudioSummary``
:80, ``CallbackSummary`` :127).  A layer adds one with ``add_summary(name, ImageSummary(x))``; the
summary writer checks it (``validate``) and writes it in the matching form.  Evaluation loops that
accumulate summaries keep the value of the last batch (``accumulate``).
"""

from __future__ import annotations

from typing import Any, Callable

import torch

Tensor = torch.Tensor


class Summary:
    """Base: wraps a value; ``value()`` is what gets written."""

    def __init__(self, _value: Any):
        self._value = _value

    def value(self) -> Any:
        return self._value

    def validate(self) -> None:
        pass

    def accumulate(self, other: "Summary") -> "Summary":
        return other


class ImageSummary(Summary):
    """``[batch, height, width, channels]`` with 1 or 3 channels; floats are expected in [0, 1]."""

    def validate(self) -> None:
        v = self._value
        if not isinstance(v, Tensor) or v.dim() != 4 or v.shape[-1] not in (1, 3):
            raise ValueError(f"ImageSummary needs [batch, height, width, 1 or 3], got {getattr(v, 'shape', type(v))}")

    def value(self) -> Tensor:
        v = self._value.detach().float().cpu()
        return v.clamp(0, 1) if self._value.is_floating_point() else v / 255.0


class AudioSummary(Summary):
    """``[samples, channels]`` (or ``[samples]``) in [-1, 1] with its sample rate."""

    def __init__(self, _value: Tensor, *, sample_rate: int = 16000):
        super().__init__(_value)
        self.sample_rate = sample_rate

    def validate(self) -> None:
        v = self._value
        if not isinstance(v, Tensor) or v.dim() not in (1, 2):
            raise ValueError(f"AudioSummary needs [samples] or [samples, channels], got {getattr(v, 'shape', type(v))}")

    def value(self) -> Tensor:
        v = self._value.detach().float().cpu()
        return (v[:, 0] if v.dim() == 2 else v).clamp(-1, 1)


class CallbackSummary(Summary):
    """``fn(*args, **kwargs)`` is evaluated on the host when the summary is written, so that costly
    formatting (rendering a plot, decoding token ids) stays out of the step."""

    def __init__(self, fn: Callable[..., Any], *args, **kwargs):
        super().__init__(None)
        self.fn, self.args, self.kwargs = fn, args, kwargs

    def value(self) -> Any:
        host = lambda x: x.detach().cpu() if isinstance(x, Tensor) else x
        return self.fn(*[host(a) for a in self.args], **{k: host(v) for k, v in self.kwargs.items()})
