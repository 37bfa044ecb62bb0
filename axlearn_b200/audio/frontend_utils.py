"""Signal-processing helpers for audio frontends (reference: axlearn/audio/frontend_utils.py:25-425).

Framing keeps a trailing PARTIAL frame (``num_frames = ceil((len - frame + hop) / hop)``, at least
one for a non-empty input): the tail is completed with ``pad_value`` -- zeros for samples, ones
for paddings, so that a frame touching padding is itself padding.  Everything works on the last
axis of a ``torch`` tensor of any rank; a batch lives on the device it came from and the FFT is the
library's batched ``rfft`` there (each GPU transforms its own shard of the batch, which is what the
reference needs a hand-sharded FFT for).
"""

from __future__ import annotations

import enum
import math
from typing import Union

import numpy as np
import torch

from axlearn_b200.audio.frontend import linear_to_mel_weight_matrix  # pylint: disable=unused-import

Tensor = torch.Tensor


class WindowType(enum.Enum):
    HANN = 0
    HAMMING = 1


class FrequencyScale(enum.Enum):
    MEL_LN = 0          # mel scale with the natural logarithm


def hertz_to_warped_scale(freq, *, freq_scale: FrequencyScale):
    if freq_scale == FrequencyScale.MEL_LN:
        return 1127.0 * np.log(1.0 + (np.asarray(freq, dtype=np.float64) / 700.0))
    raise NotImplementedError(f"Unsupported target scale {freq_scale}.")


def warped_to_hertz_scale(freq, *, freq_scale: FrequencyScale):
    if freq_scale == FrequencyScale.MEL_LN:
        return 700.0 * (np.exp(np.asarray(freq, dtype=np.float64) / 1127.0) - 1.0)
    raise NotImplementedError(f"Unsupported source scale {freq_scale}.")


def _ceil_div(numerator, denominator: int):
    return (numerator + denominator - 1) // denominator


def ms_to_samples(ms: Union[int, float], *, sample_rate: int) -> int:
    out_size = (sample_rate * ms) / 1000
    if not float(out_size).is_integer():
        raise ValueError(f"out_size must be an integer, got {out_size}.")
    return int(out_size)


def num_frames(seq_len, *, frame_size: int, hop_size: int):
    """Frames of a sequence of ``seq_len`` samples, a partial last frame included.  ``seq_len`` may
    be a tensor of lengths."""
    if isinstance(seq_len, Tensor):
        if frame_size < 1 or hop_size < 0:
            raise ValueError(f"Invalid input: frame_size={frame_size}, hop_size={hop_size}")
        n = torch.clamp(_ceil_div(seq_len - frame_size + hop_size, hop_size), min=1)
        return torch.where(seq_len == 0, torch.zeros_like(n), n)
    if seq_len < 0 or frame_size < 1 or hop_size < 0:
        raise ValueError(f"Invalid input: seq_len={seq_len}, frame_size={frame_size}, hop_size={hop_size}")
    if seq_len == 0:
        return 0
    return max(_ceil_div(seq_len - frame_size + hop_size, hop_size), 1)


def frame(x: Tensor, *, frame_size: int, hop_size: int, pad_value: float = 0) -> Tensor:
    """``[..., seq_len] -> [..., num_frames, frame_size]``.  The result is a strided VIEW of the
    (tail-padded) input: no gather, no index tensor."""
    n = num_frames(x.shape[-1], frame_size=frame_size, hop_size=hop_size)
    full = n * hop_size - hop_size + frame_size if n else 0
    if full > x.shape[-1]:
        x = torch.nn.functional.pad(x, (0, full - x.shape[-1]), value=pad_value)
    x = x[..., :full]
    if n == 0:
        return x.new_zeros(*x.shape[:-1], 0, frame_size)
    return x.unfold(-1, frame_size, hop_size)


def frame_paddings(paddings: Tensor, *, frame_size: int, hop_size: int) -> Tensor:
    """A frame is padding when any of its samples is (the completed tail counts as padding)."""
    if hop_size > frame_size:
        raise ValueError(f"hop_size {hop_size} must be smaller than frame_size {frame_size}.")
    return frame(paddings, frame_size=frame_size, hop_size=hop_size, pad_value=1).amax(dim=-1)


def pre_emphasis(x: Tensor, *, coeff) -> Tensor:
    """``[..., frame_size] -> [..., frame_size - 1]``: ``y[t] = x[t + 1] - coeff * x[t]``."""
    coeff = torch.as_tensor(coeff, dtype=x.dtype, device=x.device)
    return x[..., 1:] - coeff * x[..., :-1]


def window_coffs(window_size: int, *, window_type: WindowType, periodic: bool = True) -> Tensor:
    """Window coefficients.  ``periodic`` (the convention of spectral analysis) computes an even-sized
    window as the first ``window_size`` points of the symmetric window one longer."""
    is_even = (1 - window_size % 2) * int(periodic)
    if window_type == WindowType.HANN:
        coeffs = np.hanning(window_size + is_even)[:window_size]
    elif window_type == WindowType.HAMMING:
        coeffs = np.hamming(window_size + is_even)[:window_size]
    else:
        raise NotImplementedError(f"Unrecognized window_type {window_type}.")
    return torch.from_numpy(coeffs)


def windowing(x: Tensor, *, window_type: WindowType, periodic: bool = True) -> Tensor:
    coeffs = window_coffs(x.shape[-1], window_type=window_type, periodic=periodic).to(device=x.device)
    return (x * coeffs).to(x.dtype)


def cast_for_rfft(x: Tensor) -> Tensor:
    return x if x.dtype in (torch.float32, torch.float64) else x.float()


def fft(n: int):
    """Returns ``x -> rfft(x, n)`` over the last axis (``[..., n // 2 + 1]`` complex)."""
    return lambda x: torch.fft.rfft(cast_for_rfft(x), n=n)


def magnitude_spectrogram(ffts: Tensor, *, dtype: torch.dtype) -> Tensor:
    return ffts.abs().to(dtype)


def linear_to_log_spectrogram(x: Tensor) -> Tensor:
    return torch.log(torch.clamp(x, min=torch.finfo(x.dtype).tiny))


def linear_to_log_mel_spectrogram(x: Tensor, *, weight_matrix, mel_floor: float = 1.0) -> Tensor:
    """``[..., frames, bins] -> [..., frames, filters]``: mel projection, floor, logarithm."""
    w = torch.as_tensor(weight_matrix, device=x.device).to(x.dtype)
    return linear_to_log_spectrogram(torch.clamp(x @ w, min=mel_floor).to(x.dtype))


def next_power_of_2(n: float) -> int:
    return 2 ** math.ceil(math.log2(n))
