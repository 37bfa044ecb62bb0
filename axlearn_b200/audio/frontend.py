"""Audio front end: waveform -> log-mel filterbank features.

Parity targets in the reference: ``LogMelFrontend`` (axlearn/audio/frontend.py:130-260) with its
helpers in axlearn/audio/frontend_utils.py -- pre-emphasis (:120), framing by ``frame_size`` /
``hop_size`` in milliseconds (:60-118), Hann window (:160), magnitude spectrum with an FFT of the
next power of two (:200), triangular mel filterbank between ``lower_edge_hertz`` and
``upper_edge_hertz`` (HTK mel scale, :250-330), log with a floor, optional mean / std
normalisation per mel bin; paddings are reduced frame-wise (a frame is padding if its last sample
is).  Output ``[B, frames, num_filters, 1]`` (channels last, as the convolutional subsampler
wants) and ``[B, frames]`` paddings.
"""

from __future__ import annotations

import math
from typing import Optional, Sequence

import torch

from axlearn_b200.common.base_layer import BaseLayer
from axlearn_b200.common.config import REQUIRED, Required, config_class
from axlearn_b200.common.module import nowrap

Tensor = torch.Tensor


def next_power_of_2(n: int) -> int:
    return 1 << max(0, (n - 1).bit_length())


def hertz_to_mel(f):
    return 1127.0 * torch.log1p(torch.as_tensor(f, dtype=torch.float64) / 700.0)


def linear_to_mel_weight_matrix(*, num_filters: int, num_spectrogram_bins: int, sample_rate: float,
                                lower_edge_hertz: float, upper_edge_hertz: float) -> Tensor:
    """``[num_spectrogram_bins, num_filters]`` triangular filters, equally spaced on the mel scale;
    the DC bin gets no weight."""
    nyquist = sample_rate / 2.0
    bins_hz = torch.linspace(0.0, nyquist, num_spectrogram_bins, dtype=torch.float64)[1:]
    bins_mel = hertz_to_mel(bins_hz)[:, None]
    edges = torch.linspace(hertz_to_mel(lower_edge_hertz).item(), hertz_to_mel(upper_edge_hertz).item(),
                           num_filters + 2, dtype=torch.float64)
    lower, center, upper = edges[:-2][None], edges[1:-1][None], edges[2:][None]
    up = (bins_mel - lower) / (center - lower)
    down = (upper - bins_mel) / (upper - center)
    w = torch.clamp(torch.minimum(up, down), min=0.0)
    return torch.cat([torch.zeros(1, num_filters, dtype=torch.float64), w], dim=0).float()


def frame(x: Tensor, *, frame_size: int, hop_size: int) -> Tensor:
    """``[B, T] -> [B, num_frames, frame_size]`` (only whole frames)."""
    return x.unfold(-1, frame_size, hop_size)


def frame_paddings(paddings: Tensor, *, frame_size: int, hop_size: int) -> Tensor:
    """A frame is padding if any of its samples is (paddings are suffixes, so: its last one)."""
    return frame(paddings.float(), frame_size=frame_size, hop_size=hop_size).amax(dim=-1)


def pre_emphasis(frames: Tensor, coeff: float) -> Tensor:
    """``y[t] = x[t + 1] - coeff * x[t]`` within a frame of ``frame_size + 1`` samples."""
    return frames[..., 1:] - coeff * frames[..., :-1]


class LogMelFrontend(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        num_filters: Required[int] = REQUIRED
        sample_rate: Required[int] = REQUIRED
        frame_size_ms: Required[float] = REQUIRED
        hop_size_ms: Required[float] = REQUIRED
        pre_emphasis_coeff: Optional[float] = 0.97
        mel_floor: float = 1.0
        lower_edge_hertz: float = 125.0
        upper_edge_hertz: float = 7600.0
        fft_size: Optional[int] = None
        # Per-bin normalisation constants (sequences of num_filters values) or None.
        output_mean: Optional[Sequence[float]] = None
        output_std: Optional[Sequence[float]] = None

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        cfg = self._config
        self._frame_size = int(round(cfg.sample_rate * cfg.frame_size_ms / 1000))
        self._hop_size = int(round(cfg.sample_rate * cfg.hop_size_ms / 1000))
        if self._frame_size <= 0 or self._hop_size <= 0:
            raise ValueError("frame and hop sizes must be positive")
        self._fft_size = cfg.fft_size or next_power_of_2(self._frame_size)
        self._mel = linear_to_mel_weight_matrix(
            num_filters=cfg.num_filters, num_spectrogram_bins=self._fft_size // 2 + 1, sample_rate=cfg.sample_rate,
            lower_edge_hertz=cfg.lower_edge_hertz, upper_edge_hertz=cfg.upper_edge_hertz)

    @nowrap
    def output_shape(self, *, input_shape: Sequence[Optional[int]]):
        t = input_shape[1]
        extra = 1 if self._config.pre_emphasis_coeff is not None else 0
        frames = None if t is None else max(0, (t - self._frame_size - extra) // self._hop_size + 1)
        return [input_shape[0], frames, self._config.num_filters, 1]

    def forward(self, inputs: Tensor, *, paddings: Tensor):
        cfg = self._config
        x = inputs.float()
        size = self._frame_size + (1 if cfg.pre_emphasis_coeff is not None else 0)
        frames = frame(x, frame_size=size, hop_size=self._hop_size)
        out_paddings = frame_paddings(paddings, frame_size=size, hop_size=self._hop_size)
        if cfg.pre_emphasis_coeff is not None:
            frames = pre_emphasis(frames, cfg.pre_emphasis_coeff)
        window = torch.hann_window(self._frame_size, periodic=True, device=x.device, dtype=frames.dtype)
        spectrum = torch.fft.rfft(frames * window, n=self._fft_size).abs()
        mel = spectrum @ self._mel.to(x.device)
        out = torch.log(torch.clamp(mel, min=cfg.mel_floor))
        if cfg.output_mean is not None:
            out = out - torch.tensor(cfg.output_mean, device=x.device)
        if cfg.output_std is not None:
            out = out / torch.tensor(cfg.output_std, device=x.device)
        out = out * (1 - out_paddings)[..., None]
        return {"outputs": out[..., None].to(inputs.dtype if inputs.is_floating_point() else torch.float32),
                "paddings": out_paddings}
