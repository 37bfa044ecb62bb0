"""Balanced sampling of matched anchors / proposals (reference: axlearn/vision/samplers.py:16-111)."""

from __future__ import annotations

import dataclasses

import torch

from axlearn_b200.common import prng

Tensor = torch.Tensor


def sample(*, is_candidate: Tensor, size: Tensor, prng_key: Tensor) -> Tensor:
    """Uniformly chooses ``size[...]`` of the True positions of ``is_candidate`` (``[..., N]``)
    without replacement; all of them when there are fewer.  Returns a bool mask ``[..., N]``."""
    gen = prng.generator(prng_key, device="cpu")
    noise = torch.rand(is_candidate.shape, generator=gen).to(is_candidate.device)
    permutation = noise.argsort(dim=-1)
    inverse = permutation.argsort(dim=-1)
    shuffled = torch.gather(is_candidate, -1, permutation)
    rank = shuffled.long().cumsum(dim=-1) * shuffled
    chosen = (rank > 0) & (rank <= size[..., None])
    return torch.gather(chosen, -1, inverse)


@dataclasses.dataclass
class LabelSamples:
    """``indices`` int ``[..., sample_size]`` into the label axis; ``paddings`` bool, True where an
    index is filler because there were not enough candidates."""

    indices: Tensor
    paddings: Tensor


class LabelSampler:
    """Samples ``size`` labels: up to ``size * foreground_fraction`` foreground ones, the rest
    background (more background when foreground is short).  Ignored labels and paddings are never
    sampled."""

    def __init__(self, size: int, foreground_fraction: float, background_label: int, ignore_label: int):
        self.num_foreground = int(size * foreground_fraction)
        self.size = size
        self.background_label = background_label
        self.ignore_label = ignore_label

    def __call__(self, *, labels: Tensor, paddings: Tensor, prng_key: Tensor) -> LabelSamples:
        key1, key2 = prng.split(prng_key, 2)
        valid = ~paddings.bool()
        foreground = valid & (labels != self.ignore_label) & (labels != self.background_label)
        num_foreground = foreground.sum(dim=-1).clamp(max=self.num_foreground)
        fg = sample(is_candidate=foreground, size=num_foreground, prng_key=key1)
        background = valid & (labels == self.background_label)
        bg = sample(is_candidate=background, size=self.size - num_foreground, prng_key=key2)
        samples = fg | bg
        # Stable order: sampled positions first, by index.
        n = samples.shape[-1]
        order = torch.arange(n, device=samples.device).expand_as(samples)
        keyed = torch.where(samples, order, order + n)
        indices = keyed.argsort(dim=-1)[..., : self.size]
        if indices.shape[-1] < self.size:
            pad = self.size - indices.shape[-1]
            indices = torch.cat([indices, indices.new_zeros(*indices.shape[:-1], pad)], dim=-1)
            taken = torch.cat([torch.gather(samples, -1, indices[..., : n]),
                               samples.new_zeros(*samples.shape[:-1], pad)], dim=-1)
        else:
            taken = torch.gather(samples, -1, indices)
        return LabelSamples(indices=indices, paddings=~taken)
