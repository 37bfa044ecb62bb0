"""Vector quantisation layers.

Parity target in the reference: axlearn/common/quantizer.py -- ``RandomVectorQuantizer`` (:330:
frozen random projection + frozen normalised codebook; the BEST-RQ target generator),
``KmeansVectorQuantizer`` (:430: nearest codebook entry, straight-through estimator, k-means and
commitment losses), codebook metrics (``compute_code_coverage`` / ``compute_code_pplx`` :140-200).
Inputs are ``[B, T, D]`` split into ``num_groups`` groups of ``dim_from_all_codebooks /
num_groups``; outputs carry ``ids [B, T, G]`` and ``quantized_vectors [B, T, G, H]``.
"""

from __future__ import annotations

from typing import NamedTuple, Optional

import torch
import torch.nn.functional as F

from axlearn_b200.common.base_layer import BaseLayer, ParameterSpec
from axlearn_b200.common.config import REQUIRED, Required, config_class
from axlearn_b200.common.layers import Linear
from axlearn_b200.common.metrics import WeightedSummary
from axlearn_b200.common.param_init import gaussian_initializer

Tensor = torch.Tensor


class QuantizerOutput(NamedTuple):
    ids: Tensor                 # [B, T, G], -1 at padded positions
    quantized_vectors: Tensor   # [B, T, G, H]
    loss: Optional[Tensor] = None


def quantize_by_nearest_neighbor(inputs: Tensor, *, codebook: Tensor, metric: str = "l2") -> tuple[Tensor, Tensor]:
    """``inputs [B, T, G, H]``, ``codebook [V, G, H]`` -> (ids ``[B, T, G]``, vectors ``[B, T, G, H]``)."""
    if metric == "l2":
        dist = (inputs.float().pow(2).sum(-1, keepdim=True)
                - 2 * torch.einsum("btgh,vgh->btgv", inputs.float(), codebook.float())
                + codebook.float().pow(2).sum(-1).t()[None, None])
        ids = dist.argmin(dim=-1)
    else:                                                       # cosine / dot product
        ids = torch.einsum("btgh,vgh->btgv", inputs.float(), codebook.float()).argmax(dim=-1)
    g = torch.arange(codebook.shape[1], device=inputs.device)
    return ids, codebook[ids, g]


def compute_code_histogram(ids: Tensor, *, vocab_size: int, paddings: Tensor) -> Tensor:
    """``[G, V]`` counts over the unpadded positions."""
    live = (1 - paddings.float())[..., None].expand_as(ids).reshape(-1, ids.shape[-1])
    flat = ids.reshape(-1, ids.shape[-1]).clamp_min(0)
    hist = torch.zeros(ids.shape[-1], vocab_size, device=ids.device)
    return hist.scatter_add_(1, flat.t(), live.t())


def compute_code_coverage(hist: Tensor) -> Tensor:
    return (hist > 0).float().mean()


def compute_code_pplx(hist: Tensor) -> Tensor:
    """Mean over groups of ``exp(entropy)`` of the code distribution."""
    p = hist / hist.sum(dim=-1, keepdim=True).clamp_min(1)
    ent = -(p * torch.log(p.clamp_min(1e-30))).sum(dim=-1)
    return torch.exp(ent).mean()


class BaseQuantizer(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        codebook_dim: Required[int] = REQUIRED      # H: per-group dim
        codebook_size: Required[int] = REQUIRED     # V
        num_codebooks: int = 1                      # G

    def _add_codebook_summaries(self, ids: Tensor, paddings: Tensor) -> None:
        hist = compute_code_histogram(ids, vocab_size=self._config.codebook_size, paddings=paddings)
        n = (1 - paddings.float()).sum().clamp_min(1)
        self.add_summary("codebook/coverage", WeightedSummary(compute_code_coverage(hist), n))
        self.add_summary("codebook/pplx", WeightedSummary(compute_code_pplx(hist), n))


class RandomVectorQuantizer(BaseQuantizer):
    """Targets for masked-prediction pre-training: project with a frozen random matrix, L2
    normalise, look up the nearest entry of a frozen random codebook.  Nothing here is trained
    (mark both parameters with a ``NO_UPDATE`` learner rule)."""

    @config_class
    class Config(BaseQuantizer.Config):
        input_dim: Required[int] = REQUIRED
        normalize_codebook: bool = True
        normalize_inputs: bool = True

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("rand_proj", Linear.default_config().set(
            input_dim=cfg.input_dim, output_dim=cfg.codebook_dim * cfg.num_codebooks, bias=False))

    def _create_layer_parameter_specs(self):
        cfg = self._config
        return {"codebook": ParameterSpec(shape=(cfg.codebook_size, cfg.num_codebooks, cfg.codebook_dim),
                                          mesh_axes=(None, None, None), initializer=gaussian_initializer(1.0))}

    def forward(self, inputs: Tensor, *, paddings: Tensor) -> QuantizerOutput:
        cfg = self._config
        with torch.no_grad():
            x = self.rand_proj(inputs).reshape(*inputs.shape[:2], cfg.num_codebooks, cfg.codebook_dim)
            codebook = self.parameters["codebook"]
            if cfg.normalize_inputs:
                x = F.normalize(x.float(), dim=-1)
            if cfg.normalize_codebook:
                codebook = F.normalize(codebook.float(), dim=-1)
            ids, vectors = quantize_by_nearest_neighbor(x, codebook=codebook)
            live = (1 - paddings)[..., None]
            ids = torch.where(live > 0, ids, torch.full_like(ids, -1))
            vectors = vectors * live[..., None]
        self._add_codebook_summaries(ids, paddings)
        return QuantizerOutput(ids=ids, quantized_vectors=vectors)


class KmeansVectorQuantizer(BaseQuantizer):
    """Learned codebook (VQ-VAE): ``loss = kmeans_loss + beta * commitment_loss`` where the first
    pulls codebook entries to the (stopped) inputs and the second pulls inputs to their (stopped)
    entries; the output uses the straight-through estimator."""

    @config_class
    class Config(BaseQuantizer.Config):
        beta: float = 0.25
        normalize_codebook: bool = False

    def _create_layer_parameter_specs(self):
        cfg = self._config
        return {"codebook": ParameterSpec(shape=(cfg.codebook_size, cfg.num_codebooks, cfg.codebook_dim),
                                          mesh_axes=(None, None, "model"), initializer=gaussian_initializer(1.0))}

    def forward(self, inputs: Tensor, *, paddings: Tensor) -> QuantizerOutput:
        cfg = self._config
        b, t, _ = inputs.shape
        x = inputs.reshape(b, t, cfg.num_codebooks, cfg.codebook_dim)
        codebook = self.parameters["codebook"]
        if cfg.normalize_codebook:
            codebook = F.normalize(codebook.float(), dim=-1).to(codebook.dtype)
        ids, vectors = quantize_by_nearest_neighbor(x.detach(), codebook=codebook)
        live = (1 - paddings.float())[..., None, None]
        denom = (live.sum() * cfg.num_codebooks * cfg.codebook_dim).clamp_min(1)
        kmeans = ((vectors.float() - x.detach().float()).pow(2) * live).sum() / denom
        commitment = ((x.float() - vectors.detach().float()).pow(2) * live).sum() / denom
        loss = kmeans + cfg.beta * commitment
        out = x + (vectors - x).detach()                        # straight-through
        out = out * live.to(out.dtype)
        ids = torch.where(live[..., 0] > 0, ids, torch.full_like(ids, -1))
        self.add_summary("loss/kmeans", kmeans.detach())
        self.add_summary("loss/commitment", commitment.detach())
        self._add_codebook_summaries(ids, paddings)
        return QuantizerOutput(ids=ids, quantized_vectors=out, loss=loss)
