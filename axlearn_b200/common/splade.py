"""SPLADE pooling: a sparse lexical embedding over the vocabulary.

Reference: axlearn/common/splade.py:20-97.  Hidden states go through a masked-LM head into
vocabulary logits; the embedding is ``max_t log(1 + relu(logit_t))`` (or the sum over live
tokens).  By default the logits come from the token embedding shared by an ancestor under
``shared_token_emb`` (``attend``); ``vocab_mapping.inner_head`` can be an own ``Linear`` instead.
"""

from __future__ import annotations

from typing import Optional

import torch

from axlearn_b200.common.config import InstantiableConfig, config_class
from axlearn_b200.common.encoder import BertLMHead
from axlearn_b200.common.layers import RedirectToSharedModule, get_activation_fn
from axlearn_b200.common.poolings import BasePoolingLayer

NEG_INF = -1e15


class SpladePooling(BasePoolingLayer):
    SHARED_EMB_NAME = "shared_token_emb"

    @config_class
    class Config(BasePoolingLayer.Config):
        splade_activation_fn: str = "nn.relu"
        splade_mode: str = "max"                         # "max" or "sum"
        vocab_mapping: InstantiableConfig = BertLMHead.default_config()

    @classmethod
    def default_config(cls):
        cfg = super().default_config()
        # Logits through the token embedding that an ancestor shares (tied weights); set
        # ``vocab_mapping.inner_head`` to a ``Linear`` config for an own output matrix.
        cfg.vocab_mapping = BertLMHead.default_config().set(
            inner_head=RedirectToSharedModule.default_config().set(
                shared_module=cls.SHARED_EMB_NAME, method_map=dict(forward="attend")))
        return cfg

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("vocab_mapping", cfg.vocab_mapping.clone(input_dim=cfg.input_dim, num_classes=cfg.output_dim))

    def forward(self, tokens: torch.Tensor, paddings: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``[batch, length, hidden] -> [batch, 1, vocab]``."""
        cfg = self._config
        if cfg.splade_mode not in ("max", "sum"):
            raise ValueError(f"splade_mode {cfg.splade_mode} is not supported")
        if cfg.num_outputs != 1:
            raise NotImplementedError("SPLADE pooling has one output")
        if paddings is None:
            paddings = torch.zeros(tokens.shape[:2], dtype=torch.bool, device=tokens.device)
        pad = paddings.bool().unsqueeze(-1)
        x = self.vocab_mapping(sequence_output=tokens)["logits"]
        act = get_activation_fn(cfg.splade_activation_fn)
        if cfg.splade_mode == "max":    # pool first: log1p(act(.)) is monotone and the pooled tensor is small
            x = x.masked_fill(pad, NEG_INF).amax(dim=1, keepdim=True)
            return torch.log1p(act(x))
        return (torch.log1p(act(x)) * (~pad).to(x.dtype)).sum(dim=1, keepdim=True)
