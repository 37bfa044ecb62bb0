"""Sequence transducer (RNN-T): joint network, blank / token log-probabilities and the loss.

Reference: axlearn/common/transducer.py (log-prob conventions :77-155, ``Transducer`` :158-304,
alignment lattice :362-571, padding rules :574-660).

The lattice node ``(t, u)`` means "``t`` frames consumed, ``u`` labels emitted".  A blank moves to
``(t + 1, u)``, label ``y_u`` moves to ``(t, u + 1)``; the alignment probability is the sum over
all paths from ``(0, 0)`` that leave the lattice by a blank at ``(T - 1, U)``.  The reference
scans anti-diagonals of a tilted lattice per example under ``vmap``; here the whole batch advances
one frame row at a time and each row is solved in closed form with a log-cumsum-exp, using every
example's own ``T`` and ``U`` instead of rewriting the padded region.  Gradients come from autograd.
"""

from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.nn.functional as F

from axlearn_b200.common.base_layer import BaseLayer
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class, config_for_function
from axlearn_b200.common.layers import Linear, get_activation_fn

Tensor = torch.Tensor
_NEG_INF = -1e30


def classic_logits_to_log_probs(*, blank_id: int, blank_logit_bias: float = 0.0) -> Callable[[Tensor], dict]:
    """One softmax over the vocabulary, blank included (Graves 2012)."""

    def fn(logits: Tensor) -> dict:
        onehot = F.one_hot(torch.tensor(blank_id, device=logits.device), logits.shape[-1]).to(logits.dtype)
        lp = torch.log_softmax(logits + blank_logit_bias * onehot, dim=-1)
        return dict(log_prob_blank=lp[..., blank_id], log_prob_tokens=lp + _NEG_INF * onehot)

    return fn


def hat_logits_to_log_probs(*, blank_id: int, blank_logit_bias: float = 0.0) -> Callable[[Tensor], dict]:
    """HAT factorisation: a Bernoulli for blank, then a softmax over the labels."""

    def fn(logits: Tensor) -> dict:
        blank = logits[..., blank_id] + blank_logit_bias
        onehot = F.one_hot(torch.tensor(blank_id, device=logits.device), logits.shape[-1]).to(logits.dtype)
        tokens = torch.log_softmax(logits + _NEG_INF * onehot, dim=-1) - F.softplus(blank)[..., None]
        return dict(log_prob_blank=-F.softplus(-blank), log_prob_tokens=tokens)

    return fn


def log_probs_from_blank_and_tokens(log_prob_blank: Tensor, log_prob_tokens: Tensor, *, blank_id: int) -> Tensor:
    """``[..., vocab]`` with the blank entry taken from ``log_prob_blank``."""
    out = log_prob_tokens.clone()
    out[..., blank_id] = log_prob_blank
    return out


def log_prob_prefix_alignments(log_prob_blank: Tensor, log_prob_y: Tensor) -> Tensor:
    """``alpha [B, T, U + 1]``: log-probability of reaching node ``(t, u)``.

    ``log_prob_blank [B, T, U + 1]``, ``log_prob_y [B, T, U]``.  Row recurrence
    ``alpha[t, u] = logaddexp(alpha[t-1, u] + blank[t-1, u], alpha[t, u-1] + y[t, u-1])``; with
    ``Y[u] = sum_{j<u} y[t, j]`` the row is ``Y + logcumsumexp(from_above - Y)``.
    """
    b, t_max, u1 = log_prob_blank.shape
    blank = log_prob_blank.float()
    y_cum = torch.cat([blank.new_zeros(b, t_max, 1), torch.cumsum(log_prob_y.float(), dim=-1)], dim=-1)
    above = torch.full((b, u1), _NEG_INF, device=blank.device)
    above[:, 0] = 0.0
    rows = []
    for t in range(t_max):
        row = y_cum[:, t] + torch.logcumsumexp(above - y_cum[:, t], dim=-1)
        rows.append(row)
        above = row + blank[:, t]
    return torch.stack(rows, dim=1)


def log_prob_alignments(log_prob_blank: Tensor, log_prob_y: Tensor, *, am_lengths: Tensor,
                        label_lengths: Tensor) -> Tensor:
    """``[B]``: log-probability of all alignments of ``T_i`` frames with ``U_i`` labels."""
    alpha = log_prob_prefix_alignments(log_prob_blank, log_prob_y)
    rows = torch.arange(alpha.shape[0], device=alpha.device)
    t_last = (am_lengths - 1).clamp_min(0)
    return alpha[rows, t_last, label_lengths] + log_prob_blank.float()[rows, t_last, label_lengths]


class Transducer(BaseLayer):
    """Joint network ``proj(act(am_t + lm_u))`` and the transducer loss."""

    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        vocab_size: Required[int] = REQUIRED
        activation_fn: str = "nn.tanh"
        proj: InstantiableConfig = Linear.default_config()
        logits_to_log_probs: InstantiableConfig = config_for_function(classic_logits_to_log_probs)

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("proj", cfg.proj.clone(input_dim=cfg.input_dim, output_dim=cfg.vocab_size))
        self._logits_to_log_probs = cfg.logits_to_log_probs.instantiate()

    def predict(self, am_data: Tensor, lm_data: Tensor) -> dict:
        """``am_data [..., T, D]``, ``lm_data [..., U, D]`` -> ``log_prob_blank [..., T, U]`` and
        ``log_prob_tokens [..., T, U, vocab]``."""
        hidden = get_activation_fn(self._config.activation_fn)(am_data.unsqueeze(-2) + lm_data.unsqueeze(-3))
        return self._logits_to_log_probs(self.proj(hidden).float())

    def forward(self, *, am_data: Tensor, am_paddings: Tensor, lm_data: Tensor, lm_paddings: Tensor,
                target_labels: Tensor, frame_chunk: Optional[int] = None):
        """``am_data [B, T, D]``; ``lm_data [B, U + 1, D]`` computed from BOS + labels;
        ``lm_paddings`` has ``U_i + 1`` leading zeros per row; ``target_labels [B, U + 1]`` (entries
        past ``U_i`` are ignored).  Returns ``(loss, per_example)`` with ``log_prob_alignments``,
        ``is_valid_example`` and ``loss`` per example.

        The ``[B, T, U + 1, vocab]`` joint tensor is produced ``frame_chunk`` frames at a time and
        reduced to the two ``[B, T, U + 1]`` lattices immediately.
        """
        b, t_max, _ = am_data.shape
        u1 = lm_data.shape[1]
        labels = target_labels.clamp(0, self._config.vocab_size - 1).long()
        chunk = frame_chunk or max(1, min(t_max, (1 << 24) // max(1, b * u1 * self._config.vocab_size)))
        blanks, ys = [], []
        for lo in range(0, t_max, chunk):
            pred = self.predict(am_data[:, lo:lo + chunk], lm_data)
            blanks.append(pred["log_prob_blank"])
            idx = labels[:, None, :, None].expand(-1, pred["log_prob_tokens"].shape[1], -1, 1)
            ys.append(torch.gather(pred["log_prob_tokens"], -1, idx).squeeze(-1))
        log_prob_blank = torch.cat(blanks, dim=1)
        log_prob_y = torch.cat(ys, dim=1)[:, :, :-1]
        am_lengths = (1 - am_paddings.long()).sum(-1)
        lm_lengths = (1 - lm_paddings.long()).sum(-1)
        valid = (am_lengths > 0) & (lm_lengths > 0)
        ll = log_prob_alignments(log_prob_blank, log_prob_y, am_lengths=am_lengths,
                                 label_lengths=(lm_lengths - 1).clamp_min(0))
        per_example_loss = torch.where(valid, -ll, torch.zeros_like(ll))
        loss = per_example_loss.sum() / valid.sum().clamp_min(1)
        return loss, dict(log_prob_blank=log_prob_blank, log_prob_y=log_prob_y, log_prob_alignments=ll,
                          is_valid_example=valid, loss=per_example_loss)
