"""Speech recognition: encoder, CTC decoder head and the model that joins them.

Parity targets in the reference: ``SpeechFeatureLayer`` / ``ASREncoder`` (axlearn/audio/
encoder_asr.py:30-230: frontend -> SpecAugment -> subsampler -> input linear + dropout ->
positional embedding -> conformer stack), ``CTCDecoderModel`` (axlearn/audio/decoder_asr.py:
290-620: linear to vocabulary logits, CTC loss with blank id 0 normalised by the number of label
tokens, greedy decoding that merges repeats and drops blanks, prefix-merging beam search),
``ctc_aligner`` is not built, ``ASRModel`` (axlearn/audio/model_asr.py:20-110).
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from axlearn_b200.audio.conformer import RepeatedConformerLayer
from axlearn_b200.audio.frontend import LogMelFrontend
from axlearn_b200.audio.spectrum_augmenter import SpectrumAugmenter
from axlearn_b200.audio.subsamplers import ConvSubSampler
from axlearn_b200.common.base_layer import BaseLayer
from axlearn_b200.common.base_model import BaseModel
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.layers import Dropout, Linear
from axlearn_b200.common.metrics import WeightedSummary

Tensor = torch.Tensor


class SpeechFeatureLayer(BaseLayer):
    """``[B, samples]`` -> ``[B, frames', output_dim]`` and paddings."""

    @config_class
    class Config(BaseLayer.Config):
        output_dim: Required[int] = REQUIRED
        frontend: InstantiableConfig = LogMelFrontend.default_config()
        augmenter: Optional[InstantiableConfig] = SpectrumAugmenter.default_config()
        subsampler: InstantiableConfig = ConvSubSampler.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("frontend", cfg.frontend)
        if cfg.augmenter is not None:
            self._add_child("augmenter", cfg.augmenter)
        self._add_child("subsampler", cfg.subsampler.clone(output_dim=cfg.output_dim))

    def forward(self, inputs: Tensor, *, paddings: Tensor):
        feats = self.frontend(inputs, paddings=paddings)
        x, p = feats["outputs"], feats["paddings"]
        if "augmenter" in self._children:
            x = self.augmenter(x, paddings=p)
        sub = self.subsampler(x, paddings=p)
        x, p = sub["outputs"], sub["paddings"]
        b, t, f, c = x.shape
        return {"outputs": x.reshape(b, t, f * c), "paddings": p}


class SpeechContextNetwork(BaseLayer):
    """``input_linear`` + dropout (+ positional embedding) followed by the ``context`` stack
    (reference: axlearn/audio/encoder_asr.py ``SpeechContextNetwork``)."""

    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        output_dim: Required[int] = REQUIRED
        input_linear: InstantiableConfig = Linear.default_config().set(bias=True)
        dropout: InstantiableConfig = Dropout.default_config()
        pos_emb: Optional[InstantiableConfig] = None
        context: InstantiableConfig = RepeatedConformerLayer.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("input_linear", cfg.input_linear.clone(input_dim=cfg.input_dim, output_dim=cfg.output_dim))
        self._add_child("dropout", cfg.dropout)
        if cfg.pos_emb is not None:
            self._add_child("pos_emb", cfg.pos_emb.clone(dim=cfg.output_dim))
        self._add_child("context", cfg.context.clone(input_dim=cfg.output_dim))

    def forward(self, inputs: Tensor, *, paddings: Tensor):
        x = self.dropout(self.input_linear(inputs))
        if "pos_emb" in self._children:
            x = x + self.pos_emb(torch.arange(x.shape[1], device=x.device))[None].to(x.dtype)
        x = x * (1 - paddings)[..., None].to(x.dtype)
        return {"outputs": self.context(x, paddings=paddings), "paddings": paddings}


class ASREncoder(BaseLayer):
    """``feature`` (frontend, augmenter, subsampler) then ``context`` (input projection +
    conformer stack)."""

    @config_class
    class Config(BaseLayer.Config):
        dim: Required[int] = REQUIRED
        feature: InstantiableConfig = SpeechFeatureLayer.default_config()
        context: InstantiableConfig = SpeechContextNetwork.default_config()
        # Flattened (frequency x channels) size of the feature layer's output.
        feature_dim: Required[int] = REQUIRED

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("feature", cfg.feature)
        self._add_child("context", cfg.context.clone(input_dim=cfg.feature_dim, output_dim=cfg.dim))

    def forward(self, inputs: Tensor, *, paddings: Tensor):
        feats = self.feature(inputs, paddings=paddings)
        return self.context(feats["outputs"], paddings=feats["paddings"])


def ctc_greedy_decode(logits: Tensor, paddings: Tensor, *, blank_id: int = 0) -> list[list[int]]:
    """Best path: argmax per frame, merge repeats, drop blanks."""
    best = logits.argmax(dim=-1)
    out = []
    for seq, pad in zip(best.tolist(), paddings.tolist()):
        prev, toks = None, []
        for tok, is_pad in zip(seq, pad):
            if is_pad:
                break
            if tok != prev and tok != blank_id:
                toks.append(tok)
            prev = tok
        out.append(toks)
    return out


def ctc_prefix_beam_search(log_probs: Tensor, *, beam_size: int = 4, blank_id: int = 0) -> list[tuple[list[int], float]]:
    """Prefix-merging beam search over one utterance ``[T, V]`` of log-probabilities: hypotheses
    that collapse to the same label sequence share their probability mass.  Returns
    ``[(labels, log_prob)]`` best first."""
    import math

    def lse(*xs):
        m = max(xs)
        return m if m == -math.inf else m + math.log(sum(math.exp(x - m) for x in xs))

    beams = {(): (0.0, -math.inf)}                                  # prefix -> (log p ending in blank, not blank)
    for frame in log_probs.tolist():
        nxt: dict = {}

        def add(prefix, pb, pnb):
            old = nxt.get(prefix, (-math.inf, -math.inf))
            nxt[prefix] = (lse(old[0], pb), lse(old[1], pnb))

        for prefix, (pb, pnb) in beams.items():
            total = lse(pb, pnb)
            add(prefix, total + frame[blank_id], -math.inf)
            for v, lp in enumerate(frame):
                if v == blank_id:
                    continue
                if prefix and prefix[-1] == v:
                    add(prefix, -math.inf, pnb + lp)                # repeat without a blank: same prefix
                    add(prefix + (v,), -math.inf, pb + lp)          # after a blank: a new token
                else:
                    add(prefix + (v,), -math.inf, total + lp)
        beams = dict(sorted(nxt.items(), key=lambda kv: -lse(*kv[1]))[:beam_size])
    return [(list(p), lse(*s)) for p, s in sorted(beams.items(), key=lambda kv: -lse(*kv[1]))]


class CTCDecoderModel(BaseLayer):
    @config_class
    class Config(BaseLayer.Config):
        input_dim: Required[int] = REQUIRED
        vocab_size: Required[int] = REQUIRED
        blank_id: int = 0
        lm_head: InstantiableConfig = Linear.default_config().set(bias=True)

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("lm_head", cfg.lm_head.clone(input_dim=cfg.input_dim, output_dim=cfg.vocab_size))

    def predict(self, input_batch: dict) -> Tensor:
        """Logits ``[B, T, V]`` (padded frames zeroed)."""
        x, p = input_batch["inputs"], input_batch["paddings"]
        return self.lm_head(x) * (1 - p)[..., None].to(x.dtype)

    def forward(self, input_batch: dict):
        """``target_labels [B, U]``: values < 0 or >= vocab_size are padding.  Loss = total negative
        log-likelihood / number of label tokens; an utterance with more labels than frames is left
        out, one whose labels cannot be aligned (repeats without room for blanks) contributes 0."""
        cfg = self._config
        logits = self.predict(input_batch)
        labels = input_batch["target_labels"]
        live_labels = (labels >= 0) & (labels < cfg.vocab_size)
        label_lengths = live_labels.sum(dim=1)
        frame_lengths = (1 - input_batch["paddings"]).sum(dim=1).long()
        # Compact the live labels to the front, as the loss expects.
        order = torch.argsort((~live_labels).float(), dim=1, stable=True)
        compact = torch.gather(labels.clamp_min(0), 1, order)
        log_probs = F.log_softmax(logits.float(), dim=-1).transpose(0, 1)       # [T, B, V]
        per_example = F.ctc_loss(log_probs, compact, frame_lengths, label_lengths, blank=cfg.blank_id,
                                 reduction="none", zero_infinity=True)
        # An utterance with fewer frames than labels cannot be aligned: it is left out.
        valid = frame_lengths >= label_lengths
        denom = (label_lengths * valid).sum().clamp_min(1)
        loss = (per_example * valid).sum() / denom
        self.add_summary("loss/ctc", WeightedSummary(loss.detach(), denom))
        self.add_summary("loss/invalid_seq_percent", (~valid).float().mean())
        return loss, {"per_example_loss": per_example, "per_example_weight": valid.float()}

    def align(self, input_batch: dict) -> dict:
        """Forced alignment of ``target_labels`` to the frames: per frame the label id (blank between
        labels, -1 on padding), the label index, and the path's log-probability."""
        from axlearn_b200.audio.aligner import ctc_forced_alignment

        cfg = self._config
        labels = input_batch["target_labels"]
        log_pos = F.log_softmax(self.predict(input_batch).float(), dim=-1)
        return ctc_forced_alignment(
            log_pos=log_pos, log_pos_paddings=input_batch["paddings"], labels=labels,
            label_paddings=(labels < 0) | (labels >= cfg.vocab_size), blank_id=cfg.blank_id).asdict()

    def greedy_decode(self, input_batch: dict) -> list[list[int]]:
        return ctc_greedy_decode(self.predict(input_batch), input_batch["paddings"], blank_id=self._config.blank_id)

    def beam_search_decode(self, input_batch: dict, *, num_decodes: int = 4) -> list[list[tuple[list[int], float]]]:
        logits = self.predict(input_batch)
        lengths = (1 - input_batch["paddings"]).sum(dim=1).long().tolist()
        lp = F.log_softmax(logits.float(), dim=-1)
        return [ctc_prefix_beam_search(lp[i, :n], beam_size=num_decodes, blank_id=self._config.blank_id)
                for i, n in enumerate(lengths)]


class ASRModel(BaseModel):
    """``input_batch = {"inputs": [B, samples], "paddings": [B, samples], "target_labels": [B, U]}``."""

    @config_class
    class Config(BaseModel.Config):
        encoder: Required[InstantiableConfig] = REQUIRED
        decoder: Required[InstantiableConfig] = REQUIRED

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("encoder", cfg.encoder)
        self._add_child("decoder", cfg.decoder)

    def _encode(self, input_batch: dict) -> dict:
        enc = self.encoder(input_batch["inputs"], paddings=input_batch["paddings"])
        return {"inputs": enc["outputs"], "paddings": enc["paddings"]}

    def forward(self, input_batch: dict):
        dec_in = self._encode(input_batch)
        dec_in["target_labels"] = input_batch["target_labels"]
        if "target" in input_batch:         # BOS-prefixed decoder inputs (transducer / LAS decoders)
            dec_in["target"] = input_batch["target"]
        return self.decoder(dec_in)

    def predict(self, input_batch: dict) -> Tensor:
        return self.decoder.predict(self._encode(input_batch))

    def greedy_decode(self, input_batch: dict) -> list[list[int]]:
        return self.decoder.greedy_decode(self._encode(input_batch))

    def align(self, input_batch: dict) -> dict:
        dec_in = self._encode(input_batch)
        dec_in["target_labels"] = input_batch["target_labels"]
        return self.decoder.align(dec_in)

    def beam_search_decode(self, input_batch: dict, *, num_decodes: int = 4, **kwargs):
        dec_in = self._encode(input_batch)
        if "prefix" in input_batch:
            dec_in["prefix"] = input_batch["prefix"]
        return self.decoder.beam_search_decode(dec_in, num_decodes=num_decodes, **kwargs)
