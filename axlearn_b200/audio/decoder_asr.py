"""Transducer (RNN-T) and listen-attend-spell decoders over encoded speech frames.

Reference: axlearn/audio/decoder_asr.py (``_map_label_sequences`` :650, ``RNNPredictionNetwork``
:701, ``TransducerDecoderModel`` :768-1099, ``LASDecoderModel`` :1123-1348).  The CTC decoder lives
in ``axlearn_b200/audio/asr.py``.

Batch layout shared by the decoders: ``inputs [B, T, D]`` encoder outputs, ``paddings [B, T]``,
``target_labels [B, L]`` = labels followed by EOS (out-of-vocabulary ids are padding),
``target.input_ids [B, L]`` = BOS followed by the labels.
"""

from __future__ import annotations

import dataclasses
from typing import Callable, Optional

import torch

from axlearn_b200.common.attention import TransformerAttentionLayer
from axlearn_b200.common.base_layer import BaseLayer
from axlearn_b200.common.base_model import BaseModel
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class
from axlearn_b200.common.decoder import Decoder
from axlearn_b200.common.decoding import StopOnSubsequence
from axlearn_b200.common.layers import Embedding, Linear
from axlearn_b200.common.metrics import WeightedSummary
from axlearn_b200.common.module import child_context
from axlearn_b200.common.rnn import LSTMCell
from axlearn_b200.common.transducer import Transducer
from axlearn_b200.common.loss import cross_entropy

Tensor = torch.Tensor
NEG_INF = -1e15


@dataclasses.dataclass
class DecodeOutputs:
    raw_sequences: Tensor   # [B, num_decodes, L] as produced by the search
    sequences: Tensor       # padding and EOS replaced by 0
    paddings: Tensor        # [B, num_decodes, L] bool
    scores: Tensor          # [B, num_decodes]


def map_label_sequences(inputs: Tensor, *, remove_repeats: bool, blank_id: int = 0, pad_id: int = 0) -> dict:
    """Drops blanks, paddings and (for CTC) repeats, compacting what is left to the front.
    Returns ``sequences``, ``paddings`` and ``lengths [..., 1]``."""
    keep = (inputs != blank_id) & (inputs != pad_id)
    if remove_repeats:
        prev = torch.cat([torch.full_like(inputs[..., :1], pad_id), inputs[..., :-1]], dim=-1)
        keep = keep & (inputs != prev)
    lengths = keep.sum(-1, keepdim=True)
    order = torch.argsort((~keep).to(torch.int8), dim=-1, stable=True)
    seq = torch.gather(inputs, -1, order)
    paddings = torch.arange(inputs.shape[-1], device=inputs.device) >= lengths
    return dict(sequences=torch.where(paddings, torch.full_like(seq, pad_id), seq), paddings=paddings, lengths=lengths)


def _target_paddings(target_labels: Tensor, *, vocab_size: int) -> Tensor:
    return (target_labels < 0) | (target_labels >= vocab_size)


def _paddings_from_decode_sequence(*, sequences: Tensor, scores: Tensor, eos_id: int) -> Tensor:
    """Everything after the first EOS (and the EOS itself) is padding; so is a hypothesis whose
    score marks it as absent."""
    seen = torch.cumsum((sequences == eos_id).long(), dim=-1) > 0
    return seen | (scores <= NEG_INF / 2)


class BaseASRDecoderModel(BaseModel):
    @config_class
    class Config(BaseModel.Config):
        input_dim: Required[int] = REQUIRED
        vocab_size: Required[int] = REQUIRED

    def _input_stats_summaries(self, *, input_batch: dict, target_paddings: Tensor, is_valid_example: Tensor) -> None:
        valid = is_valid_example.float()
        n = valid.sum().clamp_min(1)
        frames = ((1 - input_batch["paddings"].float()).sum(-1) * valid).sum()
        labels = ((~target_paddings).float().sum(-1) * valid).sum()
        self.add_summary("input_stats/average_target_length", WeightedSummary(labels / n, n))
        self.add_summary("input_stats/average_source_length", WeightedSummary(frames / n, n))
        self.add_summary("input_stats/frame_packing_efficiency",
                         WeightedSummary(frames / input_batch["paddings"].numel(), input_batch["paddings"].numel()))


class RNNPredictionNetwork(BaseLayer):
    """The transducer's label-history network: embedding followed by a recurrent cell."""

    @config_class
    class Config(BaseLayer.Config):
        vocab_size: Required[int] = REQUIRED
        emb_dim: Required[int] = REQUIRED
        output_dim: Required[int] = REQUIRED
        embedding: InstantiableConfig = Embedding.default_config()
        rnn_cell: InstantiableConfig = LSTMCell.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("embedding", cfg.embedding.clone(num_embeddings=cfg.vocab_size, dim=cfg.emb_dim))
        self._add_child("rnn", cfg.rnn_cell.clone(input_dim=cfg.emb_dim, output_dim=cfg.output_dim))

    def forward(self, inputs: Tensor) -> Tensor:
        """``[B, U] -> [B, U, output_dim]``."""
        ids = inputs.clamp(0, self._config.vocab_size - 1)
        return self.rnn(self.embedding(ids).transpose(0, 1)).transpose(0, 1)

    def init_states(self, *, batch_size: int, device=None):
        return self.rnn.init_states(batch_size=batch_size, device=device)

    def extend_step(self, *, cached_states, data: Tensor):
        """``data [B]`` -> ``(states, [B, output_dim])``."""
        return self.rnn.extend_step(cached_states=cached_states, data=self.embedding(data))


class TransducerDecoderModel(BaseASRDecoderModel):
    @config_class
    class Config(BaseASRDecoderModel.Config):
        lm_dim: Required[int] = REQUIRED
        joint_dim: Required[int] = REQUIRED
        blank_id: int = 0
        bos_id: int = 1
        eos_id: int = 2
        prediction_network: InstantiableConfig = RNNPredictionNetwork.default_config()
        am_proj: InstantiableConfig = Linear.default_config()
        lm_proj: InstantiableConfig = Linear.default_config()
        transducer: InstantiableConfig = Transducer.default_config()

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        if cfg.eos_id == cfg.blank_id:
            raise ValueError(f"eos_id and blank_id must differ, got {cfg.blank_id} for both")
        self._add_child("am_proj", cfg.am_proj.clone(input_dim=cfg.input_dim, output_dim=cfg.joint_dim, bias=True))
        self._add_child("lm_proj", cfg.lm_proj.clone(input_dim=cfg.lm_dim, output_dim=cfg.joint_dim, bias=False))
        self._add_child("prediction_network", cfg.prediction_network.clone(
            vocab_size=cfg.vocab_size, output_dim=cfg.lm_dim))
        tcfg = cfg.transducer.clone(input_dim=cfg.joint_dim, vocab_size=cfg.vocab_size)
        tcfg.logits_to_log_probs.blank_id = cfg.blank_id
        self._add_child("transducer", tcfg)

    def forward(self, input_batch: dict):
        cfg = self._config
        am = self.am_proj(input_batch["inputs"])
        labels = input_batch["target_labels"]
        target_paddings = _target_paddings(labels, vocab_size=cfg.vocab_size)
        lm = self.lm_proj(self.prediction_network(input_batch["target"]["input_ids"]))
        _, per = self.transducer(am_data=am, am_paddings=input_batch["paddings"], lm_data=lm,
                                 lm_paddings=target_paddings, target_labels=labels)
        weight = per["is_valid_example"].to(per["loss"].dtype)
        loss = (per["loss"] * weight).sum() / weight.sum().clamp_min(1)
        self._input_stats_summaries(input_batch=input_batch, target_paddings=target_paddings, is_valid_example=weight)
        self.add_summary("loss/example_weight", WeightedSummary(weight.mean(), weight.shape[0]))
        self.add_summary("loss/rnnt_loss", WeightedSummary(loss.detach(), weight.sum().clamp_min(1)))
        return loss, dict(per_example_weight=weight, per_example_loss=per["loss"])

    # ---------------------------------------------------------------- decoding
    def _step_log_probs(self, am_t: Tensor, lm_u: Tensor) -> dict:
        pred = self.transducer.predict(am_t[:, None, :], lm_u[:, None, :])
        return dict(blank=pred["log_prob_blank"][:, 0, 0], tokens=pred["log_prob_tokens"][:, 0, 0])

    @torch.no_grad()
    def greedy_decode(self, input_batch: dict, *, max_decode_len: int, max_symbols_per_frame: int = 4) -> DecodeOutputs:
        """Frame-synchronous greedy search for the whole batch: at every frame emit the best
        label while it beats blank (at most ``max_symbols_per_frame`` times), then advance."""
        cfg = self._config
        am = self.am_proj(input_batch["inputs"])
        b, t_max, _ = am.shape
        live_frames = ~input_batch["paddings"].bool()
        dev = am.device
        states = self.prediction_network.init_states(batch_size=b, device=dev)
        states, lm = self.prediction_network.extend_step(
            cached_states=states, data=torch.full((b,), cfg.bos_id, dtype=torch.long, device=dev))
        lm = self.lm_proj(lm)
        out = torch.zeros(b, max_decode_len, dtype=torch.long, device=dev)
        n = torch.zeros(b, dtype=torch.long, device=dev)
        score = torch.zeros(b, device=dev)
        rows = torch.arange(b, device=dev)
        for t in range(t_max):
            for _ in range(max_symbols_per_frame):
                lp = self._step_log_probs(am[:, t], lm)
                best_lp, best = lp["tokens"].max(dim=-1)
                emit = live_frames[:, t] & (best_lp > lp["blank"]) & (n < max_decode_len) & (best != cfg.eos_id)
                if not emit.any():
                    break
                out[rows[emit], n[emit]] = best[emit]
                n = n + emit.long()
                score = score + torch.where(emit, best_lp, torch.zeros_like(best_lp))
                new_states, new_lm = self.prediction_network.extend_step(cached_states=states, data=best)
                pick = lambda new, old: torch.where(emit[:, None], new, old)
                states = {k: pick(new_states[k], states[k]) for k in states}
                lm = pick(self.lm_proj(new_lm), lm)
            lp = self._step_log_probs(am[:, t], lm)
            score = score + torch.where(live_frames[:, t], lp["blank"], torch.zeros_like(score))
        paddings = torch.arange(max_decode_len, device=dev)[None] >= n[:, None]
        return DecodeOutputs(raw_sequences=out[:, None], sequences=out[:, None], paddings=paddings[:, None],
                             scores=score[:, None])

    @torch.no_grad()
    def beam_search_decode(self, input_batch: dict, *, num_decodes: int, max_decode_len: int,
                           max_symbols_per_frame: int = 3) -> DecodeOutputs:
        """Time-synchronous beam search per utterance; hypotheses with the same label sequence
        are merged by adding their probabilities."""
        cfg = self._config
        am_all = self.am_proj(input_batch["inputs"])
        b = am_all.shape[0]
        dev = am_all.device
        lengths = (~input_batch["paddings"].bool()).sum(-1).tolist()
        seqs = torch.zeros(b, num_decodes, max_decode_len, dtype=torch.long, device=dev)
        pads = torch.ones(b, num_decodes, max_decode_len, dtype=torch.bool, device=dev)
        scores = torch.full((b, num_decodes), NEG_INF, device=dev)

        def advance(state, token):
            new_state, lm = self.prediction_network.extend_step(
                cached_states=state, data=torch.tensor([token], dtype=torch.long, device=dev))
            return new_state, self.lm_proj(lm)

        for i in range(b):
            s0, lm0 = advance(self.prediction_network.init_states(batch_size=1, device=dev), cfg.bos_id)
            beam = {(): (0.0, s0, lm0)}
            for t in range(lengths[i]):
                frontier, done = beam, {}
                for _ in range(max_symbols_per_frame + 1):
                    grown = {}
                    for labels, (lp_h, state, lm) in frontier.items():
                        lp = self._step_log_probs(am_all[i:i + 1, t], lm)
                        blank = lp_h + float(lp["blank"][0])
                        if labels in done:
                            done[labels] = (float(torch.logaddexp(torch.tensor(done[labels][0]), torch.tensor(blank))),) + done[labels][1:]
                        else:
                            done[labels] = (blank, state, lm)
                        if len(labels) >= max_decode_len:
                            continue
                        top_lp, top = lp["tokens"][0].topk(min(num_decodes, lp["tokens"].shape[-1]))
                        for tok_lp, tok in zip(top_lp.tolist(), top.tolist()):
                            if tok == cfg.eos_id:
                                continue
                            grown[labels + (tok,)] = (lp_h + tok_lp, state, lm, tok)
                    best = sorted(grown.items(), key=lambda kv: -kv[1][0])[:num_decodes]
                    frontier = {}
                    for labels, (lp_h, state, lm, tok) in best:
                        ns, nlm = advance(state, tok)
                        frontier[labels] = (lp_h, ns, nlm)
                    if not frontier:
                        break
                beam = dict(sorted(done.items(), key=lambda kv: -kv[1][0])[:num_decodes])
            for j, (labels, (lp_h, _, _)) in enumerate(sorted(beam.items(), key=lambda kv: -kv[1][0])):
                seqs[i, j, :len(labels)] = torch.tensor(labels, dtype=torch.long, device=dev)
                pads[i, j, :len(labels)] = False
                scores[i, j] = lp_h
        return DecodeOutputs(raw_sequences=seqs, sequences=seqs, paddings=pads, scores=scores)


class LASDecoderModel(BaseASRDecoderModel):
    """Listen-attend-spell: an autoregressive transformer decoder cross-attending to the frames."""

    @config_class
    class Config(BaseASRDecoderModel.Config):
        decoder: InstantiableConfig = Decoder.default_config()
        z_loss_scale: float = 0.0
        label_smoothing: float = 0.0

    @classmethod
    def default_config(cls):
        cfg = super().default_config()
        cfg.decoder.transformer.layer.cross_attention = TransformerAttentionLayer.default_config()
        return cfg

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        dec = cfg.decoder.clone(vocab_size=cfg.vocab_size)
        dec.transformer.layer.cross_attention.source_dim = cfg.input_dim
        self._add_child("decoder", dec)

    @staticmethod
    def _cross_attention_logit_biases(paddings: Tensor) -> Tensor:
        return (paddings.bool().float() * NEG_INF)[:, None, None, :]

    def forward(self, input_batch: dict):
        cfg = self._config
        labels = input_batch["target_labels"]
        target_paddings = _target_paddings(labels, vocab_size=cfg.vocab_size)
        out = self.decoder(input_batch=input_batch["target"], cross_attention_data=input_batch["inputs"],
                           cross_attention_logit_biases=self._cross_attention_logit_biases(input_batch["paddings"]))
        logits = out["logits"] if out.get("logits") is not None else self.decoder.compute_logits(out)
        valid = (~input_batch["paddings"].bool()).sum(-1) > 0
        live = (~target_paddings) & valid[:, None]
        loss, aux = cross_entropy(logits.float(), labels.clamp(0, cfg.vocab_size - 1), live_targets=live,
                                  z_loss_scale=cfg.z_loss_scale, label_smoothing=cfg.label_smoothing)
        self._input_stats_summaries(input_batch=input_batch, target_paddings=target_paddings, is_valid_example=valid)
        per_token = aux["per_token_loss"] if "per_token_loss" in aux else torch.zeros_like(live, dtype=torch.float32)
        weight = live.float().sum(-1)
        n = weight.sum()
        self.add_summary("loss", WeightedSummary(loss.detach(), n))
        self.add_summary("perplexity", WeightedSummary(torch.exp(loss.detach()), n))
        if "accuracy" in aux:
            self.add_summary("token_accuracy", WeightedSummary(aux["accuracy"], n))
        return loss, dict(per_example_loss=per_token.sum(-1), per_example_weight=weight)

    def _decode_kwargs(self, input_batch: dict, max_decode_len: int, num_decodes: int) -> dict:
        if "prefix" not in input_batch:
            raise ValueError("input_batch needs `prefix` (starting with BOS)")
        return dict(input_batch=input_batch, max_sequence_length=max_decode_len, num_decodes=num_decodes,
                    cross_attention_data=input_batch["inputs"],
                    cross_attention_logit_biases=self._cross_attention_logit_biases(input_batch["paddings"]))

    def beam_search_decode(self, input_batch: dict, *, num_decodes: int, max_decode_len: int,
                           brevity_penalty: Optional[Callable] = None) -> DecodeOutputs:
        eos = self._config.decoder.eos_token_id
        with child_context("beam_search_decode", module=self.decoder):
            out = self.decoder.beam_search_decode(
                **self._decode_kwargs(input_batch, max_decode_len, num_decodes), brevity_penalty=brevity_penalty)
        paddings = _paddings_from_decode_sequence(sequences=out.sequences, scores=out.scores[..., None], eos_id=eos)
        return DecodeOutputs(raw_sequences=out.sequences, sequences=out.sequences * (~paddings), paddings=paddings,
                             scores=out.scores)

    def sample_decode(self, input_batch: dict, *, num_decodes: int, max_decode_len: int,
                      logits_modifier=None) -> DecodeOutputs:
        eos = self._config.decoder.eos_token_id
        with child_context("sample_decode", module=self.decoder):
            out = self.decoder.sample_decode(
                **self._decode_kwargs(input_batch, max_decode_len, num_decodes), logits_modifier=logits_modifier,
                stop_decoding_condition=StopOnSubsequence([[eos]]))
        paddings = _paddings_from_decode_sequence(sequences=out.sequences, scores=out.token_scores, eos_id=eos)
        return DecodeOutputs(raw_sequences=out.sequences, sequences=out.sequences * (~paddings), paddings=paddings,
                             scores=(out.token_scores * (~paddings)).sum(-1))
