"""Autoregressive decoding: sampling and beam search over a ``tokens_to_scores`` step function.

Parity targets in the reference (axlearn/common/decoding.py): ``add_decoding_dim`` /
``flatten_decoding_dim`` / ``unflatten_decoding_dim`` (:44-75), ``brevity_penalty_fn`` (:203),
``PrefixMerger`` (:286), ``BeamSearchOutputs`` (:357), ``beam_search_decode`` (:433),
``SampleOutputs`` (:817), the stop conditions (:826-975), ``sample_decode`` (:978) and
``infer_initial_time_step`` (:1154).

Conventions shared with the reference: ``inputs[b, 0]`` is a conditioning (BOS) token that is
dropped from the outputs; ``time_step[b]`` is the index of the last prefix token of row ``b``
(tokens up to and including it are teacher-forced); each row advances from its own index, and
writes past the end of the buffer are dropped.

The loops are host loops over a fixed-shape, in-place step: sequences, scores and stop flags
are persistent device buffers updated by scatter, so a step is a constant set of launches (and
the step function is free to be a captured CUDA graph).  The termination test needs one
device-to-host read; it is made every ``check_every`` steps -- extra steps after every row has
stopped only write padding.
"""

from __future__ import annotations

import dataclasses
from typing import Any, Callable, NamedTuple, Optional, Protocol, Sequence

import torch

from axlearn_b200.common import prng
from axlearn_b200.common.utils import tree_map, vectorized_tree_map

Tensor = torch.Tensor
NEG_INF = -1.0e7


# ------------------------------------------------------------------------------------------
# The decoding (num_decodes / beam) dim.
# ------------------------------------------------------------------------------------------


def add_decoding_dim(x: Tensor, num_decodes: int) -> Tensor:
    """``[B, ...] -> [B, num_decodes, ...]`` (copies); scalars pass through."""
    if not isinstance(x, Tensor) or x.dim() == 0:
        return x
    return x.unsqueeze(1).expand(x.shape[0], num_decodes, *x.shape[1:]).contiguous()


def flatten_decoding_dim(x: Tensor) -> Tensor:
    """``[B, num_decodes, ...] -> [B * num_decodes, ...]``; scalars pass through."""
    if not isinstance(x, Tensor) or x.dim() == 0:
        return x
    return x.reshape(x.shape[0] * x.shape[1], *x.shape[2:])


def unflatten_decoding_dim(x: Tensor, batch_size: int, num_decodes: int) -> Tensor:
    if not isinstance(x, Tensor) or x.dim() == 0:
        return x
    assert x.shape[0] == batch_size * num_decodes, (x.shape, batch_size, num_decodes)
    return x.reshape(batch_size, num_decodes, *x.shape[1:])


def infer_initial_time_step(prefix: Tensor, *, pad_id: int) -> Tensor:
    """Index of the last non-pad token of each row (0 for an all-pad row)."""
    idx = torch.arange(prefix.shape[-1], device=prefix.device)
    return ((prefix != pad_id).to(idx.dtype) * idx).amax(dim=-1)


def _gather_beams(tree: Any, beam_indices: Tensor) -> Any:
    """Reorders the beam dim of every ``[B, beam, ...]`` leaf by ``beam_indices [B, new_beam]``."""

    def gather(x):
        if not isinstance(x, Tensor) or x.dim() < 2:
            return x
        idx = beam_indices.reshape(beam_indices.shape + (1,) * (x.dim() - 2)).expand(-1, -1, *x.shape[2:])
        return torch.gather(x, 1, idx)

    return vectorized_tree_map(gather, tree)


# ------------------------------------------------------------------------------------------
# Brevity penalty, prefix merging.
# ------------------------------------------------------------------------------------------


class BrevityPenaltyFn(Protocol):
    def __call__(self, *, length: Tensor, raw_scores: Tensor) -> Tensor: ...


def brevity_penalty_fn(*, alpha: float = 0.0, bp_type: str = "t5") -> BrevityPenaltyFn:
    """Length normalisation: ``raw / ((5 + len) / 6) ** alpha`` ("t5") or ``raw / len ** alpha``
    ("hf").  ``alpha = 0`` leaves scores unchanged."""
    if bp_type not in ("t5", "hf"):
        raise NotImplementedError(f"{bp_type} brevity penalty is not supported (t5, hf)")

    def fn(*, length, raw_scores: Tensor) -> Tensor:
        length = torch.as_tensor(length, dtype=raw_scores.dtype, device=raw_scores.device)
        bp = ((5.0 + length) / 6.0) ** alpha if bp_type == "t5" else length ** alpha
        return raw_scores / bp

    return fn


def compute_merge_matrix_by_prefix_ids(prefix_ids: Tensor) -> Tensor:
    """``merge[b, to, from] = 1`` iff prefix ``from`` equals prefix ``to`` and ``to`` is the first
    (highest-ranked) member of its equivalence class."""
    eq = prefix_ids[:, :, None] == prefix_ids[:, None, :]
    while eq.dim() > 3:
        eq = eq.all(dim=-1)
    eq = eq.to(torch.int64)
    seen_before = torch.nn.functional.pad(eq.cumsum(dim=1)[:, :-1, :], (0, 0, 1, 0)) > 0
    return eq * (~seen_before).to(eq.dtype)


def _merge_prefixes(merge_matrix: Tensor, *, log_probs: Tensor) -> Tensor:
    m = merge_matrix.to(log_probs.dtype)
    transfer = m * log_probs[:, None, :] + (1 - m) * NEG_INF
    return torch.logsumexp(transfer, dim=-1)


class PrefixMerger:
    """Decides which live prefixes are equivalent and should pool their probability mass
    (reference: axlearn/common/decoding.py:286-337)."""

    def init_state(self, *, tokens: Tensor) -> Any:
        raise NotImplementedError(type(self))

    def compute(self, state: Any) -> Tensor:
        raise NotImplementedError(type(self))

    def update(self, *, tokens: Tensor, state: Any) -> Any:
        raise NotImplementedError(type(self))


# ------------------------------------------------------------------------------------------
# Stop conditions.
# ------------------------------------------------------------------------------------------


class StopDecodingCondition(Protocol):
    def __call__(self, *, index: Tensor, sequences: Tensor, prefix_len: Tensor) -> Tensor:
        """``index [B]`` (position just written), ``sequences [B, N, L]``, ``prefix_len [B]``
        -> bool ``[B, N]``: the row is complete."""


class StopOnSubsequence:
    """Stops when the decoded part of a sequence ends with any of ``stopping_seqs``."""

    def __init__(self, stopping_seqs: Sequence[Sequence[int]]):
        if not stopping_seqs or any(len(s) == 0 for s in stopping_seqs):
            raise ValueError("stopping sequences must be non-empty")
        self._seqs = [list(s) for s in stopping_seqs]
        self._longest = max(len(s) for s in self._seqs)
        # Right-aligned table [S, longest] with -1 = "matches anything".
        self._table = torch.full((len(self._seqs), self._longest), -1, dtype=torch.int64)
        for i, s in enumerate(self._seqs):
            self._table[i, self._longest - len(s):] = torch.tensor(s)
        self._lens = torch.tensor([len(s) for s in self._seqs], dtype=torch.int64)

    def __call__(self, *, index: Tensor, sequences: Tensor, prefix_len: Tensor) -> Tensor:
        dev = sequences.device
        table, lens = self._table.to(dev), self._lens.to(dev)
        b, n, length = sequences.shape
        # Window of the last `longest` tokens ending at `index`.
        offs = torch.arange(-self._longest + 1, 1, device=dev)
        pos = index.long()[:, None] + offs[None]                     # [B, W]
        in_range = pos >= 0
        window = torch.gather(sequences, 2, pos.clamp(0, length - 1)[:, None, :].expand(b, n, -1))  # [B, N, W]
        match = (window[:, :, None, :] == table[None, None]) | (table[None, None] < 0)
        match = match & (in_range[:, None, None, :] | (table[None, None] < 0))
        full = match.all(dim=-1)                                      # [B, N, S]
        # The whole stopping sequence must lie in the decoded part (after the prefix).
        decoded = (index.long() - prefix_len.long() + 1)[:, None, None] >= lens[None, None]
        return (full & decoded).any(dim=-1)


class StopOnMaxLength:
    """Stops rows once ``max_num_decodes`` tokens were generated after the prefix."""

    def __init__(self, max_num_decodes: int):
        self._max = max_num_decodes

    def __call__(self, *, index: Tensor, sequences: Tensor, prefix_len: Tensor) -> Tensor:
        done = (index.long() - prefix_len.long() + 1) >= self._max
        return done[:, None].expand(-1, sequences.shape[1])


class CompositeDecodingCondition:
    """Logical OR of several conditions."""

    def __init__(self, conditions: Sequence[StopDecodingCondition]):
        if not conditions:
            raise ValueError("at least one condition is required")
        self._conditions = list(conditions)

    def __call__(self, *, index, sequences, prefix_len) -> Tensor:
        out = None
        for c in self._conditions:
            r = c(index=index, sequences=sequences, prefix_len=prefix_len)
            out = r if out is None else (out | r)
        return out


# ------------------------------------------------------------------------------------------
# Sampling.
# ------------------------------------------------------------------------------------------


@dataclasses.dataclass
class SampleOutputs:
    sequences: Tensor      # int [B, num_decodes, max_decode_len]
    token_scores: Tensor   # float32 [B, num_decodes, max_decode_len]


def _categorical(key: Tensor, logits: Tensor) -> Tensor:
    """Gumbel-max sample along the last dim, reproducible from the key alone."""
    g = prng.generator(key, logits.device)
    u = torch.rand(logits.shape, generator=g, device=logits.device, dtype=torch.float32)
    gumbel = -torch.log((-torch.log(u.clamp_min(1e-20))).clamp_min(1e-20))
    return (logits.float() + gumbel).argmax(dim=-1)


def sample_decode(
    *,
    inputs: Tensor,
    time_step: Tensor,
    cache: Any,
    tokens_to_scores: Callable[[Tensor, Any], tuple[Tensor, Any]],
    stop_decoding_condition: StopDecodingCondition,
    num_decodes: int,
    prng_key: Tensor,
    max_decode_len: Optional[int] = None,
    pad_id: int = 0,
    input_token_scores: Optional[Tensor] = None,
    check_every: Optional[int] = None,
    loop: str = "python",
) -> SampleOutputs:
    """Samples ``num_decodes`` continuations per row.

    ``tokens_to_scores([B*N, 1] ids, cache) -> ([B*N, V] scores, cache)``; sampling
    probabilities are ``softmax(scores)`` (temperature / top-k / top-p live in the callable).
    """
    del loop
    b = inputs.shape[0]
    dev = inputs.device
    if inputs.shape[0] != time_step.shape[0]:
        raise ValueError(f"inputs.shape[0] ({inputs.shape[0]}) != time_step.shape[0] ({time_step.shape[0]})")
    max_len = (inputs.shape[1] if max_decode_len is None else max_decode_len) + 1
    if inputs.shape[1] > max_len:
        raise ValueError(f"inputs.shape[1] ({inputs.shape[1]}) > max_decode_len ({max_len})")
    sequences = torch.full((b, num_decodes, max_len), pad_id, dtype=torch.int64, device=dev)
    sequences[:, :, :inputs.shape[1]] = inputs[:, None, :]
    scores = torch.zeros((b, num_decodes, max_len), dtype=torch.float32, device=dev)
    if input_token_scores is not None:
        if input_token_scores.shape[1] >= max_len:
            raise ValueError(f"token_scores.shape[1] ({input_token_scores.shape[1]}) must be < {max_len}")
        scores[:, :, 1:1 + input_token_scores.shape[1]] = input_token_scores[:, None, :].float()
    stop = torch.zeros((b, num_decodes), dtype=torch.bool, device=dev)
    cur = time_step.long().clone()
    prefix_len = time_step.long() + 1
    flat_cache = vectorized_tree_map(lambda x: flatten_decoding_dim(add_decoding_dim(x, num_decodes)), cache)
    if check_every is None:
        check_every = 8 if dev.type == "cuda" else 1
    key = prng_key
    step = 0
    while True:
        if step % check_every == 0:
            live = (cur < max_len - 1) & ~stop.all(dim=1)
            if not bool(live.any()):
                break
        step += 1
        ids = torch.gather(sequences, 2, cur.clamp(max=max_len - 1)[:, None, None].expand(b, num_decodes, 1))
        flat_scores, flat_cache = tokens_to_scores(ids.reshape(b * num_decodes, 1), flat_cache)
        cand = flat_scores.reshape(b, num_decodes, -1).float()
        step_key, key = prng.split(key, 2)
        nxt = _categorical(step_key, cand)                                  # [B, N]
        logp = torch.gather(cand, 2, nxt[..., None]).squeeze(-1)
        nxt = torch.where(stop, torch.full_like(nxt, pad_id), nxt)
        logp = torch.where(stop, torch.zeros_like(logp), logp)
        nxt_index = cur + 1
        writable = (nxt_index <= max_len - 1)[:, None].expand(b, num_decodes)
        widx = nxt_index.clamp(max=max_len - 1)[:, None, None].expand(b, num_decodes, 1)
        old_tok = torch.gather(sequences, 2, widx).squeeze(-1)
        old_sc = torch.gather(scores, 2, widx).squeeze(-1)
        sequences.scatter_(2, widx, torch.where(writable, nxt, old_tok)[..., None])
        scores.scatter_(2, widx, torch.where(writable, logp, old_sc)[..., None])
        should_stop = stop_decoding_condition(
            index=nxt_index.clamp(max=max_len - 1), sequences=sequences, prefix_len=prefix_len)
        stop = stop | should_stop
        cur = nxt_index
    return SampleOutputs(sequences=sequences[:, :, 1:], token_scores=scores[:, :, 1:])


# ------------------------------------------------------------------------------------------
# Beam search.
# ------------------------------------------------------------------------------------------


@dataclasses.dataclass
class BeamSearchOutputs:
    sequences: Tensor       # finished (ending in EOS): int [B, num_decodes, max_decode_len]
    scores: Tensor          # float32 [B, num_decodes], length-normalised
    live_sequences: Tensor  # reached max length without EOS
    live_scores: Tensor     # float32 [B, num_decodes], no normalisation


def beam_search_decode(
    *,
    inputs: Tensor,
    time_step: Tensor,
    cache: Any,
    tokens_to_scores: Callable[[Tensor, Any], tuple[Tensor, Any]],
    eos_id: int,
    num_decodes: int,
    max_decode_len: Optional[int] = None,
    brevity_penalty: Optional[BrevityPenaltyFn] = None,
    pad_id: int = 0,
    prefix_merger: Optional[PrefixMerger] = None,
    loop: str = "python",
) -> BeamSearchOutputs:
    """Beam search with separate live and finished beams.

    ``tokens_to_scores`` must return log-probabilities.  Each step scores
    ``beam * vocab`` candidates per row, keeps the best ``2 * beam`` (so that ``beam`` live
    candidates survive even if half end in EOS), moves candidates ending in EOS to the finished
    set (length-normalised by ``brevity_penalty``) and keeps the best ``beam`` of each set.
    Within the prefix, the next token is forced to the given one.
    """
    del loop
    b = inputs.shape[0]
    dev = inputs.device
    beam = num_decodes
    max_len = (inputs.shape[1] if max_decode_len is None else max_decode_len) + 1
    bp = brevity_penalty or brevity_penalty_fn(alpha=0.0)
    cur = time_step.long().clone()
    live_seqs = torch.full((b, beam, max_len), pad_id, dtype=torch.int64, device=dev)
    live_seqs[:, :, :inputs.shape[1]] = inputs[:, None, :]
    # Only beam 0 is alive at the start, so that identical beams do not fill the top-k.
    live_scores = torch.full((b, beam), NEG_INF, dtype=torch.float32, device=dev)
    live_scores[:, 0] = 0.0
    fin_seqs = torch.full((b, beam, max_len), pad_id, dtype=torch.int64, device=dev)
    fin_scores = torch.full((b, beam), NEG_INF, dtype=torch.float32, device=dev)
    beam_cache = vectorized_tree_map(lambda x: add_decoding_dim(x, beam), cache)
    merger_state = prefix_merger.init_state(tokens=live_seqs) if prefix_merger is not None else None

    def done() -> bool:
        not_at_end = cur < max_len - 1
        # Best possible future score of a live beam vs worst kept finished score.
        best_live = bp(length=torch.tensor(float(max_len - 1), device=dev), raw_scores=live_scores.amax(dim=1))
        worst_fin = fin_scores.amin(dim=1)
        improvable = best_live > worst_fin
        return not bool((not_at_end & improvable).any())

    while not done():
        ids = torch.gather(live_seqs, 2, cur.clamp(max=max_len - 1)[:, None, None].expand(b, beam, 1))
        flat_cache = vectorized_tree_map(flatten_decoding_dim, beam_cache)
        flat_lp, flat_cache = tokens_to_scores(ids.reshape(b * beam, 1), flat_cache)
        new_cache = vectorized_tree_map(lambda x: unflatten_decoding_dim(x, b, beam), flat_cache)
        cand = flat_lp.reshape(b, beam, -1).float()
        vocab = cand.shape[-1]
        nxt_index = cur + 1
        row_active = nxt_index <= max_len - 1                       # [B]
        # Inside the prefix the given token is the only candidate.
        in_prefix = (nxt_index < inputs.shape[1]) & (
            torch.gather(inputs, 1, nxt_index.clamp(max=inputs.shape[1] - 1)[:, None]).squeeze(1) != pad_id)
        in_prefix = in_prefix & (nxt_index <= time_step.long())
        forced = torch.gather(inputs, 1, nxt_index.clamp(max=inputs.shape[1] - 1)[:, None]).squeeze(1)
        forced_mask = torch.full((b, vocab), NEG_INF, device=dev)
        forced_mask.scatter_(1, forced[:, None].clamp(0, vocab - 1), 0.0)
        cand = torch.where(in_prefix[:, None, None], forced_mask[:, None, :].expand(-1, beam, -1), cand)
        if prefix_merger is not None:
            merged = _merge_prefixes(prefix_merger.compute(merger_state), log_probs=live_scores)
            total = cand + merged[..., None]
        else:
            total = cand + live_scores[..., None]
        flat_total = total.reshape(b, beam * vocab)
        k2 = min(2 * beam, beam * vocab)
        top_scores, top_idx = flat_total.topk(k2, dim=1)
        top_beam = top_idx // vocab
        top_tok = top_idx % vocab
        top_seqs = _gather_beams(live_seqs, top_beam)
        widx = nxt_index.clamp(max=max_len - 1)[:, None, None].expand(b, k2, 1)
        top_seqs.scatter_(2, widx, top_tok[..., None])
        is_eos = top_tok == eos_id
        # Live candidates: non-EOS, best `beam`.
        live_cand = top_scores + is_eos.float() * NEG_INF
        new_live_scores, sel = live_cand.topk(beam, dim=1)
        new_live_seqs = _gather_beams(top_seqs, sel)
        new_live_beam = torch.gather(top_beam, 1, sel)
        new_beam_cache = _gather_beams(new_cache, new_live_beam)
        # Finished candidates: EOS ones, normalised, merged with the previous finished set.
        length = (nxt_index.float())[:, None]
        fin_cand = bp(length=length, raw_scores=top_scores) + (~is_eos).float() * NEG_INF
        all_fin_scores = torch.cat([fin_scores, fin_cand], dim=1)
        all_fin_seqs = torch.cat([fin_seqs, top_seqs], dim=1)
        new_fin_scores, fsel = all_fin_scores.topk(beam, dim=1)
        new_fin_seqs = _gather_beams(all_fin_seqs, fsel)
        # Rows that already reached the end keep their state.
        act = row_active[:, None]
        live_scores = torch.where(act, new_live_scores, live_scores)
        live_seqs = torch.where(act[..., None], new_live_seqs, live_seqs)
        fin_scores = torch.where(act, new_fin_scores, fin_scores)
        fin_seqs = torch.where(act[..., None], new_fin_seqs, fin_seqs)
        beam_cache = new_beam_cache
        if prefix_merger is not None:
            merger_state = _gather_beams(merger_state, new_live_beam)
            merger_state = prefix_merger.update(
                tokens=torch.gather(new_live_seqs, 2, widx[:, :beam]).squeeze(-1), state=merger_state)
        cur = nxt_index
    return BeamSearchOutputs(
        sequences=fin_seqs[:, :, 1:], scores=fin_scores,
        live_sequences=live_seqs[:, :, 1:], live_scores=live_scores)


# ------------------------------------------------------------------------------------------
# Glue to ``Decoder`` (used by ``DecodingLayer``).
# ------------------------------------------------------------------------------------------


def log_probs_from_logits(logits: Tensor, *, logits_modifier: Optional[Callable] = None) -> Tensor:
    lp = torch.log_softmax(logits.float(), dim=-1)
    if logits_modifier is not None:
        lp = torch.log_softmax(logits_modifier(lp), dim=-1)
    return lp


def _pad_to(prefix: Tensor, max_sequence_length: int, pad_id: int) -> Tensor:
    if prefix.shape[1] > max_sequence_length:
        raise ValueError(f"prefix length {prefix.shape[1]} exceeds max_sequence_length {max_sequence_length}")
    out = torch.full((prefix.shape[0], max_sequence_length), pad_id, dtype=prefix.dtype, device=prefix.device)
    out[:, :prefix.shape[1]] = prefix
    return out


def _cross_kwargs(cross_attention_data, cross_attention_logit_biases) -> dict:
    if cross_attention_data is None:
        return {}
    return dict(cross_attention_data=cross_attention_data, cross_attention_logit_biases=cross_attention_logit_biases)


def _decoder_step_fn(decoder, *, logits_modifier=None, cross_attention_data=None, cross_attention_logit_biases=None):
    expanded: dict = {}

    def cross(rows: int) -> dict:
        """Encoder outputs repeated per hypothesis: decoding runs ``[batch * num_decodes]`` rows."""
        if cross_attention_data is None:
            return {}
        if rows not in expanded:
            rep = rows // cross_attention_data.shape[0]
            bias = cross_attention_logit_biases
            expanded[rows] = _cross_kwargs(
                cross_attention_data.repeat_interleave(rep, dim=0),
                None if bias is None else bias.repeat_interleave(rep, dim=0))
        return expanded[rows]

    def tokens_to_scores(token_ids: Tensor, cache: Any):
        with torch.no_grad():
            states, out = decoder.extend_step(cached_states=cache, input_ids=token_ids, **cross(token_ids.shape[0]))
        return log_probs_from_logits(out["logits"][:, -1, :], logits_modifier=logits_modifier), states

    return tokens_to_scores


def sample_decode_with_decoder(decoder, *, input_batch: dict, num_decodes: int, max_sequence_length: int,
                               logits_modifier=None, stop_decoding_condition=None, prng_key=None,
                               temperature: float = 1.0, cross_attention_data=None,
                               cross_attention_logit_biases=None, **_unused) -> SampleOutputs:
    """Prefills the prompt in one pass, samples the first token from the last prompt position,
    then extends one token at a time (reference: axlearn/common/decoder.py:286-372)."""
    cfg = decoder.config
    prefix = input_batch["prefix"]
    if temperature != 1.0:
        from axlearn_b200.common import logit_modifiers

        scale = logit_modifiers.scale_by(temperature)
        logits_modifier = scale if logits_modifier is None else logit_modifiers.chain(scale, logits_modifier)
    input_ids = _pad_to(prefix, max_sequence_length, cfg.pad_token_id)
    prefill_len = infer_initial_time_step(prefix, pad_id=cfg.pad_token_id) + 1
    if cross_attention_data is None and prefix.is_cuda:
        fast = _sample_decode_on_engine(
            decoder, input_ids=input_ids, prefill_len=prefill_len, num_decodes=num_decodes,
            max_sequence_length=max_sequence_length, logits_modifier=logits_modifier,
            stop_decoding_condition=stop_decoding_condition, prng_key=prng_key)
        if fast is not None:
            return fast
    with torch.no_grad():
        states, out = decoder.prefill_states(
            time_step=prefill_len.to(torch.int32), input_batch={**input_batch, "input_ids": input_ids},
            max_sequence_length=max_sequence_length,
            **_cross_kwargs(cross_attention_data, cross_attention_logit_biases))
        h = out["hidden_states"]
        last = torch.gather(h, 1, (prefill_len - 1).clamp(min=0)[:, None, None].expand(-1, 1, h.shape[-1]))
        logits = decoder.compute_logits({"hidden_states": last})
    lp = log_probs_from_logits(logits, logits_modifier=logits_modifier)[:, 0, :]
    key = prng_key if prng_key is not None else prng.PRNGKey(0)
    first_key, decode_key = prng.split(key, 2)
    first = _categorical(first_key, lp)
    b = input_ids.shape[0]
    rows = torch.arange(b, device=input_ids.device)
    can_write = prefill_len < input_ids.shape[1]
    input_ids = input_ids.clone()
    input_ids[rows[can_write], prefill_len[can_write]] = first[can_write].to(input_ids.dtype)
    init_scores = torch.zeros((b, max_sequence_length - 1), dtype=torch.float32, device=input_ids.device)
    ok = can_write & (prefill_len - 1 < init_scores.shape[1])
    init_scores[rows[ok], (prefill_len - 1)[ok]] = lp[rows, first][ok]
    return sample_decode(
        inputs=input_ids, time_step=prefill_len.clamp(max=max_sequence_length - 1), cache=states,
        tokens_to_scores=_decoder_step_fn(decoder, logits_modifier=logits_modifier,
                                          cross_attention_data=cross_attention_data,
                                          cross_attention_logit_biases=cross_attention_logit_biases),
        stop_decoding_condition=stop_decoding_condition or StopOnSubsequence([[cfg.eos_token_id]]),
        num_decodes=num_decodes, prng_key=decode_key, max_decode_len=max_sequence_length - 1,
        pad_id=cfg.pad_token_id, input_token_scores=init_scores)


def _sample_decode_on_engine(decoder, *, input_ids: Tensor, prefill_len: Tensor, num_decodes: int,
                             max_sequence_length: int, logits_modifier, stop_decoding_condition, prng_key):
    """The same sampling loop with the CUDA-graph decode engine as its ``tokens -> scores``
    function (paged KV cache inside the engine, one graph replay per token): used when the decoder
    is the Fuji shape the engine implements, on one GPU.  Returns None otherwise."""
    from axlearn_b200.inference import decode_engine

    cfg = decoder.config
    b = input_ids.shape[0]
    engine = decode_engine.engine_for_decoder(decoder, batch=b * num_decodes, max_len=max_sequence_length)
    if engine is None:
        return None
    longest = int(prefill_len.max().item())
    prompts = input_ids[:, :max(longest, 1)].repeat_interleave(num_decodes, dim=0)
    engine.prefill(prompts, lengths=prefill_len.repeat_interleave(num_decodes))
    logits = engine.logits[::num_decodes].clone()                       # one row per prompt
    lp = log_probs_from_logits(logits[:, None, :], logits_modifier=logits_modifier)[:, 0, :]
    key = prng_key if prng_key is not None else prng.PRNGKey(0)
    first_key, decode_key = prng.split(key, 2)
    first = _categorical(first_key, lp)
    rows = torch.arange(b, device=input_ids.device)
    can_write = prefill_len < input_ids.shape[1]
    input_ids = input_ids.clone()
    input_ids[rows[can_write], prefill_len[can_write]] = first[can_write].to(input_ids.dtype)
    init_scores = torch.zeros((b, max_sequence_length - 1), dtype=torch.float32, device=input_ids.device)
    ok = can_write & (prefill_len - 1 < init_scores.shape[1])
    init_scores[rows[ok], (prefill_len - 1)[ok]] = lp[rows, first][ok]

    def tokens_to_scores(token_ids: Tensor, cache: Any):
        step_logits = engine.step_logits(token_ids[:, 0])
        return log_probs_from_logits(step_logits[:, None, :], logits_modifier=logits_modifier)[:, 0, :], cache

    return sample_decode(
        inputs=input_ids, time_step=prefill_len.clamp(max=max_sequence_length - 1), cache={},
        tokens_to_scores=tokens_to_scores,
        stop_decoding_condition=stop_decoding_condition or StopOnSubsequence([[cfg.eos_token_id]]),
        num_decodes=num_decodes, prng_key=decode_key, max_decode_len=max_sequence_length - 1,
        pad_id=cfg.pad_token_id, input_token_scores=init_scores)


def beam_search_decode_with_decoder(decoder, *, input_batch: dict, num_decodes: int, max_sequence_length: int,
                                    brevity_penalty=None, cross_attention_data=None,
                                    cross_attention_logit_biases=None, **_unused) -> BeamSearchOutputs:
    """Prefills all prompt tokens except the last, then beam-searches from it (reference:
    axlearn/common/decoder.py:217-284)."""
    cfg = decoder.config
    prefix = input_batch["prefix"]
    input_ids = _pad_to(prefix, max_sequence_length, cfg.pad_token_id)
    time_step = infer_initial_time_step(prefix, pad_id=cfg.pad_token_id)
    with torch.no_grad():
        states, _ = decoder.prefill_states(
            time_step=time_step.to(torch.int32), input_batch={**input_batch, "input_ids": input_ids},
            max_sequence_length=max_sequence_length,
            **_cross_kwargs(cross_attention_data, cross_attention_logit_biases))
    return beam_search_decode(
        inputs=input_ids, time_step=time_step, cache=states,
        tokens_to_scores=_decoder_step_fn(decoder, cross_attention_data=cross_attention_data,
                                          cross_attention_logit_biases=cross_attention_logit_biases),
        eos_id=cfg.eos_token_id, num_decodes=num_decodes,
        max_decode_len=max_sequence_length - 1, brevity_penalty=brevity_penalty, pad_id=cfg.pad_token_id)
