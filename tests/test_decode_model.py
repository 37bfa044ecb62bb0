"""Incremental decoding through the model stack must agree with the full forward pass."""

import torch

from axlearn_b200.common import prng
from axlearn_b200.common.module import functional
from axlearn_b200.experiments.text.gpt import fuji


def _model(num_kv_heads=None):
    cfg = fuji.model_config(num_layers=2, hidden_dim=64, num_heads=4, num_kv_heads=num_kv_heads, vocab_size=97,
                            rope_theta=1e4, shared_lm_head=False, ffn_dim=128)
    model = cfg.set(name="model").instantiate(parent=None)
    params = model.initialize_parameters_recursively(prng.PRNGKey(0))
    return model, params


def _call(model, params, method, input_batch, **kwargs):
    out, _ = functional(model, prng.PRNGKey(1), params, dict(input_batch=input_batch, **kwargs),
                        is_training=False, method=method)
    return out


def test_greedy_sample_decode_matches_teacher_forced_argmax():
    model, params = _model(num_kv_heads=2)
    prefix = torch.tensor([[1, 17, 23, 5, 0, 0], [1, 9, 0, 0, 0, 0]])
    from axlearn_b200.common import logit_modifiers

    out = _call(model, params, "sample_decode", {"prefix": prefix}, num_decodes=1, max_sequence_length=12,
                logits_modifier=logit_modifiers.top_k_logits(1, break_ties="smallest_index"))
    seqs = out.sequences[:, 0]                       # [B, 11]: tokens 1.. of each row
    full = torch.cat([prefix[:, :1], seqs], dim=1)   # with the conditioning token back in front
    # Teacher-forced logits over the decoded sequence.
    logits = _call(model, params, "extract_logits", {"input_ids": full})
    plen = [4, 2]
    for b in range(2):
        stopped = False
        for t in range(plen[b], 12):
            if stopped:
                assert full[b, t] == 0
                continue
            assert full[b, t] == logits[b, t - 1].argmax(), (b, t)
            stopped = full[b, t] == 1   # eos id of the tiny config
    # Prefix preserved.
    assert full[0, :4].tolist() == [1, 17, 23, 5] and full[1, :2].tolist() == [1, 9]


def test_beam_search_top_beam_scores_are_consistent():
    model, params = _model()
    prefix = torch.tensor([[1, 11, 12, 0]])
    out = _call(model, params, "beam_search_decode", {"prefix": prefix}, num_decodes=3, max_sequence_length=8)
    assert out.live_sequences.shape == (1, 3, 7)
    live = torch.cat([prefix[:, :1], out.live_sequences[0, :1]], dim=1)
    logits = _call(model, params, "extract_logits", {"input_ids": live})
    lp = torch.log_softmax(logits.float(), dim=-1)
    score = sum(lp[0, t - 1, live[0, t]].item() for t in range(3, 8))
    assert abs(score - out.live_scores[0, 0].item()) < 1e-3 * max(1.0, abs(score))
