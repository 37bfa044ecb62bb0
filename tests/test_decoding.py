"""Sampling / beam search / logit modifiers against brute-force references on CPU."""

import itertools
import math

import pytest
import torch

from axlearn_b200.common import decoding, logit_modifiers, prng


def _markov_scores(vocab, seed=0):
    """A first-order Markov LM: next-token log-probs depend on the current token only."""
    g = torch.Generator().manual_seed(seed)
    table = torch.log_softmax(torch.randn(vocab, vocab, generator=g) * 2.0, dim=-1)

    def tokens_to_scores(ids, cache):
        cache = dict(cache)
        cache["steps"] = cache["steps"] + 1
        return table[ids[:, 0]], cache

    return table, tokens_to_scores


def test_decoding_dim_helpers():
    x = torch.arange(6).reshape(2, 3)
    y = decoding.add_decoding_dim(x, 4)
    assert y.shape == (2, 4, 3) and torch.equal(y[:, 2], x)
    flat = decoding.flatten_decoding_dim(y)
    assert flat.shape == (8, 3)
    assert torch.equal(decoding.unflatten_decoding_dim(flat, 2, 4), y)
    assert decoding.add_decoding_dim(torch.tensor(3), 4).dim() == 0


def test_infer_initial_time_step():
    prefix = torch.tensor([[5, 0, 7, 0], [0, 0, 0, 0], [1, 2, 3, 4]])
    assert decoding.infer_initial_time_step(prefix, pad_id=0).tolist() == [2, 0, 3]


def test_brevity_penalty():
    raw = torch.tensor([[-6.0, -3.0]])
    t5 = decoding.brevity_penalty_fn(alpha=1.0, bp_type="t5")(length=torch.tensor(7.0), raw_scores=raw)
    assert torch.allclose(t5, raw / 2.0)
    hf = decoding.brevity_penalty_fn(alpha=2.0, bp_type="hf")(length=torch.tensor(3.0), raw_scores=raw)
    assert torch.allclose(hf, raw / 9.0)
    with pytest.raises(NotImplementedError):
        decoding.brevity_penalty_fn(bp_type="x")


def test_merge_matrix():
    ids = torch.tensor([[[1, 2], [3, 4], [1, 2], [3, 4], [5, 6]]])
    m = decoding.compute_merge_matrix_by_prefix_ids(ids)[0]
    expect = torch.zeros(5, 5, dtype=torch.int64)
    expect[0, 0] = expect[0, 2] = expect[1, 1] = expect[1, 3] = expect[4, 4] = 1
    assert torch.equal(m, expect)
    lp = torch.log(torch.tensor([[0.1, 0.2, 0.3, 0.1, 0.3]]))
    merged = decoding._merge_prefixes(m[None], log_probs=lp)  # pylint: disable=protected-access
    assert torch.allclose(merged[0, :2].exp(), torch.tensor([0.4, 0.3]), atol=1e-5)
    assert merged[0, 2] < -1e6


def test_stop_on_subsequence():
    cond = decoding.StopOnSubsequence([[7, 8], [9]])
    seqs = torch.tensor([[[1, 2, 7, 8, 0, 0], [1, 2, 3, 9, 0, 0], [1, 7, 8, 4, 0, 0]]])
    out = cond(index=torch.tensor([3]), sequences=seqs, prefix_len=torch.tensor([2]))
    assert out.tolist() == [[True, True, False]]
    # A match that lies (partly) inside the prefix does not count.
    out = cond(index=torch.tensor([3]), sequences=seqs, prefix_len=torch.tensor([3]))
    assert out.tolist() == [[False, True, False]]


def test_stop_on_max_length_and_composite():
    cond = decoding.CompositeDecodingCondition([decoding.StopOnMaxLength(2), decoding.StopOnSubsequence([[9]])])
    seqs = torch.zeros(2, 1, 6, dtype=torch.int64)
    seqs[1, 0, 2] = 9
    out = cond(index=torch.tensor([3, 2]), sequences=seqs, prefix_len=torch.tensor([2, 2]))
    assert out.tolist() == [[True], [True]]
    out = cond(index=torch.tensor([2, 1]), sequences=seqs, prefix_len=torch.tensor([2, 2]))
    assert out.tolist() == [[False], [False]]


def test_sample_decode_teacher_forcing_and_scores():
    vocab = 11
    table, fn = _markov_scores(vocab)
    inputs = torch.tensor([[1, 4, 6, 0, 0, 0], [1, 0, 0, 0, 0, 0]])
    time_step = torch.tensor([2, 0])
    out = decoding.sample_decode(
        inputs=inputs, time_step=time_step, cache={"steps": torch.zeros(2)}, tokens_to_scores=fn,
        stop_decoding_condition=decoding.StopOnSubsequence([[3]]), num_decodes=3, prng_key=prng.PRNGKey(1),
        max_decode_len=8, pad_id=0)
    assert out.sequences.shape == (2, 3, 8)
    # The prefix (minus the dropped first token) is preserved.
    assert (out.sequences[0, :, :2] == torch.tensor([4, 6])).all()
    full = torch.cat([inputs[:, None, :1].expand(-1, 3, -1), out.sequences], dim=-1)
    for b in range(2):
        for n in range(3):
            stopped = False
            for t in range(int(time_step[b]) + 1, 9):
                tok, prev = int(full[b, n, t]), int(full[b, n, t - 1])
                if stopped:
                    assert tok == 0 and out.token_scores[b, n, t - 1] == 0
                    continue
                assert math.isclose(out.token_scores[b, n, t - 1].item(), table[prev, tok].item(), rel_tol=1e-5)
                stopped = tok == 3
    # Different decodes of a row are different samples (with overwhelming probability).
    assert not torch.equal(out.sequences[1, 0], out.sequences[1, 1]) or not torch.equal(out.sequences[1, 1], out.sequences[1, 2])


def test_sample_decode_is_reproducible_and_check_every_invariant():
    vocab = 7
    _, fn = _markov_scores(vocab, seed=3)
    kw = dict(inputs=torch.tensor([[1, 0, 0, 0]]), time_step=torch.tensor([0]), tokens_to_scores=fn,
              stop_decoding_condition=decoding.StopOnSubsequence([[2]]), num_decodes=2,
              prng_key=prng.PRNGKey(5), max_decode_len=10)
    a = decoding.sample_decode(cache={"steps": torch.zeros(1)}, check_every=1, **kw)
    b = decoding.sample_decode(cache={"steps": torch.zeros(1)}, check_every=4, **kw)
    assert torch.equal(a.sequences, b.sequences) and torch.equal(a.token_scores, b.token_scores)


def test_beam_search_matches_exhaustive_search():
    vocab, length, beam = 5, 4, 3
    eos = 2
    table, fn = _markov_scores(vocab, seed=7)
    inputs = torch.tensor([[1, 0, 0, 0, 0]])
    out = decoding.beam_search_decode(
        inputs=inputs, time_step=torch.tensor([0]), cache={"steps": torch.zeros(1)}, tokens_to_scores=fn,
        eos_id=eos, num_decodes=beam, max_decode_len=length)
    # Exhaustive: all sequences that end with their first EOS within `length` tokens.
    finished = []
    for n in range(1, length + 1):
        for body in itertools.product([t for t in range(vocab) if t != eos], repeat=n - 1):
            seq = list(body) + [eos]
            prev, score = 1, 0.0
            for t in seq:
                score += table[prev, t].item()
                prev = t
            finished.append((score, seq))
    finished.sort(key=lambda x: -x[0])
    # With beam 3 over a 5-token vocabulary the search is not exact in general, but the best
    # hypothesis of this model is found, scores are exact for the returned sequences, and they are
    # sorted.
    best_score, best_seq = finished[0]
    got = out.sequences[0, 0].tolist()
    assert got[:len(best_seq)] == best_seq and all(t == 0 for t in got[len(best_seq):])
    assert math.isclose(out.scores[0, 0].item(), best_score, rel_tol=1e-5)
    lookup = {tuple(s): sc for sc, s in finished}
    for j in range(beam):
        seq = out.sequences[0, j].tolist()
        if out.scores[0, j] < -1e6:
            continue
        seq = seq[:seq.index(eos) + 1]
        assert math.isclose(out.scores[0, j].item(), lookup[tuple(seq)], rel_tol=1e-5)
    assert (out.scores[0, :-1] >= out.scores[0, 1:]).all()


def test_beam_search_respects_prefix():
    vocab = 6
    _, fn = _markov_scores(vocab, seed=9)
    inputs = torch.tensor([[1, 4, 5, 0, 0, 0]])
    out = decoding.beam_search_decode(
        inputs=inputs, time_step=torch.tensor([2]), cache={"steps": torch.zeros(1)}, tokens_to_scores=fn,
        eos_id=2, num_decodes=2, max_decode_len=5)
    assert (out.live_sequences[0, :, :2] == torch.tensor([4, 5])).all()
    ok = out.scores[0] > -1e6
    assert (out.sequences[0, ok][:, :2] == torch.tensor([4, 5])).all()


def test_logit_modifiers():
    logits = torch.log(torch.tensor([[0.5, 0.25, 0.125, 0.125], [0.1, 0.2, 0.3, 0.4]]))
    out = logit_modifiers.top_p_logits(0.7)(logits)
    assert (out[0] > -1e6).tolist() == [True, True, False, False]
    assert (out[1] > -1e6).tolist() == [False, False, True, True]
    out = logit_modifiers.top_k_logits(3)(logits)
    assert (out[0] > -1e6).tolist() == [True, True, True, True]  # tie at the third value keeps both
    out = logit_modifiers.top_k_logits(3, break_ties="smallest_index")(logits)
    assert (out[0] > -1e6).tolist() == [True, True, True, False]
    assert torch.allclose(logit_modifiers.scale_by(2.0)(logits), logits / 2)
    with pytest.raises(ValueError):
        logit_modifiers.scale_by(1e-6)
    chained = logit_modifiers.chain(logit_modifiers.scale_by(0.5), logit_modifiers.top_k_logits(1))(logits)
    assert (chained > -1e6).sum(dim=-1).tolist() == [1, 1]
