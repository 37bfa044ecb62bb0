"""Transducer loss against brute-force lattice sums; RNN-T and LAS decoder models."""
import itertools
import math

import torch

from axlearn_b200.audio import decoder_asr as da
from axlearn_b200.common import prng, transducer
from axlearn_b200.common.module import functional


def _brute_force(blank, y, t_len, u_len):
    """Sum over every monotone path of t_len blanks and u_len labels ending with a blank."""
    total = -math.inf
    for labels_at in itertools.combinations(range(t_len + u_len - 1), u_len):
        t = u = 0
        lp = 0.0
        for step in range(t_len + u_len - 1):
            if step in labels_at:
                lp += y[t][u]
                u += 1
            else:
                lp += blank[t][u]
                t += 1
        if t != t_len - 1 or u != u_len:
            continue
        lp += blank[t_len - 1][u_len]
        total = lp if total == -math.inf else max(total, lp) + math.log1p(math.exp(-abs(total - lp)))
    return total


def test_alignment_log_prob_matches_brute_force_with_ragged_lengths():
    torch.manual_seed(0)
    b, t, u = 3, 4, 3
    blank = -torch.rand(b, t, u + 1) * 2
    y = -torch.rand(b, t, u) * 2
    am_len = torch.tensor([4, 2, 3])
    lab_len = torch.tensor([3, 1, 0])
    got = transducer.log_prob_alignments(blank, y, am_lengths=am_len, label_lengths=lab_len)
    for i in range(b):
        want = _brute_force(blank[i].tolist(), y[i].tolist(), int(am_len[i]), int(lab_len[i]))
        assert abs(float(got[i]) - want) < 1e-4, (i, float(got[i]), want)


def test_log_prob_conventions_are_normalised():
    logits = torch.randn(5, 7)
    for fn in (transducer.classic_logits_to_log_probs(blank_id=2, blank_logit_bias=0.3),
               transducer.hat_logits_to_log_probs(blank_id=2, blank_logit_bias=-0.2)):
        out = fn(logits)
        total = out["log_prob_blank"].exp() + out["log_prob_tokens"].exp().sum(-1)
        torch.testing.assert_close(total, torch.ones(5), rtol=1e-5, atol=1e-5)
        full = transducer.log_probs_from_blank_and_tokens(out["log_prob_blank"], out["log_prob_tokens"], blank_id=2)
        torch.testing.assert_close(full.exp().sum(-1), torch.ones(5), rtol=1e-5, atol=1e-5)


def test_transducer_layer_loss_ignores_padding_and_has_gradients():
    cfg = transducer.Transducer.default_config().set(name="t", input_dim=6, vocab_size=5)
    cfg.logits_to_log_probs.blank_id = 0
    layer = cfg.instantiate(parent=None)
    params = layer.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    params = {"proj": {k: v.clone().requires_grad_(True) for k, v in params["proj"].items()}}
    am = torch.randn(2, 5, 6)
    lm = torch.randn(2, 4, 6)
    am_pad = torch.tensor([[0, 0, 0, 1, 1], [0, 0, 0, 0, 0]])
    lm_pad = torch.tensor([[0, 0, 0, 1], [0, 0, 1, 1]])
    labels = torch.tensor([[1, 3, 4, 0], [2, 4, 0, 0]])
    kw = dict(am_data=am, am_paddings=am_pad, lm_data=lm, lm_paddings=lm_pad, target_labels=labels)
    (loss, per), _ = functional(layer, None, params, kw, is_training=True)
    loss.backward()
    assert params["proj"]["weight"].grad.abs().sum() > 0
    # Same result when the padded region holds other data and when frames are chunked.
    am2, lm2 = am.clone(), lm.clone()
    am2[0, 3:] = 7.0
    lm2[1, 2:] = -3.0
    (loss2, per2), _ = functional(layer, None, params, dict(kw, am_data=am2, lm_data=lm2, frame_chunk=2), is_training=True)
    torch.testing.assert_close(per2["loss"], per["loss"], rtol=1e-5, atol=1e-5)
    # Example 0 alone, cut to its true size.
    (loss0, _), _ = functional(layer, None, params, dict(
        am_data=am[:1, :3], am_paddings=am_pad[:1, :3], lm_data=lm[:1, :3], lm_paddings=lm_pad[:1, :3],
        target_labels=labels[:1, :3]), is_training=True)
    torch.testing.assert_close(loss0, per["loss"][0], rtol=1e-5, atol=1e-5)
    assert per["is_valid_example"].all() and loss > 0


def _asr_batch(b=2, t=6, d=8, vocab=10):
    torch.manual_seed(1)
    labels = torch.tensor([[4, 5, 6, 2, -1], [7, 3, 2, -1, -1]])          # labels, EOS (2), padding
    ids = torch.tensor([[1, 4, 5, 6, 0], [1, 7, 3, 0, 0]])                # BOS (1), labels
    return dict(inputs=torch.randn(b, t, d), paddings=torch.tensor([[0] * 6, [0, 0, 0, 0, 1, 1]]).bool(),
                target_labels=labels, target=dict(input_ids=ids))


def test_transducer_decoder_model_trains_and_decodes_what_it_learnt():
    cfg = da.TransducerDecoderModel.default_config().set(name="rnnt", input_dim=8, vocab_size=10, lm_dim=12, joint_dim=16)
    cfg.prediction_network.emb_dim = 6
    model = cfg.instantiate(parent=None)
    params = model.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    from axlearn_b200.common.utils import flatten_items, tree_map
    params = tree_map(lambda p: p.clone().requires_grad_(True), params)
    leaves = [p for _, p in flatten_items(params)]
    opt = torch.optim.Adam(leaves, lr=0.03)
    batch = _asr_batch()
    first = None
    for _ in range(150):
        (loss, aux), _ = functional(model, prng.PRNGKey(1), params, [batch], is_training=True)
        first = first if first is not None else float(loss)
        opt.zero_grad()
        loss.backward()
        opt.step()
    assert float(loss) < 0.2 * first
    assert aux["per_example_loss"].shape == (2,)
    out, _ = functional(model, None, params, dict(input_batch=batch, max_decode_len=5), is_training=False, method="greedy_decode")
    assert out.sequences[0, 0, :3].tolist() == [4, 5, 6] and out.paddings[0, 0].tolist() == [False] * 3 + [True] * 2
    assert out.sequences[1, 0, :2].tolist() == [7, 3] and int((~out.paddings[1, 0]).sum()) == 2
    beams, _ = functional(model, None, params, dict(input_batch=batch, num_decodes=3, max_decode_len=5),
                          is_training=False, method="beam_search_decode")
    assert beams.sequences.shape == (2, 3, 5)
    assert beams.sequences[0, 0, :3].tolist() == [4, 5, 6] and beams.sequences[1, 0, :2].tolist() == [7, 3]
    assert (beams.scores[:, 0] >= beams.scores[:, 1]).all()
    # The merged beam score of the best hypothesis is close to the full alignment likelihood.
    assert float(beams.scores[0, 0]) <= 1e-3 and float(beams.scores[0, 0]) > -1.0


def test_map_label_sequences():
    x = torch.tensor([[0, 3, 3, 0, 3, 5, 9, 9]])
    ctc = da.map_label_sequences(x, remove_repeats=True, blank_id=0, pad_id=9)
    assert ctc["sequences"][0, :3].tolist() == [3, 3, 5] and int(ctc["lengths"]) == 3
    assert ctc["sequences"][0, 3:].tolist() == [9] * 5
    rnnt = da.map_label_sequences(x, remove_repeats=False, blank_id=0, pad_id=9)
    assert rnnt["sequences"][0, :4].tolist() == [3, 3, 3, 5] and rnnt["paddings"][0].tolist() == [False] * 4 + [True] * 4


def test_las_decoder_model_loss_and_decoding_respect_frame_paddings():
    cfg = da.LASDecoderModel.default_config().set(name="las", input_dim=8, vocab_size=10)
    cfg.decoder.set(dim=16, pad_token_id=0, eos_token_id=2)
    cfg.decoder.transformer.set(num_layers=1)
    cfg.decoder.transformer.layer.self_attention.attention.num_heads = 2
    cfg.decoder.transformer.layer.cross_attention.attention.num_heads = 2
    cfg.decoder.transformer.layer.feed_forward.hidden_dim = 32
    model = cfg.instantiate(parent=None)
    params = model.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    batch = _asr_batch()
    (loss, aux), _ = functional(model, prng.PRNGKey(1), params, [batch], is_training=False)
    assert torch.isfinite(loss) and aux["per_example_weight"].tolist() == [4.0, 3.0]
    noisy = dict(batch, inputs=batch["inputs"].clone())
    noisy["inputs"][1, 4:] = 50.0                                   # padded frames are not attended to
    (loss2, _), _ = functional(model, prng.PRNGKey(1), params, [noisy], is_training=False)
    torch.testing.assert_close(loss2, loss, rtol=1e-5, atol=1e-5)
    dec_batch = dict(inputs=batch["inputs"], paddings=batch["paddings"], prefix=torch.tensor([[1], [1]]))
    beams, _ = functional(model, None, params, dict(input_batch=dec_batch, num_decodes=2, max_decode_len=6),
                          is_training=False, method="beam_search_decode")
    assert beams.sequences.shape[:2] == (2, 2) and beams.paddings.dtype == torch.bool
    assert ((beams.sequences == 0) | ~beams.paddings).all()
    beams_noisy, _ = functional(model, None, params, dict(input_batch=dict(dec_batch, inputs=noisy["inputs"]),
                                                          num_decodes=2, max_decode_len=6),
                                is_training=False, method="beam_search_decode")
    assert torch.equal(beams_noisy.raw_sequences, beams.raw_sequences)
    samples, _ = functional(model, prng.PRNGKey(3), params, dict(input_batch=dec_batch, num_decodes=2, max_decode_len=6),
                            is_training=False, method="sample_decode")
    assert samples.sequences.shape[:2] == (2, 2) and torch.isfinite(samples.scores).all()
