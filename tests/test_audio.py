"""Audio stack: log-mel frontend, SpecAugment, subsampler, conformer, CTC model."""

import math

import pytest
import torch

from axlearn_b200.audio.asr import (
    ASREncoder,
    ASRModel,
    CTCDecoderModel,
    SpeechFeatureLayer,
    ctc_greedy_decode,
    ctc_prefix_beam_search,
)
from axlearn_b200.audio.conformer import ConformerLayer, LConvLayer
from axlearn_b200.audio.frontend import LogMelFrontend, linear_to_mel_weight_matrix
from axlearn_b200.audio.spectrum_augmenter import MaskSampler, SpectrumAugmenter
from axlearn_b200.audio.subsamplers import ConvSubSampler
from axlearn_b200.common import prng
from axlearn_b200.common.module import functional


def _run(layer, inputs, *, params=None, is_training=False, method="forward", seed=1):
    if params is None:
        params = layer.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    out, _ = functional(layer, prng.PRNGKey(seed), params, inputs, is_training=is_training, method=method)
    return out, params


def _frontend_cfg():
    return LogMelFrontend.default_config().set(
        name="frontend", num_filters=16, sample_rate=8000, frame_size_ms=25, hop_size_ms=10, mel_floor=1e-3)


def test_mel_matrix_and_frontend_find_a_tone():
    w = linear_to_mel_weight_matrix(num_filters=16, num_spectrogram_bins=129, sample_rate=8000,
                                    lower_edge_hertz=125, upper_edge_hertz=3800)
    assert w.shape == (129, 16) and (w >= 0).all() and w[0].sum() == 0
    assert (w.sum(dim=0) > 0).all()                           # every filter covers some bin
    peaks = w.argmax(dim=0)
    assert (peaks[1:] > peaks[:-1]).all()                     # centres increase with the filter index
    layer = _frontend_cfg().instantiate(parent=None)
    t = torch.arange(8000) / 8000.0
    low = torch.sin(2 * math.pi * 300 * t)[None] * 1000
    high = torch.sin(2 * math.pi * 3000 * t)[None] * 1000
    paddings = torch.zeros(1, 8000)
    lo, _ = _run(layer, dict(inputs=low, paddings=paddings))
    hi, _ = _run(layer, dict(inputs=high, paddings=paddings))
    assert lo["outputs"].shape == tuple(layer.output_shape(input_shape=[1, 8000]))
    assert lo["outputs"][0, :, :, 0].mean(dim=0).argmax() < hi["outputs"][0, :, :, 0].mean(dim=0).argmax()
    # Frames that reach into the padded tail are padding and zeroed.
    paddings[0, 4000:] = 1
    half, _ = _run(layer, dict(inputs=low, paddings=paddings))
    n_live = int((1 - half["paddings"]).sum())
    assert 0 < n_live < half["paddings"].shape[1]
    assert half["outputs"][0, n_live:].abs().sum() == 0
    torch.testing.assert_close(half["outputs"][0, :n_live], lo["outputs"][0, :n_live])


def test_spec_augment_masks_only_in_training():
    cfg = SpectrumAugmenter.default_config().set(
        name="aug",
        freq_mask_sampler=MaskSampler.default_config().set(max_num_masks=2, max_mask_length=3),
        time_mask_sampler=MaskSampler.default_config().set(max_num_masks_ratio=0.1, max_mask_length_ratio=0.1))
    layer = cfg.instantiate(parent=None)
    x = torch.ones(3, 50, 16, 1)
    paddings = torch.zeros(3, 50)
    paddings[2, 30:] = 1
    same, _ = _run(layer, dict(inputs=x, paddings=paddings), is_training=False)
    assert torch.equal(same, x)
    out, _ = _run(layer, dict(inputs=x, paddings=paddings), is_training=True)
    masked = 1 - out[..., 0]
    assert 0 < masked.sum() < masked.numel() * 0.6
    # Masks are whole rows (time) or whole columns (frequency).
    rows = masked.amin(dim=2)               # frames masked at every frequency
    cols = masked.amin(dim=1)
    rebuilt = torch.clamp(rows[:, :, None] + cols[:, None, :], max=1)
    assert torch.equal(rebuilt, masked)
    assert cols.sum(dim=1).max() <= 6       # at most 2 masks of width <= 3
    out2, _ = _run(layer, dict(inputs=x, paddings=paddings), is_training=True, seed=7)
    assert not torch.equal(out, out2)


def test_subsampler_shapes_and_paddings():
    layer = ConvSubSampler.default_config().set(name="sub", output_dim=8).instantiate(parent=None)
    x = torch.randn(2, 40, 16, 1)
    paddings = torch.zeros(2, 40)
    paddings[1, 20:] = 1
    out, _ = _run(layer, dict(inputs=x, paddings=paddings))
    assert out["outputs"].shape == (2, 10, 4, 8) == tuple(layer.output_shape(input_shape=[2, 40, 16, 1]))
    assert out["paddings"].shape == (2, 10) and out["paddings"][0].sum() == 0
    live = int((1 - out["paddings"][1]).sum())
    assert 4 <= live <= 6 and out["outputs"][1, live:].abs().sum() == 0


def test_conformer_layer_ignores_padded_frames():
    layer = ConformerLayer.default_config().set(name="conf", input_dim=32, num_heads=4).instantiate(parent=None)
    x = torch.randn(2, 12, 32)
    paddings = torch.zeros(2, 12)
    paddings[1, 7:] = 1
    out, params = _run(layer, dict(inputs=x, paddings=paddings))
    assert out.shape == x.shape and out[1, 7:].abs().sum() == 0
    x2 = x.clone()
    x2[1, 7:] = 99.0                        # garbage in the padded tail changes nothing
    out2, _ = _run(layer, dict(inputs=x2, paddings=paddings), params=params)
    torch.testing.assert_close(out2[1, :7], out[1, :7], rtol=1e-4, atol=1e-5)
    # Limited context: frame 0 does not see frame 5 when right_context = 2.
    local = ConformerLayer.default_config().set(name="conf", input_dim=32, num_heads=4, left_context=2,
                                                right_context=2).instantiate(parent=None)
    bias = local._attention_bias(paddings, torch.float32)  # pylint: disable=protected-access
    assert bias[0, 0, 0, 5] < -1e8 and bias[0, 0, 0, 2] == 0
    lconv = LConvLayer.default_config().set(name="lconv", input_dim=32).instantiate(parent=None)
    y, _ = _run(lconv, dict(inputs=x, paddings=paddings))
    assert y.shape == x.shape


def test_ctc_decoding_helpers():
    v = 4
    path = [0, 1, 1, 0, 1, 2, 2, 0]
    logits = torch.full((1, 8, v), -5.0)
    for t, tok in enumerate(path):
        logits[0, t, tok] = 5.0
    assert ctc_greedy_decode(logits, torch.zeros(1, 8)) == [[1, 1, 2]]
    pads = torch.zeros(1, 8)
    pads[0, 4:] = 1
    assert ctc_greedy_decode(logits, pads) == [[1]]
    beams = ctc_prefix_beam_search(torch.log_softmax(logits[0], dim=-1), beam_size=3)
    assert beams[0][0] == [1, 1, 2] and beams[0][1] > beams[1][1]
    # Mass of paths that collapse to the same labels is merged: two frames, P(a) = 0.4 each frame,
    # P(blank) = 0.6: "a" can be a-, -a, aa = 0.24 + 0.24 + 0.16 = 0.64 > blank-only 0.36.
    lp = torch.log(torch.tensor([[0.6, 0.4], [0.6, 0.4]]))
    best = ctc_prefix_beam_search(lp, beam_size=2)
    assert best[0][0] == [1] and math.exp(best[0][1]) == pytest.approx(0.64, abs=1e-6)


def _asr_model():
    feature = SpeechFeatureLayer.default_config().set(
        frontend=_frontend_cfg(), augmenter=None, subsampler=ConvSubSampler.default_config().set(hidden_dim=4))
    enc = ASREncoder.default_config().set(dim=32, feature=feature.set(output_dim=4), feature_dim=4 * 4)
    enc.context.context.set(num_layers=1)
    enc.context.context.layer.set(num_heads=4)
    enc.context.context.layer.lconv.conv_norm.decay = 0.9
    dec = CTCDecoderModel.default_config().set(input_dim=32, vocab_size=6)
    return ASRModel.default_config().set(name="asr", encoder=enc, decoder=dec).instantiate(parent=None)


def test_asr_model_learns_a_tiny_mapping():
    """Two 'words' (a low and a high tone): a few steps of Adam separate them."""
    model = _asr_model()
    t = torch.arange(4000) / 8000.0
    wave = torch.stack([torch.sin(2 * math.pi * 300 * t), torch.sin(2 * math.pi * 2500 * t)]) * 1000
    batch = {"inputs": wave, "paddings": torch.zeros(2, 4000), "target_labels": torch.tensor([[1, 2, -1], [3, -1, -1]])}
    params = model.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    from axlearn_b200.common.utils import flatten_items

    leaves = [t_.requires_grad_() for p_, t_ in flatten_items(params) if "moving_" not in p_]
    opt = torch.optim.Adam(leaves, lr=5e-3)
    losses = []
    for step in range(200):
        (loss, aux), oc = functional(model, prng.PRNGKey(step), params, dict(input_batch=batch), is_training=True)
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(loss.item())
        # Batch-norm statistics travel as state updates (here through the stacked conformer layers).
        flat_params = dict(flatten_items(params))
        updates = flatten_items(oc.state_updates)
        assert any(p.endswith("conv_norm/moving_mean") for p, _ in updates)
        with torch.no_grad():
            for path, value in updates:
                flat_params[path].copy_(value)
    assert losses[-1] < 0.1 * losses[0], (losses[0], losses[-1])
    with torch.no_grad():
        decoded, _ = functional(model, prng.PRNGKey(0), params, dict(input_batch=batch), is_training=False,
                                method="greedy_decode")
        beams, _ = functional(model, prng.PRNGKey(0), params, dict(input_batch=batch), is_training=False,
                              method="beam_search_decode")
    assert decoded == [[1, 2], [3]]
    assert [b[0][0] for b in beams] == [[1, 2], [3]]
