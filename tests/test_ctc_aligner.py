"""CTC forced alignment against brute force over all frame paths."""
import itertools

import torch

from axlearn_b200.audio.aligner import ctc_forced_alignment


def _collapse(path, blank=0):
    out, prev = [], None
    for p in path:
        if p != prev and p != blank:
            out.append(p)
        prev = p
    return out


def test_alignment_is_the_best_path_that_collapses_to_the_labels():
    torch.manual_seed(0)
    t, v = 6, 4
    log_pos = torch.log_softmax(torch.randn(3, t, v), dim=-1)
    labels = torch.tensor([[1, 2, -1], [3, 3, 1], [2, -1, -1]])
    frames = [6, 6, 4]
    paddings = torch.tensor([[0] * 6, [0] * 6, [0, 0, 0, 0, 1, 1]])
    out = ctc_forced_alignment(log_pos=log_pos, log_pos_paddings=paddings, labels=labels, label_paddings=labels < 0)
    for i in range(3):
        want = [int(x) for x in labels[i] if x >= 0]
        best, best_path = -1e9, None
        for path in itertools.product(range(v), repeat=frames[i]):
            if _collapse(path) != want:
                continue
            s = sum(float(log_pos[i, f, p]) for f, p in enumerate(path))
            if s > best:
                best, best_path = s, path
        assert abs(float(out.alignment_score[i]) - best) < 1e-4
        got = out.alignment[i, :frames[i]].tolist()
        assert _collapse(got) == want
        assert abs(sum(float(log_pos[i, f, p]) for f, p in enumerate(got)) - best) < 1e-4
        assert (out.alignment[i, frames[i]:] == -1).all()
        idx = out.alignment_indices[i, :frames[i]]
        assert [want[j] for j in idx[idx >= 0].tolist()] == [p for p in got if p != 0]


def test_labels_that_do_not_fit_are_reported():
    log_pos = torch.log_softmax(torch.randn(1, 3, 4), dim=-1)
    labels = torch.tensor([[2, 2, 2]])                          # needs 5 frames (blanks between repeats)
    out = ctc_forced_alignment(log_pos=log_pos, log_pos_paddings=torch.zeros(1, 3), labels=labels, label_paddings=labels < 0)
    assert out.alignment_score[0] == float("-inf") and (out.alignment[0] == 0).all()


def test_decoder_model_align_and_typed_summaries(tmp_path):
    from axlearn_b200.audio.asr import CTCDecoderModel
    from axlearn_b200.common import prng
    from axlearn_b200.common.module import functional
    from axlearn_b200.common.summary import AudioSummary, CallbackSummary, ImageSummary
    from axlearn_b200.common.summary_writer import SummaryWriter

    model = CTCDecoderModel.default_config().set(name="ctc", input_dim=6, vocab_size=5).instantiate(parent=None)
    params = model.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    batch = dict(inputs=torch.randn(2, 7, 6), paddings=torch.zeros(2, 7), target_labels=torch.tensor([[1, 2, -1], [3, -1, -1]]))
    out, _ = functional(model, None, params, dict(input_batch=batch), is_training=False, method="align")
    assert out["alignment"].shape == (2, 7) and torch.isfinite(out["alignment_score"]).all()
    assert _collapse(out["alignment"][0].tolist()) == [1, 2] and _collapse(out["alignment"][1].tolist()) == [3]

    writer = SummaryWriter.default_config().set(name="w", dir=str(tmp_path)).instantiate(parent=None)
    writer(1, {"image": ImageSummary(torch.rand(2, 8, 8, 3)), "audio": AudioSummary(torch.rand(800) * 2 - 1, sample_rate=8000),
               "text": CallbackSummary(lambda ids: " ".join(str(int(i)) for i in ids), torch.tensor([4, 5])),
               "hist": torch.randn(16), "loss": torch.tensor(0.5)})
    writer.flush()
    import json
    row = json.loads((tmp_path / "summaries.jsonl").read_text().splitlines()[-1])
    assert row["text"] == "4 5" and row["loss"] == 0.5 and row["image"].startswith("<ImageSummary")
    import pytest
    with pytest.raises(ValueError):
        writer(2, {"bad": ImageSummary(torch.rand(8, 8))})


def test_alignment_to_segments_and_host_aligner():
    import numpy as np

    from axlearn_b200.audio.aligner import CtcAligner, alignment_to_segments

    seg = alignment_to_segments(torch.tensor([[0, 1, 1, 2, -1], [0, 0, 0, 0, 0], [3, 0, 3, 3, -1]]), blank_id=0)
    assert seg[0].tolist() == [[1, 3], [3, 4], [-1, -1], [-1, -1], [-1, -1]]
    assert seg[1].tolist() == [[-1, -1]] * 5
    assert seg[2].tolist() == [[0, 2], [2, 4], [-1, -1], [-1, -1], [-1, -1]]

    aligner = CtcAligner(vocab_size=4)
    rng = np.random.default_rng(0)
    logits = rng.normal(size=(8, 4)).astype(np.float32)
    truth = np.array([2, 2, 1], dtype=np.int32)
    # Make the intended path clearly the best one.
    path = [2, 2, 0, 2, 1, 1, 0, 0]
    for t, s in enumerate(path):
        logits[t, s] += 10
    log_post = logits - np.log(np.exp(logits).sum(-1, keepdims=True))
    got = aligner.align(log_post, truth)
    assert got.tolist() == path
    boundary = aligner.alignment_to_boundary(got, truth)
    assert boundary.tolist() == [[0, 3, 4], [3, 4, 8]]
    assert aligner.align(log_post[:2], np.array([1, 2, 3], dtype=np.int32)) is None     # too few frames
    import pytest as _pytest
    with _pytest.raises(ValueError):
        aligner.align(log_post, truth.astype(np.int64))
    with _pytest.raises(ValueError):
        aligner.alignment_to_boundary(got, np.array([1, 2], dtype=np.int32))
