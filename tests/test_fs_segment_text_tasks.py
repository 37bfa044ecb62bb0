"""File-system functions, best-fit packing, MLM masking and T5 span corruption."""
import numpy as np
import pytest

from axlearn_b200.common import file_system as fs
from axlearn_b200.common import input_text_tasks as tt
from axlearn_b200.common.segment_tree import BestFitSegmentTree, SegmentTree, best_fit_pack


def test_file_system_local_and_registered_backend(tmp_path):
    d = str(tmp_path / "a" / "b")
    fs.makedirs(d)
    with fs.open(d + "/x.txt", "w") as f:
        f.write("hello")
    assert fs.readfile("file://" + d + "/x.txt") == "hello" and fs.isdir(d) and fs.listdir(d) == ["x.txt"]
    fs.copy(d + "/x.txt", d + "/y.txt")
    with pytest.raises(fs.OpError):
        fs.copy(d + "/x.txt", d + "/y.txt")
    fs.copy(d + "/x.txt", d + "/y.txt", overwrite=True)
    assert [p.rsplit("/", 1)[1] for p in fs.glob([d + "/*.txt"])] == ["x.txt", "y.txt"]
    fs.remove(d + "/y.txt")
    assert not fs.exists(d + "/y.txt")
    with pytest.raises(fs.NotFoundError):
        fs.readfile(d + "/missing")
    with pytest.raises(fs.OpError):
        fs.exists("s3://bucket/key")

    class Memory:
        files = {}

        def exists(self, path):
            return path in self.files

        def open(self, path, mode="r"):
            import io
            if "w" in mode:
                buf = io.BytesIO()
                files, key = self.files, path
                buf.close = lambda: files.__setitem__(key, buf.getvalue())
                return buf
            return io.BytesIO(self.files[path])

    fs.register_backend("mem", Memory())
    fs.copy(d + "/x.txt", "mem://copy")
    assert Memory.files["mem://copy"] == b"hello"
    fs.rmtree(str(tmp_path / "a"))
    assert not fs.exists(d)


def test_segment_tree_and_best_fit():
    t = SegmentTree(6, max, -1, values=[3, 1, 4, 1, 5, 9])
    assert t.reduce() == 9 and t.reduce(0, 4) == 4 and t.reduce(3, 4) == 1
    t.update(5, 0)
    assert t.reduce() == 5 and t.leftmost(0, lambda m: m >= 4) == 2 and t.leftmost(3, lambda m: m >= 4) == 4
    assert t.leftmost(0, lambda m: m >= 7) == -1
    b = BestFitSegmentTree(10)
    assert b.place(6) == (10, 4) and b.place(5) == (10, 5)
    assert b.place(4) == (4, 0)                                 # the tighter of the two open bins
    assert b.place(5) == (5, 0) and b.place(3) == (10, 7)
    bins = best_fit_pack([6, 5, 4, 5, 3, 7, 2], 10)
    assert bins == [[0, 2], [1, 3], [4, 5], [6]]
    rng = np.random.default_rng(0)
    lengths = rng.integers(1, 60, 500).tolist()
    packed = best_fit_pack(lengths, 64)
    assert sorted(i for b_ in packed for i in b_) == list(range(500))
    assert all(sum(lengths[i] for i in b_) <= 64 for b_ in packed)
    assert len(packed) <= 1.1 * sum(lengths) / 64 + 1           # close to the volume bound


def test_mlm_actions_and_mask():
    rng = np.random.default_rng(0)
    a = tt.iid_mlm_actions(20000, rng=rng)
    sel = a != tt.MLMAction.DO_NOTHING
    assert abs(sel.mean() - 0.15) < 0.01
    assert abs((a[sel] == tt.MLMAction.MASK).mean() - 0.8) < 0.03 and abs((a[sel] == tt.MLMAction.SWAP).mean() - 0.1) < 0.03
    ids = np.arange(5, 25)
    ids[0], ids[-1] = 1, 2                                       # CLS, SEP
    actions = np.full(20, tt.MLMAction.MASK)
    out = tt.apply_mlm_mask(ids, actions, mask_id=4, vocab_size=100, rng=rng, special_ids=(0, 1, 2))
    assert out["input_ids"][0] == 1 and out["input_ids"][-1] == 2 and (out["input_ids"][1:-1] == 4).all()
    assert out["target_labels"][0] == 0 and (out["target_labels"][1:-1] == ids[1:-1]).all()
    starts = np.array([1, 0, 0, 1, 1, 0, 1, 0, 0, 0, 1, 1], dtype=bool)
    ww = tt.whole_word_mlm_actions(starts, rng=rng, select_token_prob=0.4)
    word_id = np.cumsum(starts) - 1
    for w in range(word_id.max() + 1):
        assert len(set(ww[word_id == w])) == 1                  # a word is treated as a whole
    assert (ww != 0).any()


def test_t5_span_corruption_round_trips():
    rng = np.random.default_rng(1)
    mask = tt.random_spans_noise_mask(200, rng=rng)
    assert not mask[0] and abs(mask.sum() - 30) <= 1
    runs = np.flatnonzero(np.diff(np.concatenate([[0], mask.astype(int)])) == 1)
    assert abs(len(runs) - 10) <= 1
    ids = np.arange(100, 150)
    ex = tt.apply_t5_mask(ids, vocab_size=1000, rng=rng)
    src, tgt = ex["source_ids"], ex["target_ids"]
    assert tgt[-1] == 1 and tgt[0] == 999
    # Stitching the target's spans back into the source at their sentinels restores the input.
    spans, cur = {}, None
    for t in tgt[:-1]:
        if t >= 900:
            cur = int(t)
            spans[cur] = []
        else:
            spans[cur].append(int(t))
    rebuilt = []
    for s in src:
        rebuilt.extend(spans[int(s)] if s >= 900 else [int(s)])
    assert rebuilt == ids.tolist()
    ar = tt.make_t5_autoregressive_inputs(ex, max_source_len=64, max_target_len=24)
    assert ar["source"]["input_ids"].shape == (64,) and ar["target_labels"].shape == (24,)
    assert ar["target"]["input_ids"][0] == 0 and (ar["target"]["input_ids"][1:len(tgt)] == tgt[:-1][:23]).all()
