"""Composable input pipeline: determinism, sharding, mixtures, packing, eval padding, resume."""
import json

import numpy as np
import pytest
import torch

from axlearn_b200.common import input_pipeline as ip


def _take(stage, n):
    out = []
    for _ in range(n):
        try:
            out.append(next(stage))
        except StopIteration:
            break
    return out


def test_read_shuffles_per_epoch_and_shards_disjointly():
    src = ip.RangeSource(10)
    a = [x["index"] for x in ip.read(src, shuffle=True, seed=3, num_epochs=2)]
    assert sorted(a[:10]) == list(range(10)) and sorted(a[10:]) == list(range(10)) and a[:10] != a[10:]
    assert a == [x["index"] for x in ip.read(src, shuffle=True, seed=3, num_epochs=2)]
    parts = [[x["index"] for x in ip.read(src, shuffle=True, seed=3, shard_index=i, shard_count=3)] for i in range(3)]
    assert sorted(sum(parts, [])) == list(range(10)) and [len(p) for p in parts] == [4, 3, 3]
    assert [x["index"] for x in ip.read(ip.RangeSource(2), shard_index=2, shard_count=3)] == []


def test_every_stage_resumes_exactly():
    def build():
        a = ip.read(ip.RangeSource(50), shuffle=True, seed=1, num_epochs=None).map(lambda x: {"v": x["index"]})
        b = ip.read(ip.RangeSource(7, key="v"), num_epochs=None).filter(lambda x: x["v"] % 2 == 0)
        return ip.sample_from_datasets([a, b], [0.7, 0.3], seed=5).batch(4).prefetch(3)

    ref = [b["v"].tolist() for b in _take(build(), 12)]
    s = build()
    head = [b["v"].tolist() for b in _take(s, 5)]
    state = json.loads(json.dumps(s.state()))                     # JSON-serialisable
    tail_same_object = [b["v"].tolist() for b in _take(s, 7)]
    s2 = build()
    s2.set_state(state)
    tail = [b["v"].tolist() for b in _take(s2, 7)]
    assert head + tail == ref and head + tail_same_object == ref


def test_mixture_follows_weights_and_survives_exhaustion():
    a = ip.read(ip.ListSource([{"k": 0}] * 1000), num_epochs=None)
    b = ip.read(ip.ListSource([{"k": 1}] * 1000), num_epochs=None)
    ks = [x["k"] for x in _take(ip.sample_from_datasets([a, b], [3, 1], seed=0), 4000)]
    assert abs(np.mean(ks) - 0.25) < 0.03
    short = ip.read(ip.ListSource([{"k": 0}] * 3))
    long = ip.read(ip.ListSource([{"k": 1}] * 20))
    assert sum(x["k"] == 1 for x in ip.sample_from_datasets([short, long], [1, 1], seed=0)) == 20
    short = ip.read(ip.ListSource([{"k": 0}] * 3))
    long = ip.read(ip.ListSource([{"k": 1}] * 200))
    assert len(list(ip.sample_from_datasets([short, long], [1, 1], seed=0, stop_on_first_exhausted=True))) < 50
    assert [x["k"] for x in ip.concatenate([ip.read(ip.ListSource([{"k": 0}] * 2)), ip.read(ip.ListSource([{"k": 1}]))])] == [0, 0, 1]


def test_packing_keeps_examples_whole_and_marks_segments():
    rng = np.random.default_rng(0)
    docs = [{"input_ids": rng.integers(1, 99, n), "target_labels": rng.integers(1, 99, n)} for n in rng.integers(2, 9, 40)]
    rows = list(ip.read(ip.ListSource(docs)).pack(length=16, window=10))
    total = sum(len(d["input_ids"]) for d in docs)
    assert sum(int((r["input_segment_ids"] > 0).sum()) for r in rows) == total
    for r in rows:
        seg, pos = r["input_segment_ids"], r["input_positions"]
        live = seg > 0
        assert (r["target_labels"][~live] == -1).all() and (r["input_ids"][~live] == 0).all()
        starts = np.flatnonzero(np.diff(np.concatenate([[0], seg])) > 0)
        assert (pos[starts] == 0).all()
    assert len(rows) < len(docs) / 2                               # actually packs
    s = ip.read(ip.ListSource(docs)).pack(length=16, window=10)
    first = _take(s, 7)
    st = s.state()
    rest = list(s)
    s2 = ip.read(ip.ListSource(docs)).pack(length=16, window=10)
    s2.set_state(st)
    rest2 = list(s2)
    assert len(rest) == len(rest2) and all((a["input_ids"] == b["input_ids"]).all() for a, b in zip(rest, rest2))


def test_eval_padding_marks_invalid_rows_and_rekey():
    ds = ip.read(ip.ListSource([{"input_ids": np.arange(4) + i, "target_labels": np.arange(4) + i} for i in range(5)]))
    batches = list(ip.pad_for_evaluation(ds, per_feed_batch_size=2, num_batches=4))
    assert len(batches) == 4
    assert [b["is_valid"].tolist() for b in batches] == [[True, True], [True, True], [True, False], [False, False]]
    assert (batches[2]["target_labels"][1] == -1).all()
    out = list(ip.rekey(ip.read(ip.RangeSource(2)), {"x": "index", "y": None}, default_value=7))
    assert out == [{"x": 0, "y": 7}, {"x": 1, "y": 7}]


def test_file_sources(tmp_path):
    p = tmp_path / "a.jsonl"
    p.write_text("\n".join(json.dumps({"text": f"line {i}"}) for i in range(5)) + "\n")
    q = tmp_path / "b.jsonl"
    q.write_text(json.dumps({"text": "other"}) + "\n")
    src = ip.JsonLinesSource([str(p), str(q)])
    assert len(src) == 6 and src[3]["text"] == "line 3" and src[5]["text"] == "other"
    tok = tmp_path / "tokens.bin"
    np.arange(100, dtype=np.uint16).tofile(tok)
    ts = ip.TokenFileSource(str(tok), length=8)
    assert len(ts) == 12 and ts[1]["input_ids"].tolist() == list(range(8, 16)) and ts[1]["target_labels"][-1] == 16
    pa = pytest.importorskip("pyarrow")
    import pyarrow.parquet as pq
    pq.write_table(pa.table({"a": list(range(10)), "b": [str(i) for i in range(10)]}), tmp_path / "t.parquet", row_group_size=4)
    ps = ip.ParquetSource([str(tmp_path / "t.parquet")], columns=["a"])
    assert len(ps) == 10 and ps[9] == {"a": 9} and ps[0] == {"a": 0}


def test_pipeline_input_batches_per_feed_and_resumes():
    def source(shard_index, shard_count):
        return ip.read(ip.RangeSource(64), shuffle=True, seed=2, num_epochs=None,
                       shard_index=shard_index, shard_count=shard_count).map(
            lambda x: {"input_ids": np.full(4, x["index"], dtype=np.int32)})

    def make(feed):
        return ip.PipelineInput.default_config().set(
            name="in", source=source, global_batch_size=8, num_feeds=2, feed_index=feed, prefetch=2).instantiate(parent=None)

    a, b = make(0), make(1)
    ia, ib = iter(a.dataset()), iter(b.dataset())
    seen = []
    for _ in range(4):
        x, y = next(ia), next(ib)
        assert x["input_ids"].shape == (4, 4) and x["input_ids"].dtype == torch.int32
        seen += x["input_ids"][:, 0].tolist() + y["input_ids"][:, 0].tolist()
    assert sorted(seen) == sorted(set(seen)) and len(seen) == 32         # feeds are disjoint within the epoch
    state = a.get_state()
    want = [next(ia)["input_ids"][:, 0].tolist() for _ in range(3)]
    c = make(0)
    c.set_state(state)
    ic = iter(c.dataset())
    assert [next(ic)["input_ids"][:, 0].tolist() for _ in range(3)] == want
    ev = ip.PipelineInput.default_config().set(
        name="ev", source=lambda i, n: ip.read(ip.RangeSource(5), shard_index=i, shard_count=n).map(
            lambda x: {"target_labels": np.full(2, x["index"])}),
        global_batch_size=4, num_feeds=1, is_training=False, prefetch=0).instantiate(parent=None)
    batches = list(ev.dataset())
    assert len(batches) == 2 and batches[1]["is_valid"].tolist() == [True, False, False, False]


def test_best_fit_packing_uses_fewer_rows():
    rng = np.random.default_rng(3)
    docs = [{"input_ids": np.ones(n, dtype=np.int32), "target_labels": np.ones(n, dtype=np.int32)}
            for n in rng.integers(1, 33, 400)]
    first = list(ip.read(ip.ListSource(docs)).pack(length=32, window=100))
    best = list(ip.read(ip.ListSource(docs)).pack(length=32, window=100, method="best_fit"))
    tokens = sum(len(d["input_ids"]) for d in docs)
    assert sum(int((r["input_segment_ids"] > 0).sum()) for r in best) == tokens
    assert len(best) <= len(first) and len(best) <= 1.08 * tokens / 32 + 4
