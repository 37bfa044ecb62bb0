"""Logical <-> physical input dispatch and elastic (scale-down) input."""

import pytest
import torch

from axlearn_b200.common.elastic_input import ElasticInput, ElasticSpmdInputDispatcher
from axlearn_b200.common.input_dispatch import PHYSICAL_TO_LOGICAL_KEY, InputDispatcher, SpmdInputDispatcher
from axlearn_b200.common.input_fake import FakeLmInput


def _dispatcher(**kw):
    return InputDispatcher.default_config().set(name="d", **kw).instantiate(parent=None)


def test_logical_batch_not_divisible_by_feeds_round_trips():
    # 6 logical rows over 4 feeds: 3 logical feeds of 2 rows; every feed pads to 2 physical rows.
    feeds = [_dispatcher(global_logical_batch_size=6, num_physical_feeds=4, physical_feed_index=i) for i in range(4)]
    assert feeds[0].num_logical_feeds == 3 and feeds[0].feed_logical_batch_size == 2
    assert [f.logical_feed_index for f in feeds] == [0, 1, 2, None]
    assert [f.feed_read_config()["shard_index"] for f in feeds] == [0, 1, 2, 0]
    logical = torch.arange(6 * 3).reshape(6, 3)
    physical = []
    for i, f in enumerate(feeds):
        shard = f.feed_read_config()["shard_index"]
        rows = logical[shard * 2:(shard + 1) * 2]
        physical.append(f.logical_to_physical_batch({"x": rows, "meta": {"y": rows[:, 0]}}))
    # Per-feed view: the logical feeds return their rows, the padding feed returns nothing.
    assert feeds[1].physical_to_logical_batch(physical[1])["x"].equal(logical[2:4])
    assert feeds[3].physical_to_logical_batch(physical[3])["x"].shape[0] == 0
    # Global view: concatenating the feeds' physical batches gives back the logical batch.
    glob = {"x": torch.cat([p["x"] for p in physical]), "meta": {"y": torch.cat([p["meta"]["y"] for p in physical])},
            PHYSICAL_TO_LOGICAL_KEY: torch.cat([p[PHYSICAL_TO_LOGICAL_KEY] for p in physical])}
    out = feeds[0].physical_to_logical_batch(glob)
    assert out["x"].equal(logical) and out["meta"]["y"].equal(logical[:, 0])


def test_small_logical_batch_pads_to_one_row_per_feed():
    d = _dispatcher(global_logical_batch_size=2, num_physical_feeds=8, physical_feed_index=5,
                    logical_feed_indices=[1, 5])
    assert d.feed_physical_batch_size == 1 and d.logical_feed_index == 1
    p = d.logical_to_physical_batch({"x": torch.tensor([[7.0]])})
    assert p[PHYSICAL_TO_LOGICAL_KEY].tolist() == [1]
    shapes = d.logical_to_physical_shapes({"x": type("S", (), {"shape": (1, 1), "dtype": torch.float32})()})
    assert shapes["x"].shape == (1, 1) and shapes[PHYSICAL_TO_LOGICAL_KEY].shape == (1,)


def test_invalid_configurations_are_rejected():
    with pytest.raises(ValueError):
        _dispatcher(global_logical_batch_size=6, num_physical_feeds=4, physical_feed_index=0,
                    logical_feed_indices=[0, 0, 1])
    with pytest.raises(ValueError):
        _dispatcher(global_logical_batch_size=6, num_physical_feeds=4, physical_feed_index=4)
    with pytest.raises(ValueError):
        SpmdInputDispatcher.default_config().set(name="s", global_logical_batch_size=6, num_feeds=4,
                                                 feed_index=0).instantiate(parent=None)
    d = _dispatcher(global_logical_batch_size=4, num_physical_feeds=2, physical_feed_index=0)
    with pytest.raises(ValueError):
        d.logical_to_physical_batch({"x": torch.zeros(3, 1)})


def _elastic_cfg(num_slices, feed_index):
    return ElasticSpmdInputDispatcher.default_config().set(
        name="e", global_logical_batch_size=16, num_max_slices=4, feeds_per_slice=2, num_slices=num_slices,
        feed_index=feed_index)


def test_elastic_dispatcher_feed_arithmetic():
    full = _elastic_cfg(4, 3).instantiate(parent=None)
    assert not full.is_in_elastic_mode and full.step_batch_size == 2
    assert full.feed_read_config() == dict(num_shards=8, shard_index=3)
    # Two of four slices alive: 4 surviving feeds share 4 missing feeds -> 2 extra rows each, a
    # missing feed's batch (2 rows) is one mini-batch.
    d = _elastic_cfg(2, 1).instantiate(parent=None)
    assert d.is_in_elastic_mode and d.step_batch_size == 4
    assert d.elastic_feed_index == 5 and d.elastic_feed_mini_batch_index == 0
    # Three of four alive: 6 survivors share 2 missing feeds of 2 rows -> not evenly divisible.
    with pytest.raises(ValueError):
        _elastic_cfg(3, 0).instantiate(parent=None)
    with pytest.raises(ValueError):
        ElasticSpmdInputDispatcher.default_config().set(
            name="e", global_logical_batch_size=16, num_max_slices=2, feeds_per_slice=2, num_slices=3,
            feed_index=0).instantiate(parent=None)


@pytest.mark.parametrize("num_slices", [4, 2, 1])
def test_elastic_input_keeps_the_global_batch(num_slices):
    """The union of what the surviving processes step on is the batch of the full job."""
    source = FakeLmInput.default_config().set(global_batch_size=16, source_length=5, vocab_size=100, seed=3)
    full = next(iter(source.clone(name="full", num_feeds=1, feed_index=0).instantiate(parent=None).dataset()))
    want = sorted(tuple(r.tolist()) for r in full["input_ids"])
    rows = []
    alive = 2 * num_slices
    for feed in range(alive):
        inp = ElasticInput.default_config().set(
            name="elastic", input=source, dispatcher=_elastic_cfg(num_slices, feed)).instantiate(parent=None)
        batch = next(iter(inp.dataset()))
        assert batch["input_ids"].shape[0] == 16 // alive
        assert batch["target_labels"].shape[0] == 16 // alive
        rows += [tuple(r.tolist()) for r in batch["input_ids"]]
    assert sorted(rows) == want
