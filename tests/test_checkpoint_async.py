"""Asynchronous, bounded, data-sharded checkpoint writes; commit across processes without a collective."""

import json
import os
import threading
import time

import numpy as np
import torch

from axlearn_b200.common import checkpointer as ck
from axlearn_b200.common.checkpointer import TensorStoreStateStorage, read_index_file, read_state_tensors


def _state():
    torch.manual_seed(0)
    return {"a": torch.randn(64, 32), "b": {"c": torch.randn(16, 8).to(torch.bfloat16), "step": torch.tensor(7)},
            "d": torch.arange(24, dtype=torch.int32).reshape(2, 3, 4)}


def test_single_process_save_is_async_and_bounded(tmp_path):
    cfg = TensorStoreStateStorage.default_config().set(max_concurrent_gb=4096 / (1 << 30))  # 4 KiB
    storage = cfg.instantiate()
    state = _state()
    d = str(tmp_path / "step_00000001")
    storage.save_to_dir(step=1, state=state, ckpt_dir=d)
    storage.wait_until_finished()
    assert dict(read_index_file(d))["step"] == 1
    back = read_state_tensors(d)
    assert torch.equal(back["a"], state["a"]) and torch.equal(back["b/c"], state["b"]["c"])
    # "a" alone (8 KiB) exceeds the 4 KiB budget: it is admitted only when nothing else is staged.
    assert storage.peak_staged_bytes <= max(64 * 32 * 4, 4096)


def test_data_shard_rule():
    # 4 holders, every holder writes a quarter of dim 0.
    assert ck._data_shard((8, 6), 4, 2, -1) == (0, 4, 2)
    # dim 0 is not divisible by 4, dim 1 is.
    assert ck._data_shard((6, 8), 4, 3, -1) == (1, 4, 3)
    # degree capped at 2: holders 2 and 3 write nothing.
    assert ck._data_shard((8, 8), 4, 1, 2) == (0, 2, 1)
    assert ck._data_shard((8, 8), 4, 3, 2) is None
    # nothing divisible by 4 or 3, fall back to 2; then to the first holder alone.
    assert ck._data_shard((2, 5), 4, 1, -1) == (0, 2, 1)
    assert ck._data_shard((5, 7), 4, 0, -1) == (0, 1, 0) and ck._data_shard((5, 7), 4, 1, -1) is None
    # switched off: only the first holder writes.
    assert ck._data_shard((8, 8), 4, 0, None) == (0, 1, 0) and ck._data_shard((8, 8), 4, 1, None) is None


def test_multi_process_commit_by_markers(tmp_path, monkeypatch):
    """Three "processes" (threads with patched rank) write slices of replicated arrays; process 0
    writes the index only after every marker exists; no collective is issued from the threads."""
    d = str(tmp_path / "step_00000005")
    os.makedirs(d)
    state = _state()
    nproc = 3
    tls = threading.local()
    monkeypatch.setattr(ck.coll, "process_index", lambda: getattr(tls, "rank", 0))
    monkeypatch.setattr(ck.coll, "process_count", lambda: nproc)
    monkeypatch.setattr(ck.coll, "barrier", lambda *a, **k: None)
    storages = []
    started = []

    def proc(rank, delay):
        tls.rank = rank
        time.sleep(delay)
        st = TensorStoreStateStorage.default_config().set(max_data_shard_degree=-1, timeout_secs=30).instantiate()
        storages.append(st)
        t0 = time.time()
        st.save_to_dir(step=5, state=state, ckpt_dir=d)
        started.append(time.time() - t0)
        # The commit thread inherits no thread-local: give it the rank through the closure above.
        st.wait_until_finished()

    # The commit runs on a helper thread of each storage: make process_index work there too.
    ranks_by_thread = {}
    orig_thread = threading.Thread

    class RankThread(orig_thread):
        def __init__(self, *a, **k):
            super().__init__(*a, **k)
            self._rank = getattr(tls, "rank", 0)

        def run(self):
            tls.rank = self._rank
            super().run()

    monkeypatch.setattr(ck.threading, "Thread", RankThread)
    threads = [orig_thread(target=proc, args=(r, 0.3 if r == 2 else 0.0)) for r in range(nproc)]
    for t in threads:
        t.start()
    time.sleep(0.15)
    assert not os.path.exists(os.path.join(d, "index"))  # process 2 has not written yet
    for t in threads:
        t.join()
    assert dict(read_index_file(d))["step"] == 5
    assert not [n for n in os.listdir(d) if n.startswith(".done.")]
    back = read_state_tensors(d)
    for key, want in (("a", state["a"]), ("b/c", state["b"]["c"]), ("d", state["d"]), ("b/step", state["b"]["step"])):
        assert torch.equal(back[key], want), key
    # "a" [64, 32] was written as three?  64 % 3 != 0 and 32 % 3 != 0 -> degree 2 along dim 0.
    meta = json.load(open(os.path.join(d, "gda", "a", ".zarray")))
    assert meta["chunks"] == [32, 32] and sorted(os.listdir(os.path.join(d, "gda", "a"))) == [".zarray", "0.0", "1.0"]
    # "d" [2, 3, 4]: 3 holders split dim 1.
    assert json.load(open(os.path.join(d, "gda", "d", ".zarray")))["chunks"] == [2, 1, 4]


def test_zarr_bytes_are_reader_independent(tmp_path):
    """The chunk files are raw C-order little-endian arrays described by ``.zarray``: check them
    with numpy alone, without this package's reader."""
    storage = TensorStoreStateStorage.default_config().instantiate()
    state = _state()
    d = str(tmp_path / "step_00000002")
    storage.save_to_dir(step=2, state=state, ckpt_dir=d)
    storage.wait_until_finished()
    for path, want in (("a", state["a"].numpy()), ("d", state["d"].numpy())):
        adir = os.path.join(d, "gda", path)
        meta = json.load(open(os.path.join(adir, ".zarray")))
        assert meta["zarr_format"] == 2 and meta["order"] == "C" and meta["compressor"] is None
        assert meta["shape"] == list(want.shape) and meta["chunks"] == list(want.shape)
        raw = open(os.path.join(adir, ".".join("0" for _ in want.shape)), "rb").read()
        got = np.frombuffer(raw, dtype=np.dtype(meta["dtype"])).reshape(meta["chunks"])
        np.testing.assert_array_equal(got, want)
    # bfloat16 is stored under the name TensorStore uses, two bytes per element.
    meta = json.load(open(os.path.join(d, "gda", "b", "c", ".zarray")))
    assert meta["dtype"] == "bfloat16"
    raw = open(os.path.join(d, "gda", "b", "c", "0.0"), "rb").read()
    assert len(raw) == 16 * 8 * 2
    bits = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
    np.testing.assert_array_equal(bits.view(np.float32).reshape(16, 8), state["b"]["c"].float().numpy())
    # Scalars: chunk file "0".
    assert os.path.exists(os.path.join(d, "gda", "b", "step", "0"))
    index = json.load(open(os.path.join(d, "index")))
    assert index[0] == ["step", 2] and ["a", {"dtype": "float32", "shape": "(64, 32)"}] in index
