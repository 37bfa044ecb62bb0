"""Composable, deterministic and checkpointable host input pipelines.

Covers the roles of the reference's two dataset stacks: axlearn/common/input_grain.py
(``sample_from_datasets`` :150, ``shard_dataset`` :192, ``prefetch_dataset`` :215, ``rekey`` :262,
``pad_for_evaluation`` :298, per-feed ``Input`` :583-763), axlearn/common/input_grain_lm.py
(windowed and streaming packing) and axlearn/common/input_tf_data.py (mixtures :845, batching
:560, eval padding :1290, ``Input`` :1420).

Design: every stage is an iterator object whose whole position is a small JSON-like ``state()``
that ``set_state`` restores exactly, so a checkpoint resumes the stream mid-epoch without
replaying it.  Random stages draw from counter-based generators (seed, epoch, index), never from
global state.  The last stage collates into pinned host tensors and, optionally, stays a few
batches ahead on a background thread so that the host never stalls the device.
"""

from __future__ import annotations

import bisect
import json
import os
import queue
import threading
from typing import Any, Callable, Iterable, Iterator, Optional, Sequence

import numpy as np
import torch

from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class, maybe_instantiate
from axlearn_b200.common.input_base import Input
from axlearn_b200.parallel.mesh import current_mesh


# ------------------------------------------------------------------------------------------
# Sources: random access by index.
# ------------------------------------------------------------------------------------------


class Source:
    def __len__(self) -> int:
        raise NotImplementedError(type(self))

    def __getitem__(self, index: int) -> dict:
        raise NotImplementedError(type(self))


class ListSource(Source):
    def __init__(self, items: Sequence[dict]):
        self._items = items

    def __len__(self):
        return len(self._items)

    def __getitem__(self, index):
        return self._items[index]


class RangeSource(Source):
    def __init__(self, n: int, key: str = "index"):
        self._n, self._key = n, key

    def __len__(self):
        return self._n

    def __getitem__(self, index):
        if not 0 <= index < self._n:
            raise IndexError(index)
        return {self._key: index}


class JsonLinesSource(Source):
    """One JSON object per line over one or more files; line offsets are indexed once."""

    def __init__(self, paths: Sequence[str]):
        self._paths = list(paths)
        self._offsets: list[np.ndarray] = []
        for p in self._paths:
            offs, pos = [], 0
            with open(p, "rb") as f:
                for line in f:
                    if line.strip():
                        offs.append(pos)
                    pos += len(line)
            self._offsets.append(np.asarray(offs, dtype=np.int64))
        self._starts = np.cumsum([0] + [len(o) for o in self._offsets])

    def __len__(self):
        return int(self._starts[-1])

    def __getitem__(self, index):
        f = bisect.bisect_right(self._starts, index) - 1
        with open(self._paths[f], "rb") as fh:
            fh.seek(int(self._offsets[f][index - self._starts[f]]))
            return json.loads(fh.readline())


class TokenFileSource(Source):
    """A flat binary file of token ids (memory-mapped) cut into fixed windows: the layout that
    pre-tokenised corpora use.  Example ``i`` = tokens ``[i * stride, i * stride + length]``."""

    def __init__(self, path: str, *, length: int, dtype: str = "uint16", stride: Optional[int] = None):
        self._tokens = np.memmap(path, dtype=np.dtype(dtype), mode="r")
        self._length, self._stride = length, stride or length
        self._n = max(0, (len(self._tokens) - length - 1) // self._stride + 1)

    def __len__(self):
        return self._n

    def __getitem__(self, index):
        lo = index * self._stride
        window = np.asarray(self._tokens[lo:lo + self._length + 1], dtype=np.int32)
        return {"input_ids": window[:-1], "target_labels": window[1:]}


class TFRecordSource(Source):
    """``tf.train.Example`` records of TFRecord files (the format of the reference's tfds datasets,
    axlearn/common/input_tf_data.py:204-330).  The frame offsets of every file are indexed once
    from the length headers, so access is random; ``features`` optionally maps a feature name to
    ``"bytes"`` / ``"str"`` / ``"int"`` / ``"float"`` (scalar: first value) -- unnamed features
    come back as the arrays / byte lists that ``tfrecord.decode_example`` produces."""

    def __init__(self, paths: Sequence[str], features: Optional[dict[str, str]] = None, *, check_crc: bool = False):
        import struct

        self._paths, self._features, self._check_crc = list(paths), features, check_crc
        self._offsets: list[np.ndarray] = []
        for p in self._paths:
            offs, pos, size = [], 0, os.path.getsize(p)
            with open(p, "rb") as f:
                while pos + 12 <= size:
                    f.seek(pos)
                    (length,) = struct.unpack("<Q", f.read(8))
                    offs.append(pos)
                    pos += 12 + length + 4
            if pos != size:
                raise ValueError(f"{p}: truncated TFRecord file")
            self._offsets.append(np.asarray(offs, dtype=np.int64))
        self._starts = np.cumsum([0] + [len(o) for o in self._offsets])

    def __len__(self):
        return int(self._starts[-1])

    def __getitem__(self, index):
        from axlearn_b200.common import tfrecord

        f = bisect.bisect_right(self._starts, index) - 1
        with open(self._paths[f], "rb") as fh:
            fh.seek(int(self._offsets[f][index - self._starts[f]]))
            record = next(tfrecord.read_tfrecords(fh, check_crc=self._check_crc))
        ex = tfrecord.decode_example(record)
        if self._features is None:
            return ex
        out = {}
        for name, kind in self._features.items():
            v = ex[name]
            if kind == "bytes":
                out[name] = v[0]
            elif kind == "str":
                out[name] = v[0].decode("utf-8")
            elif kind in ("int", "float"):
                out[name] = v[0].item()
            else:
                out[name] = v
        return out


class ParquetSource(Source):
    """Rows of parquet files through pyarrow (row groups are cached one at a time)."""

    def __init__(self, paths: Sequence[str], columns: Optional[Sequence[str]] = None):
        import pyarrow.parquet as pq

        self._files = [pq.ParquetFile(p) for p in paths]
        self._columns = list(columns) if columns else None
        counts = [f.metadata.row_group(g).num_rows for f in self._files for g in range(f.num_row_groups)]
        self._groups = [(f, g) for f in self._files for g in range(f.num_row_groups)]
        self._starts = np.cumsum([0] + counts)
        self._cached: tuple[int, Any] = (-1, None)

    def __len__(self):
        return int(self._starts[-1])

    def __getitem__(self, index):
        g = bisect.bisect_right(self._starts, index) - 1
        if self._cached[0] != g:
            f, rg = self._groups[g]
            self._cached = (g, f.read_row_group(rg, columns=self._columns).to_pylist())
        return self._cached[1][index - self._starts[g]]


# ------------------------------------------------------------------------------------------
# Stages.
# ------------------------------------------------------------------------------------------


class Stage:
    """An iterator with an exact, restorable position."""

    def __iter__(self):
        return self

    def __next__(self) -> Any:
        raise NotImplementedError(type(self))

    def state(self) -> dict:
        raise NotImplementedError(type(self))

    def set_state(self, state: dict) -> None:
        raise NotImplementedError(type(self))

    # Fluent composition.
    def map(self, fn: Callable[[Any], Any]) -> "Stage":
        return _Map(self, fn)

    def filter(self, fn: Callable[[Any], bool]) -> "Stage":
        return _Filter(self, fn)

    def batch(self, batch_size: int, *, drop_remainder: bool = True) -> "Stage":
        return _Batch(self, batch_size, drop_remainder)

    def unbatch(self) -> "Stage":
        return _Unbatch(self)

    def pack(self, *, length: int, keys: Sequence[str] = ("input_ids", "target_labels"), window: int = 64,
             method: str = "first_fit") -> "Stage":
        """``method``: ``first_fit`` (arrival order) or ``best_fit`` (tightest open row, found with a
        segment tree: fewer, fuller rows on long-tailed length distributions)."""
        return _Pack(self, length, tuple(keys), window, method)

    def prefetch(self, buffer_size: int = 4) -> "Stage":
        return _Prefetch(self, buffer_size)


class _Read(Stage):
    """Reads ``source`` in a per-epoch order: identity, or a seeded permutation; this process
    takes positions ``shard_index, shard_index + shard_count, ...`` of the order."""

    def __init__(self, source: Source, *, shuffle: bool, seed: int, num_epochs: Optional[int],
                 shard_index: int, shard_count: int):
        self._src, self._shuffle, self._seed = source, shuffle, seed
        self._epochs, self._si, self._sc = num_epochs, shard_index, shard_count
        self._epoch, self._pos = 0, shard_index
        self._perm: Optional[np.ndarray] = None
        self._perm_epoch = -1

    def _order(self) -> Optional[np.ndarray]:
        if not self._shuffle:
            return None
        if self._perm_epoch != self._epoch:
            rng = np.random.Generator(np.random.Philox(key=[self._seed, self._epoch]))
            self._perm, self._perm_epoch = rng.permutation(len(self._src)), self._epoch
        return self._perm

    def __next__(self):
        n = len(self._src)
        if n <= self._si:
            raise StopIteration
        while self._pos >= n:       # every epoch starts again at this shard's first position
            self._epoch += 1
            self._pos = self._si
        if self._epochs is not None and self._epoch >= self._epochs:
            raise StopIteration
        order = self._order()
        index = int(order[self._pos]) if order is not None else self._pos
        self._pos += self._sc
        return self._src[index]

    def state(self):
        return {"epoch": self._epoch, "pos": self._pos}

    def set_state(self, state):
        self._epoch, self._pos = int(state["epoch"]), int(state["pos"])


def read(source: Source, *, shuffle: bool = False, seed: int = 0, num_epochs: Optional[int] = 1,
         shard_index: int = 0, shard_count: int = 1) -> Stage:
    """``num_epochs=None`` repeats forever (a new permutation per epoch when shuffling)."""
    return _Read(source, shuffle=shuffle, seed=seed, num_epochs=num_epochs, shard_index=shard_index,
                 shard_count=shard_count)


class _Wrap(Stage):
    def __init__(self, parent: Stage):
        self._parent = parent

    def state(self):
        return {"parent": self._parent.state()}

    def set_state(self, state):
        self._parent.set_state(state["parent"])


class _Map(_Wrap):
    def __init__(self, parent, fn):
        super().__init__(parent)
        self._fn = fn

    def __next__(self):
        return self._fn(next(self._parent))


class _Filter(_Wrap):
    def __init__(self, parent, fn):
        super().__init__(parent)
        self._fn = fn

    def __next__(self):
        while True:
            x = next(self._parent)
            if self._fn(x):
                return x


def _stack(rows: Sequence[dict]) -> dict:
    out = {}
    for k in rows[0]:
        v0 = rows[0][k]
        out[k] = _stack([r[k] for r in rows]) if isinstance(v0, dict) else np.stack([np.asarray(r[k]) for r in rows])
    return out


class _Batch(_Wrap):
    def __init__(self, parent, batch_size, drop_remainder):
        super().__init__(parent)
        self._n, self._drop = batch_size, drop_remainder

    def __next__(self):
        rows = []
        for _ in range(self._n):
            try:
                rows.append(next(self._parent))
            except StopIteration:
                break
        if not rows or (self._drop and len(rows) < self._n):
            raise StopIteration
        return _stack(rows)


class _Unbatch(_Wrap):
    def __init__(self, parent):
        super().__init__(parent)
        self._rows: list = []
        self._i = 0

    def __next__(self):
        while self._i >= len(self._rows):
            b = next(self._parent)
            n = len(next(iter(b.values())))
            self._rows, self._i = [{k: v[j] for k, v in b.items()} for j in range(n)], 0
        self._i += 1
        return self._rows[self._i - 1]

    def state(self):
        # The current batch is re-read on restore: the parent's state before it plus an offset.
        raise NotImplementedError("unbatch is for evaluation streams and is not checkpointed")


class _Pack(_Wrap):
    """Windowed first-fit packing of variable-length examples into ``length``-token rows with
    ``input_segment_ids`` / ``input_positions``.  ``window`` examples are drawn at a time and every
    row is completed inside its window, so the position is restorable at window boundaries."""

    def __init__(self, parent, length, keys, window, method="first_fit"):
        super().__init__(parent)
        if method not in ("first_fit", "best_fit"):
            raise ValueError(f"unknown packing method {method}")
        self._len, self._keys, self._window, self._method = length, keys, window, method
        self._ready: list[dict] = []
        self._i = 0
        self._at_window: dict = parent.state()

    def _fill(self):
        self._at_window = self._parent.state()
        bins: list[list[dict]] = []
        room: list[int] = []
        if self._method == "best_fit":
            from axlearn_b200.common.segment_tree import best_fit_pack

            examples = []
            for _ in range(self._window):
                try:
                    examples.append(next(self._parent))
                except StopIteration:
                    break
            if not examples:
                raise StopIteration
            packed = best_fit_pack([len(ex[self._keys[0]]) for ex in examples], self._len)
            self._ready, self._i = [self._emit([examples[i] for i in b]) for b in packed], 0
            return
        for _ in range(self._window):
            try:
                ex = next(self._parent)
            except StopIteration:
                break
            n = min(len(ex[self._keys[0]]), self._len)
            for b, r in enumerate(room):
                if r >= n:
                    bins[b].append(ex)
                    room[b] -= n
                    break
            else:
                bins.append([ex])
                room.append(self._len - n)
        if not bins:
            raise StopIteration
        self._ready, self._i = [self._emit(b) for b in bins], 0

    def _emit(self, examples: list[dict]) -> dict:
        row = {k: np.zeros(self._len, dtype=np.int32) for k in self._keys}
        if "target_labels" in row:
            row["target_labels"][:] = -1
        seg = np.zeros(self._len, dtype=np.int32)
        pos = np.zeros(self._len, dtype=np.int32)
        at = 0
        for s, ex in enumerate(examples, start=1):
            n = min(len(ex[self._keys[0]]), self._len)
            for k in self._keys:
                row[k][at:at + n] = np.asarray(ex[k][:n])
            seg[at:at + n] = s
            pos[at:at + n] = np.arange(n)
            at += n
        row["input_segment_ids"], row["input_positions"] = seg, pos
        return row

    def __next__(self):
        if self._i >= len(self._ready):
            self._fill()
        self._i += 1
        return self._ready[self._i - 1]

    def state(self):
        return {"parent": self._at_window, "emitted": self._i}

    def set_state(self, state):
        self._parent.set_state(state["parent"])
        self._ready, self._i = [], 0
        if state["emitted"]:
            self._fill()
            self._i = int(state["emitted"])


class _Mixture(Stage):
    """Draws every element from child ``k`` with probability ``weights[k]``; draw ``i`` uses the
    generator keyed by (seed, i), so the sequence of choices depends on nothing else."""

    def __init__(self, children: Sequence[Stage], weights: Sequence[float], seed: int, stop_on_first_exhausted: bool):
        if len(children) != len(weights) or not children:
            raise ValueError("one weight per dataset")
        w = np.asarray(weights, dtype=np.float64)
        if (w < 0).any() or w.sum() <= 0:
            raise ValueError(f"invalid weights {weights}")
        self._children, self._cdf = list(children), np.cumsum(w / w.sum())
        self._seed, self._count, self._stop_first = seed, 0, stop_on_first_exhausted
        self._alive = [True] * len(children)

    def __next__(self):
        while any(self._alive):
            u = np.random.Generator(np.random.Philox(key=[self._seed, self._count])).random()
            self._count += 1
            k = min(int(np.searchsorted(self._cdf, u, side="right")), len(self._children) - 1)
            if not self._alive[k]:
                continue
            try:
                return next(self._children[k])
            except StopIteration:
                self._alive[k] = False
                if self._stop_first:
                    break
        raise StopIteration

    def state(self):
        return {"count": self._count, "alive": list(self._alive), "children": [c.state() for c in self._children]}

    def set_state(self, state):
        self._count, self._alive = int(state["count"]), list(state["alive"])
        for c, s in zip(self._children, state["children"]):
            c.set_state(s)


def sample_from_datasets(sources: Sequence[Stage], weights: Sequence[float], *, seed: int = 0,
                         stop_on_first_exhausted: bool = False) -> Stage:
    return _Mixture(sources, weights, seed, stop_on_first_exhausted)


class _Concat(Stage):
    def __init__(self, children):
        self._children, self._k = list(children), 0

    def __next__(self):
        while self._k < len(self._children):
            try:
                return next(self._children[self._k])
            except StopIteration:
                self._k += 1
        raise StopIteration

    def state(self):
        return {"k": self._k, "children": [c.state() for c in self._children]}

    def set_state(self, state):
        self._k = int(state["k"])
        for c, s in zip(self._children, state["children"]):
            c.set_state(s)


def concatenate(sources: Sequence[Stage]) -> Stage:
    return _Concat(sources)


class _PadForEval(_Wrap):
    """Batches an evaluation stream, padding the last batch (and, across processes, whole extra
    batches up to ``num_batches``) with zero rows; ``target_labels`` of padding rows are -1 so
    they carry no loss, and ``is_valid`` marks real rows."""

    def __init__(self, parent, per_feed_batch_size, num_batches):
        super().__init__(parent)
        self._n, self._total, self._done = per_feed_batch_size, num_batches, 0
        self._template: Optional[dict] = None

    def __next__(self):
        rows = []
        for _ in range(self._n):
            try:
                rows.append(next(self._parent))
            except StopIteration:
                break
        if rows:
            self._template = rows[0]
        if not rows and (self._total is None or self._done >= self._total or self._template is None):
            raise StopIteration
        real = len(rows)
        while len(rows) < self._n:
            pad = {k: np.zeros_like(np.asarray(v)) for k, v in self._template.items()}
            if "target_labels" in pad:
                pad["target_labels"] = pad["target_labels"] - 1
            rows.append(pad)
        self._done += 1
        batch = _stack(rows)
        batch["is_valid"] = np.arange(self._n) < real
        return batch

    def state(self):
        return {"parent": self._parent.state(), "done": self._done}

    def set_state(self, state):
        super().set_state(state)
        self._done = int(state["done"])


def pad_for_evaluation(ds: Stage, *, per_feed_batch_size: int, num_batches: Optional[int] = None) -> Stage:
    return _PadForEval(ds, per_feed_batch_size, num_batches)


def rekey(ds: Stage, key_map: dict[str, Optional[str]], *, default_value: Any = None,
          retain_original_inputs: bool = False) -> Stage:
    """``{new key: old key}``; a missing or ``None`` source gives ``default_value``."""

    def fn(ex: dict) -> dict:
        out = dict(ex) if retain_original_inputs else {}
        for new, old in key_map.items():
            out[new] = ex.get(old, default_value) if old is not None else default_value
        return out

    return ds.map(fn)


class _Prefetch(_Wrap):
    """Keeps up to ``buffer_size`` elements ready on a background thread.  ``state()`` is the
    parent's state *before* the next element this stage will return, so nothing in the buffer is
    lost on restore."""

    _END = object()

    def __init__(self, parent, buffer_size):
        super().__init__(parent)
        self._size = max(1, buffer_size)
        self._q: Optional[queue.Queue] = None
        self._thread: Optional[threading.Thread] = None
        self._stop = threading.Event()
        self._unplaced: Optional[dict] = None

    def _start(self):
        self._q = queue.Queue(maxsize=self._size)
        self._stop.clear()
        self._unplaced = None

        def work(q: queue.Queue, stop: threading.Event):
            while not stop.is_set():
                before = self._parent.state()
                try:
                    item = (before, next(self._parent))
                except StopIteration:
                    item = (before, self._END)
                except Exception as e:  # pylint: disable=broad-except
                    item = (before, e)
                placed = False
                while not stop.is_set():
                    try:
                        q.put(item, timeout=0.1)
                        placed = True
                        break
                    except queue.Full:
                        continue
                if not placed:      # stopped with an element in hand: the stream resumes before it
                    self._unplaced = before
                    return
                if item[1] is self._END or isinstance(item[1], Exception):
                    return

        self._thread = threading.Thread(target=work, args=(self._q, self._stop), daemon=True)
        self._thread.start()

    def _shutdown(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
            self._thread, self._q = None, None

    def __next__(self):
        if self._q is None:
            self._start()
        before, item = self._q.get()
        if item is self._END:
            self._shutdown()
            raise StopIteration
        if isinstance(item, Exception):
            self._shutdown()
            raise item
        return item

    def state(self):
        if self._q is None:
            return {"parent": self._parent.state()}
        # Drain: stop the worker, then the parent's own state minus what is still buffered is
        # exactly the ``before`` of the oldest buffered item (or the parent's state if empty).
        self._stop.set()
        self._thread.join()
        pending = []
        while True:
            try:
                pending.append(self._q.get_nowait())
            except queue.Empty:
                break
        st = pending[0][0] if pending else (self._unplaced or self._parent.state())
        self._thread, self._q = None, None
        self._parent.set_state(st)
        return {"parent": st}

    def set_state(self, state):
        self._shutdown()
        self._parent.set_state(state["parent"])

    def __del__(self):
        try:
            self._shutdown()
        except Exception:  # pylint: disable=broad-except
            pass


# ------------------------------------------------------------------------------------------
# The Input module.
# ------------------------------------------------------------------------------------------


def to_tensors(batch: dict, *, pin: Optional[bool] = None) -> dict:
    pin = torch.cuda.is_available() if pin is None else pin
    out = {}
    for k, v in batch.items():
        if isinstance(v, dict):
            out[k] = to_tensors(v, pin=pin)
            continue
        t = torch.from_numpy(np.ascontiguousarray(v)) if isinstance(v, np.ndarray) else torch.as_tensor(v)
        out[k] = t.pin_memory() if pin else t
    return out


class PipelineInput(Input):
    """``source(shard_index, shard_count) -> Stage`` of examples; this module batches per feed,
    prefetches and converts to (pinned) tensors.  The feed is this process's coordinate along the
    batch axes of the mesh unless ``num_feeds`` / ``feed_index`` are given."""

    @config_class
    class Config(Input.Config):
        source: Required[Any] = REQUIRED        # config or callable (shard_index, shard_count) -> Stage
        global_batch_size: Required[int] = REQUIRED
        is_training: bool = True
        prefetch: int = 4
        pad_for_eval_num_batches: Optional[int] = None
        num_feeds: Optional[int] = None
        feed_index: Optional[int] = None

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._stage: Optional[Stage] = None
        self._pending_state: Optional[dict] = None

    def _feeds(self) -> tuple[int, int]:
        cfg = self._config
        if cfg.num_feeds is not None:
            return cfg.num_feeds, cfg.feed_index or 0
        mesh = current_mesh()
        if mesh is None:
            return 1, 0
        axes = mesh.present_axes(("data", "expert", "fsdp"))
        return mesh.axis_size(axes), mesh.axis_index(axes)

    def _make_source(self) -> Callable[[int, int], Stage]:
        """``(shard_index, shard_count) -> Stage`` of examples; subclasses add per-example stages."""
        cfg = self._config
        return maybe_instantiate(cfg.source) if isinstance(cfg.source, InstantiableConfig) else cfg.source

    def _build(self) -> Stage:
        cfg = self._config
        feeds, index = self._feeds()
        if cfg.global_batch_size % feeds:
            raise ValueError(f"global batch {cfg.global_batch_size} is not divisible by {feeds} feeds")
        ds = self._make_source()(index, feeds)
        per_feed = cfg.global_batch_size // feeds
        if cfg.is_training:
            ds = ds.batch(per_feed, drop_remainder=True)
        else:
            ds = pad_for_evaluation(ds, per_feed_batch_size=per_feed, num_batches=cfg.pad_for_eval_num_batches)
        return ds.prefetch(cfg.prefetch) if cfg.prefetch else ds

    def dataset(self) -> Iterator[dict]:
        if self._stage is None:
            self._stage = self._build()
            if self._pending_state is not None:
                self._stage.set_state(self._pending_state)
                self._pending_state = None
        for batch in self._stage:
            yield to_tensors(batch)

    def get_state(self) -> dict:
        if self._stage is None:
            return self._pending_state or {}
        return self._stage.state()

    def set_state(self, state: dict) -> None:
        if not state:
            return
        if self._stage is None:
            self._pending_state = state
        else:
            self._stage.set_state(state)
