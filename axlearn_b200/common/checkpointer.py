"""Checkpointing with the reference's on-disk layout.

Layout (a hard compatibility target; axlearn/common/checkpointer.py:60-63, 353-364, 494-608
and axlearn/common/array_serialization.py:153-166, 355-360 in the reference)::

    {dir}/step_{step:08d}/
        index                      JSON list of [path, value]; first entry ["step", N];
                                   tensors -> {"dtype": "float32", "shape": "(4096, 11008)"}
        gda/{path}/.zarray         zarr v2 metadata; chunk shape = shard shape
        gda/{path}/{i}.{j}...      one raw chunk per shard, named by dot-joined shard
                                   coordinates ("0" for scalars)
        python_{process}/{path}    serialized python savables (e.g. input iterator state)

``index`` is written last, after every process has finished its chunks, so a directory
without ``index`` is incomplete and ignored; garbage collection deletes ``index`` first.
Paths come from ``flatten_items(state, "/")`` (dict keys sorted, tuples by position,
NamedTuples by field name), e.g. ``learner/optimizer/1/0/mu/decoder/.../weight``.

Each process writes the shards it owns with replica id 0.  Saving copies device tensors to
pinned host memory (the only part that blocks training) and writes files on a background
thread; the next save waits for the previous one.  Restoring reads, for every leaf, only the
chunks that intersect the slice this rank needs under the *current* mesh, so a checkpoint
written on one mesh can be read on another.
"""

from __future__ import annotations

import ast
import json
import math
import os
import re
import shutil
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Any, Callable, NamedTuple, Optional, Sequence

import numpy as np
import torch

from axlearn_b200.common.config import (
    REQUIRED,
    Configurable,
    InstantiableConfig,
    Required,
    config_class,
    config_for_function,
)
from axlearn_b200.common.module import Module
from axlearn_b200.common.utils import TensorSpec, flatten_items, tree_map
from axlearn_b200.parallel import collectives as coll
from axlearn_b200.parallel.mesh import current_mesh

STEP_NUM_DIGITS = 8
STEP_PREFIX = "step"
_STEP_RE = re.compile(rf"{STEP_PREFIX}_(\d{{{STEP_NUM_DIGITS}}})")


class CheckpointValidationType(str):
    """How strictly the stored structure must match the restore target."""


EXACT = CheckpointValidationType("EXACT")
EXACT_UP_TO_DTYPE = CheckpointValidationType("EXACT_UP_TO_DTYPE")
CONTAINS_STATE = CheckpointValidationType("CONTAINS_STATE")
CONTAINS_STATE_UP_TO_DTYPE = CheckpointValidationType("CONTAINS_STATE_UP_TO_DTYPE")


def parse_step_from_dir(step_dir: str) -> int:
    m = _STEP_RE.fullmatch(os.path.basename(os.path.normpath(step_dir)))
    if not m:
        raise ValueError(f"Not a checkpoint step dir: {step_dir}")
    return int(m.group(1))


def build_step_dir(base_dir: str, *, step: int) -> str:
    if not 0 <= step < 10**STEP_NUM_DIGITS:
        raise ValueError(f"step must be in [0, 10^{STEP_NUM_DIGITS}): {step}")
    return os.path.join(base_dir, f"{STEP_PREFIX}_{step:0{STEP_NUM_DIGITS}d}")


def checkpoint_paths(base_dir: str) -> list[str]:
    """Committed (``index`` present) step dirs, oldest first."""
    if not os.path.isdir(base_dir):
        return []
    out = []
    for name in sorted(os.listdir(base_dir)):
        if _STEP_RE.fullmatch(name) and os.path.exists(os.path.join(base_dir, name, "index")):
            out.append(os.path.join(base_dir, name))
    return out


def latest_checkpoint_path(base_dir: str) -> Optional[str]:
    paths = checkpoint_paths(base_dir)
    return paths[-1] if paths else None


# ------------------------------------------------------------------------------------------
# dtype names.
# ------------------------------------------------------------------------------------------

_DTYPE_NAMES = {
    torch.float32: "float32", torch.float64: "float64", torch.float16: "float16",
    torch.bfloat16: "bfloat16", torch.int32: "int32", torch.int64: "int64", torch.int16: "int16",
    torch.int8: "int8", torch.uint8: "uint8", torch.bool: "bool", torch.uint32: "uint32",
    torch.uint16: "uint16", torch.float8_e4m3fn: "float8_e4m3fn", torch.float8_e5m2: "float8_e5m2",
}
_NAME_TO_DTYPE = {v: k for k, v in _DTYPE_NAMES.items()}
# zarr dtype strings; bfloat16/fp8 use tensorstore's extension names.
_ZARR_DTYPE = {
    "float32": "<f4", "float64": "<f8", "float16": "<f2", "bfloat16": "bfloat16", "int32": "<i4",
    "int64": "<i8", "int16": "<i2", "int8": "|i1", "uint8": "|u1", "bool": "|b1", "uint32": "<u4",
    "uint16": "<u2", "float8_e4m3fn": "float8_e4m3fn", "float8_e5m2": "float8_e5m2",
}
_ZARR_TO_NAME = {v: k for k, v in _ZARR_DTYPE.items()}
# Storage view for dtypes numpy lacks.
_VIEW_AS = {torch.bfloat16: torch.int16, torch.float8_e4m3fn: torch.uint8, torch.float8_e5m2: torch.uint8,
            torch.uint32: torch.int32, torch.uint16: torch.int16}


def _to_numpy_bytes(t: torch.Tensor) -> np.ndarray:
    t = t.detach().contiguous()
    if t.dtype in _VIEW_AS:
        t = t.view(_VIEW_AS[t.dtype])
    return t.numpy()


def _from_bytes(buf: bytes, dtype: torch.dtype, shape: Sequence[int]) -> torch.Tensor:
    store = _VIEW_AS.get(dtype, dtype)
    np_dtype = torch.empty((), dtype=store).numpy().dtype
    arr = np.frombuffer(buf, dtype=np_dtype).reshape(tuple(shape)).copy()
    t = torch.from_numpy(arr)
    return t.view(dtype) if store is not dtype else t


# ------------------------------------------------------------------------------------------
# Index file.
# ------------------------------------------------------------------------------------------


def _leaf_entry(value: Any) -> Any:
    if isinstance(value, torch.Tensor):
        return {"dtype": _DTYPE_NAMES[value.dtype], "shape": str(tuple(value.shape))}
    if isinstance(value, TensorSpec):
        return {"dtype": _DTYPE_NAMES[value.dtype], "shape": str(tuple(value.shape))}
    if isinstance(value, (int, float, str, bool)) or value is None:
        return value
    return str(type(value))


def write_index_file(ckpt_dir: str, *, step: int, entries: Sequence[tuple[str, Any]]) -> None:
    payload = [["step", int(step)]] + [[p, e] for p, e in entries]
    tmp = os.path.join(ckpt_dir, f".index.tmp.{os.getpid()}")
    with open(tmp, "w") as f:
        json.dump(payload, f)
    os.replace(tmp, os.path.join(ckpt_dir, "index"))


def read_index_file(ckpt_dir: str) -> list[tuple[str, Any]]:
    with open(os.path.join(ckpt_dir, "index")) as f:
        return [(p, v) for p, v in json.load(f)]


def read_state_spec(ckpt_dir: str) -> dict:
    """Tree of ``TensorSpec`` (and verbatim leaves) describing a stored checkpoint."""
    from axlearn_b200.common.utils import unflatten_items

    items = []
    for path, v in read_index_file(ckpt_dir):
        if path == "step":
            continue
        if isinstance(v, dict) and "dtype" in v and "shape" in v:
            v = TensorSpec(shape=tuple(ast.literal_eval(v["shape"])), dtype=_NAME_TO_DTYPE[v["dtype"]])
        items.append((path, v))
    return unflatten_items(items)


# ------------------------------------------------------------------------------------------
# Array storage (zarr v2, raw chunks).
# ------------------------------------------------------------------------------------------


def read_state_tensors(ckpt_dir: str) -> dict[str, torch.Tensor]:
    """Reads every array of a committed checkpoint in full: ``{path: tensor}`` (offline
    inspection, tests, conversion tools)."""
    out = {}
    for path, value in read_index_file(ckpt_dir):
        if isinstance(value, dict) and "shape" in value and "dtype" in value:
            shape = tuple(ast.literal_eval(value["shape"])) if isinstance(value["shape"], str) else tuple(value["shape"])
            out[path] = _read_array(ckpt_dir, path, want=tuple(slice(0, d) for d in shape), dtype=None)
    return out


class _Shard(NamedTuple):
    path: str
    host: torch.Tensor  # CPU copy of this rank's shard.
    global_shape: tuple
    coords: tuple  # Chunk coordinates of this shard.
    write_chunk: bool
    write_meta: bool


def _compressor_meta(name: Optional[str]) -> Optional[dict]:
    """``None`` (raw chunks, the default here) or the zarr-v2 compressor entry.  ``"zstd"`` is what
    the reference's writer puts into its tensorstore spec (level 1)."""
    if name in (None, "", "none"):
        return None
    if name == "zstd":
        return {"id": "zstd", "level": 1}
    if name in ("zlib", "gzip"):
        return {"id": name, "level": 1}
    raise ValueError(f"unknown chunk compressor {name!r}")


def _encode_chunk(raw: bytes, compressor: Optional[dict]) -> bytes:
    if compressor is None:
        return raw
    cid, level = compressor.get("id"), int(compressor.get("level", 1))
    if cid == "zstd":
        import pyarrow as pa

        return pa.Codec("zstd", compression_level=level).compress(raw, asbytes=True)
    if cid == "zlib":
        import zlib

        return zlib.compress(raw, level)
    if cid == "gzip":
        import gzip

        return gzip.compress(raw, compresslevel=level)
    raise ValueError(f"cannot write chunks with compressor {compressor!r}")


def _decode_chunk(raw: bytes, compressor: Optional[dict], nbytes: int) -> bytes:
    """Undoes the zarr-v2 ``compressor`` of one chunk (``nbytes`` = size of the decoded chunk)."""
    if compressor is None:
        return raw
    cid = compressor.get("id")
    if cid == "zstd":
        import pyarrow as pa

        return pa.Codec("zstd").decompress(raw, decompressed_size=nbytes, asbytes=True)
    if cid == "zlib":
        import zlib

        return zlib.decompress(raw)
    if cid == "gzip":
        import gzip

        return gzip.decompress(raw)
    raise ValueError(f"chunks compressed with {compressor!r} cannot be read here (supported: none, zstd, zlib, gzip)")


def _zarray_meta(global_shape: Sequence[int], chunk_shape: Sequence[int], dtype_name: str,
                 compressor: Optional[dict] = None) -> dict:
    return {
        "chunks": list(chunk_shape) if len(chunk_shape) else [],
        "compressor": compressor,
        "dimension_separator": ".",
        "dtype": _ZARR_DTYPE[dtype_name],
        "fill_value": None,
        "filters": None,
        "order": "C",
        "shape": list(global_shape),
        "zarr_format": 2,
    }


def _write_shard(ckpt_dir: str, s: _Shard, compressor: Optional[dict] = None) -> int:
    adir = os.path.join(ckpt_dir, "gda", s.path)
    os.makedirs(adir, exist_ok=True)
    if s.write_meta:
        meta = _zarray_meta(s.global_shape, tuple(s.host.shape), _DTYPE_NAMES[s.host.dtype], compressor)
        with open(os.path.join(adir, ".zarray"), "w") as f:
            json.dump(meta, f)
    if s.write_chunk:
        name = ".".join(str(c) for c in s.coords) if s.coords else "0"
        arr = _to_numpy_bytes(s.host)
        with open(os.path.join(adir, name), "wb") as f:
            f.write(_encode_chunk(arr.tobytes(), compressor))
        return arr.nbytes
    return 0


def _read_array(ckpt_dir: str, path: str, *, want: tuple[slice, ...], dtype: Optional[torch.dtype]) -> torch.Tensor:
    """Reads the region ``want`` (slices in global coordinates) of a stored array."""
    adir = os.path.join(ckpt_dir, "gda", path)
    with open(os.path.join(adir, ".zarray")) as f:
        meta = json.load(f)
    stored = _NAME_TO_DTYPE[_ZARR_TO_NAME[meta["dtype"]]]
    shape, chunks = tuple(meta["shape"]), tuple(meta["chunks"])
    compressor = meta.get("compressor")
    if meta.get("filters"):
        raise ValueError(f"{path}: zarr filters are not supported")
    if meta.get("order", "C") != "C":
        raise ValueError(f"{path}: only C-order chunks are supported")
    sep = meta.get("dimension_separator", ".")
    itemsize = torch.empty((), dtype=stored).element_size()

    def load_chunk(name: str, chunk_shape: tuple) -> Optional[torch.Tensor]:
        file = os.path.join(adir, name)
        if not os.path.exists(file):
            return None                      # never written: every element is the fill value
        with open(file, "rb") as f:
            raw = f.read()
        return _from_bytes(_decode_chunk(raw, compressor, int(np.prod(chunk_shape, dtype=np.int64)) * itemsize),
                           stored, chunk_shape)

    fill = meta.get("fill_value") or 0
    if not shape:
        t = load_chunk("0", ())
        if t is None:
            t = torch.full((), fill, dtype=stored)
        return t if dtype is None or dtype == stored else t.to(dtype)
    out_shape = tuple(s.stop - s.start for s in want)
    out = torch.empty(out_shape, dtype=stored)
    ranges = []
    for s, c in zip(want, chunks):
        ranges.append(range(s.start // c, (s.stop - 1) // c + 1) if s.stop > s.start else range(0))
    for coords in np.ndindex(*[len(r) for r in ranges]):
        cidx = tuple(r[i] for r, i in zip(ranges, coords))
        # A chunk file always holds a whole chunk; at the array's edge the part beyond `shape` is padding.
        chunk = load_chunk(sep.join(str(c) for c in cidx), chunks)
        src, dst = [], []
        for d, (ci, c, s) in enumerate(zip(cidx, chunks, want)):
            lo, hi = max(s.start, ci * c), min(s.stop, (ci + 1) * c)
            src.append(slice(lo - ci * c, hi - ci * c))
            dst.append(slice(lo - s.start, hi - s.start))
        if chunk is None:
            out[tuple(dst)] = fill
        else:
            out[tuple(dst)] = chunk[tuple(src)]
    return out if dtype is None or dtype == stored else out.to(dtype)


# ------------------------------------------------------------------------------------------
# Policies.
# ------------------------------------------------------------------------------------------


def every_n_steps_policy(n: int = 1, *, min_step: int = 1) -> Callable[..., bool]:
    def fn(*, step: int, evaler_summaries: Optional[dict] = None) -> bool:
        return step >= min_step and step % n == 0

    return fn


def every_n_steps_and_last_policy(n: int = 1, *, min_step: int = 1, max_step: int) -> Callable[..., bool]:
    base = every_n_steps_policy(n, min_step=min_step)

    def fn(*, step: int, evaler_summaries: Optional[dict] = None) -> bool:
        return base(step=step) or step == max_step

    return fn


class BestMetricPolicy(Configurable):
    """Saves when ``metric`` (an evaler summary, addressed as ``evaler/name``) improves."""

    @config_class
    class Config(Configurable.Config):
        metric: Required[tuple] = REQUIRED  # (evaler_name, metric_name)
        mode: str = "max"

    def __init__(self, cfg):
        super().__init__(cfg)
        self.best: Optional[float] = None

    def __call__(self, *, step: int, evaler_summaries: Optional[dict] = None) -> bool:
        cfg = self._config
        ev, name = cfg.metric
        if not evaler_summaries or evaler_summaries.get(ev) is None:
            return False
        flat = dict(flatten_items(evaler_summaries[ev]))
        if name not in flat:
            raise ValueError(f"metric {name} not found in evaler {ev} summaries: {list(flat)}")
        v = flat[name]
        v = float(v.value() if hasattr(v, "value") else v)
        better = self.best is None or (v > self.best if cfg.mode == "max" else v < self.best)
        if better:
            self.best = v
        return better


# ------------------------------------------------------------------------------------------
# State storage.
# ------------------------------------------------------------------------------------------


class _ByteBudget:
    """Bounds the bytes that sit in host staging buffers waiting to be written."""

    def __init__(self, limit: Optional[int]):
        self._limit = limit
        self._used = 0
        self._cv = threading.Condition()

    def acquire(self, n: int) -> None:
        if self._limit is None:
            return
        with self._cv:
            # A single array larger than the whole budget is admitted once nothing else is in flight.
            while self._used > 0 and self._used + n > self._limit:
                self._cv.wait()
            self._used += n

    def release(self, n: int) -> None:
        if self._limit is None:
            return
        with self._cv:
            self._used -= n
            self._cv.notify_all()


def _data_shard(local_shape: Sequence[int], replicas: int, replica: int, max_degree: Optional[int]):
    """How replica ``replica`` of ``replicas`` holders of the same shard takes part in writing it:
    ``(dim, degree, index)`` = it writes slice ``index`` of ``degree`` along ``dim``; or None
    when it writes nothing.  The first dim divisible by the degree is split (reference:
    axlearn/common/array_serialization.py:189-240); without ``max_degree`` only replica 0 writes."""
    if not max_degree or replicas <= 1:
        return (0, 1, 0) if replica == 0 else None
    degree = replicas if max_degree < 0 else min(replicas, max_degree)
    while degree > 1:
        for dim, size in enumerate(local_shape):
            if size % degree == 0 and size >= degree:
                return (dim, degree, replica) if replica < degree else None
        degree -= 1
    return (0, 1, 0) if replica == 0 else None


class TensorStoreStateStorage(Configurable):
    """Writes/reads a state tree in the layout described in the module docstring.

    Saving is asynchronous in every process (reference: ``BoundedDataShardedAsyncCheckpointManager``,
    axlearn/common/array_serialization.py:1199-1337): ``save_to_dir`` only *enqueues* the
    device-to-host copies on the current stream (so the next training step, queued behind them,
    cannot overwrite what is being copied) and returns; worker threads wait for each copy and
    write the chunk; host staging is bounded by ``max_concurrent_gb`` (the call blocks while the
    budget is exhausted); replicated arrays are written in slices by up to
    ``max_data_shard_degree`` of their holders.  Commit needs no collective: every process drops
    a marker file once its chunks are on disk and process 0 writes ``index`` when all markers
    are there, so the index-last rule holds across processes without a barrier on a helper thread.
    """

    @config_class
    class Config(Configurable.Config):
        timeout_secs: float = 3600
        # Upper bound on host staging memory in flight (GiB); None = unbounded.
        max_concurrent_gb: Optional[float] = None
        max_concurrent_restore_gb: Optional[float] = 32
        # Up to this many holders of a replicated array each write a slice of it (-1 = all of
        # them, None / 0 = only the first holder writes).
        max_data_shard_degree: Optional[int] = None
        num_io_threads: int = 8
        # Chunk compression: None (raw, the fastest to write from pinned host memory) or "zstd"
        # (what the reference's tensorstore writer uses, level 1), "zlib", "gzip".  The reader
        # handles all of them whatever this says.
        compressor: Optional[str] = None

    def __init__(self, cfg):
        super().__init__(cfg)
        self._pool = ThreadPoolExecutor(max_workers=cfg.num_io_threads, thread_name_prefix="ckpt-io")
        self._pending: Optional[threading.Thread] = None
        self._error: Optional[BaseException] = None
        self.peak_staged_bytes = 0  # observed high-water mark of host staging (tests, summaries)

    # ---------------------------------------------------------------- save
    def save_to_dir(self, *, step: int, state: Any, ckpt_dir: str, specs: Optional[Any] = None,
                    on_commit_callback: Optional[Callable[..., None]] = None) -> None:
        cfg = self._config
        self.wait_until_finished()
        mesh = current_mesh()
        rank, nproc = coll.process_index(), coll.process_count()
        if rank == 0:
            os.makedirs(ckpt_dir, exist_ok=True)
        coll.barrier("ckpt-mkdir")
        spec_map = dict(flatten_items(specs, is_leaf=lambda x: isinstance(x, TensorSpec))) if specs is not None else {}
        entries: list[tuple[str, Any]] = []
        python_items: list[tuple[str, Any]] = []
        budget = _ByteBudget(int(cfg.max_concurrent_gb * (1 << 30)) if cfg.max_concurrent_gb else None)
        futures = []
        staged = {"now": 0, "peak": 0}
        lock = threading.Lock()

        def write_when_copied(shard: _Shard, event, nbytes: int):
            try:
                if event is not None:
                    event.synchronize()  # this array's device-to-host copy has landed
                _write_shard(ckpt_dir, shard, _compressor_meta(cfg.compressor))
            finally:
                with lock:
                    staged["now"] -= nbytes
                budget.release(nbytes)

        for path, value in flatten_items(state):
            if isinstance(value, torch.Tensor):
                spec = spec_map.get(path)
                mesh_axes = getattr(spec, "mesh_axes", None)
                if mesh is not None and mesh.size > 1 and mesh_axes is not None and len(mesh_axes) == value.dim():
                    sizes = [mesh.axis_size(mesh.present_axes(ax)) for ax in mesh_axes]
                    gshape = tuple(d * n for d, n in zip(value.shape, sizes))
                    coords = [mesh.axis_index(mesh.present_axes(ax)) for ax in mesh_axes]
                    replicas = mesh.size // max(1, math.prod(sizes))
                    part = _data_shard(value.shape, replicas, mesh.replica_id(mesh_axes), cfg.max_data_shard_degree)
                else:
                    gshape, coords = tuple(value.shape), [0 for _ in value.shape]
                    part = _data_shard(value.shape, nproc, rank, cfg.max_data_shard_degree)
                entries.append((path, {"dtype": _DTYPE_NAMES[value.dtype], "shape": str(gshape)}))
                if part is None:
                    continue
                dim, degree, index = part
                piece = value
                if degree > 1:
                    width = value.shape[dim] // degree
                    piece = value.narrow(dim, index * width, width)
                    coords[dim] = coords[dim] * degree + index
                nbytes = piece.numel() * piece.element_size()
                budget.acquire(nbytes)  # blocks the caller while too much is staged already
                with lock:
                    staged["now"] += nbytes
                    staged["peak"] = max(staged["peak"], staged["now"])
                host, event = self._to_host(piece)
                shard = _Shard(path, host, gshape, tuple(coords), True, all(c == 0 for c in coords))
                futures.append(self._pool.submit(write_when_copied, shard, event, nbytes))
            elif hasattr(value, "get_state"):
                entries.append((path, str(type(value))))
                python_items.append((path, value.get_state()))
            else:
                entries.append((path, _leaf_entry(value)))

        def commit():
            try:
                for f in futures:
                    f.result()
                self.peak_staged_bytes = staged["peak"]
                if python_items:
                    pdir = os.path.join(ckpt_dir, f"python_{rank}")
                    for path, st in python_items:
                        fp = os.path.join(pdir, path)
                        os.makedirs(os.path.dirname(fp), exist_ok=True)
                        with open(fp, "w") as f:
                            json.dump(st, f)
                _commit_across_processes(ckpt_dir, rank=rank, nproc=nproc, timeout_secs=cfg.timeout_secs)
                if rank == 0:
                    # Markers go first: the callback may move the directory, and a crash between
                    # the two leaves an uncommitted checkpoint either way.
                    _clear_commit_markers(ckpt_dir)
                    if on_commit_callback is not None:
                        on_commit_callback(ckpt_dir=ckpt_dir, step=step, entries=entries)
                    else:
                        write_index_file(ckpt_dir, step=step, entries=entries)
            except BaseException as e:  # pylint: disable=broad-except
                self._error = e

        self._pending = threading.Thread(target=commit, name="ckpt-commit", daemon=True)
        self._pending.start()

    def _to_host(self, t: torch.Tensor):
        """``(host copy, event)``: the copy is enqueued on the current stream; ``event`` (None for
        CPU tensors) fires when it has landed."""
        t = t.detach()
        if not t.is_cuda:
            return t.clone(), None
        host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
        host.copy_(t, non_blocking=True)
        event = torch.cuda.Event()
        event.record(torch.cuda.current_stream(t.device))
        return host, event

    def wait_until_finished(self) -> None:
        if self._pending is not None:
            self._pending.join()
            self._pending = None
        self._raise_if_failed()

    def _raise_if_failed(self) -> None:
        if self._error is not None:
            e, self._error = self._error, None
            raise RuntimeError("checkpoint save failed") from e

    def stop(self) -> None:
        self.wait_until_finished()

    # ---------------------------------------------------------------- restore
    def restore_from_dir(self, *, step: int, state: Any, ckpt_dir: str, specs: Optional[Any] = None,
                         validation: CheckpointValidationType = EXACT, device=None) -> Any:
        """``state`` is the target structure: tensors (or TensorSpecs) give shape/dtype of
        this rank's shard; returns a tree of the same structure holding restored values."""
        stored = dict(read_index_file(ckpt_dir))
        if stored.get("step") != step:
            raise ValueError(f"index step {stored.get('step')} != requested {step}")
        stored.pop("step")
        mesh = current_mesh()
        spec_map = dict(flatten_items(specs, is_leaf=lambda x: isinstance(x, TensorSpec))) if specs is not None else {}
        target = flatten_items(state, is_leaf=lambda x: isinstance(x, TensorSpec))
        target_paths = {p for p, _ in target}
        up_to_dtype = validation in (EXACT_UP_TO_DTYPE, CONTAINS_STATE_UP_TO_DTYPE)
        if validation in (EXACT, EXACT_UP_TO_DTYPE):
            extra = set(stored) - target_paths
            if extra:
                raise ValueError(f"checkpoint has entries not in the target state: {sorted(extra)[:5]}...")
        missing = target_paths - set(stored)
        if missing:
            raise ValueError(f"target state entries missing from checkpoint: {sorted(missing)[:5]}...")

        def restore_leaf(path: str, tgt: Any) -> Any:
            entry = stored[path]
            if isinstance(tgt, (torch.Tensor, TensorSpec)):
                if not (isinstance(entry, dict) and "shape" in entry):
                    raise ValueError(f"{path}: checkpoint holds {entry!r}, target is a tensor")
                gshape = tuple(ast.literal_eval(entry["shape"]))
                sdtype = _NAME_TO_DTYPE[entry["dtype"]]
                if not up_to_dtype and sdtype != tgt.dtype:
                    raise ValueError(f"{path}: dtype {sdtype} != target {tgt.dtype}")
                spec = spec_map.get(path)
                mesh_axes = getattr(spec, "mesh_axes", None)
                if mesh is not None and mesh.size > 1 and mesh_axes is not None and len(mesh_axes) == len(gshape):
                    want = mesh.shard_slices(gshape, mesh_axes)
                else:
                    want = tuple(slice(0, d) for d in gshape)
                local_shape = tuple(s.stop - s.start for s in want)
                if tuple(tgt.shape) != local_shape:
                    raise ValueError(f"{path}: stored shape {gshape} gives local {local_shape}, target {tuple(tgt.shape)}")
                t = _read_array(ckpt_dir, path, want=want, dtype=tgt.dtype)
                dev = device if device is not None else (tgt.device if isinstance(tgt, torch.Tensor) else None)
                return t.to(dev) if dev is not None and torch.device(dev).type != "cpu" else t
            if hasattr(tgt, "set_state"):
                fp = os.path.join(ckpt_dir, f"python_{coll.process_index()}", path)
                with open(fp) as f:
                    tgt.set_state(json.load(f))
                return tgt
            return entry

        # Host memory held by arrays that were read but not yet handed over is bounded by
        # max_concurrent_restore_gb (reference: axlearn/common/array_serialization.py:549-720).
        cfg = self._config
        budget = _ByteBudget(int(cfg.max_concurrent_restore_gb * (1 << 30)) if cfg.max_concurrent_restore_gb else None)

        def bounded(path: str, tgt: Any, nbytes: int):
            try:
                return restore_leaf(path, tgt)
            finally:
                budget.release(nbytes)

        futures = {}
        for p, t in target:
            nbytes = 0
            if isinstance(t, (torch.Tensor, TensorSpec)):
                elem = torch.empty((), dtype=t.dtype).element_size() if t.dtype is not None else 4
                nbytes = math.prod(tuple(t.shape)) * elem
            budget.acquire(nbytes)
            futures[p] = self._pool.submit(bounded, p, t, nbytes)
        restored = {p: f.result() for p, f in futures.items()}
        return _fill_like(state, restored)


def _commit_across_processes(ckpt_dir: str, *, rank: int, nproc: int, timeout_secs: float) -> None:
    """Index-last commit without a collective: every process drops ``.done.<rank>`` once its
    chunks are on disk; process 0 returns when all ``nproc`` markers exist (the others return at
    once).  Runs on a helper thread, where a process-group barrier must not be issued."""
    if nproc <= 1:
        return
    marker = os.path.join(ckpt_dir, f".done.{rank}")
    with open(marker + ".tmp", "w") as f:
        f.write(str(time.time()))
    os.replace(marker + ".tmp", marker)
    if rank != 0:
        return
    deadline = time.time() + timeout_secs
    while True:
        if all(os.path.exists(os.path.join(ckpt_dir, f".done.{r}")) for r in range(nproc)):
            return
        if time.time() > deadline:
            raise TimeoutError(f"not every process finished writing {ckpt_dir} within {timeout_secs} s")
        time.sleep(0.02)


def _clear_commit_markers(ckpt_dir: str) -> None:
    for name in os.listdir(ckpt_dir):
        if name.startswith(".done."):
            try:
                os.remove(os.path.join(ckpt_dir, name))
            except FileNotFoundError:
                pass


def _fill_like(structure: Any, values: dict[str, Any], prefix: str = "") -> Any:
    """Rebuilds ``structure`` with leaves replaced from ``values`` keyed by path."""
    from axlearn_b200.common.utils import _children

    if structure is None:
        return None
    kids = None if isinstance(structure, TensorSpec) else _children(structure)
    if kids is None:
        return values[prefix]
    new = [( k, _fill_like(v, values, f"{prefix}/{k}" if prefix else k)) for k, v in kids]
    if isinstance(structure, dict):
        out = type(structure)()
        orig_keys = {str(k): k for k in structure.keys()}
        for k, v in new:
            out[orig_keys[k]] = v
        return out
    if isinstance(structure, tuple) and hasattr(type(structure), "_fields"):
        return type(structure)(*[v for _, v in new])
    return type(structure)(v for _, v in new)


# ------------------------------------------------------------------------------------------
# Checkpointer.
# ------------------------------------------------------------------------------------------


class BaseCheckpointer(Module):
    @config_class
    class Config(Module.Config):
        dir: Required[str] = REQUIRED
        save_policy: InstantiableConfig = config_for_function(every_n_steps_policy)


class Checkpointer(BaseCheckpointer):
    """Saves / restores trainer state under ``{dir}/step_XXXXXXXX`` and garbage-collects old
    checkpoints (reference: axlearn/common/checkpointer.py:1005-1273)."""

    @config_class
    class Config(BaseCheckpointer.Config):
        storage: InstantiableConfig = TensorStoreStateStorage.default_config()
        gc_loop_interval_seconds: float = 60
        keep_last_n: int = 1
        keep_every_n_steps: Optional[int] = None
        summary_writer: Optional[InstantiableConfig] = None

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._allow_contextless = True
        self._storage: TensorStoreStateStorage = cfg.storage.instantiate()
        self._save_policy = cfg.save_policy.instantiate()
        self._gc_thread: Optional[threading.Thread] = None
        self._gc_stop = threading.Event()
        self._within_context = False

    @classmethod
    def latest_checkpoint_path(cls, base_dir: str) -> Optional[str]:
        return latest_checkpoint_path(base_dir)

    @classmethod
    def checkpoint_paths(cls, base_dir: str) -> list[str]:
        return checkpoint_paths(base_dir)

    def __enter__(self):
        self._within_context = True
        return self

    def __exit__(self, exc_type, exc, tb):
        self.stop(has_exception=exc_type is not None)
        self._within_context = False
        return False

    def ckpt_dir(self, step: int) -> str:
        return build_step_dir(self._config.dir, step=step)

    def save(self, *, step: int, state: Any, specs: Optional[Any] = None,
             evaler_summaries: Optional[dict] = None, force: bool = False,
             pre_save_check: Optional[Callable[[], None]] = None) -> bool:
        """Saves if the policy says so; returns whether a save was started.  ``pre_save_check``
        runs once the policy has decided to save and before anything is written; it may raise
        to veto the save (the trainer uses it to refuse a state computed by a kernel that
        reported an error)."""
        if not force and not self._save_policy(step=step, evaler_summaries=evaler_summaries):
            return False
        if pre_save_check is not None:
            pre_save_check()
        ckpt_dir = self.ckpt_dir(step)
        if os.path.exists(os.path.join(ckpt_dir, "index")):
            raise ValueError(f"checkpoint {ckpt_dir} already exists")
        self._storage.save_to_dir(step=step, state=state, ckpt_dir=ckpt_dir, specs=specs)
        if coll.process_index() == 0:
            self._run_garbage_collection(exclude_step=step)
        return True

    def wait_until_finished(self) -> None:
        self._storage.wait_until_finished()

    def restore(self, *, step: Optional[int] = None, state: Any, specs: Optional[Any] = None,
                validation: CheckpointValidationType = EXACT, device=None) -> tuple[Optional[int], Any]:
        """Restores ``step`` (or the latest committed step).  Returns ``(step, state)``;
        ``(None, state)`` unchanged when no checkpoint exists and ``step`` was None."""
        self._storage.wait_until_finished()
        cfg = self._config
        if step is None:
            path = latest_checkpoint_path(cfg.dir)
            if path is None:
                return None, state
            step = parse_step_from_dir(path)
        else:
            path = self.ckpt_dir(step)
            if not os.path.exists(os.path.join(path, "index")):
                raise ValueError(f"checkpoint {path} does not exist or is incomplete")
        restored = self._storage.restore_from_dir(
            step=step, state=state, ckpt_dir=path, specs=specs, validation=validation, device=device)
        coll.barrier("ckpt-restore")
        return step, restored

    def stop(self, *, has_exception: bool = False) -> None:
        """Waits for in-flight saves (skipped after an exception, so a failed rank cannot
        deadlock the others in a barrier)."""
        if not has_exception:
            self._storage.wait_until_finished()
        self._gc_stop.set()

    # ---------------------------------------------------------------- garbage collection
    def _run_garbage_collection(self, *, exclude_step: Optional[int] = None) -> None:
        cfg = self._config
        base = cfg.dir
        if not os.path.isdir(base):
            return
        all_dirs = sorted(
            os.path.join(base, n) for n in os.listdir(base) if _STEP_RE.fullmatch(n))
        committed = [d for d in all_dirs if os.path.exists(os.path.join(d, "index"))]
        uncommitted = [d for d in all_dirs if d not in committed]
        keep: set = set(committed[-max(cfg.keep_last_n, 1):])
        # The newest uncommitted dir may be a save in flight.
        if uncommitted:
            keep.add(uncommitted[-1])
        if exclude_step is not None:
            keep.add(self.ckpt_dir(exclude_step))
        if cfg.keep_every_n_steps:
            last_kept = None
            for d in committed:
                s = parse_step_from_dir(d)
                if last_kept is None or s >= last_kept + cfg.keep_every_n_steps:
                    if s % cfg.keep_every_n_steps == 0 or last_kept is None:
                        keep.add(d)
                        last_kept = s
        for d in all_dirs:
            if d in keep:
                continue
            idx = os.path.join(d, "index")
            if os.path.exists(idx):
                os.remove(idx)  # Un-commit first so that a crash leaves no half-deleted ckpt.
            shutil.rmtree(d, ignore_errors=True)
