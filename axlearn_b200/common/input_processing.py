"""Dataset processors: the composable source -> processor -> batcher input stack.

Parity target: the reference's tf.data stack (axlearn/common/input_tf_data.py:125-1560) --
``BuildDatasetFn`` / ``DatasetToDatasetFn``, ``chain``, ``with_processor``, ``sample_from_datasets``,
``concatenate_datasets``, ``take`` / ``unbatch`` / ``select_fields`` / ``remove_fields`` /
``filter_examples`` / ``squeeze_fields`` / ``rekey`` / ``shuffle`` / ``unpack`` /
``extract_from_sequence`` / ``add_static_fields`` / ``skip_on_error``, ``batch`` with
per-feed batch sizes, evaluation padding (``_pad_for_evaluation``: every feed yields the same
number of batches, padded with ``pad_example_fn`` examples) and logical feeds, ``pad_to_batch`` /
``pack_to_batch`` / ``trim_to_batch`` / ``trim_and_pad_tensor``, and the ``Input`` module built
from ``source`` / ``processor`` / ``batcher`` configs.

There is no tf.data here.  A *dataset* is any iterable of examples (dicts of numpy arrays, Python
scalars or strings); a ``BuildDatasetFn`` takes no arguments and returns one; a
``DatasetToDatasetFn`` maps a dataset to a dataset.  Everything is lazy (generators), so an
infinite source works for training, and deterministic given its seeds.  The heavy lifting
(decoding, tokenisation) runs on host threads in ``input_pipeline._Prefetch`` when wrapped by
``PipelineInput``; these processors are the per-example logic.
"""

from __future__ import annotations

import copy
import itertools
from typing import Any, Callable, Iterable, Iterator, Mapping, Optional, Sequence, Union

import numpy as np

from axlearn_b200.common.config import (
    REQUIRED,
    ConfigOr,
    InstantiableConfig,
    Required,
    config_class,
    maybe_instantiate,
)
from axlearn_b200.common.input_base import Input as BaseInput
from axlearn_b200.parallel import collectives as coll

Example = dict
Dataset = Iterable[Example]
BuildDatasetFn = Callable[[], Dataset]
DatasetToDatasetFn = Callable[[Dataset], Dataset]
PadExampleFn = Callable[[Example], Example]


# ------------------------------------------------------------------------------------------
# Combinators.
# ------------------------------------------------------------------------------------------


def map_over_dataset(fn: Callable[[Example], Example]) -> DatasetToDatasetFn:
    """Lifts a per-example function to a dataset processor."""

    def process(ds: Dataset) -> Iterator[Example]:
        for ex in ds:
            yield fn(ex)

    return process


def identity() -> DatasetToDatasetFn:
    return lambda ds: ds


def chain(*processors: ConfigOr[DatasetToDatasetFn], is_training: Optional[bool] = None) -> DatasetToDatasetFn:
    """Applies processors left to right.  Configs are instantiated (with ``is_training`` set on
    those that have the field)."""
    fns = []
    for p in processors:
        if isinstance(p, InstantiableConfig):
            if is_training is not None and "is_training" in p:
                p = p.clone(is_training=is_training)
            p = p.instantiate()
        fns.append(p)

    def process(ds: Dataset) -> Dataset:
        for fn in fns:
            ds = fn(ds)
        return ds

    return process


def with_processor(source: ConfigOr[BuildDatasetFn], *, processor: ConfigOr[DatasetToDatasetFn],
                   is_training: Optional[bool] = None) -> BuildDatasetFn:
    if isinstance(source, InstantiableConfig) and is_training is not None and "is_training" in source:
        source = source.clone(is_training=is_training)
    src, proc = maybe_instantiate(source), chain(processor, is_training=is_training)
    return lambda: proc(src())


def sample_from_datasets(*, sources: Sequence[ConfigOr[BuildDatasetFn]], weights: Sequence[float], seed: int = 0,
                         is_training: bool = True) -> BuildDatasetFn:
    """Draws each next example from source ``i`` with probability ``weights[i]``; sources with
    weight 0 are never read; the mixture ends when a sampled source is exhausted (training
    sources are expected to repeat)."""
    if len(sources) != len(weights):
        raise ValueError("sources and weights must have the same length")
    if not any(w > 0 for w in weights):
        raise ValueError("at least one weight must be positive")
    built = [maybe_instantiate(s.clone(is_training=is_training) if isinstance(s, InstantiableConfig)
                               and "is_training" in s else s) for s in sources]

    def fn() -> Iterator[Example]:
        rng = np.random.default_rng(seed)
        p = np.asarray(weights, dtype=np.float64)
        p = p / p.sum()
        its = [iter(b()) if w > 0 else None for b, w in zip(built, weights)]
        while True:
            i = int(rng.choice(len(its), p=p))
            try:
                yield next(its[i])
            except StopIteration:
                return

    return fn


def concatenate_datasets(*, sources: Sequence[ConfigOr[BuildDatasetFn]], is_training: bool = False) -> BuildDatasetFn:
    built = [maybe_instantiate(s.clone(is_training=is_training) if isinstance(s, InstantiableConfig)
                               and "is_training" in s else s) for s in sources]
    return lambda: itertools.chain.from_iterable(b() for b in built)


def take(num_examples: int) -> DatasetToDatasetFn:
    return lambda ds: itertools.islice(ds, num_examples)


def unbatch() -> DatasetToDatasetFn:
    """Splits every example along the leading dim of its fields."""

    def process(ds: Dataset) -> Iterator[Example]:
        for ex in ds:
            n = len(next(iter(ex.values())))
            for i in range(n):
                yield {k: v[i] for k, v in ex.items()}

    return process


def select_fields(fields: Sequence[str]) -> DatasetToDatasetFn:
    return map_over_dataset(lambda ex: {k: ex[k] for k in fields})


def remove_fields(fields: Sequence[str]) -> DatasetToDatasetFn:
    drop = set(fields)
    return map_over_dataset(lambda ex: {k: v for k, v in ex.items() if k not in drop})


def filter_examples(filter_fn: Callable[[Example], bool]) -> DatasetToDatasetFn:
    return lambda ds: (ex for ex in ds if filter_fn(ex))


def squeeze_fields(axis: Mapping[str, Optional[Union[int, tuple]]]) -> DatasetToDatasetFn:
    def fn(ex: Example) -> Example:
        ex = dict(ex)
        for k, ax in axis.items():
            ex[k] = np.squeeze(np.asarray(ex[k]), axis=ax)
        return ex

    return map_over_dataset(fn)


def skip_on_error(*, log_warning: bool = False) -> DatasetToDatasetFn:
    """Drops examples whose production raised (decoding errors and the like)."""

    def process(ds: Dataset) -> Iterator[Example]:
        it = iter(ds)
        while True:
            try:
                yield next(it)
            except StopIteration:
                return
            except Exception as e:  # pylint: disable=broad-except
                if log_warning:
                    print(f"input_processing: skipped an example: {type(e).__name__}: {e}", flush=True)

    return process


def extract_from_sequence(in_key: str, out_key: str, idx: Union[int, slice] = 0) -> DatasetToDatasetFn:
    def fn(ex: Example) -> Example:
        ex = dict(ex)
        ex[out_key] = ex[in_key][idx]
        return ex

    return map_over_dataset(fn)


def _get_path(ex: Any, path: str, separator: Optional[str]):
    if separator is None or not isinstance(path, str):
        return (path in ex), (ex.get(path) if isinstance(ex, dict) else None)
    node = ex
    for part in path.split(separator):
        if not isinstance(node, dict) or part not in node:
            return False, None
        node = node[part]
    return True, node


def rekey(key_map: dict[str, Optional[str]], *, default_value: Any = "", retain_original_inputs: bool = False,
          separator: Optional[str] = None) -> DatasetToDatasetFn:
    """``output[new] = input[old]`` for every ``new: old`` in ``key_map`` (``default_value`` when
    ``old`` is falsy or absent and a default is given); ``separator`` enables nested paths."""

    def fn(ex: Example) -> Example:
        out = dict(ex) if retain_original_inputs else {}
        for new, old in key_map.items():
            found, value = (False, None) if not old else _get_path(ex, old, separator)
            if not found:
                if default_value is None:
                    continue
                value = default_value
            if separator is None:
                out[new] = value
            else:
                node = out
                parts = new.split(separator)
                for part in parts[:-1]:
                    node = node.setdefault(part, {})
                node[parts[-1]] = value
        return out

    return map_over_dataset(fn)


def shuffle(shuffle_buffer_size: int, *, seed: int = 0) -> DatasetToDatasetFn:
    """Buffered shuffle: the next example is a uniformly random element of a sliding buffer."""

    def process(ds: Dataset) -> Iterator[Example]:
        if shuffle_buffer_size <= 0:
            yield from ds
            return
        rng = np.random.default_rng(seed)
        buf: list = []
        for ex in ds:
            if len(buf) < shuffle_buffer_size:
                buf.append(ex)
                continue
            i = int(rng.integers(len(buf)))
            out, buf[i] = buf[i], ex
            yield out
        rng.shuffle(buf)
        yield from buf

    return process


def unpack(key_map: dict[str, tuple]) -> DatasetToDatasetFn:
    """``output[new] = input[p0][p1]...`` for every ``new: (p0, p1, ...)``; other fields stay."""

    def fn(ex: Example) -> Example:
        ex = dict(ex)
        for new, path in key_map.items():
            node = ex
            for part in path:
                node = node[part]
            ex[new] = node
        return ex

    return map_over_dataset(fn)


def add_static_fields(key_map: dict[str, Any]) -> DatasetToDatasetFn:
    def fn(ex: Example) -> Example:
        ex = dict(ex)
        ex.update(copy.deepcopy(key_map))
        return ex

    return map_over_dataset(fn)


def ragged_to_tensor(feature_shapes: dict[str, Sequence[Optional[int]]], default_value: int = 0) -> DatasetToDatasetFn:
    """Pads lists of variable-length lists to rectangular arrays of the given shapes (None =
    the longest along that dim)."""

    def pad(value, shape):
        rows = [np.asarray(r) for r in value]
        width = shape[-1] if shape[-1] is not None else max((len(r) for r in rows), default=0)
        n = shape[0] if shape[0] is not None else len(rows)
        out = np.full((n, width), default_value, dtype=rows[0].dtype if rows else np.int32)
        for i, r in enumerate(rows[:n]):
            out[i, : min(width, len(r))] = r[:width]
        return out

    def fn(ex: Example) -> Example:
        ex = dict(ex)
        for k, shape in feature_shapes.items():
            ex[k] = pad(ex[k], shape)
        return ex

    return map_over_dataset(fn)


# ------------------------------------------------------------------------------------------
# Shaping single examples.
# ------------------------------------------------------------------------------------------


def trim_and_pad_tensor(t: Any, max_len: int, pad_id: int = 0) -> np.ndarray:
    """Trims or right-pads the LAST dim of ``t`` to ``max_len``."""
    t = np.asarray(t)
    if t.shape[-1] >= max_len:
        return t[..., :max_len]
    pad = [(0, 0)] * (t.ndim - 1) + [(0, max_len - t.shape[-1])]
    return np.pad(t, pad, constant_values=pad_id)


def trim_and_pad(feature_lengths: dict[str, int], pad_id: int = 0) -> DatasetToDatasetFn:
    def fn(ex: Example) -> Example:
        ex = dict(ex)
        for k, n in feature_lengths.items():
            ex[k] = trim_and_pad_tensor(ex[k], n, pad_id)
        return ex

    return map_over_dataset(fn)


def pad_to_batch(batch_size: int, pad_value: int = 0) -> DatasetToDatasetFn:
    """Pads the FIRST dim of every field to ``batch_size``."""

    def pad(v):
        v = np.asarray(v)
        if v.shape[0] > batch_size:
            raise ValueError(f"leading dim {v.shape[0]} exceeds batch_size {batch_size}")
        return np.pad(v, [(0, batch_size - v.shape[0])] + [(0, 0)] * (v.ndim - 1), constant_values=pad_value)

    return map_over_dataset(lambda ex: {k: pad(v) for k, v in ex.items()})


def trim_to_batch(batch_size: int) -> DatasetToDatasetFn:
    return map_over_dataset(lambda ex: {k: np.asarray(v)[:batch_size] for k, v in ex.items()})


def pack_to_batch(batch_size: int, pad_value: int = 0) -> DatasetToDatasetFn:
    """Concatenates consecutive examples along their first dim into elements of exactly
    ``batch_size`` rows (padded); an example that does not fit the open element starts a new one."""

    def process(ds: Dataset) -> Iterator[Example]:
        padder = pad_to_batch(batch_size, pad_value)
        cur: Optional[dict] = None
        rows = 0
        for ex in ds:
            ex = {k: np.asarray(v) for k, v in ex.items()}
            n = next(iter(ex.values())).shape[0]
            if n > batch_size:
                raise ValueError(f"an element with {n} rows cannot be packed into batches of {batch_size}")
            if cur is not None and rows + n > batch_size:
                yield from padder([cur])
                cur, rows = None, 0
            cur = ex if cur is None else {k: np.concatenate([cur[k], ex[k]], axis=0) for k in cur}
            rows += n
        if cur is not None:
            yield from padder([cur])

    return process


def default_pad_example_fn(example: Example) -> Example:
    """A padding example: zeros (empty strings) shaped like ``example``."""

    def zero(v):
        if isinstance(v, str):
            return ""
        if isinstance(v, bytes):
            return b""
        a = np.asarray(v)
        if a.dtype.kind in "US":
            return np.full(a.shape, "", dtype=a.dtype)
        return np.zeros_like(a)

    return {k: (default_pad_example_fn(v) if isinstance(v, dict) else zero(v)) for k, v in example.items()}


# ------------------------------------------------------------------------------------------
# Batching.
# ------------------------------------------------------------------------------------------


def _stack(rows: Sequence[Example]) -> Example:
    out = {}
    for k in rows[0]:
        vals = [r[k] for r in rows]
        if isinstance(vals[0], dict):
            out[k] = _stack(vals)
        elif isinstance(vals[0], (str, bytes)):
            out[k] = np.asarray(vals, dtype=object)
        else:
            out[k] = np.stack([np.asarray(v) for v in vals])
    return out


def _max_over_feeds(n: int) -> int:
    """Largest ``n`` over the data feeds (processes), so that all of them yield equally many
    evaluation batches (the "last batch" problem of multi-process evaluation)."""
    if coll.process_count() <= 1:
        return n
    import torch
    import torch.distributed as dist

    t = torch.tensor([n], dtype=torch.int64)
    if dist.get_backend() == "nccl":
        t = t.cuda()
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return int(t.item())


def per_feed_batch(feed_batch_size: int, *, is_training: bool, pad_example_fn: PadExampleFn = default_pad_example_fn,
                   post_batch_processor: Optional[ConfigOr[DatasetToDatasetFn]] = None,
                   repeat: Optional[int] = None) -> DatasetToDatasetFn:
    """Batches one feed's examples.  Training drops a short last batch and repeats forever (or
    ``repeat`` times); evaluation pads the last batch with ``pad_example_fn`` examples and, with
    several processes, pads every feed to the same number of batches."""
    if repeat is not None and (not isinstance(repeat, int) or repeat <= 0):
        raise ValueError(f"Invalid repeat (must be a positive integer): {repeat}")
    post = chain(post_batch_processor) if post_batch_processor is not None else None

    def batches_once(ds: Dataset) -> Iterator[Example]:
        rows: list = []
        template = None
        count = 0
        for ex in ds:
            template = ex if template is None else template
            rows.append(ex)
            count += 1
            if len(rows) == feed_batch_size:
                yield _stack(rows)
                rows = []
        if is_training:
            return
        # Evaluation: pad to a whole number of batches, the same on every feed.
        target = count + (-count) % feed_batch_size
        target = _max_over_feeds(target)
        if template is None and target > 0:
            raise ValueError("an empty evaluation feed cannot be padded: no example to shape the padding after")
        while count < target:
            rows.append(pad_example_fn(template))
            count += 1
            if len(rows) == feed_batch_size:
                yield _stack(rows)
                rows = []

    def process(ds: Dataset) -> Iterator[Example]:
        def run():
            if not is_training and repeat is None:
                yield from batches_once(ds)
                return
            n = 0
            while repeat is None or n < repeat:
                produced = False
                for b in batches_once(ds):
                    produced = True
                    yield b
                n += 1
                if not produced:
                    return  # an empty pass would repeat forever

        out = run()
        return post(out) if post is not None else out

    return process


def batch(global_batch_size: int, *, is_training: bool, pad_example_fn: PadExampleFn = default_pad_example_fn,
          global_logical_batch_size: Optional[int] = None, logical_feed_indices: Optional[Sequence[int]] = None,
          prefetch_buffer_size: Optional[int] = None,
          post_batch_processor: Optional[ConfigOr[DatasetToDatasetFn]] = None,
          repeat: Optional[int] = None) -> DatasetToDatasetFn:
    """Global batch size -> this feed's batches.  ``global_logical_batch_size`` with
    ``logical_feed_indices``: only those feeds draw real examples (``logical / len(indices)`` each);
    every feed's batch is then padded to the physical ``global_batch_size / feeds`` rows, and feeds
    outside the set yield padding only."""
    del prefetch_buffer_size  # prefetching is the job of input_pipeline's background stage
    feeds = coll.process_count()
    if global_batch_size % feeds:
        raise ValueError(f"global_batch_size ({global_batch_size}) must be divisible by the number of data feeds ({feeds}).")
    if (global_logical_batch_size is None) != (logical_feed_indices is None):
        raise ValueError("Must provide both | neither global_logical_batch_size and logical_feed_indices.")
    physical = global_batch_size // feeds
    if global_logical_batch_size is None:
        return per_feed_batch(physical, is_training=is_training, pad_example_fn=pad_example_fn,
                              post_batch_processor=post_batch_processor, repeat=repeat)
    logical_feed_indices = list(logical_feed_indices)
    if global_logical_batch_size % len(logical_feed_indices):
        raise ValueError(f"global_logical_batch_size ({global_logical_batch_size}) must be divisible by the number of "
                         f"logical data feeds ({len(logical_feed_indices)}).")
    logical = global_logical_batch_size // len(logical_feed_indices)
    if logical > physical:
        raise ValueError("a feed's logical batch cannot exceed its physical batch")
    me = coll.process_index()
    inner = per_feed_batch(logical, is_training=is_training, pad_example_fn=pad_example_fn, repeat=repeat)
    post = chain(post_batch_processor) if post_batch_processor is not None else None

    def process(ds: Dataset) -> Iterator[Example]:
        def run():
            for b in inner(ds):
                rows = [{k: v[i] for k, v in b.items()} for i in range(logical)]
                if me not in logical_feed_indices:
                    rows = []
                pad = pad_example_fn({k: v[0] for k, v in b.items()})
                yield _stack(rows + [pad] * (physical - len(rows)))

        out = run()
        return post(out) if post is not None else out

    return process


# ------------------------------------------------------------------------------------------
# The Input module.
# ------------------------------------------------------------------------------------------


class Input(BaseInput):
    """``source`` (BuildDatasetFn) -> ``processor`` -> ``batcher`` (both DatasetToDatasetFn)."""

    @config_class
    class Config(BaseInput.Config):
        is_training: Required[bool] = REQUIRED
        source: Required[InstantiableConfig] = REQUIRED
        processor: Required[InstantiableConfig] = REQUIRED
        batcher: Required[InstantiableConfig] = REQUIRED

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)

        def with_mode(c):
            return c.clone(is_training=cfg.is_training) if "is_training" in c else c

        self._source = with_mode(cfg.source).instantiate()
        self._processor = with_mode(cfg.processor).instantiate()
        self._batcher = with_mode(cfg.batcher).instantiate()

    @property
    def source(self) -> BuildDatasetFn:
        return self._source

    @property
    def processor(self) -> DatasetToDatasetFn:
        return self._processor

    def dataset(self) -> Iterator[dict]:
        from axlearn_b200.common.input_pipeline import to_tensors

        for b in self._batcher(self._processor(self._source())):
            yield to_tensors(b)


def disable_shuffle_recursively(cfg: InstantiableConfig) -> None:
    """Sets every ``shuffle_buffer_size`` / ``shuffle`` knob under ``cfg`` to "off" (evaluation,
    deterministic runs)."""
    from axlearn_b200.common.config import ConfigBase

    def visit(node):
        if isinstance(node, ConfigBase):
            if "shuffle_buffer_size" in node:
                node.shuffle_buffer_size = 0
            if "shuffle" in node and isinstance(node.shuffle, bool):
                node.shuffle = False
            for _, v in node.items():
                visit(v)
        elif isinstance(node, (list, tuple)):
            for v in node:
                visit(v)
        elif isinstance(node, dict):
            for v in node.values():
                visit(v)

    visit(cfg)
