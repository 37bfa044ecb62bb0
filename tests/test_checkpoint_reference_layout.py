"""A checkpoint laid out BY HAND the way the reference's writer lays it out -- ``index`` as
``json.dumps([["step", n], [path, {"dtype", "shape"}], ...])`` (axlearn/common/checkpointer.py:353-358,
:523) and one tensorstore zarr-v2 array per tensor under ``gda/<path>`` with the metadata jax's
serialisation puts into the spec (zstd level 1, "." separator, full-size edge chunks, unwritten
chunks = fill value) -- must restore through this framework's checkpointer.  And what this
framework writes with ``compressor="zstd"`` must decode with nothing but the zarr-v2 rules."""

import json
import os

import numpy as np
import pyarrow as pa
import torch

from axlearn_b200.common.checkpointer import Checkpointer, TensorStoreStateStorage, every_n_steps_policy
from axlearn_b200.common.config import config_for_function


def _write_zarr(adir, arr: np.ndarray, chunks, *, dtype_str=None, skip=()):
    """The files a zarr-v2 writer with a zstd compressor produces for ``arr``."""
    os.makedirs(adir)
    meta = {"chunks": list(chunks), "compressor": {"id": "zstd", "level": 1}, "dimension_separator": ".",
            "dtype": dtype_str or arr.dtype.str, "fill_value": None, "filters": None, "order": "C",
            "shape": list(arr.shape), "zarr_format": 2}
    with open(os.path.join(adir, ".zarray"), "w") as f:
        json.dump(meta, f)
    codec = pa.Codec("zstd", compression_level=1)
    if arr.ndim == 0:
        with open(os.path.join(adir, "0"), "wb") as f:
            f.write(codec.compress(arr.tobytes(), asbytes=True))
        return
    grid = [(-(-s // c)) for s, c in zip(arr.shape, chunks)]
    for idx in np.ndindex(*grid):
        if idx in skip:
            continue
        full = np.zeros(chunks, dtype=arr.dtype)                 # edge chunks are stored at full size
        sl = tuple(slice(i * c, min((i + 1) * c, s)) for i, c, s in zip(idx, chunks, arr.shape))
        part = arr[sl]
        full[tuple(slice(0, n) for n in part.shape)] = part
        with open(os.path.join(adir, ".".join(map(str, idx))), "wb") as f:
            f.write(codec.compress(full.tobytes(), asbytes=True))


def test_restores_a_reference_style_checkpoint(tmp_path):
    rng = np.random.default_rng(0)
    w = rng.standard_normal((10, 6)).astype("<f4")               # 4 x 4 chunks: ragged edges in both dims
    emb = rng.standard_normal((8, 4)).astype("<f4")
    emb_bf16 = (emb.view("<u4") >> 16).astype("<u2")             # the bits of the bf16 truncation
    sparse = np.zeros((4, 4), dtype="<i4")
    sparse[2:, :] = 7                                            # chunk (0, 0) is all fill value and never written
    step_dir = tmp_path / "step_00000300"
    gda = step_dir / "gda"
    _write_zarr(gda / "model" / "linear" / "weight", w, (4, 4))
    _write_zarr(gda / "model" / "emb" / "weight", emb_bf16, (8, 4), dtype_str="bfloat16")
    _write_zarr(gda / "model" / "table", sparse, (2, 4), skip={(0, 0)})
    _write_zarr(gda / "learner" / "count", np.array(300, dtype="<i4"), ())
    index = [["step", 300],
             ["model/linear/weight", {"dtype": "float32", "shape": "(10, 6)"}],
             ["model/emb/weight", {"dtype": "bfloat16", "shape": "(8, 4)"}],
             ["model/table", {"dtype": "int32", "shape": "(4, 4)"}],
             ["learner/count", {"dtype": "int32", "shape": "()"}],
             ["learner/name", "adamw"]]
    (step_dir / "index").write_text(json.dumps(index))

    ck = Checkpointer.default_config().set(name="ckpt", dir=str(tmp_path)).instantiate(parent=None)
    target = {"model": {"linear": {"weight": torch.zeros(10, 6)}, "emb": {"weight": torch.zeros(8, 4, dtype=torch.bfloat16)},
                        "table": torch.zeros(4, 4, dtype=torch.int32)},
              "learner": {"count": torch.zeros((), dtype=torch.int32), "name": "?"}}
    step, got = ck.restore(state=target)
    assert step == 300
    torch.testing.assert_close(got["model"]["linear"]["weight"], torch.from_numpy(w.astype(np.float32)), rtol=0, atol=0)
    want_emb = torch.from_numpy(emb_bf16.astype(np.int16)).view(torch.bfloat16)
    assert torch.equal(got["model"]["emb"]["weight"], want_emb)
    assert torch.equal(got["model"]["table"], torch.from_numpy(sparse.astype(np.int32)))
    assert int(got["learner"]["count"]) == 300 and got["learner"]["name"] == "adamw"


def test_zstd_chunks_written_here_decode_by_the_zarr_rules(tmp_path):
    torch.manual_seed(0)
    state = {"a": torch.randn(16, 8), "b": torch.randn(5).bfloat16(), "n": torch.tensor(3)}
    cfg = Checkpointer.default_config().set(
        name="ckpt", dir=str(tmp_path), save_policy=config_for_function(every_n_steps_policy),
        storage=TensorStoreStateStorage.default_config().set(compressor="zstd"))
    ck = cfg.instantiate(parent=None)
    ck.save(step=1, state=state)
    ck.wait_until_finished()
    adir = tmp_path / "step_00000001" / "gda" / "a"
    meta = json.loads((adir / ".zarray").read_text())
    assert meta["compressor"] == {"id": "zstd", "level": 1} and meta["zarr_format"] == 2
    raw = pa.Codec("zstd").decompress((adir / "0.0").read_bytes(), decompressed_size=16 * 8 * 4, asbytes=True)
    np.testing.assert_array_equal(np.frombuffer(raw, dtype=meta["dtype"]).reshape(meta["chunks"]), state["a"].numpy())
    assert (adir / "0.0").stat().st_size != 16 * 8 * 4            # really compressed, not raw
    _, back = ck.restore(state={k: torch.zeros_like(v) for k, v in state.items()})
    for k in state:
        assert torch.equal(back[k], state[k])
