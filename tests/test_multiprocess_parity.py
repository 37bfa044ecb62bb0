"""Sharded training on several CPU (gloo) ranks must reproduce single-process training.

Each case trains the tiny Fuji for a few steps on a mesh (FSDP, tensor parallel, both) with the
same global batch and seed as a single-process run and compares the per-step losses and the
re-assembled parameters.  Ranks are real processes talking over gloo on 127.0.0.1.
"""

import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, REPO)
from tests.helpers import from_plain, to_plain  # noqa: E402  pylint: disable=wrong-import-position


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _train(directory, mesh_axes: dict, steps: int, num_kv_heads=None):
    mesh_axes = dict(mesh_axes)
    seq_mode = mesh_axes.pop("seq_parallel_mode", None)
    tp_seq = mesh_axes.pop("tp_sequence_parallel", False)
    sys.path.insert(0, REPO)
    from axlearn_b200.common import prng
    from axlearn_b200.experiments.text.gpt.common import mesh_shape_from_axes
    from tests.helpers import tiny_fuji_trainer_config

    cfg = tiny_fuji_trainer_config(
        directory, max_step=steps, save_every_n_steps=1000, mesh_shape=mesh_shape_from_axes(**mesh_axes),
        hidden=64, heads=4, ffn=128, vocab=512, seq=32, batch=4, layers=2, num_kv_heads=num_kv_heads)
    if seq_mode is not None:
        cfg.model.decoder.transformer.layer.self_attention.attention.seq_parallel_mode = seq_mode
    if tp_seq:
        cfg.model.decoder.transformer.tp_sequence_parallel = True
    trainer = cfg.instantiate(parent=None)
    trainer.init(prng.PRNGKey(0))
    losses = []
    data = iter(trainer.input.dataset())
    for _ in range(steps):
        losses.append(trainer.train_step(next(data))["loss"].item())
    return trainer, losses


def _worker(rank, world, port, directory, mesh_axes, steps, out_queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        trainer, losses = _train(os.path.join(directory, f"r{rank}"), mesh_axes, steps)
        # Reassemble one FSDP/TP-sharded weight to compare with the single-process run.
        from axlearn_b200.parallel import collectives as coll

        w = trainer.trainer_state["model"]["decoder"]["transformer"]["repeat"]["layer"]["feed_forward"]["linear2"]["weight"]
        spec = (("model", "expert", "fsdp", "seq"), None)
        with trainer.mesh():
            full = w
            for dim, entry in enumerate(spec):
                # A dim split over several axes is major-to-minor: undo the minor axis first.
                for axis in reversed(trainer.mesh().present_axes(entry)):
                    full = coll.all_gather_raw(
                        full, trainer.mesh().group(axis), trainer.mesh().axis_size(axis), dim + 1)
        if rank == 0:
            out_queue.put(to_plain((losses, full.clone())))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mesh_axes", [
    dict(fsdp=2), dict(model=2), dict(fsdp=2, model=2), dict(data=2), dict(seq=2),
    # Context parallelism: queries stay sequence-sharded, K / V are gathered over the seq axis.
    dict(seq=2, seq_parallel_mode="allgather_kv"),
    # Tensor parallelism with sequence-sharded norm / residual regions (all-gather into the
    # column-parallel linears, reduce-scatter out of the row-parallel ones).
    dict(model=2, tp_sequence_parallel=True), dict(fsdp=2, model=2, tp_sequence_parallel=True),
])
def test_sharded_matches_single_process(tmp_path, mesh_axes):
    steps = 3
    world = 1
    for v in mesh_axes.values():
        world *= v if isinstance(v, int) and not isinstance(v, bool) else 1
    ref_trainer, ref_losses = _train(tmp_path / "single", {}, steps)
    ref_w = ref_trainer.trainer_state["model"]["decoder"]["transformer"]["repeat"]["layer"]["feed_forward"]["linear2"]["weight"]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, str(tmp_path), mesh_axes, steps, q)) for r in range(world)]
    for p in procs:
        p.start()
    losses, full_w = from_plain(q.get(timeout=300))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 1e-4 * abs(b), (losses, ref_losses)
    assert torch.allclose(full_w, ref_w, atol=2e-5, rtol=1e-4)
