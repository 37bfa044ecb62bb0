"""Pipeline parallelism on gloo ranks must reproduce the same model run on one process."""

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


def _train(directory, mesh_axes: dict, steps: int, schedule: str = "gpipe", microbatches: int = 2, overlap: bool = True):
    sys.path.insert(0, REPO)
    from axlearn_b200.common import prng
    from axlearn_b200.common.pipeline import PipelinedTransformerLayer
    from axlearn_b200.experiments.text.gpt.common import mesh_shape_from_axes
    from tests.helpers import tiny_fuji_trainer_config

    from axlearn_b200.common.pipeline import GPipeSchedule, StreamSchedule

    stack = PipelinedTransformerLayer.default_config().set(num_stages=2, num_microbatches=microbatches)
    stack.pipeline.schedule = (StreamSchedule if schedule == "stream" else GPipeSchedule).default_config()
    stack.pipeline.overlap_transfers = overlap
    cfg = tiny_fuji_trainer_config(
        directory, max_step=steps, save_every_n_steps=1000, mesh_shape=mesh_shape_from_axes(**mesh_axes),
        hidden=32, heads=2, ffn=64, vocab=128, seq=16, batch=4, layers=4, stack_cfg=stack)
    trainer = cfg.instantiate(parent=None)
    trainer.init(prng.PRNGKey(0))
    losses = []
    data = iter(trainer.input.dataset())
    for _ in range(steps):
        losses.append(trainer.train_step(next(data))["loss"].item())
    stages = trainer.trainer_state["model"]["decoder"]["transformer"]["pipeline"]["layer"]
    w = stages["layer1"]["feed_forward"]["linear2"]["weight"]
    emb = trainer.trainer_state["model"]["decoder"]["emb"]["token_emb"]["weight"]
    return losses, w.clone(), emb.clone()


def _worker(rank, world, port, directory, steps, q, schedule="gpipe", microbatches=2, overlap=True):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q.put(to_plain((rank,) + _train(os.path.join(directory, f"r{rank}"), dict(pipeline=2), steps, schedule, microbatches, overlap)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("schedule,microbatches,overlap", [("gpipe", 2, True), ("stream", 4, True), ("stream", 2, False)])
def test_two_stage_pipeline_matches_single_process(tmp_path, schedule, microbatches, overlap):
    steps, world = 3, 2
    ref_losses, ref_w, ref_emb = _train(tmp_path / "single", {}, steps, "gpipe", microbatches)
    assert ref_w.shape[0] == 2       # both stages live on the one rank
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, str(tmp_path), steps, q, schedule, microbatches, overlap)) for r in range(world)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(world):
        rank, losses, w, emb = from_plain(q.get(timeout=120))
        got[rank] = (losses, w, emb)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for r in range(world):
        for a, b in zip(got[r][0], ref_losses):
            assert abs(a - b) < 1e-4 * abs(b), (got[r][0], ref_losses)
        # Rank r holds stage r only.
        assert got[r][1].shape[0] == 1
        assert torch.allclose(got[r][1][0], ref_w[r], atol=3e-5, rtol=1e-3)
        assert torch.allclose(got[r][2], ref_emb, atol=3e-5, rtol=1e-3)


def test_schedules_describe_the_pass():
    from axlearn_b200.common.pipeline import GPipeSchedule, StreamSchedule

    g = GPipeSchedule.default_config().set(num_stages=3, num_microbatches=6).instantiate()
    assert g.num_iterations == 8 and abs(g.bubble_fraction() - 0.25) < 1e-9
    assert g.stage_and_microbatch_at(0) == [(0, 0)] and g.stage_and_microbatch_at(2) == [(0, 2), (1, 1), (2, 0)]
    assert g.stage_and_microbatch_at(7) == [(2, 5)]
    assert [g.output_owner(i) for i in range(6)] == [2] * 6
    s = StreamSchedule.default_config().set(num_stages=3, num_microbatches=6).instantiate()
    assert [s.output_owner(i) for i in range(6)] == [0, 0, 1, 1, 2, 2]
    with pytest.raises(ValueError):
        StreamSchedule.default_config().set(num_stages=4, num_microbatches=6).instantiate()
