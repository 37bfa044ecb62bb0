"""Expert-parallel MoE training on gloo ranks must reproduce single-process training."""

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


def _train(directory, mesh_axes: dict, steps: int, num_groups: int):
    sys.path.insert(0, REPO)
    from axlearn_b200.common import prng
    from axlearn_b200.experiments.text.gpt import envy
    from axlearn_b200.experiments.text.gpt.common import (
        adamw_decoupled_learner_config,
        get_trainer_config_fn,
        mesh_shape_from_axes,
    )

    model = envy.preset("test", num_groups=num_groups)
    learner = adamw_decoupled_learner_config(peak_lr=3e-3, max_step=steps, weight_decay=0.1, lr_warmup_steps=1)
    cfg = get_trainer_config_fn(
        model_cfg=model, learner_cfg=learner, max_step=steps, train_batch_size=4, max_sequence_length=16,
        vocab_size=512, mesh_shape=mesh_shape_from_axes(**mesh_axes), save_every_n_steps=1000)()
    cfg.dir = str(directory)
    cfg.device = "cpu"
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
        # Each rank holds half of the batch: one routing group per rank = two in total.
        trainer, losses = _train(os.path.join(directory, f"r{rank}"), mesh_axes, steps, num_groups=2 // world)
        layer = trainer.trainer_state["model"]["decoder"]["transformer"]["repeat"]["layer"]["feed_forward"]
        out_queue.put(to_plain((rank, losses, layer["wo_weight"].clone(), layer["gate_weight"].clone())))
    finally:
        dist.destroy_process_group()


def test_expert_parallel_matches_single_process(tmp_path):
    steps, world = 3, 2
    ref_trainer, ref_losses = _train(tmp_path / "single", {}, steps, num_groups=2)
    ref_layer = ref_trainer.trainer_state["model"]["decoder"]["transformer"]["repeat"]["layer"]["feed_forward"]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, str(tmp_path), dict(expert=2), steps, q))
             for r in range(world)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(world):
        rank, losses, wo, gate = from_plain(q.get(timeout=120))
        got[rank] = (losses, wo, gate)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for a, b in zip(got[0][0], ref_losses):
        assert abs(a - b) < 1e-4 * abs(b), (got[0][0], ref_losses)
    # Experts live on their rank: rank r holds experts [2r, 2r + 2) of every layer.
    full_wo = torch.cat([got[0][1], got[1][1]], dim=1)
    assert full_wo.shape == ref_layer["wo_weight"].shape
    # Adam turns round-off in near-zero gradients (unfilled expert slots) into steps of the size
    # of the learning rate, so single elements may differ; the bulk must agree.
    d = (full_wo - ref_layer["wo_weight"]).abs()
    assert d.mean() < 5e-5 and d.max() < 3 * 3e-3, (d.max(), d.mean())
    dg = (got[0][2] - ref_layer["gate_weight"]).abs()
    assert dg.mean() < 5e-5, dg.mean()
