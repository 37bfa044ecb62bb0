"""Expert-parallel drop-free MoE (grouped-GEMM layer) on gloo ranks must reproduce single-process
training: tokens are all-gathered over the expert axis, every rank runs its own experts, partial
outputs are reduce-scattered back."""

import os
import socket
import sys

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


def _train(directory, mesh_axes: dict, steps: int):
    sys.path.insert(0, REPO)
    from axlearn_b200.common import prng
    from axlearn_b200.experiments.text.gpt import envy
    from axlearn_b200.experiments.text.gpt.common import (
        adamw_decoupled_learner_config,
        get_trainer_config_fn,
        mesh_shape_from_axes,
    )

    # fp32 compute: with experts on several ranks a token's K expert outputs are summed across
    # ranks in the activation dtype (three bf16 roundings instead of one), which is harmless for
    # training but not bit-comparable.  The load-balance loss is a product of per-batch means (not additive over ranks), so it is
    # switched off for the comparison; the z-loss is a plain mean and stays.
    model = envy.preset("test", drop_free=True, load_balance_loss_weight=0.0)
    learner = adamw_decoupled_learner_config(peak_lr=3e-3, max_step=steps, weight_decay=0.1, lr_warmup_steps=1)
    cfg = get_trainer_config_fn(
        model_cfg=model, learner_cfg=learner, max_step=steps, train_batch_size=4, max_sequence_length=16,
        vocab_size=512, mesh_shape=mesh_shape_from_axes(**mesh_axes), save_every_n_steps=1000,
        train_dtype=torch.float32)()
    cfg.dir = str(directory)
    cfg.device = "cpu"
    trainer = cfg.instantiate(parent=None)
    trainer.init(prng.PRNGKey(0))
    losses = []
    data = iter(trainer.input.dataset())
    for _ in range(steps):
        losses.append(trainer.train_step(next(data))["loss"].item())
    return trainer, losses


def _ffn(trainer):
    return trainer.trainer_state["model"]["decoder"]["transformer"]["repeat"]["layer"]["feed_forward"]


def _worker(rank, world, port, directory, mesh_axes, steps, out_queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        trainer, losses = _train(os.path.join(directory, f"r{rank}"), mesh_axes, steps)
        layer = _ffn(trainer)
        out_queue.put(to_plain((rank, losses, layer["wo_weight"].clone(), layer["gate_weight"].clone())))
    finally:
        dist.destroy_process_group()


def test_dropfree_expert_parallel_matches_single_process(tmp_path):
    steps, world = 3, 2
    ref_trainer, ref_losses = _train(tmp_path / "single", {}, steps)
    ref_layer = _ffn(ref_trainer)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, str(tmp_path), dict(expert=2), steps, q))
             for r in range(world)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(world):
        rank, losses, wo, gate = from_plain(q.get(timeout=180))
        got[rank] = (losses, wo, gate)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for a, b in zip(got[0][0], ref_losses):
        assert abs(a - b) < 1e-4 * abs(b), (got[0][0], ref_losses)
    # Experts live on their rank: rank r holds its half of the experts of every layer.
    full_wo = torch.cat([got[0][1], got[1][1]], dim=1)
    assert full_wo.shape == ref_layer["wo_weight"].shape
    d = (full_wo - ref_layer["wo_weight"]).abs()
    assert d.mean() < 5e-5 and d.max() < 3 * 3e-3, (d.max(), d.mean())
    dg = (got[0][2] - ref_layer["gate_weight"]).abs()
    assert dg.mean() < 5e-5, dg.mean()
