"""Two-GPU expert parallelism: the peer-memory exchange (rows pushed into / pulled out of the
owning GPU's memory) against the library all-to-all path.  Spawns one process per GPU."""

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
pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(rank, world, port, directory, peer, queue, drop_free=False, axis="expert"):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0", AXB_MOE_PEER_EXCHANGE="1" if peer else "0")
    sys.path.insert(0, REPO)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from axlearn_b200.common import prng
        from axlearn_b200.experiments.text.gpt import envy
        from axlearn_b200.experiments.text.gpt.common import (
            adamw_decoupled_learner_config,
            get_trainer_config_fn,
            mesh_shape_from_axes,
        )
        from axlearn_b200.ops import cuda_ops

        model = envy.preset("test", hidden_dim=256, num_heads=2, num_kv_heads=2, moe_ffn_dim=512, num_groups=1,
                            drop_free=drop_free, **(dict(load_balance_loss_weight=0.0) if drop_free else {}))
        learner = adamw_decoupled_learner_config(peak_lr=1e-3, max_step=4, weight_decay=0.1, lr_warmup_steps=1)
        cfg = get_trainer_config_fn(
            model_cfg=model, learner_cfg=learner, max_step=4, train_batch_size=4 * world, max_sequence_length=64,
            vocab_size=512, mesh_shape=mesh_shape_from_axes(**{axis: world}), save_every_n_steps=1000)()
        cfg.dir = os.path.join(directory, f"{'peer' if peer else 'nccl'}_{axis}_{rank}")
        cfg.device = f"cuda:{rank}"
        cfg.train_dtype = torch.bfloat16
        trainer = cfg.instantiate(parent=None)
        trainer.init(prng.PRNGKey(0))
        data = iter(trainer.input.dataset())
        losses = [trainer.train_step(next(data))["loss"].item() for _ in range(3)]
        torch.cuda.synchronize()
        cuda_ops.check_status()
        layer = trainer.trainer_state["model"]["decoder"]["transformer"]["repeat"]["layer"]["feed_forward"]
        queue.put(to_plain((rank, losses, layer["wo_weight"].float().cpu(), layer["gate_weight"].float().cpu(),
                            cuda_ops.launch_count)))
    finally:
        dist.destroy_process_group()


def _launch(tmp_path, peer, **kwargs):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_run, args=(r, world, port, str(tmp_path), peer, q), kwargs=kwargs) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    for _ in range(world):
        rank, *rest = from_plain(q.get(timeout=600))
        results[rank] = rest
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    return results


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_exchange_matches_all_to_all(tmp_path):
    ref = _launch(tmp_path, peer=False)
    got = _launch(tmp_path, peer=True)
    assert got[0][3] > ref[0][3], "the peer path must launch its push / pull / flag kernels"
    for rank in (0, 1):
        for a, b in zip(got[rank][0], ref[rank][0]):
            assert abs(a - b) < 2e-3 * abs(b), (got[rank][0], ref[rank][0])
        for i in (1, 2):
            a, b = got[rank][i], ref[rank][i]
            assert (a - b).abs().max().item() < 2e-2 * b.abs().max().item()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_dropfree_expert_parallel_matches_replicated_experts(tmp_path):
    """Grouped-GEMM experts split over two GPUs (tokens all-gathered, outputs reduce-scattered)
    against the same model with every expert on both GPUs (plain data parallelism)."""
    ref = _launch(tmp_path, peer=False, drop_free=True, axis="data")
    got = _launch(tmp_path, peer=False, drop_free=True, axis="expert")
    for rank in (0, 1):
        for a, b in zip(got[rank][0], ref[rank][0]):
            assert abs(a - b) < 2e-3 * abs(b), (got[rank][0], ref[rank][0])
        a, b = got[rank][2], ref[rank][2]                       # router weights: replicated in both
        assert (a - b).abs().max().item() < 2e-2 * b.abs().max().item()
    wo = torch.cat([got[0][1], got[1][1]], dim=1)              # [L, E, H, M] from the two halves
    assert wo.shape == ref[0][1].shape
    # Adam turns round-off in near-zero gradients into steps of the size of the learning rate, so
    # single elements may differ by up to 2 * lr per step; the bulk must agree.
    d = (wo - ref[0][1]).abs()
    assert d.mean().item() < 2e-4 and d.max().item() < 3 * 2 * 1e-3 + 1e-3, (d.mean().item(), d.max().item())
