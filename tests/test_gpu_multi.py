"""Two-GPU checks of the fused FSDP path against the library-collective path.

Needs two visible GPUs (skipped otherwise).  Each case spawns one process per GPU over NCCL on
127.0.0.1, trains a small Fuji for two steps on both paths from the same initial state, and
compares losses and the per-layer gradient shards after the first backward.
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
pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(rank, world, port, directory, fused, queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), AXB200_FUSED_FSDP="1" if fused else "0", NCCL_NVLS_ENABLE="0")
    sys.path.insert(0, REPO)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from axlearn_b200.common import prng
        from axlearn_b200.common.base_layer import RematSpec, nothing_saveable
        from axlearn_b200.common.utils import flatten_items
        from axlearn_b200.experiments.text.gpt.common import mesh_shape_from_axes
        from axlearn_b200.ops import cuda_ops
        from tests.helpers import tiny_fuji_trainer_config

        cfg = tiny_fuji_trainer_config(
            os.path.join(directory, f"{'fused' if fused else 'nccl'}_{rank}"), max_step=4, save_every_n_steps=1000,
            train_dtype=torch.bfloat16, device=f"cuda:{rank}", mesh_shape=mesh_shape_from_axes(fsdp=world),
            hidden=512, heads=4, ffn=1024, vocab=4096, seq=256, batch=4 * world, layers=3, scan_chunk=512,
            shared_lm_head=True)
        cfg.model.decoder.transformer.layer.remat_spec = RematSpec(prevent_cse=False, policy=nothing_saveable)
        trainer = cfg.instantiate(parent=None)
        trainer.init(prng.PRNGKey(0))
        data = iter(trainer.input.dataset())
        losses, grads = [], None
        for step in range(2):
            out = trainer.train_step(next(data))
            losses.append(out["loss"].item())
            if step == 0:
                stacked = trainer._shadows["decoder"]["transformer"]["repeat"]["layer"]  # pylint: disable=protected-access
                grads = {p: t.grad.float().cpu() for p, t in flatten_items(stacked)}
        torch.cuda.synchronize()
        cuda_ops.check_status()
        queue.put(to_plain((rank, losses, grads, cuda_ops.launch_count)))
    finally:
        dist.destroy_process_group()


def _launch(tmp_path, fused):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_run, args=(r, world, port, str(tmp_path), fused, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    for _ in range(world):
        rank, losses, grads, launches = from_plain(q.get(timeout=600))
        results[rank] = (losses, grads, launches)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    return results


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_fsdp_matches_library_collectives(tmp_path):
    ref = _launch(tmp_path, fused=False)
    got = _launch(tmp_path, fused=True)
    assert got[0][2] > ref[0][2], "the fused path must launch its own signal/reduce kernels"
    for rank in (0, 1):
        for a, b in zip(got[rank][0], ref[rank][0]):
            assert abs(a - b) < 5e-3 * abs(b), (got[rank][0], ref[rank][0])
        bad = []
        for path, g in got[rank][1].items():
            r = ref[rank][1][path]
            scale = r.abs().max().item() + 1e-8
            # Per-layer errors make it obvious which slice of a stacked gradient is off.
            per_layer = [round((g[i] - r[i]).abs().max().item() / scale, 4) for i in range(g.shape[0])]
            if max(per_layer) >= 3e-2:
                bad.append((path, per_layer))
        assert not bad, (rank, bad)


def _run_tp(rank, world, port, directory, peer, big, queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), AXB200_TP_PEER="1" if peer else "0", NCCL_NVLS_ENABLE="0")
    sys.path.insert(0, REPO)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from axlearn_b200.common import prng
        from axlearn_b200.common.base_layer import RematSpec, nothing_saveable
        from axlearn_b200.common.utils import flatten_items
        from axlearn_b200.experiments.text.gpt.common import mesh_shape_from_axes
        from axlearn_b200.ops import cuda_ops
        from tests.helpers import tiny_fuji_trainer_config

        dims = dict(hidden=1024, heads=8, ffn=2048, seq=1024) if big else dict(hidden=512, heads=4, ffn=1024, seq=256)
        cfg = tiny_fuji_trainer_config(
            os.path.join(directory, f"tp_{'peer' if peer else 'nccl'}_{rank}"), max_step=4, save_every_n_steps=1000,
            train_dtype=torch.bfloat16, device=f"cuda:{rank}", mesh_shape=mesh_shape_from_axes(model=world),
            vocab=4096, batch=4, layers=2, scan_chunk=512, shared_lm_head=True, **dims)
        cfg.model.decoder.transformer.layer.remat_spec = RematSpec(prevent_cse=False, policy=nothing_saveable)
        trainer = cfg.instantiate(parent=None)
        trainer.init(prng.PRNGKey(0))
        data = iter(trainer.input.dataset())
        losses = []
        for _ in range(3):
            losses.append(trainer.train_step(next(data))["loss"].item())
        torch.cuda.synchronize()
        cuda_ops.check_status()
        stacked = trainer.trainer_state["model"]["decoder"]["transformer"]["repeat"]["layer"]
        w = {p: t.float().cpu() for p, t in flatten_items(stacked) if "linear2" in p or "o_proj" in p}
        queue.put(to_plain((rank, losses, w, cuda_ops.launch_count)))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("big", [False, True])
def test_tensor_parallel_peer_reductions_match_library_all_reduce(tmp_path, big):
    """model=2: reductions over peer memory (GEMM-epilogue stores + one summing kernel) against NCCL
    all-reduces, three training steps from the same initial state."""
    world = 2
    results = {}
    for peer in (False, True):
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        port = _free_port()
        procs = [ctx.Process(target=_run_tp, args=(r, world, port, str(tmp_path), peer, big, q)) for r in range(world)]
        for p in procs:
            p.start()
        got = {}
        for _ in range(world):
            rank, losses, w, launches = from_plain(q.get(timeout=600))
            got[rank] = (losses, w, launches)
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
        results[peer] = got
    for rank in range(world):
        ref_losses, ref_w, ref_launches = results[False][rank]
        losses, w, launches = results[True][rank]
        assert launches > ref_launches, "the peer path must launch its own push / sum kernels"
        for a, b in zip(losses, ref_losses):
            assert abs(a - b) < 5e-3 * abs(b), (losses, ref_losses)
        for path, t in w.items():
            assert (t - ref_w[path]).abs().max() < 2e-2 * ref_w[path].abs().max() + 1e-6, path


def _run_nvls(rank, world, port, queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), AXB200_NVLS="1")
    sys.path.insert(0, REPO)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from axlearn_b200.ops import cuda_ops
        from axlearn_b200.parallel import nvls

        dev = torch.device("cuda", rank)
        try:
            reducer = nvls.MultimemAllReduce(1 << 22, group=dist.group.WORLD, device=dev)
        except RuntimeError as e:
            queue.put((rank, "unavailable", str(e)))
            return
        worst = 0.0
        for n, seed in ((1 << 22, 0), (8 * 1000, 1), (1 << 20, 2)):
            g = torch.Generator(device=dev).manual_seed(seed * 10 + rank)
            x = torch.randn(n, device=dev, generator=g).bfloat16()
            got = reducer.all_reduce(x)
            ref = x.float().clone()
            dist.all_reduce(ref)
            torch.cuda.synchronize()
            cuda_ops.check_status()
            worst = max(worst, ((got.float() - ref).abs() / (ref.abs() + 1.0)).max().item())
        queue.put((rank, "ok", worst))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_multimem_all_reduce_matches_library():
    """In-switch all-reduce (multimem.ld_reduce / multimem.st on a multicast-bound symmetric buffer)
    against NCCL; skipped where the system offers no multicast address."""
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_run_nvls, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    if any(status == "unavailable" for _, status, _ in results):
        pytest.skip(f"no multicast: {results[0][2]}")
    for _, status, worst in results:
        assert status == "ok" and worst < 2e-2, results
