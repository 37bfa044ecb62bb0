"""Memory planning from parameter specs and the mesh (no devices involved)."""

import pytest

from axlearn_b200.common import aot_compilation
from axlearn_b200.common.aot_compilation import GIB, plan_training_memory
from axlearn_b200.experiments.text.gpt import fuji


def test_fuji_7b_plan_on_eight_gpus():
    cfg = fuji.trainer_configs()["fuji-7B-v2"]()
    plan = plan_training_memory(cfg, num_gpus=8, per_gpu_batch=4, seq_len=4096)
    assert plan.mesh["fsdp"] == 8 and plan.mesh["data"] == 1
    assert 6.5e9 < plan.total_params < 6.8e9
    # Everything but the (replicated) norm scales is sharded 8 ways.
    assert plan.local_params == pytest.approx(plan.total_params / 8, rel=0.17)
    b = plan.bytes_per_gpu
    assert b["fp32 master parameters"] == pytest.approx(4 * plan.local_params)
    assert b["optimizer moments (x2, fp32)"] == pytest.approx(8 * plan.local_params)
    assert b["layer-input checkpoints (full remat)"] == pytest.approx(2 * 4 * 4096 * 4096 * 32)
    assert 0.5 * GIB < b["FSDP gather buffers (2 layers)"] < 1.0 * GIB       # 2 x 202 M bf16 parameters
    assert plan.fits and "fits" in plan.table()
    # Twice the GPUs over the data axis: same per-GPU state.
    plan16 = plan_training_memory(cfg, num_gpus=16, per_gpu_batch=4, seq_len=4096)
    assert plan16.mesh["data"] == 2
    assert plan16.bytes_per_gpu["fp32 master parameters"] == pytest.approx(b["fp32 master parameters"])


def test_70b_does_not_fit_eight_gpus_and_cli(capsys):
    cfg = fuji.trainer_configs()["fuji-70B-v2"]()
    plan = plan_training_memory(cfg, num_gpus=8, per_gpu_batch=1, seq_len=4096)
    assert not plan.fits
    state = sum(v for k, v in plan.bytes_per_gpu.items() if "master" in k or "moments" in k)
    assert state > 95 * GIB
    rc = aot_compilation.main(["--module", "text.gpt.c4_trainer", "--config", "fuji-7B-v2", "--num_gpus", "8", "--per_gpu_batch", "4", "--json"])
    assert rc == 0 and '"fits": true' in capsys.readouterr().out
    with pytest.raises(ValueError):           # fsdp=8 x data=-1 cannot be laid out on 3 GPUs
        plan_training_memory(fuji.trainer_configs()["fuji-7B-v2"](), num_gpus=3)
