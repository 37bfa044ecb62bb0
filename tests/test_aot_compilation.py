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


def test_cost_analysis_matches_hand_counts():
    from axlearn_b200.common.aot_compilation import analyze_training_cost
    from axlearn_b200.experiments.text.gpt import c4_trainer

    cfg = c4_trainer.named_trainer_configs()["fuji-7B-v2"]()
    cost = analyze_training_cost(cfg, num_gpus=8, per_gpu_batch=4, seq_len=4096)
    assert cost.tokens_per_gpu == 4 * 4096
    # 6.48 B matrix parameters in the layer stack (8 passes with full remat) + the 134 M LM head (6).
    stack = 32 * (3 * 4096 * 4096 + 4096 * 4096 + 3 * 4096 * 11008)
    expect = 16384 * (8.0 * stack + 6.0 * 32768 * 4096)
    assert abs(cost.gemm_flops - expect) / expect < 1e-6
    per_pass = 4 * 32 * (4.0 * 4096 * 4096 * 4096 * 0.5)
    assert abs(cost.attention_flops - 4.5 * per_pass) / cost.attention_flops < 1e-6
    assert set(cost.collective_bytes) == {"parameter all-gathers", "gradient reduce-scatters"}
    # One bf16 copy of the model is gathered three times (forward, recomputation, backward) and
    # scattered once, 7/8 of it over the links.
    assert abs(cost.collective_bytes["gradient reduce-scatters"] - 2.0 * 6.61e9 * 7 / 8) / 1.2e10 < 0.05
    assert abs(cost.collective_bytes["parameter all-gathers"] / cost.collective_bytes["gradient reduce-scatters"] - 3.0) < 1e-6
    assert 600 < cost.compute_ms < 900 and "tokens/s per GPU" in cost.table()
    tp = analyze_training_cost(cfg.clone(mesh_shape=(1, 1, 1, 4, 1, 2)), num_gpus=8, per_gpu_batch=4, seq_len=4096)
    assert "tensor-parallel all-reduces" in tp.collective_bytes and abs(tp.gemm_flops * 2 - cost.gemm_flops) / cost.gemm_flops < 1e-6


def test_topology_flag_and_reference_entry_point(capsys):
    import json

    from axlearn_b200.experiments import run_aot_compilation

    rc = run_aot_compilation.main(["--module", "text.gpt.c4_trainer", "--config", "fuji-7B-v2", "--topology", "gpu-b200-16",
                                   "--json"])
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rc == 0 and out["fits"] and out["mesh"]["fsdp"] * out["mesh"]["data"] == 16
