"""Evaler: policies, summary accumulation over eval batches, composite / global calculators, and
evaluation from inside the trainer loop."""

import torch

from axlearn_b200.common import evaler, prng
from axlearn_b200.common.config import config_for_function
from axlearn_b200.common.input_fake import FakeLmInput
from axlearn_b200.common.metrics import WeightedSummary
from axlearn_b200.experiments.text.gpt import fuji
from tests.helpers import tiny_fuji_trainer_config


def _model():
    cfg = fuji.model_config(num_layers=1, hidden_dim=32, num_heads=2, num_kv_heads=None, vocab_size=64,
                            rope_theta=1e4, shared_lm_head=True, ffn_dim=64)
    model = cfg.set(name="model").instantiate(parent=None)
    return model, model.initialize_parameters_recursively(prng.PRNGKey(0))


def _input(batches=3):
    return FakeLmInput.default_config().set(
        global_batch_size=4, source_length=16, vocab_size=64, total_num_batches=batches, is_training=False)


def test_every_n_steps_policy():
    p = evaler.every_n_steps_policy(n=5, min_step=3, max_step=12)
    assert [s for s in range(1, 14) if p(step=s, train_summaries={})] == [5, 10, 12]


def test_spmd_evaler_accumulates_model_summaries(tmp_path):
    model, params = _model()
    cfg = evaler.SpmdEvaler.default_config().set(
        name="eval", input=_input(3), dir=str(tmp_path),
        eval_policy=config_for_function(evaler.every_n_steps_policy).set(n=2))
    ev = cfg.instantiate(parent=None, model=model)
    key = prng.PRNGKey(1)
    _, summaries, outputs = ev.eval_step(1, prng_key=key, model_params=params)
    assert summaries is None and outputs is None          # policy says no
    _, summaries, outputs = ev.eval_step(2, prng_key=key, model_params=params, return_aux=True)
    assert len(outputs) == 3
    loss = summaries["loss"]
    # Weights are live-target counts (targets equal to the padding id do not count).
    assert isinstance(loss, WeightedSummary) and 3 * 4 * 16 - 12 <= float(loss.weight) <= 3 * 4 * 16
    # The accumulated loss is the (weighted) mean of the per-batch losses.
    per_batch = torch.stack([o["loss"] for o in outputs])
    assert abs(float(loss.mean) - per_batch.mean().item()) < 2e-2
    assert (tmp_path / "summaries" / "eval").exists()


def test_composite_and_global_calculators(tmp_path):
    model, params = _model()

    def metric_fn(outputs):
        n = sum(o.predict_outputs["hidden_states"].shape[0] for o in outputs)
        return {"num_examples": n}

    calc = evaler.CompositeMetricCalculator.default_config().set(metric_calculators={
        "summaries": evaler.ModelSummaryAccumulator.default_config(),
        "global": evaler.GlobalMetricCalculator.default_config().set(metric_fn=metric_fn),
    })
    ev = evaler.SpmdEvaler.default_config().set(
        name="eval", input=_input(2), dir=str(tmp_path), metric_calculator=calc).instantiate(parent=None, model=model)
    _, summaries, _ = ev.eval_step(1, prng_key=prng.PRNGKey(0), model_params=params)
    assert "summaries/loss" in summaries and float(summaries["global/num_examples"].mean) == 8


def test_trainer_runs_evalers_and_best_metric_policy_sees_them(tmp_path):
    cfg = tiny_fuji_trainer_config(tmp_path, max_step=4, save_every_n_steps=100, hidden=32, heads=2, ffn=64,
                                   vocab=64, seq=16, batch=4, layers=1)
    cfg.evalers = {"heldout": evaler.SpmdEvaler.default_config().set(
        input=FakeLmInput.default_config().set(global_batch_size=4, source_length=16, vocab_size=64,
                                               total_num_batches=2),
        eval_policy=config_for_function(evaler.every_n_steps_policy).set(n=2))}
    trainer = cfg.instantiate(parent=None)
    trainer.run(prng.PRNGKey(0))
    assert trainer.heldout.last_eval_seconds is not None
    files = list((tmp_path / "summaries" / "heldout").iterdir())
    assert files


def test_evaler_traces_chosen_batches_and_writes_outputs(tmp_path):
    import json
    import os

    from axlearn_b200.common.inference import JsonlOutputWriter

    model, params = _model()
    cfg = evaler.SpmdEvaler.default_config().set(
        name="eval", input=_input(3), dir=str(tmp_path), trace_at_iters=[1],
        output_writer=JsonlOutputWriter.default_config().set(output_dir=str(tmp_path / "out"), include_inputs=True),
        eval_policy=config_for_function(evaler.every_n_steps_policy).set(n=1))
    ev = cfg.instantiate(parent=None, model=model)
    key = prng.PRNGKey(1)
    for step in range(1, 6):
        ev.eval_step(step, prng_key=key, model_params=params)
    traces = sorted(os.listdir(tmp_path / "summaries" / "eval" / "traces"))
    # Batch 1 of the first THREE evaluations only.
    assert traces == [f"eval_step{s:08d}_batch1.json" for s in (1, 2, 3)]
    with open(tmp_path / "summaries" / "eval" / "traces" / traces[0]) as f:
        assert "traceEvents" in json.load(f)
    rows = [json.loads(line) for line in open(ev.output_writer.path)]
    assert len(rows) == 5 * 3 * 4 and "inputs/input_ids" in rows[0]          # 5 evals x 3 batches x 4 examples
