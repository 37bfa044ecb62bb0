"""InferenceRunner / InferencePipeline: restore a trained model and run its methods."""

import json
import os

import torch

from axlearn_b200.common import inference, prng
from axlearn_b200.common.checkpointer import latest_checkpoint_path
from axlearn_b200.common.input_fake import FakeLmInput
from axlearn_b200.common.module import functional
from tests.helpers import tiny_fuji_trainer_config


def test_runner_reproduces_trainer_outputs_and_pipeline_writes_records(tmp_path):
    cfg = tiny_fuji_trainer_config(tmp_path / "run", max_step=2, save_every_n_steps=2, hidden=32, heads=2, ffn=64,
                                   vocab=64, seq=16, batch=4, layers=2)
    trainer = cfg.instantiate(parent=None)
    trainer.run(prng.PRNGKey(0))
    ckpt = latest_checkpoint_path(os.path.join(str(tmp_path / "run"), "checkpoints"))

    rcfg = inference.InferenceRunner.config_from_trainer(cfg).set(name="runner", device="cpu")
    rcfg.init_state_builder.dir = ckpt
    runner = rcfg.instantiate(parent=None)
    assert runner.step == 2
    ids = torch.randint(2, 64, (3, 16))
    batch = {"input_ids": ids}
    out = runner.create_method_runner(method="extract_logits")(batch)
    ref, _ = functional(trainer.model, prng.PRNGKey(0), trainer.trainer_state["model"], dict(input_batch=batch),
                        is_training=False, method="extract_logits")
    assert torch.allclose(out.output_batch, ref, atol=1e-5)

    pcfg = inference.InferencePipeline.default_config().set(
        name="pipe", model_method="predict",
        input=FakeLmInput.default_config().set(global_batch_size=2, source_length=16, vocab_size=64,
                                               total_num_batches=3, is_training=False),
        runner=rcfg, output_writer=inference.JsonlOutputWriter.default_config().set(
            output_dir=str(tmp_path / "out"), output_keys=["hidden_states"]))
    pipe = pcfg.instantiate(parent=None)
    assert pipe.run() == 3
    pipe.output_writer.close()
    lines = open(pipe.output_writer.path, encoding="utf-8").read().strip().split("\n")
    assert len(lines) == 6
    rec = json.loads(lines[0])
    assert len(rec["inputs/input_ids"]) == 16 and len(rec["hidden_states"]) == 16 and len(rec["hidden_states"][0]) == 32
