"""The launcher records the resolved config and its flags before it runs the trainer
(reference: axlearn/common/launch_trainer.py:192-217)."""

import json

from axlearn_b200.common import launch_trainer


def test_launcher_writes_config_and_flags_and_trains(tmp_path):
    run_dir = tmp_path / "run"
    launch_trainer.main(["--module", "text.gpt.c4_trainer", "--config", "fuji-test-v1", "--trainer_dir", str(run_dir),
                         "--max_step", "2", "--device", "cpu"])
    text = (run_dir / "trainer_config").read_text()
    assert "max_step: 2" in text and "model.decoder.transformer.num_layers" in text
    flags = json.loads((run_dir / "launch_trainer_flags").read_text())
    assert flags["config"] == "fuji-test-v1" and flags["max_step"] == 2 and flags["trainer_dir"] == str(run_dir)
