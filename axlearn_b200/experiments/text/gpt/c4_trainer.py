"""Named LM trainer configs (the module passed as ``--module=text.gpt.c4_trainer``).

Parity target: axlearn/experiments/text/gpt/c4_trainer.py:111 ``named_trainer_configs``.
With ``--data_dir=FAKE`` (or no dataset reachable) inputs are synthetic uniform-random tokens.
"""

from __future__ import annotations

from axlearn_b200.experiments.text.gpt import fuji


def named_trainer_configs() -> dict:
    configs = {}
    configs.update(fuji.trainer_configs())
    from axlearn_b200.experiments.text.gpt import envy  # pylint: disable=import-outside-toplevel

    configs.update(envy.trainer_configs())
    return configs
