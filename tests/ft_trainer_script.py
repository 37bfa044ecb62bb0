"""Trainer entry point with host-side fault injection, used by the fault-tolerance tests.

``AXB_FAULT=crash@N`` raises inside step N, ``AXB_FAULT=hang@N`` sleeps forever inside step N;
the fault fires only while the file ``AXB_FAULT_MARKER`` does not exist (it is created when the
fault fires), i.e. once per test.  All arguments go to ``launch_trainer``.
"""

import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from axlearn_b200.common import launch_trainer  # noqa: E402
from axlearn_b200.common.trainer import SpmdTrainer  # noqa: E402

fault = os.environ.get("AXB_FAULT", "")
marker = os.environ.get("AXB_FAULT_MARKER", "")
if fault:
    kind, at = fault.split("@")
    original = SpmdTrainer._run_step  # pylint: disable=protected-access

    def faulty(self, batch):
        if self.step == int(at) and marker and not os.path.exists(marker):
            with open(marker, "w", encoding="utf-8") as f:
                f.write(kind)
            if kind == "crash":
                raise RuntimeError(f"injected crash at step {self.step}")
            while True:           # "hang": the process stays alive but makes no progress
                time.sleep(1.0)
        return original(self, batch)

    SpmdTrainer._run_step = faulty  # pylint: disable=protected-access

launch_trainer.main()
