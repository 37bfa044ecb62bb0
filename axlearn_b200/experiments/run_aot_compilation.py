"""Plans a trainer config without hardware (reference: axlearn/experiments/run_aot_compilation.py).

    python -m axlearn_b200.experiments.run_aot_compilation --module=text.gpt.c4_trainer --config=fuji-7B-v2 \\
        --topology=gpu-b200-64 [--cost]

The reference compiles the training step ahead of time for a TPU topology and prints what the
compiler reports.  Nothing is compiled here; the same question -- does this config fit this many
accelerators, and what will a step cost -- is answered from the parameter specs and the mesh by
``common/aot_compilation.py`` (per-GPU memory plan; ``--cost``: FLOPs, bytes per collective and a
step-time estimate at the measured rates).  This module is that tool under the reference's name.
"""

from axlearn_b200.common.aot_compilation import main

if __name__ == "__main__":
    raise SystemExit(main())
