"""Hot ops with two implementations each: hand-written sm_100a CUDA kernels (used whenever
the operands live on a GPU in a supported dtype) and plain PyTorch (``reference``; used on
CPU and as the numerics oracle).  Layers call the functions exported here and never pick a
backend themselves.

On a machine with a GPU the CUDA extension is mandatory: if it is missing or fails to load,
the first GPU call raises instead of silently falling back.
"""

from axlearn_b200.ops.dispatch import (  # noqa: F401
    attention,
    cross_entropy,
    linear,
    lm_head_cross_entropy,
    add_rms_norm,
    rms_norm,
    rms_norm_keep_input,
    share_input_grad,
    rope,
    swiglu,
    use_reference_ops,
)
