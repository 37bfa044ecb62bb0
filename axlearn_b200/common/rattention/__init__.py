"""Sliding-window attention plus residual linear attention over the tokens outside the window."""

from axlearn_b200.common.rattention.rattention import (  # noqa: F401
    GroupRMSNorm,
    RAttention,
    feature_map,
    residual_linear_attention,
    residual_linear_attention_reference,
)
