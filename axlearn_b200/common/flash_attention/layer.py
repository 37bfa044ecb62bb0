"""FlashAttention: drop-in attention layer that always routes to the fused kernels.

Parity targets in the reference (axlearn/common/flash_attention/layer.py): ``FlashAttention``
(:30-384), ``FlashBlockSizeModifier`` (:434), ``BackendOverrideModifier`` (:464).

The reference picks among cuDNN / Pallas-Triton / XLA per backend and wraps the call in
``shard_map``.  Here there is one backend: the sm_100a kernels behind
``axlearn_b200.ops.attention`` (tcgen05 flash forward/backward for training and prefill,
split-KV kernels for decode), already invoked per rank on local heads.  Causal, segment-id,
sliding-window and logit-cap masks run inside the kernels; an arbitrary additive bias, dropout
or a logit sink take the reference-math path of the parent class.

``backend_overrides`` selects among the kernel generations that ship in the library
(``{"forward": "v3" | "v2" | "v1", "backward": "fused" | "split"}``; ``"split"`` is the
bit-reproducible backward).  ``gpu_block_size`` / ``tpu_block_size`` are accepted so that the
reference's configs and ``FlashBlockSizeModifier`` rules apply unchanged, but the sm_100a kernels
work on fixed 128 x 128 tiles (one tcgen05 accumulator of 128 TMEM lanes): any other value is
ignored with a one-time note rather than forwarded.
"""

from __future__ import annotations

import contextlib
import warnings
from typing import Optional

from axlearn_b200.common.attention import GroupedQueryAttention
from axlearn_b200.common.config import ConfigModifier, Required, REQUIRED, config_class


class FlashAttention(GroupedQueryAttention):
    @config_class
    class Config(GroupedQueryAttention.Config):
        # Kernel tile size along the key axis (the kernels choose their own tiling when None).
        tpu_block_size: int = 512
        gpu_block_size: Optional[int] = None
        backend_overrides: Optional[dict] = None
        mha_dim_to_partition_spec: dict = {}
        output_dim_to_partition_spec: dict = {}

    _KERNEL_TILE = 128
    _warned_block_size = False

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        overrides = dict(cfg.backend_overrides or {})
        unknown = set(overrides) - {"forward", "backward"}
        if unknown:
            raise ValueError(f"unknown backend_overrides keys {sorted(unknown)}; expected 'forward' / 'backward'")
        if overrides.get("forward", "v3") not in ("v1", "v2", "v3"):
            raise ValueError(f"backend_overrides['forward'] must be v1, v2 or v3, got {overrides['forward']!r}")
        if overrides.get("backward", "fused") not in ("fused", "split"):
            raise ValueError(f"backend_overrides['backward'] must be fused or split, got {overrides['backward']!r}")
        self._overrides = overrides
        bs = cfg.gpu_block_size
        if bs is not None and bs != self._KERNEL_TILE and not FlashAttention._warned_block_size:
            FlashAttention._warned_block_size = True
            warnings.warn(f"gpu_block_size={bs} ignored: the sm_100a attention kernels use {self._KERNEL_TILE}-row tiles")

    @contextlib.contextmanager
    def _kernel_selection(self):
        if not self._overrides:
            yield
            return
        from axlearn_b200.ops import flash_sm100

        prev = flash_sm100.FORWARD_VARIANT, flash_sm100.BACKWARD_VARIANT
        flash_sm100.FORWARD_VARIANT = self._overrides.get("forward", prev[0])
        flash_sm100.BACKWARD_VARIANT = self._overrides.get("backward", prev[1])
        try:
            yield
        finally:
            flash_sm100.FORWARD_VARIANT, flash_sm100.BACKWARD_VARIANT = prev

    def _forward_for_mode(self, **kwargs):
        with self._kernel_selection():
            return super()._forward_for_mode(**kwargs)


class FlashBlockSizeModifier(ConfigModifier):
    @config_class
    class Config(ConfigModifier.Config):
        tpu_block_size: Optional[int] = 512
        gpu_block_size: Optional[int] = None

    def __call__(self, cfg):
        c = self._config

        def visit(node):
            from axlearn_b200.common.config import ConfigBase

            if isinstance(node, ConfigBase):
                if getattr(node, "klass", None) is FlashAttention:
                    if c.tpu_block_size is not None:
                        node.tpu_block_size = c.tpu_block_size
                    node.gpu_block_size = c.gpu_block_size
                for _, v in node.items():
                    visit(v)
            elif isinstance(node, (list, tuple)):
                for x in node:
                    visit(x)
            elif isinstance(node, dict):
                for x in node.values():
                    visit(x)

        visit(cfg)
        return cfg


class BackendOverrideModifier(ConfigModifier):
    @config_class
    class Config(ConfigModifier.Config):
        backend_overrides: Optional[dict] = None

    def __call__(self, cfg):
        c = self._config

        def visit(node):
            from axlearn_b200.common.config import ConfigBase

            if isinstance(node, ConfigBase):
                if getattr(node, "klass", None) is FlashAttention:
                    node.backend_overrides = c.backend_overrides
                for _, v in node.items():
                    visit(v)

        visit(cfg)
        return cfg
