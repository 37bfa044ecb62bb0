"""FlashAttention: drop-in attention layer that always routes to the fused kernels.

Parity targets in the reference (axlearn/common/flash_attention/layer.py): ``FlashAttention``
(:30-384), ``FlashBlockSizeModifier`` (:434), ``BackendOverrideModifier`` (:464).

The reference picks among cuDNN / Pallas-Triton / XLA per backend and wraps the call in
``shard_map``.  Here there is one backend: the sm_100a kernels behind
``axlearn_b200.ops.attention`` (tcgen05 flash forward/backward for training and prefill,
split-KV kernels for decode), already invoked per rank on local heads; unsupported bias forms
fall back to the reference-math path of the parent class.  The block-size knob is kept for
config compatibility and forwarded to the kernel launcher.
"""

from __future__ import annotations

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
