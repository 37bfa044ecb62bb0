"""Runtime options of a job: kernel-selection knobs, NCCL and allocator settings.

The reference tunes its runs through per-accelerator compiler option dictionaries which become
``XLA_FLAGS`` / ``compiler_options`` and can be overridden from one environment variable
(axlearn/common/compiler_options.py:18-310).  Nothing is compiled here, so the counterpart is the
set of ENVIRONMENT variables which the kernels, the collectives and the libraries underneath read
when they are first used:

* ``default_runtime_options(instance_type=..., num_gpus=..., num_nodes=...)`` returns the
  dictionary for an accelerator type and topology;
* ``AXB200_RUNTIME_OPTIONS_OVERRIDE="KEY=value,KEY2=value2"`` overrides or adds entries (same
  format and tolerance of malformed pairs as the reference's ``XLA_OPTIONS_OVERRIDE``);
* ``apply(options)`` exports them into ``os.environ`` (before the first CUDA / NCCL use) without
  touching variables which the user already set; ``env_flags_from_options`` renders them as a
  ``K=V K2=V2`` prefix for a command line (what job builders put in the container command).

``KNOBS`` documents every framework-owned variable with its default and meaning; a test keeps the
table in step with the variables that the sources read through ``os.environ`` / ``getenv``.
"""

from __future__ import annotations

import logging
import os
import re
from typing import Mapping, Optional, Union

OptionValue = Union[str, bool, int]
OVERRIDE_ENV = "AXB200_RUNTIME_OPTIONS_OVERRIDE"

# name -> (default, meaning).  Only knobs meant for users; the ``*_CASE`` variables of the C++ unit
# drivers and the launcher-set topology variables (``AXB_NUM_SLICES``, ``AXB_SLICE_INDEX``) are not
# options.
KNOBS: dict[str, tuple[str, str]] = {
    "AXB200_GEMM": ("2cta", "2cta: CTA-pair 256x256 tiles where the shape allows; 1cta: single-CTA kernels only."),
    "AXB_GEMM_SKINNY": ("2", "GEMMs of one row block: 0 general tiles, 1 64-column tiles, 2 64-column tiles and split-K."),
    "AXB_GEMM2_GROUP_M": ("", "Row blocks per raster group of the CTA-pair GEMM (empty: per-mode default)."),
    "AXB200_FLASH_FWD": ("v3", "Flash-attention forward kernel: v3 (scores in registers), v2 or v1."),
    "AXB200_FLASH_BWD": ("fused", "Flash-attention backward: fused (one kernel, 5 GEMMs) or split (dK/dV + dQ kernels)."),
    "AXB200_RMSNORM": ("warp", "RMSNorm kernels: warp (rows held in registers, where the width allows) or plain."),
    "AXB_DECODE_ATTN": ("", "head: the per-head decode-attention kernel for every layout (no row-contiguous kernel); head1 / head2: also at most 1 / 2 query heads per CTA."),
    "AXB200_MOE_GROUP_BLOCK": ("256", "Rows to which each expert's token run is padded (256: CTA-pair grouped GEMM; 128: single CTA)."),
    "AXB_MOE_PEER_EXCHANGE": ("1", "0: NCCL all-to-all for expert parallelism; 1: peer-memory exchange kernels; force: also when sizes are small."),
    "AXB200_FUSED_FSDP": ("1", "0: NCCL all-gather / reduce-scatter for FSDP instead of the GEMM-fused peer-memory paths."),
    "AXB200_COMM_SMS": ("16", "SMs left to communication kernels while a GEMM overlaps with them (0 on one GPU)."),
    "AXB200_TP_PEER": ("1", "0: NCCL all-reduce for tensor parallelism instead of the one-shot peer-memory all-reduce."),
    "AXB200_TP_PEER_MAX_BYTES": (str(2 << 30), "Largest staging buffer of the one-shot peer all-reduce; larger messages go to NCCL."),
    "AXB200_NVLS": ("0", "1: bind symmetric buffers to an NVLink multicast object and reduce with multimem instructions."),
    "AXB200_DECODE_ENGINE": ("1", "0: sample_decode stays on the eager extend_step path instead of the CUDA-graph engine."),
    "AXB_DECODE_FUSED_PUSH": ("", "1 / 0 forces the fused-epilogue push of the decode all-reduce on or off (empty: by rank count)."),
    "AXB200_STACK_SUMMARY": ("1", "0: exceptions keep their full tracebacks instead of the summary that drops framework-internal frames."),
}


def infer_gpu_type(instance_type: str) -> str:
    """``"gpu-b200-8"`` / ``"a4-highgpu-8g"`` / ``"b200"`` -> ``"b200"``; raises for anything that
    is not a GPU instance type this framework knows."""
    name = instance_type.lower()
    if re.search(r"(^|[-_])b200([-_]|$)", name) or name.startswith("a4-"):
        return "b200"
    if re.search(r"(^|[-_])gb200([-_]|$)", name) or name.startswith("a4x-"):
        return "gb200"
    raise ValueError(f"not a supported GPU instance type: {instance_type!r}")


def default_runtime_options(*, instance_type: str = "b200", num_gpus: int = 8, num_nodes: int = 1,
                            deterministic: bool = False) -> dict[str, OptionValue]:
    """Environment for one job.  Values are what this framework was measured with on 8 x B200 behind
    NVSwitch; multi-node jobs add the settings that matter once traffic leaves the NVLink domain."""
    infer_gpu_type(instance_type)
    options: dict[str, OptionValue] = {
        # The caching allocator grows segments in place instead of fragmenting 180 GB into fixed blocks.
        "PYTORCH_CUDA_ALLOC_CONF": "expandable_segments:True",
        # Kernels of different streams are picked up in launch order: the communication kernels that
        # a GEMM overlaps with must not queue behind it.
        "CUDA_DEVICE_MAX_CONNECTIONS": 32,
        "TORCH_NCCL_AVOID_RECORD_STREAMS": True,
        "TORCH_NCCL_ASYNC_ERROR_HANDLING": 1,
        "AXB200_FUSED_FSDP": num_gpus > 1,
        "AXB200_TP_PEER": num_gpus > 1,
        "AXB200_COMM_SMS": 16,
    }
    if num_gpus > 1:
        # In-switch reduction for NCCL's own all-reduce / reduce-scatter on one NVSwitch domain.
        options["NCCL_NVLS_ENABLE"] = 1
    if num_nodes > 1:
        options.update({
            "NCCL_CROSS_NIC": 0,
            "NCCL_NET_GDR_LEVEL": "PIX",
            "NCCL_IB_QPS_PER_CONNECTION": 4,
            # Expert-parallel exchanges across nodes fall back to NCCL all-to-all.
            "AXB_MOE_PEER_EXCHANGE": 0,
        })
    if deterministic:
        options.update({"CUBLAS_WORKSPACE_CONFIG": ":4096:8", "NCCL_ALGO": "Ring"})
    return _apply_overrides_from_env(options)


def _apply_overrides_from_env(options: Mapping[str, OptionValue]) -> dict[str, OptionValue]:
    override = os.environ.get(OVERRIDE_ENV)
    out = dict(options)
    if not override:
        return out
    for pair in override.split(","):
        if not pair:
            continue
        if "=" not in pair:
            logging.warning("Invalid runtime option override (missing '='): %s", pair)
            continue
        key, value = (part.strip() for part in pair.split("=", 1))
        if not key:
            logging.warning("Empty key in runtime option override: %s", pair)
            continue
        if key in out:
            logging.info("Overriding runtime option %s: %s -> %s", key, out[key], value)
        else:
            logging.info("Adding runtime option %s: %s", key, value)
        out[key] = value
    return out


def _render(value: OptionValue) -> str:
    if isinstance(value, bool):
        return "1" if value else "0"
    return str(value)


def env_from_options(options: Mapping[str, OptionValue]) -> dict[str, str]:
    return {k: _render(v) for k, v in options.items()}


def env_flags_from_options(options: Mapping[str, OptionValue]) -> str:
    """``K=V K2=V2`` for the front of a shell command."""
    return " ".join(f"{k}={v}" for k, v in env_from_options(options).items())


def apply(options: Mapping[str, OptionValue], *, environ: Optional[dict] = None, overwrite: bool = False) -> dict[str, str]:
    """Exports ``options``; a variable that is already set wins unless ``overwrite``.  Returns what
    was written.  Must run before the first kernel / collective: the knobs are read once."""
    environ = os.environ if environ is None else environ
    written = {}
    for k, v in env_from_options(options).items():
        if overwrite or k not in environ:
            environ[k] = v
            written[k] = v
    return written
