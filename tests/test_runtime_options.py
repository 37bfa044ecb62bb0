"""Runtime options (the counterpart of axlearn/common/compiler_options.py)."""

import os
import re
import subprocess

import pytest

from axlearn_b200.common import runtime_options as ro


def test_gpu_type():
    assert ro.infer_gpu_type("gpu-b200-8") == ro.infer_gpu_type("a4-highgpu-8g") == ro.infer_gpu_type("B200") == "b200"
    assert ro.infer_gpu_type("a4x-highgpu-4g") == "gb200"
    with pytest.raises(ValueError):
        ro.infer_gpu_type("tpu-v5p-128")


def test_defaults_and_topology(monkeypatch):
    monkeypatch.delenv(ro.OVERRIDE_ENV, raising=False)
    one = ro.default_runtime_options(num_gpus=1)
    assert one["AXB200_FUSED_FSDP"] is False and "NCCL_NVLS_ENABLE" not in one
    node = ro.default_runtime_options(num_gpus=8)
    assert node["AXB200_FUSED_FSDP"] is True and node["NCCL_NVLS_ENABLE"] == 1 and "NCCL_CROSS_NIC" not in node
    multi = ro.default_runtime_options(num_gpus=8, num_nodes=4, deterministic=True)
    assert multi["AXB_MOE_PEER_EXCHANGE"] == 0 and multi["NCCL_ALGO"] == "Ring"
    flags = ro.env_flags_from_options(node)
    assert "AXB200_FUSED_FSDP=1" in flags.split() and "PYTORCH_CUDA_ALLOC_CONF=expandable_segments:True" in flags.split()


def test_env_override(monkeypatch):
    monkeypatch.setenv(ro.OVERRIDE_ENV, "AXB200_COMM_SMS=24,,bad,=x,NEW_KEY=a=b, NCCL_NVLS_ENABLE = 0 ")
    opts = ro.default_runtime_options(num_gpus=8)
    assert opts["AXB200_COMM_SMS"] == "24" and opts["NEW_KEY"] == "a=b" and opts["NCCL_NVLS_ENABLE"] == "0"
    assert "bad" not in opts and "" not in opts


def test_apply_respects_user_settings():
    env = {"AXB200_COMM_SMS": "8"}
    written = ro.apply({"AXB200_COMM_SMS": 16, "AXB200_TP_PEER": True}, environ=env)
    assert env == {"AXB200_COMM_SMS": "8", "AXB200_TP_PEER": "1"} and written == {"AXB200_TP_PEER": "1"}
    ro.apply({"AXB200_COMM_SMS": 16}, environ=env, overwrite=True)
    assert env["AXB200_COMM_SMS"] == "16"


def test_knob_table_matches_the_sources():
    root = os.path.dirname(os.path.dirname(os.path.abspath(ro.__file__)))
    read = set()
    pattern = re.compile(r"(?:environ(?:\.get)?[\[(]|getenv\()\s*\"((?:AXB200|AXB)_[A-Z0-9_]+)\"")
    for dirpath, _, files in os.walk(root):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cc", ".cpp")) and f != "runtime_options.py":
                with open(os.path.join(dirpath, f), encoding="utf-8", errors="ignore") as fh:
                    read |= set(pattern.findall(fh.read()))
    # Variables of the C++ unit drivers and the ones a launcher sets to describe the topology.
    read = {n for n in read if not n.endswith("_CASE")} - {"AXB_NUM_SLICES", "AXB_SLICE_INDEX", ro.OVERRIDE_ENV}
    assert read - set(ro.KNOBS) == set(), read - set(ro.KNOBS)
    assert set(ro.KNOBS) - read == set(), set(ro.KNOBS) - read
