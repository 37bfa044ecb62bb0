"""GPU system characteristics table."""

import pytest

from axlearn_b200.cloud.gcp import system_characteristics as sc
from axlearn_b200.cloud.gcp.jobset_utils import ACCELERATOR_LABELS


def test_table_is_consistent_with_the_job_builders():
    for machine, label in ACCELERATOR_LABELS.items():
        assert sc.get_system_characteristics(machine).gke_accelerator == label
    b200 = sc.get_system_characteristics("b200-8")
    assert b200.gce_machine_type == "a4-highgpu-8g" and b200.chips_per_vm == 8 and b200.memory_gb_per_chip == 180
    assert b200.accelerator_type == sc.AcceleratorType["GPU"] and b200.topology == "N/A"
    with pytest.raises(ValueError):
        sc.get_system_characteristics("v5p-8")


def test_multi_node_instance_types():
    vm, n = sc.parse_gpu_instance_type("gpu-b200-64")
    assert vm.device_type == "b200-8" and n == 8
    assert sc.parse_gpu_instance_type("gpu-a100-40gb-16")[1] == 2
    assert sc.parse_gpu_instance_type("a3-ultragpu-8g") == (sc.get_system_characteristics("h200-141gb-8"), 1)
    with pytest.raises(ValueError, match="multiple"):
        sc.parse_gpu_instance_type("gpu-b200-12")
    with pytest.raises(ValueError, match="family"):
        sc.parse_gpu_instance_type("gpu-x9-8")
