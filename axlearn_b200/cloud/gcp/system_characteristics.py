"""GCP accelerator system characteristics (reference: axlearn/cloud/gcp/system_characteristics.py).

The reference's table is mostly TPU slices; a GPU framework needs the GPU machine families.  A
user-facing instance type is ``<gpu>-<GPUs per VM>`` (``b200-8``, as the reference's
``h100-80gb-8``); ``gpu-<gpu>-<total GPUs>`` names a multi-node job (``gpu-b200-64`` = 8 VMs).
"""

from __future__ import annotations

import dataclasses
import re

AcceleratorType = {"TPU": 1, "GPU": 2, "CPU": 3}  # pylint: disable=invalid-name


@dataclasses.dataclass(frozen=True)
class SystemCharacteristics:
    topology: str                 # "N/A" for GPU machines: NVLink domains are whole VMs
    vms_per_slice: int
    gke_accelerator: str          # the cloud.google.com/gke-accelerator node label
    gce_machine_type: str
    chips_per_vm: int
    accelerator_type: int
    device_type: str
    memory_gb_per_chip: int = 0


def _gpu(name: str, label: str, machine: str, chips: int, mem: int) -> SystemCharacteristics:
    return SystemCharacteristics("N/A", 1, label, machine, chips, AcceleratorType["GPU"], name, mem)


USER_FACING_NAME_TO_SYSTEM_CHARACTERISTICS = {
    "a100-40gb-1": _gpu("a100-40gb-1", "nvidia-tesla-a100", "a2-highgpu-1g", 1, 40),
    "a100-40gb-2": _gpu("a100-40gb-2", "nvidia-tesla-a100", "a2-highgpu-2g", 2, 40),
    "a100-40gb-4": _gpu("a100-40gb-4", "nvidia-tesla-a100", "a2-highgpu-4g", 4, 40),
    "a100-40gb-8": _gpu("a100-40gb-8", "nvidia-tesla-a100", "a2-highgpu-8g", 8, 40),
    "h100-80gb-8": _gpu("h100-80gb-8", "nvidia-h100-80gb", "a3-highgpu-8g", 8, 80),
    "h100-mega-80gb-8": _gpu("h100-mega-80gb-8", "nvidia-h100-mega-80gb", "a3-megagpu-8g", 8, 80),
    "h200-141gb-8": _gpu("h200-141gb-8", "nvidia-h200-141gb", "a3-ultragpu-8g", 8, 141),
    "b200-8": _gpu("b200-8", "nvidia-b200", "a4-highgpu-8g", 8, 180),
    "gb200-4": _gpu("gb200-4", "nvidia-gb200", "a4x-highgpu-4g", 4, 186),
}

GCE_MACHINE_TYPE_TO_SYSTEM_CHARACTERISTICS = {c.gce_machine_type: c for c in USER_FACING_NAME_TO_SYSTEM_CHARACTERISTICS.values()}


def get_system_characteristics(instance_type: str) -> SystemCharacteristics:
    """By user-facing name or GCE machine type."""
    found = (USER_FACING_NAME_TO_SYSTEM_CHARACTERISTICS.get(instance_type)
             or GCE_MACHINE_TYPE_TO_SYSTEM_CHARACTERISTICS.get(instance_type))
    if found is None:
        raise ValueError(f"unknown instance type {instance_type!r}; known: {sorted(USER_FACING_NAME_TO_SYSTEM_CHARACTERISTICS)}")
    return found


def parse_gpu_instance_type(instance_type: str) -> tuple[SystemCharacteristics, int]:
    """``gpu-<family>-<total GPUs>`` -> (characteristics of one VM, number of VMs); a bare user-facing
    name or machine type is one VM."""
    m = re.fullmatch(r"gpu-([a-z0-9-]+?)-(\d+)", instance_type)
    if m is None:
        return get_system_characteristics(instance_type), 1
    family, total = m.group(1), int(m.group(2))
    candidates = [c for name, c in USER_FACING_NAME_TO_SYSTEM_CHARACTERISTICS.items() if name.rsplit("-", 1)[0] == family]
    if not candidates:
        raise ValueError(f"unknown GPU family {family!r} in {instance_type!r}")
    vm = max(candidates, key=lambda c: c.chips_per_vm)
    if total % vm.chips_per_vm:
        raise ValueError(f"{instance_type}: {total} GPUs is not a multiple of {vm.chips_per_vm} per {vm.gce_machine_type}")
    return vm, total // vm.chips_per_vm
