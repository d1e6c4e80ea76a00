"""NVLink topology check run at Buffer construction.

The reference only checks devices whose name contains 'PCIE': at most two ranks, and NVML must report
an NVLink P2P path for each pair (deep_ep/utils.py:64-101). The same rule is applied here; on SXM/HGX
parts (B200) every pair is connected through NVSwitch and nothing needs checking.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist


def check_pairs(physical_ids, nvml) -> None:
    """Assert that every pair of the given physical GPU indices has an NVLink P2P path according to ``nvml``
    (a ``pynvml``-like module; tests pass a fake)."""
    nvml.nvmlInit()
    try:
        handles = [nvml.nvmlDeviceGetHandleByIndex(i) for i in physical_ids]
        for i, a in enumerate(handles):
            for j, b in enumerate(handles):
                if i >= j:
                    continue
                status = nvml.nvmlDeviceGetP2PStatus(a, b, nvml.NVML_P2P_CAPS_INDEX_NVLINK)
                assert status == nvml.NVML_P2P_STATUS_OK, \
                    f"GPU {physical_ids[i]} and GPU {physical_ids[j]} are not connected via NVLink"
    finally:
        nvml.nvmlShutdown()


def check_nvlink_connections(group: Optional["dist.ProcessGroup"], nvml=None, device_name: Optional[str] = None) -> None:
    """Assert that PCIe-form-factor GPUs of the group are NVLink-bridged (at most two ranks, NVML P2P status OK).
    ``nvml`` and ``device_name`` let tests inject a fake NVML and a device name."""
    if group is None:
        return
    if device_name is None:
        if not torch.cuda.is_available():
            return
        device_name = torch.cuda.get_device_name(torch.cuda.current_device())
    if "PCIE" not in device_name.upper():
        return
    assert group.size() <= 2, "PCIe GPUs only have pairwise NVLink connections"
    if nvml is None:
        import pynvml as nvml  # provided by nvidia-ml-py
    devices = os.environ.get("CUDA_VISIBLE_DEVICES", "0,1,2,3,4,5,6,7").strip(",").split(",")
    local = torch.cuda.current_device() if torch.cuda.is_available() else int(os.environ.get("LOCAL_RANK", "0"))
    physical = int(devices[local])
    ids = [None] * group.size()
    dist.all_gather_object(ids, physical, group)
    check_pairs(ids, nvml)
