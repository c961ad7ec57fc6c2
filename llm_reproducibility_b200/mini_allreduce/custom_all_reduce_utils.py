"""Eligibility probes for the peer-to-peer all-reduce (reference: mini_allreduce/custom_all_reduce_utils.py)."""
import logging
import os
from typing import List

import torch

logger = logging.getLogger(__name__)

try:
    import pynvml

    _HAS_NVML = True
except Exception as exc:  # pragma: no cover - depends on the image
    _HAS_NVML = False
    logger.warning("pynvml not available: %r", exc)


def gpu_p2p_access_check(src: int, tgt: int) -> bool:
    """True if device `src` can map device `tgt`'s memory (driver report)."""
    if os.getenv("SGLANG_SKIP_P2P_CHECK", "0") == "1":
        logger.info("Skipping P2P check; using driver report only.")
    return torch.cuda.can_device_access_peer(src, tgt)


def is_full_nvlink(physical_device_ids: List[int], world_size: int, nvml=None) -> bool:
    """True if every pair of the given GPUs is connected by NVLink (NVML P2P status).

    `nvml` lets tests substitute a fake of the pynvml module.
    """
    nvml = nvml or (pynvml if _HAS_NVML else None)
    if nvml is None:
        logger.warning("NVML unavailable; assuming no full NVLink.")
        return False
    nvml.nvmlInit()
    try:
        handles = [nvml.nvmlDeviceGetHandleByIndex(i) for i in physical_device_ids]
        for i in range(len(handles)):
            for j in range(i + 1, len(handles)):
                try:
                    st = nvml.nvmlDeviceGetP2PStatus(handles[i], handles[j], nvml.NVML_P2P_CAPS_INDEX_NVLINK)
                except nvml.NVMLError:
                    logger.exception("NVLink detection failed; assuming False.")
                    return False
                if st != nvml.NVML_P2P_STATUS_OK:
                    return False
        return True
    finally:
        nvml.nvmlShutdown()


def is_weak_contiguous(inp: torch.Tensor) -> bool:
    """Contiguous, or occupying exactly the tail of its storage (e.g. a permuted contiguous slice)."""
    return inp.is_contiguous() or (
        inp.untyped_storage().nbytes() - inp.storage_offset() * inp.element_size()
        == inp.numel() * inp.element_size()
    )
