"""Helpers shared by the host-side modules."""

from __future__ import annotations

import torch


def to_device(t: torch.Tensor, device) -> torch.Tensor:
    """Copy a host tensor to ``device`` without stalling the CPU.

    A copy from pageable memory makes the host wait for the stream; staging the
    source in pinned memory and copying with ``non_blocking=True`` lets the host
    run ahead (the caching pinned allocator keeps the staging buffer alive until
    the copy has run).  Same role as the reference's ``echokv_vllm/_util.py:8-20``.
    """
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError("echokv_b200 runs on CUDA devices only")
    return t.pin_memory().to(device, non_blocking=True)
