"""Absolute canary: a full-precision K_ref ring per layer and the per-tier attention KL.

    delta_b = KL( softmax(Q . K~_b^T * s) || softmax(Q . K_ref^T * s) ),   b in {2, 4, 8}

K_ref holds the most recent ``window`` keys in float32, captured by the write
kernel before they are quantized, so the measurement never reads the cache and
the controller's own decisions cannot feed back into it.  K~_b is the storage
round trip of K_ref in the cache's exact K format (per channel over consecutive
groups of ``k_group`` tokens).  Interface of the reference's
``echokv_vllm/canary.py`` (``ring_view`` :19-23, ``KRefRing`` :26-56,
``canary_kl`` :59-89); the arithmetic runs in one CUDA kernel
(``csrc/canary.cu``) for all layers at once.
"""

from __future__ import annotations

import torch

from echokv_b200 import _native as N
from echokv_b200.quant import SUPPORTED_BITS


def ring_view(buf: torch.Tensor, pos: int, fill: int, dim: int = 0) -> torch.Tensor:
    """The ``fill`` keys of a ring buffer along ``dim``, oldest first (``pos`` = next write)."""
    if fill < buf.shape[dim]:
        return buf.narrow(dim, 0, fill)
    return torch.roll(buf, -pos, dims=dim)


class KRefRing:
    """Host-driven circular buffer of the last ``window`` keys, ``[window, H, D]`` float32 on the GPU."""

    def __init__(self, window: int) -> None:
        if window < 2:
            raise ValueError("K_ref window must be >= 2")
        self.window = window
        self.buf: torch.Tensor | None = None
        self.fill = 0
        self.pos = 0

    def push(self, keys: torch.Tensor) -> None:
        keys = keys[-self.window:].float()
        t = keys.shape[0]
        if t == 0:
            return
        if self.buf is None:
            self.buf = torch.zeros(self.window, *keys.shape[1:], device=keys.device)
        head = min(t, self.window - self.pos)
        self.buf[self.pos: self.pos + head] = keys[:head]
        if head < t:
            self.buf[: t - head] = keys[head:]
        self.pos = (self.pos + t) % self.window
        self.fill = min(self.window, self.fill + t)

    def view(self) -> torch.Tensor | None:
        if self.buf is None or self.fill < 2:
            return None
        return ring_view(self.buf, self.pos, self.fill)


def canary_kl_ring(query: torch.Tensor, kref: torch.Tensor, ring_pos: int, ring_fill: int, k_group: int,
                   softmax_scale: float, out: torch.Tensor | None = None) -> torch.Tensor:
    """KL at 2, 4 and 8 bits for every layer: float32 ``[L, 3]``.

    ``query`` ``[L, nq, Hq, D]`` (any supported dtype), ``kref`` float32 ``[L, W, H, D]`` ring
    buffers with write cursor ``ring_pos`` and ``ring_fill`` valid keys.  Only the newest
    ``floor(fill / k_group) * k_group`` keys are scored (a partial group would sit in the cache's
    full-precision residual and contribute no error).
    """
    N.require_cuda(query, kref)
    if query.dim() != 4 or kref.dim() != 4 or query.shape[0] != kref.shape[0] or query.shape[3] != kref.shape[3]:
        raise ValueError("query must be [L, nq, Hq, D] and kref [L, W, H, D]")
    if kref.dtype != torch.float32 or kref.stride(3) != 1 or query.stride(3) != 1:
        raise ValueError("kref must be float32 and both tensors contiguous in the last dim")
    if (ring_fill // k_group) * k_group == 0:
        raise ValueError(f"K_ref has {ring_fill} keys, fewer than k_group={k_group}")
    L, nq, hq, d = query.shape
    w, h = kref.shape[1], kref.shape[2]
    if out is None:
        out = torch.empty(L, 3, dtype=torch.float32, device=query.device)
    N.check(N.lib.echokv_canary_kl(
        query.data_ptr(), N.dtype_code(query.dtype), query.stride(0), query.stride(1), query.stride(2),
        kref.data_ptr(), kref.stride(0), kref.stride(1), kref.stride(2), ring_pos, ring_fill, w,
        L, nq, hq, h, d, k_group, float(softmax_scale), out.data_ptr(), N.stream_ptr(query.device)))
    return out


def canary_kl(query: torch.Tensor, kref: torch.Tensor, bits: tuple[int, ...], k_group: int,
              softmax_scale: float) -> torch.Tensor:
    """Mean per-head, per-query KL at each tier in ``bits``; float32 ``[..., len(bits)]``.

    ``query`` ``[..., nq, Hq, D]``; ``kref`` ``[..., W, H, D]`` oldest key first; leading dims
    (e.g. layers) are independent problems.
    """
    for b in bits:
        if b not in SUPPORTED_BITS:
            raise ValueError(f"unsupported bits: {b}")
    lead = query.shape[:-3]
    q4 = query.reshape(-1, *query.shape[-3:])
    k4 = kref.reshape(-1, *kref.shape[-3:]).float().contiguous()
    if q4.stride(3) != 1:
        q4 = q4.contiguous()
    full = canary_kl_ring(q4, k4, 0, k4.shape[1], k_group, softmax_scale)
    cols = [SUPPORTED_BITS.index(b) for b in bits]
    return full[:, cols].reshape(*lead, len(bits))


def tp_mean(x: torch.Tensor, group=None) -> torch.Tensor:
    """Average ``x`` over the tensor-parallel ranks (each rank's canary sees only its own KV heads),
    so every rank takes the same tier decision -- the reference's ``backend._tp_mean``
    (echokv_vllm/backend.py:665-675).  One small all-reduce (NCCL on GPUs); a no-op without a
    process group or with a single rank."""
    import torch.distributed as dist

    if not dist.is_available() or not dist.is_initialized():
        return x
    world = dist.get_world_size(group)
    if world == 1:
        return x
    dist.all_reduce(x, op=dist.ReduceOp.SUM, group=group)
    return x.div_(world)
