"""Launchers of the quantize-on-write kernels (``csrc/write.cu``).

Same call surface as the reference's ``echokv_vllm/kernels/write.py``
(``write_tokens`` :29-36, ``finalize_k`` :39-50) plus ``write_step``, the two in one launch; all read everything from
device metadata, so a CUDA graph can capture them.  There is no PyTorch path.
"""

from __future__ import annotations

import torch

from echokv_b200 import _native as N


def _rows_hd(t: torch.Tensor, what: str) -> torch.Tensor:
    if t.dim() != 3 or t.stride(2) != 1:
        raise ValueError(f"{what} must be [rows, H, D] with a contiguous last dim")
    return t


def scatter_i64(dst: torch.Tensor, idx: torch.Tensor, val: torch.Tensor) -> None:
    """``dst[idx] = val`` for int64 device tensors (one tiny kernel, no host sync)."""
    n = idx.numel()
    if n:
        N.check(N.lib.echokv_scatter_i64(dst.data_ptr(), idx.data_ptr(), val.data_ptr(), n, N.stream_ptr(dst.device)))


def write_tokens(store, key: torch.Tensor, value: torch.Tensor, meta, kref: torch.Tensor | None = None) -> None:
    """Store the ``meta.n_rows`` token rows of ``key`` / ``value`` as ``meta.tok`` says."""
    if meta.n_rows == 0:
        return
    N.require_cuda(key, value, meta.tok, kref)
    key, value = _rows_hd(key, "key"), _rows_hd(value, "value")
    if key.dtype != value.dtype:
        raise TypeError("key and value must share a dtype")
    if kref is not None and (kref.dtype != torch.float32 or kref.stride(2) != 1):
        raise ValueError("the K_ref ring must be float32 [W, H, D] with a contiguous last dim")
    tok = meta.tok
    N.check(N.lib.echokv_write_tokens(
        store.c_layout, store.c_pages,
        key.data_ptr(), key.stride(0), key.stride(1), value.data_ptr(), value.stride(0), value.stride(1),
        N.dtype_code(key.dtype), tok.data_ptr(), tok.stride(0), store.c_res,
        N.ptr(kref), 0 if kref is None else kref.stride(0), 0 if kref is None else kref.stride(1),
        meta.n_rows, N.stream_ptr(key.device)))


def finalize_k(store, key: torch.Tensor, meta, full_grid: bool = False) -> None:
    """Quantize every completed K group per channel and store its codes and stats.

    ``full_grid`` launches one CTA per token row, masked by the device-side
    count, so the host never needs the count (CUDA-graph capture).
    """
    n = meta.n_rows if full_grid else meta.n_fin
    if not n or meta.fin.numel() == 0:  # an empty ``fin`` buffer can only mean a count of 0
        return
    N.require_cuda(key, meta.fin)
    key = _rows_hd(key, "key")
    N.check(N.lib.echokv_finalize_k(
        store.c_layout, store.c_pages, key.data_ptr(), key.stride(0), key.stride(1), N.dtype_code(key.dtype),
        meta.fin.data_ptr(), meta.fin_count.data_ptr(), store.c_res, n, N.stream_ptr(key.device)))


def _stash_vector_ok(src: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> bool:
    row_bytes = out[0].numel() * out.element_size()
    return not (src.dtype != out.dtype or src.shape[1:] != out.shape[1:] or not out.is_contiguous()
                or not src[0].is_contiguous() or rows.dtype != torch.long or rows.numel() < out.shape[0] or row_bytes % 16
                or (src.stride(0) * src.element_size()) % 16 or src.data_ptr() % 16 or out.data_ptr() % 16)


def write_step(store, key: torch.Tensor, value: torch.Tensor, meta, kref: torch.Tensor | None = None,
               full_grid: bool = False, stash: tuple | None = None) -> None:
    """``finalize_k`` + ``write_tokens`` + ``gather_rows(*stash)`` of one layer in one launch.

    ``stash`` = (source rows, int64 row indices on the device, destination): the canary's query
    rows.  Stores the same bytes as the three calls in that order (which is how steps of more than
    1,024 rows run inside the library).
    """
    if stash is not None and not _stash_vector_ok(*stash):
        write_step(store, key, value, meta, kref, full_grid, None)
        gather_rows(*stash)
        return
    n_fin = (meta.n_rows if full_grid else meta.n_fin) if meta.fin.numel() else 0
    if meta.n_rows == 0 and n_fin == 0 and stash is None:
        return
    N.require_cuda(key, value, meta.tok, meta.fin, kref)
    key, value = _rows_hd(key, "key"), _rows_hd(value, "value")
    if key.dtype != value.dtype:
        raise TypeError("key and value must share a dtype")
    if kref is not None and (kref.dtype != torch.float32 or kref.stride(2) != 1):
        raise ValueError("the K_ref ring must be float32 [W, H, D] with a contiguous last dim")
    tok = meta.tok
    if stash is None:
        s_args = (None, 0, None, 0, None, 0)
    else:
        src, rows, out = stash
        N.require_cuda(src, rows, out)
        s_args = (src.data_ptr(), src.stride(0) * src.element_size(), rows.data_ptr(), out.shape[0], out.data_ptr(),
                  out[0].numel() * out.element_size())
    N.check(N.lib.echokv_write_step(
        store.c_layout, store.c_pages,
        key.data_ptr(), key.stride(0), key.stride(1), value.data_ptr(), value.stride(0), value.stride(1),
        N.dtype_code(key.dtype), tok.data_ptr(), tok.stride(0), store.c_res,
        N.ptr(kref), 0 if kref is None else kref.stride(0), 0 if kref is None else kref.stride(1),
        meta.n_rows, N.ptr(meta.fin) if n_fin else None, N.ptr(meta.fin_count) if n_fin else None, n_fin,
        *s_args, N.stream_ptr(key.device)))


def gather_rows(src: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    """``out[i] = src[rows[i]]`` along dim 0 (the canary's query stash; graph-capturable, indices on the device)."""
    N.require_cuda(src, rows, out)
    row_bytes = out[0].numel() * out.element_size()
    if not _stash_vector_ok(src, rows, out):
        torch.index_select(src, 0, rows[: out.shape[0]], out=out)  # shapes the vector kernel does not take
        return
    N.check(N.lib.echokv_gather_rows(src.data_ptr(), src.stride(0) * src.element_size(), rows.data_ptr(), out.shape[0],
                                     out.data_ptr(), row_bytes, N.stream_ptr(src.device)))
