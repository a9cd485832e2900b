"""Chunked-prefill attention over the tiered store (launchers for ``csrc/read.cu`` / ``csrc/prefill.cu``).

Call surface of the reference's ``echokv_vllm/kernels/prefill.py``
(``prefill_attention`` :170-207, ``dequant_dense`` :90-115,
``build_dequant_work`` :77-87).  A chunk's queries attend to the request's
whole stored context (this chunk included, already written), with a
bottom-right causal mask.  There is no PyTorch path.

Two device paths:
  * row path: every query token is handed to the split-K decode kernel as a
    sequence whose length is its causal limit.  Each token re-reads its context,
    so this is for short chunks (the reference's fused path has the same
    trade-off, kernels/prefill.py:10-13).
  * dense path: dequantize every context once into ``[total_ctx, H, D]`` in the
    model dtype, then run the tensor-core attention kernel over it.
"""

from __future__ import annotations

import itertools

import torch

from echokv_b200 import _native as N
from echokv_b200._util import to_device
from echokv_b200.kernels.decode import decode_attention

ROW_PATH_MAX_CHUNK = 64  # longer chunks take the dense path when it is available


def build_dequant_work(prefill, req_of, block_size: int, device) -> torch.Tensor:
    """Work list ``[n, 4]`` int32: (request, block index, dense row of the block's first token, ctx);
    contexts are packed back to back in ``prefill`` order."""
    rows = [(r, bi, g0 + bi * block_size, ctx)
            for (_, _, ctx, g0), r in zip(prefill, req_of) for bi in range(-(-ctx // block_size))]
    return to_device(torch.tensor(rows, dtype=torch.int32).reshape(-1, 4), device)


def dequant_dense(store, work: torch.Tensor, total_ctx: int, block_table: torch.Tensor, dtype):
    """Dense ``[total_ctx, H, D]`` K and V (``dtype``) of the contexts in ``work``."""
    L = store.layout
    k = torch.empty(total_ctx, L.num_kv_heads, L.head_size, device=store.device, dtype=dtype)
    v = torch.empty_like(k)
    if work.numel():
        N.require_cuda(work, block_table)
        if block_table.dtype != torch.int32 or block_table.stride(1) != 1:
            block_table = block_table.to(torch.int32).contiguous()
        N.check(N.lib.echokv_dequant_dense(
            store.c_layout, store.c_pages, store.c_res, work.data_ptr(), work.shape[0],
            block_table.data_ptr(), block_table.stride(0), k.data_ptr(), v.data_ptr(), k.stride(0), k.stride(1),
            N.dtype_code(dtype), N.stream_ptr(store.device)))
    return k, v


def build_rows(prefill, req_of, device):
    """Row-path metadata: per query token its row, its request and its causal limit (device int64)."""
    q_rows, reqs, lens = [], [], []
    for (qs, qe, ctx, _), r in zip(prefill, req_of):
        nq = qe - qs
        q_rows.extend(range(qs, qe))
        reqs.extend([r] * nq)
        lens.extend(range(ctx - nq + 1, ctx + 1))
    packed = to_device(torch.tensor([q_rows, reqs, lens], dtype=torch.long), device)
    return packed[0], packed[1], packed[2], (max(lens) if lens else 0)


def build_dense(prefill, req_of, block_size: int, device):
    """Dense-path metadata, once per step for all layers: the dequantization work list, the total
    context rows, the chunk table ``[n, 4]`` int32 (q_start, q_end, ctx, dense_start) on the device and
    the longest chunk.  Contexts are packed back to back in ``prefill`` order; the fourth field of the
    incoming tuples is recomputed, not trusted."""
    packed, at = [], 0
    for qs, qe, ctx, _ in prefill:
        packed.append((qs, qe, ctx, at))
        at += ctx
    chunks = to_device(torch.tensor(packed, dtype=torch.int32).reshape(-1, 4), device)
    return build_dequant_work(packed, req_of, block_size, device), at, chunks, max(qe - qs for qs, qe, _, _ in packed)


def dense_attention(query: torch.Tensor, k: torch.Tensor, v: torch.Tensor, chunks: torch.Tensor, max_chunk: int,
                    out: torch.Tensor, softmax_scale: float) -> None:
    """Bottom-right causal attention of each chunk's queries over its dense context (``csrc/prefill.cu``).
    ``query [T, Hq, D]`` and ``k``/``v [total_ctx, H, D]`` share one 16-bit dtype; ``out [T, Hq, D]``."""
    N.require_cuda(query, k, v, chunks, out)
    if query.dtype != k.dtype or k.dtype != v.dtype or k.stride() != v.stride():
        raise ValueError("query, K and V must share a dtype and K, V a layout")
    if query.stride(2) != 1 or k.stride(2) != 1 or out.stride(2) != 1:
        raise ValueError("the head dimension must be contiguous")
    N.check(N.lib.echokv_prefill(
        query.data_ptr(), query.stride(0), query.stride(1), k.data_ptr(), v.data_ptr(), k.stride(0), k.stride(1),
        k.shape[0], N.dtype_code(query.dtype), chunks.data_ptr(), chunks.shape[0], max_chunk, out.data_ptr(), out.stride(0),
        out.stride(1), N.dtype_code(out.dtype), softmax_scale, query.shape[1], k.shape[1], query.shape[2],
        N.stream_ptr(query.device)))


def dense_supported(store, query: torch.Tensor) -> bool:
    return query.dtype in (torch.float16, torch.bfloat16) and store.layout.head_size in (64, 128)


def prefill_attention(store, query: torch.Tensor, output: torch.Tensor, prefill, req_of, block_table: torch.Tensor,
                      softmax_scale: float, tiles=None, gather=None, dense=None, rows=None) -> None:
    """Write attention for every prefill chunk into ``output [T, Hq, D]``.

    ``prefill`` holds ``(q_start, q_end, ctx, dense_start)`` per chunk and ``req_of`` the
    block-table row of each.  ``dense`` (from ``build_dense``) selects the dense path; ``rows``
    (from ``build_rows``) lets the metadata builder prepare the row path's indices once per step
    for all layers.  With neither, chunks longer than ``ROW_PATH_MAX_CHUNK`` take the dense path
    when the dtype and head size allow it.  ``tiles`` and ``gather`` belong to the reference's
    Triton and PyTorch paths and are ignored.
    """
    if not prefill:
        return
    out3 = output.view(output.shape[0], -1, query.shape[-1])
    if dense is None and rows is None and dense_supported(store, query) and \
            max(qe - qs for qs, qe, _, _ in prefill) > ROW_PATH_MAX_CHUNK:
        dense = build_dense(prefill, req_of, store.layout.block_size, query.device)
    if dense is not None and dense_supported(store, query):
        work, total, chunks, max_chunk = dense
        k, v = dequant_dense(store, work, total, block_table, query.dtype)
        dense_attention(query, k, v, chunks, max_chunk, out3, softmax_scale)
        return
    if rows is None:
        rows = build_rows(prefill, req_of, query.device)
    q_rows, reqs, lens, max_len = rows
    decode_attention(store, query, block_table, lens, softmax_scale, q_rows=q_rows, bt_rows=reqs, out=out3,
                     max_len=max_len)
