"""Launcher of split-K paged decode attention (``csrc/decode*.cu``).

Same call surface as the reference's ``echokv_vllm/kernels/decode.py``
``decode_attention`` (:44-92).  There is no PyTorch path.
"""

from __future__ import annotations

import torch

from echokv_b200 import _native as N

BLOCKS_PER_SPLIT = 16
MAX_DECODE_SPLITS = 64  # upper bound of the split grid (backend.py:67-69 of the reference caps its fixed grid alike)
EAGER_MAX_SPLITS = 32   # calls that size their own grid (the prefill row path): their scratch grows with rows x splits
MIN_SPLIT_TOKENS = 64   # smallest split `choose_blocks_per_split` proposes
ITEM_COST_TILES = 4     # fixed cost of a (sequence, split) work item in units of one 16-token tile's work


def decode_parallelism(store, num_q_heads: int) -> int:
    """Work items the split kernel has in work at once on the current device (0: generic kernel)."""
    return int(N.lib.echokv_decode_parallelism(store.c_layout, int(num_q_heads)))


def choose_blocks_per_split(lens, block_size: int, num_splits: int, slots: int) -> int:
    """Blocks per split for one decode step of sequences with cache lengths ``lens``.

    The split kernel works on ``slots`` (sequence, split) items at a time, so the step takes
    ``ceil(items / slots)`` waves of one item's time each: a split of b blocks costs ``b * block_size / 16 +
    ITEM_COST_TILES``.  Every split count up to ``num_splits`` is tried on the mean sequence and the
    cheapest wins (ties: fewer, larger splits, which leave less to merge); splits hold an even number of tiles.  The value is a launch
    parameter shared by all sequences of the step, so for a given value results stay batch-invariant.
    """
    import numpy as np

    lens = np.asarray(lens)
    live = lens[lens > 0]
    if live.size == 0 or slots <= 0:
        return BLOCKS_PER_SPLIT
    nb = int(np.ceil(np.mean(-(-live // block_size))))
    tiles = max(1, block_size // 16)
    floor = max(1, MIN_SPLIT_TOKENS // block_size)
    best = None
    for s in range(1, max(1, num_splits) + 1):
        b = max(floor, -(-nb // s))
        if (b * tiles) & 1:
            b += 1  # the kernel works a split off in pairs of tiles: an odd count leaves one tile on the slower single path
        used = -(-nb // b)
        waves = -(-(int(live.size) * used) // slots)
        cost = waves * (b * tiles + ITEM_COST_TILES)
        if best is None or cost < best[0] or (cost == best[0] and b > best[1]):
            best = (cost, b)
    return best[1]


class _Scratch:
    """Per-device split-partials buffer, grown on demand.

    The buffer starts zeroed: its first 256 bytes are the split kernel's work-queue state, which every
    call leaves at zero.  A CUDA graph holds the address of the buffer it was captured with, so a buffer that a capture has
    used is never freed: when a later call needs more bytes (more sequences than the captured sizes, the
    row path of a long prefill, another model in the same process) a larger buffer takes over and the old
    one is kept alive for the graphs that point at it.
    """

    def __init__(self) -> None:
        self.buf: dict[torch.device, torch.Tensor] = {}
        self.captured: set[torch.device] = set()
        self.retired: list[torch.Tensor] = []

    def get(self, device, nbytes: int) -> torch.Tensor:
        cur = self.buf.get(device)
        capturing = torch.cuda.is_current_stream_capturing()
        if cur is None or cur.numel() < nbytes:
            if capturing:
                raise RuntimeError("decode scratch must be sized before CUDA-graph capture (run one eager step first)")
            if cur is not None and device in self.captured:
                self.retired.append(cur)
                self.captured.discard(device)
            cur = self.buf[device] = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        if capturing:
            self.captured.add(device)
        return cur


_scratch = _Scratch()


def decode_attention(store, query: torch.Tensor, block_table: torch.Tensor, seq_lens: torch.Tensor,
                     softmax_scale: float, blocks_per_split: int = BLOCKS_PER_SPLIT,
                     q_rows: torch.Tensor | None = None, bt_rows: torch.Tensor | None = None,
                     out: torch.Tensor | None = None, max_len: int | None = None,
                     num_splits: int | None = None, bps_dev: torch.Tensor | None = None) -> torch.Tensor:
    """Attention of one query token per sequence over each sequence's cache.

    Sequence ``i`` uses query row ``q_rows[i]`` and block-table row ``bt_rows[i]``
    (default: row ``i``) with cache length ``seq_lens[i]``.  Without ``out``
    returns float32 ``[S, Hq, D]``; with ``out`` writes sequence ``i`` to
    ``out[q_rows[i]]`` in ``out``'s dtype; length-0 sequences (CUDA-graph padding)
    leave their row untouched.  Each sequence is cut into at most ``num_splits``
    splits of ``max(blocks_per_split, ceil(blocks / num_splits))`` blocks -- a
    function of the sequence alone, so results are batch-invariant.  ``bps_dev`` (one int32 on the
    device, or the low half of an int64) raises ``blocks_per_split`` at run time: a captured graph
    keeps reading it, so the host can size the splits for every replayed step.
    """
    L = store.layout
    N.require_cuda(query, block_table, seq_lens, out)
    if query.dim() != 3 or query.shape[2] != L.head_size:
        raise ValueError("query must be [T, Hq, D]")
    if query.stride(2) != 1:
        query = query.contiguous()
    hq = query.shape[1]
    s = seq_lens.shape[0]
    dev = query.device
    if block_table.dtype != torch.int32 or block_table.stride(1) != 1:
        block_table = block_table.to(torch.int32).contiguous()
    lens = seq_lens if seq_lens.dtype == torch.long and seq_lens.is_contiguous() else seq_lens.long().contiguous()
    if q_rows is not None and (q_rows.dtype != torch.long or not q_rows.is_contiguous()):
        q_rows = q_rows.long().contiguous()
    if bt_rows is not None and (bt_rows.dtype != torch.long or not bt_rows.is_contiguous()):
        bt_rows = bt_rows.long().contiguous()
    if out is None:
        out = torch.empty(query.shape[0], hq, L.head_size, device=dev, dtype=torch.float32)
    if out.stride(2) != 1:
        raise ValueError("out must have a contiguous last dim")
    if num_splits is None:
        width = block_table.shape[1]
        max_blocks = width if max_len is None else min(width, -(-max_len // L.block_size))
        num_splits = max(1, min(-(-max_blocks // blocks_per_split), EAGER_MAX_SPLITS))
    if s == 0:
        return out
    nbytes = N.lib.echokv_decode_scratch_bytes(s, hq, L.head_size, num_splits)
    scratch = _scratch.get(dev, nbytes)
    if bps_dev is not None:
        N.require_cuda(bps_dev)
        if bps_dev.dtype not in (torch.int32, torch.int64) or bps_dev.numel() < 1:
            raise TypeError("bps_dev must hold one int32 / int64 on the device")
    N.check(N.lib.echokv_decode_ex(
        store.c_layout, store.c_pages, store.c_res,
        query.data_ptr(), query.stride(0), query.stride(1), N.dtype_code(query.dtype), N.ptr(q_rows),
        block_table.data_ptr(), block_table.stride(0), N.ptr(bt_rows), lens.data_ptr(),
        scratch.data_ptr(), scratch.numel(),
        out.data_ptr(), out.stride(0), out.stride(1), N.dtype_code(out.dtype),
        float(softmax_scale), int(num_splits), int(blocks_per_split), N.ptr(bps_dev), s, hq, N.stream_ptr(dev)))
    return out
