"""Per-block mixed-precision paged KV store inside a vLLM page budget (host side).

Drop-in for the reference's ``echokv_vllm/tiered_cache.py`` (``TieredLayout``
:76-147, ``TieredKVCache`` :150-482) with the device work done by the sm_100a
kernels of ``libechokv_b200.so``.  The byte layout of a page is unchanged (and
checked bit for bit against the reference):

    header   block_size bytes: [0] tier (0 never opened, else 2/4/8), [1] mask of
             K groups sealed early, [4:16] three int32 ids of extra pool chunks
    V stats  fp16 scale, fp16 min, each [block_size, H, D / v_group]
    K stats  fp16 scale, fp16 min, each [block_size / k_group, H, D]
    data     mem_bits / 2 chunks of block_size * H * D / 2 bytes; token rows are
             [K codes | V codes]; chunk j holds tokens [j * tpc, (j + 1) * tpc),
             tpc = 2 * block_size / bits

A block's tier is fixed when its offset 0 is written (forward-only rule).  An
INT2 block lives in chunk 0 of its own page; INT4 needs one extra chunk and
INT8 three, taken from a per-layer pool of the chunk slots 1.. of every page.
The pool is managed on the host (every input of an allocation decision is
host-known); the device only receives 16-byte page headers.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch
from torch.profiler import record_function

from echokv_b200 import _native as N
from echokv_b200._util import to_device
from echokv_b200.quant import EXTRA_CHUNKS, SUPPORTED_BITS
from echokv_b200.write_plan import Eviction, SharedState, WriteMeta, WritePlan, stage_plan

NEXTRA = EXTRA_CHUNKS


@dataclass(frozen=True)
class TieredLayout:
    num_kv_heads: int
    head_size: int
    block_size: int
    mem_bits: int
    k_group: int = 32
    v_group: int = 32

    def __post_init__(self) -> None:
        if self.mem_bits not in (2, 4, 6, 8):
            raise ValueError(f"mem_bits must be one of 2/4/6/8, got {self.mem_bits}")
        if self.block_size % 16:
            raise ValueError(f"block_size must be a multiple of 16, got {self.block_size}")
        if self.block_size % self.k_group or self.block_size // self.k_group > 8:
            raise ValueError(f"block_size {self.block_size} must be 1-8 multiples of k_group {self.k_group}")
        if self.head_size % self.v_group or self.head_size % 4:
            raise ValueError(f"head_size {self.head_size} must be divisible by v_group {self.v_group} and by 4")

    @staticmethod
    def per_token_bytes(num_kv_heads: int, head_size: int, mem_bits: int, k_group: int = 32,
                        v_group: int = 32) -> int:
        """Bytes per token the pool must budget: header byte + V stats + K stats + data at mem_bits,
        rounded up to whole float32 elements."""
        hd = num_kv_heads * head_size
        stats = 4 * num_kv_heads * (head_size // v_group) + 4 * hd // k_group
        return (1 + stats + (mem_bits // 2) * hd // 2 + 3) // 4 * 4

    @property
    def k_groups_per_block(self) -> int:
        return self.block_size // self.k_group

    @property
    def v_groups(self) -> int:
        return self.head_size // self.v_group

    @property
    def chunks_per_page(self) -> int:
        return self.mem_bits // 2

    @property
    def chunk_bytes(self) -> int:
        return self.block_size * self.num_kv_heads * self.head_size // 2

    @property
    def offsets(self) -> dict[str, int]:
        v_stats = self.block_size * self.num_kv_heads * self.v_groups * 2
        k_stats = self.k_groups_per_block * self.num_kv_heads * self.head_size * 2
        names = ("v_scale", "v_min", "k_scale", "k_min", "data", "end")
        sizes = (v_stats, v_stats, k_stats, k_stats, self.chunks_per_page * self.chunk_bytes)
        out, at = {}, self.block_size
        for name, size in zip(names, sizes + (0,)):
            out[name] = at
            at += size
        return out

    @property
    def page_bytes(self) -> int:
        return self.offsets["end"]

    def side_bytes(self, bits: int) -> int:
        return self.num_kv_heads * self.head_size * bits // 8

    def row_bytes(self, bits: int) -> int:
        return 2 * self.side_bytes(bits)

    def tokens_per_chunk(self, bits: int) -> int:
        return 2 * self.block_size // bits

    def native(self) -> N.Layout:
        return N.Layout(self.num_kv_heads, self.head_size, self.block_size, self.mem_bits, self.k_group, self.v_group)


class ChunkPool:
    """Host free list of the spare chunk slots (1 .. k_c-1 of every page) of one layer.

    Chunk id = page * chunks_per_page + slot.  The initial order and the
    pop-from-the-tail discipline define which ids a block gets, so they follow
    the reference exactly (tiered_cache.py:199-202, :286-295): the page headers
    must come out identical.
    """

    def __init__(self, num_blocks: int, chunks_per_page: int) -> None:
        ids = np.arange(num_blocks * chunks_per_page).reshape(num_blocks, chunks_per_page)[:, 1:]
        self.free: list[int] = ids.reshape(-1)[::-1].tolist()
        self.size = len(self.free)
        self.tier = np.zeros(num_blocks, dtype=np.int64)  # host copy of every block's tier
        self.table = np.zeros((num_blocks, 3), dtype=np.int64)  # extra chunk ids per block

    def release(self, block: int, new_tier: int) -> None:
        n = NEXTRA.get(int(self.tier[block]), 0)
        self.free.extend(self.table[block, :n].tolist())
        self.tier[block] = new_tier

    def allot(self, blocks: np.ndarray, target_bits: int) -> np.ndarray:
        """Greedy in block order: as many blocks as fit at the target tier, then the next tier down."""
        tiers = np.full(blocks.size, 2, dtype=np.int64)
        done = 0
        for bits in (8, 4):
            if bits > target_bits:
                continue
            per = NEXTRA[bits]
            take = min(blocks.size - done, len(self.free) // per)
            if take <= 0:
                continue
            cut = len(self.free) - take * per
            ids = self.free[cut:][::-1]
            del self.free[cut:]
            self.table[blocks[done: done + take], :per] = np.asarray(ids, dtype=np.int64).reshape(take, per)
            tiers[done: done + take] = bits
            done += take
        self.tier[blocks] = tiers
        return tiers

    def headers(self, blocks: np.ndarray) -> np.ndarray:
        hdr = np.zeros((blocks.size, 16), dtype=np.uint8)
        hdr[:, 0] = self.tier[blocks]
        hdr[:, 4:] = np.ascontiguousarray(self.table[blocks].astype(np.int32)).view(np.uint8)
        return hdr


class TieredKVCache:
    """One layer's tiered store over ``pages``: a uint8 ``[num_blocks, >= page_bytes]`` CUDA view."""

    def __init__(self, layout: TieredLayout, pages: torch.Tensor, residual_slots: int = 256,
                 residual_dtype: torch.dtype = torch.float32, residual: torch.Tensor | None = None,
                 shared: SharedState | None = None) -> None:
        if pages.dtype != torch.uint8 or pages.dim() != 2:
            raise ValueError("pages must be a 2-D uint8 tensor")
        if pages.shape[1] < layout.page_bytes:
            raise ValueError(f"page has {pages.shape[1]} bytes, layout needs {layout.page_bytes}")
        if pages.stride(1) != 1 or pages.stride(0) % 16 != 0:
            raise ValueError("pages must be byte-contiguous with a 16-byte aligned row stride")
        N.require_cuda(pages)
        L = layout
        n = pages.shape[0]
        h, d, bs = L.num_kv_heads, L.head_size, L.block_size
        self.layout = L
        self.num_blocks = n
        self.device = pages.device
        self.pages = pages
        o = L.offsets
        self.header = pages[:, :16]
        self.tag = pages[:, 0]
        self.sealed = pages[:, 1]
        self.table = pages[:, 4:16].view(torch.int32)

        def half(a: str, b: str, *shape):
            return pages[:, o[a]: o[b]].view(torch.float16).view(n, *shape)

        self.v_scale = half("v_scale", "v_min", bs, h, L.v_groups)
        self.v_min = half("v_min", "k_scale", bs, h, L.v_groups)
        self.k_scale = half("k_scale", "k_min", L.k_groups_per_block, h, d)
        self.k_min = half("k_min", "data", L.k_groups_per_block, h, d)
        self.data = pages[:, o["data"]: o["end"]].view(n, L.chunks_per_page, L.chunk_bytes)
        pages[:, :bs].zero_()

        self.pool = ChunkPool(n, L.chunks_per_page)
        self.pool_size = self.pool.size

        if residual is None:
            residual = torch.zeros(residual_slots + 1, L.k_group, h, d, dtype=residual_dtype, device=self.device)
        if residual.shape[1:] != (L.k_group, h, d) or residual.shape[0] < 2 or residual.stride(3) != 1:
            raise ValueError(f"residual buffer shape {tuple(residual.shape)} does not match layout")
        slots = residual.shape[0] - 1  # the last row is spare
        if shared is None:
            shared = SharedState(n, bs, L.k_group, slots, kref_window=L.k_group, device=self.device)
        if shared.num_blocks != n or shared.planner.num_slots > slots:
            raise ValueError("shared state does not match this layer's cache")
        self.shared = shared
        self.res_k = residual
        self.res_group = shared.res_group
        self.block_res = shared.block_res
        self.planner = shared.planner

        # ctypes descriptors, built once (the C ABI takes them by pointer)
        self._c_layout = L.native()
        self._c_pages = N.Pages(pages.data_ptr(), pages.stride(0), n, 0, 0)
        self._c_res = N.Residual(residual.data_ptr(), N.dtype_code(residual.dtype), 0, residual.stride(0),
                                 residual.stride(1), residual.stride(2), self.block_res.data_ptr(),
                                 self.res_group.data_ptr())
        self.c_layout, self.c_pages, self.c_res = C.byref(self._c_layout), C.byref(self._c_pages), C.byref(self._c_res)

        self._mark_h = np.zeros(n, dtype=np.int64)
        self._tok_tier = np.zeros(9, dtype=np.int64)
        self.reset_counters()

    @property
    def max_tier(self) -> int:
        """Upper bound (2/4/8) the caller knows for the tier of every block of this layer, or 0.
        Informational: the kernels do not depend on it (the decode kernel's shared-memory stages have
        one size for every tier, so a layer may change tier under a captured graph)."""
        return self._c_pages.max_tier

    @max_tier.setter
    def max_tier(self, bits: int) -> None:
        if bits not in (0, 2, 4, 8):
            raise ValueError("max_tier must be 0 (unknown), 2, 4 or 8")
        self._c_pages.max_tier = bits

    # reference-compatible host mirrors
    @property
    def _tag_h(self) -> np.ndarray:
        return self.pool.tier

    @property
    def _table_h(self) -> np.ndarray:
        return self.pool.table

    @property
    def _free(self) -> list:
        return self.pool.free

    # -- counters ----------------------------------------------------------
    def _settle(self, blocks: np.ndarray) -> None:
        """Book tokens written since the last settlement to the tier the block had then."""
        cum = self.shared.cum_h[blocks]
        np.add.at(self._tok_tier, self.pool.tier[blocks], cum - self._mark_h[blocks])
        self._mark_h[blocks] = cum

    @property
    def tokens_written(self) -> dict[int, int]:
        pending = np.bincount(self.pool.tier, weights=self.shared.cum_h - self._mark_h, minlength=9)
        return {b: int(self._tok_tier[b] + pending[b]) for b in SUPPORTED_BITS}

    def reset_counters(self) -> None:
        self._tok_tier[:] = 0
        self._mark_h[:] = self.shared.cum_h
        self.blocks_opened = {b: 0 for b in SUPPORTED_BITS}
        self.downgraded_blocks = 0
        self.demoted_blocks = 0
        self.sealed_groups = 0

    @property
    def pool_free(self) -> int:
        return len(self.pool.free)

    @property
    def residual_free(self) -> int:
        return len(self.planner.free)

    # -- chunk pool (host-side decisions) ---------------------------------
    def open_blocks(self, blocks, target_bits: int, protect=None) -> tuple[np.ndarray, np.ndarray]:
        """(Re)open ``blocks`` (unique ids) at ``target_bits`` or the best tier that fits.

        Old extra chunks return to the pool first.  If the pool cannot give every
        block the target tier, the least recently written full blocks are demoted
        to INT2 in place (never ``protect`` blocks or the ones opened here); only
        then do new blocks open lower.  Returns ``(blocks, headers [n, 16] uint8)``.
        """
        if target_bits not in SUPPORTED_BITS:
            raise ValueError(f"unsupported target bits {target_bits}")
        if torch.is_tensor(blocks):
            blocks = blocks.cpu().numpy()
        blocks = np.asarray(blocks, dtype=np.int64)
        self._settle(blocks)
        for b in blocks.tolist():
            self.pool.release(b, 0)
        short = NEXTRA[target_bits] * blocks.size - len(self.pool.free)
        if short > 0:
            keep = set(blocks.tolist())
            if protect is not None:
                keep |= set(np.asarray(protect).tolist())
            self._demote_lru(short, keep)
        tiers = self.pool.allot(blocks, target_bits)
        for bits in SUPPORTED_BITS:
            self.blocks_opened[bits] += int((tiers == bits).sum())
        self.downgraded_blocks += int((tiers < target_bits).sum())
        return blocks, self.pool.headers(blocks)

    def write_headers(self, blocks: torch.Tensor, headers: torch.Tensor) -> None:
        """Apply ``open_blocks`` headers (device ``[n]`` int64 ids, ``[n, 16]`` uint8)."""
        N.check(N.lib.echokv_write_headers(self.c_pages, blocks.data_ptr(), headers.data_ptr(), blocks.numel(),
                                           N.stream_ptr(self.device)))

    def _demote_lru(self, chunks_needed: int, keep: set) -> None:
        """Requantize the least recently written full INT4/INT8 blocks to INT2, freeing their chunks."""
        tier = self.pool.tier
        full = np.flatnonzero((tier >= 4) & (self.shared.fill_h == self.layout.block_size))
        ranked = full[np.argsort(self.shared.last_h[full], kind="stable")]
        victims, freed = [], 0
        for b in ranked.tolist():
            if freed >= chunks_needed:
                break
            if b in keep:
                continue
            victims.append(b)
            freed += NEXTRA[int(tier[b])]
        if not victims:
            return
        vb = to_device(torch.tensor(victims, dtype=torch.long), self.device)
        nbytes = N.lib.echokv_demote_scratch_bytes(self.c_layout, len(victims))
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        N.check(N.lib.echokv_demote_blocks(self.c_layout, self.c_pages, self.c_res, vb.data_ptr(), len(victims),
                                           scratch.data_ptr(), nbytes, N.stream_ptr(self.device)))
        varr = np.asarray(victims, dtype=np.int64)
        self._settle(varr)
        for b in victims:
            self.pool.release(b, 2)
        self.demoted_blocks += len(victims)

    # -- write ------------------------------------------------------------
    def _seal(self, ev: Eviction) -> None:
        """Quantize the ``fill`` keys of an evicted residual slot against their own stats."""
        if ev.fill <= 0:
            return
        bits = int(self.pool.tier[ev.block]) or 2
        mask = self.planner.sealed.get(ev.block, 1 << ev.group)
        N.check(N.lib.echokv_seal_group(self.c_layout, self.c_pages, self.c_res, ev.slot, ev.block, ev.group,
                                        ev.fill, bits, mask & 0xFF, N.stream_ptr(self.device)))
        self.sealed_groups += 1

    def prepare(self, plan: WritePlan, target_bits: int):
        """Host side of a step's writes for this layer: seal evicted groups, open blocks.
        Returns the opened blocks' page headers (see ``open_blocks``) or None."""
        for ev in plan.evictions:
            self._seal(ev)
        opens = plan.open_np
        if plan.touched_np.size:
            # a write into a block nothing opened (no offset-0 write seen): open it now
            fresh = plan.touched_np[self.pool.tier[plan.touched_np] == 0]
            if fresh.size:
                opens = np.union1d(opens, fresh)
        if not opens.size:
            return None
        return self.open_blocks(opens, target_bits, protect=plan.touched_np)

    def apply(self, meta: WriteMeta, key: torch.Tensor, value: torch.Tensor, kref: torch.Tensor | None = None,
              capturing: bool = False, stash: tuple | None = None) -> None:
        """Device side: quantize and store ``key`` / ``value`` ``[*, H, D]`` as ``meta`` says, in one launch
        (completed K groups, token rows and, with ``stash`` = (query, row indices, destination), the canary's
        query rows).  ``capturing`` gives the group pass its full grid, masked by the device count."""
        from echokv_b200.kernels.write import write_step

        with record_function("echokv.write.step"):
            write_step(self, key, value, meta, kref, full_grid=capturing, stash=stash)

    def write(self, key: torch.Tensor, value: torch.Tensor, slots: torch.Tensor, target_bits: int,
              kref: torch.Tensor | None = None) -> None:
        """Standalone path: plan, prepare, stage and apply in one call (``slots`` -1 = skip)."""
        plan = self.planner.plan(slots.detach().cpu())
        opened = self.prepare(plan, target_bits)
        self.shared.commit(plan)
        meta, extra = stage_plan(plan, self.device, opened)
        self.shared.apply_res_map(*extra[:4])
        if opened is not None:
            self.write_headers(extra[4], extra[5])
        self.apply(meta, key, value, kref)

    # -- read -------------------------------------------------------------
    def gather(self, blk: torch.Tensor, off: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """Dequantized K and V (float32 ``[n, H, D]``) of the tokens at (blk, off)."""
        L = self.layout
        n = blk.numel()
        blk = blk.to(self.device, torch.long).contiguous()
        off = off.to(self.device, torch.long).contiguous()
        k = torch.empty(n, L.num_kv_heads, L.head_size, device=self.device)
        v = torch.empty_like(k)
        N.check(N.lib.echokv_gather(self.c_layout, self.c_pages, self.c_res, blk.data_ptr(), off.data_ptr(), n,
                                    k.data_ptr(), v.data_ptr(), N.stream_ptr(self.device)))
        return k, v

    def tier_histogram(self) -> dict[int, int]:
        """Blocks currently tagged at each tier."""
        return {b: int((self.tag == b).sum()) for b in SUPPORTED_BITS}
