"""The per-step path of one KV-cache group, independent of vLLM.

``GroupRunner`` owns what the reference's metadata builder and attention impls
own between them (``echokv_vllm/backend.py``: ``_Staging`` :144-229,
``EchoKVMetadataBuilder._plan`` :463-496, ``EchoKVAttentionImpl`` buffers
:532-542): the layers' stores over their slices of the paged pool, one
``SharedState``, every layer's residual buffer, K_ref ring and canary stash, and
a persistent staging buffer that receives each step's int64 metadata with one
pinned host-to-device copy.  ``plan_step`` does every host-side decision once
per step for all layers; ``write`` and ``decode`` only launch kernels on device
metadata at fixed addresses, so a CUDA graph can capture a decode step and
replay it.  The vLLM backend (``backend.py``) is a thin adapter over this class;
the benchmark drives it directly.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from echokv_b200.canary import canary_kl_ring, tp_mean
from echokv_b200.controller import LayerController
from echokv_b200.quant import SUPPORTED_BITS
from echokv_b200.kernels.decode import (BLOCKS_PER_SPLIT, MAX_DECODE_SPLITS, MIN_SPLIT_TOKENS, choose_blocks_per_split,
                                        decode_attention, decode_parallelism)
from echokv_b200.kernels.write import gather_rows
from echokv_b200.tiered_cache import TieredKVCache, TieredLayout
from echokv_b200.write_plan import SharedState, WriteMeta


class Staging:
    """One step's int64 metadata in one device buffer, filled by one host-to-device copy.

    Element layout (every region starts at an even element = 16-byte boundary):

        [0] n_fin  [1] blocks per decode split | canary rows (nq) | decode rows, requests, lengths (3 x cap)
        | token arrays slot, residual, sealed, kref (4 x cap) | completed groups (cap x w) | tail

    Steps with at most ``cap`` rows / groups use the persistent buffer, whose
    graph-visible regions (everything before the tail) keep their addresses;
    larger steps (long prefills, never graph-replayed) get a buffer of their own
    size.  The tail (residual-map updates, page headers) is consumed by ops the
    builder launches itself; a tail that does not fit is uploaded separately so
    the graph-visible regions never move.
    """

    RING = 4  # pinned host buffers in flight

    def __init__(self, cap: int, nq: int, w: int, tail: int, device) -> None:
        self.cap = cap + (cap & 1)
        self.nq, self.w, self.tail = nq, w, tail + (tail & 1)
        self.o_dec = 2 + nq + (nq & 1)
        self.device = torch.device(device)
        self.size = self.o_dec + 7 * self.cap + self.cap * w + (self.cap * w & 1) + self.tail
        self.dev = torch.zeros(self.size, dtype=torch.long, device=self.device)
        self.host = [torch.zeros(self.size, dtype=torch.long).pin_memory() for _ in range(self.RING)]
        self.done: list[torch.cuda.Event | None] = [None] * self.RING
        self.turn = 0

    def _offsets(self, cd: int, ct: int, cf: int):
        o_tok = self.o_dec + 3 * cd
        o_fin = o_tok + 4 * ct
        o_tail = o_fin + cf * self.w
        return o_tok, o_fin, o_tail + (o_tail & 1)

    def stage(self, n_fin: int, canary: np.ndarray, decode, tok, fin: np.ndarray, tail: list[np.ndarray], bps: int = 0):
        """Upload a step; returns device views ``(fin_count, canary, [3 decode], tok [4, t], fin, tail views,
        blocks per split)``."""
        s, t = decode[0].size, tok[0].size
        fits = max(s, t, n_fin) <= self.cap
        tail_sizes = [a.size + (a.size & 1) for a in tail]
        tail_own = fits and sum(tail_sizes) > self.tail
        if fits:
            cd = ct = cf = self.cap
            i = self.turn
            if self.done[i] is not None:
                self.done[i].synchronize()  # the copy that last used this pinned buffer
            hbuf = self.host[i]
            h = hbuf.numpy()
        else:
            cd, ct, cf = s + (s & 1), t + (t & 1), n_fin
            total = self._offsets(cd, ct, cf)[2] + sum(tail_sizes)
            hbuf = torch.zeros(total, dtype=torch.long).pin_memory()
            h = hbuf.numpy()
        o_tok, o_fin, o_tail = self._offsets(cd, ct, cf)
        h[0], h[1] = n_fin, bps
        h[2: 2 + self.nq] = canary
        for k, a in enumerate(decode):
            h[self.o_dec + k * cd: self.o_dec + k * cd + s] = a
        for k, a in enumerate(tok):
            h[o_tok + k * ct: o_tok + k * ct + t] = a
        h[o_fin: o_fin + n_fin * self.w] = fin.reshape(-1)
        end = o_tail
        tail_dev = None
        if tail_own:
            th = torch.zeros(sum(tail_sizes), dtype=torch.long).pin_memory()
            o = 0
            for a, n in zip(tail, tail_sizes):
                th.numpy()[o: o + a.size] = a.reshape(-1)
                o += n
            tail_dev = th.to(self.device, non_blocking=True)
        else:
            for a, n in zip(tail, tail_sizes):
                h[end: end + a.size] = a.reshape(-1)
                end += n
        if fits:
            dev = self.dev
            dev[:end].copy_(hbuf[:end], non_blocking=True)
            ev = self.done[self.turn] or torch.cuda.Event()
            ev.record()
            self.done[self.turn] = ev
            self.turn = (self.turn + 1) % self.RING
        else:
            dev = hbuf.to(self.device, non_blocking=True)
        src, o = (tail_dev, 0) if tail_own else (dev, o_tail)
        views = []
        for a, n in zip(tail, tail_sizes):
            views.append(src[o: o + a.size])
            o += n
        return (
            dev[0:1],
            dev[2: 2 + self.nq],
            [dev[self.o_dec + k * cd: self.o_dec + k * cd + s] for k in range(3)],
            dev[o_tok: o_tok + 4 * ct].view(4, ct)[:, :t],
            dev[o_fin: o_fin + cf * self.w].view(cf, self.w),
            views,
            dev[1:2],
        )


@dataclass
class StepMeta:
    """Device-side description of one step, shared by every layer."""

    write: WriteMeta
    canary_rows: torch.Tensor
    decode_rows: torch.Tensor | None
    decode_reqs: torch.Tensor | None
    decode_lens: torch.Tensor | None
    num_splits: int
    bps_dev: torch.Tensor | None = None  # blocks per decode split of this step (one int64 on the device)


class GroupRunner:
    """All layers of one KV-cache group: stores, shared planner state, staging."""

    def __init__(self, layout: TieredLayout, caches: list[torch.Tensor], num_q_heads: int, scale: float,
                 controllers: list[LayerController], residual_slots: int, model_dtype: torch.dtype,
                 kref_window: int = 64, canary_max_q: int = 8, cap: int = 512, max_model_len: int = 8192,
                 residuals: list[torch.Tensor] | None = None, krefs: list[torch.Tensor] | None = None,
                 stashes: list[torch.Tensor] | None = None) -> None:
        if len(caches) != len(controllers):
            raise ValueError("one controller per layer")
        dev = caches[0].device
        self.layout, self.device = layout, dev
        self.num_q_heads, self.scale = num_q_heads, float(scale)
        self.controllers = controllers
        n = caches[0].shape[0]
        self.shared = SharedState(n, layout.block_size, layout.k_group, residual_slots, kref_window, dev)
        h, d, g = layout.num_kv_heads, layout.head_size, layout.k_group
        self.stores: list[TieredKVCache] = []
        self.krefs: list[torch.Tensor] = []
        self.stashes: list[torch.Tensor] = []
        # one allocation for all layers' K_ref rings / stashes: the canary kernel reads them in place
        self._kref_all = None if krefs else torch.zeros(len(caches), kref_window, h, d, dtype=torch.float32, device=dev)
        self._stash_all = None if stashes else torch.zeros(len(caches), canary_max_q, num_q_heads, d,
                                                           dtype=model_dtype, device=dev)
        for i, pages in enumerate(caches):
            res = residuals[i] if residuals else torch.zeros(residual_slots + 1, g, h, d, dtype=model_dtype, device=dev)
            self.stores.append(TieredKVCache(layout, pages, residual=res, shared=self.shared))
            self.krefs.append(krefs[i] if krefs else self._kref_all[i])
            self.stashes.append(stashes[i] if stashes else self._stash_all[i])
        self.canary_max_q = canary_max_q
        self.cap = cap
        tail = cap * (4 + 3 * len(caches)) + 64
        self.staging = Staging(cap, canary_max_q, 3 + g, tail, dev)
        # The split grid is fixed (a graph replays it); how many of its splits a step uses follows from the
        # blocks per split chosen for that step in `plan_step`, never less than `split_floor` blocks.
        max_blocks = -(-max_model_len // layout.block_size)
        self.split_floor = max(1, MIN_SPLIT_TOKENS // layout.block_size)
        self.num_splits = max(1, min(-(-max_blocks // self.split_floor), MAX_DECODE_SPLITS))
        with torch.cuda.device(dev):
            self.decode_slots = decode_parallelism(self.stores[0], num_q_heads)

    # -- host side, once per step ---------------------------------------------------------
    def plan_step(self, slots_cpu, decode=None, canary: np.ndarray | None = None) -> StepMeta:
        """Plan the step's writes for every layer, open blocks at each layer's current tier, and
        upload all metadata with one copy.  ``decode`` = (query rows, request rows, lengths)."""
        shared = self.shared
        plan = shared.planner.plan(slots_cpu)
        store0 = self.stores[0]
        opens = plan.open_np
        if plan.touched_np.size:
            fresh = plan.touched_np[store0.pool.tier[plan.touched_np] == 0]
            if fresh.size:
                opens = np.union1d(opens, fresh)
        opened = []
        if opens.size or plan.evictions:
            for st, ctl in zip(self.stores, self.controllers):
                for ev in plan.evictions:
                    st._seal(ev)
                if opens.size:
                    opened.append(st.open_blocks(opens, ctl.bits, protect=plan.touched_np))
        shared.commit(plan)
        tail = [plan.res_map_block, plan.res_map_value, plan.res_group_slot, plan.res_group_value]
        for blocks, headers in opened:
            tail += [blocks, np.ascontiguousarray(headers).view(np.int64).reshape(-1)]
        empty = np.zeros(0, dtype=np.int64)
        dec = decode if decode is not None else (empty, empty, empty)
        can = np.zeros(self.canary_max_q, dtype=np.int64) if canary is None else canary
        bps = BLOCKS_PER_SPLIT
        if self.decode_slots and dec[2].size:
            bps = choose_blocks_per_split(dec[2], self.layout.block_size, self.num_splits, self.decode_slots)
        fin_count, canary_rows, dviews, tok, fin, views, bps_dev = self.staging.stage(
            plan.n_fin, can, dec, (plan.tok_slot, plan.tok_res, plan.tok_sealed, plan.tok_kref), plan.fin, tail, bps)
        shared.apply_res_map(*views[:4])
        for st, ids, hdr in zip(self.stores, views[4::2], views[5::2]):
            st.write_headers(ids, hdr.view(torch.uint8).view(-1, 16))
        write = WriteMeta(tok=tok, fin=fin, fin_count=fin_count, n_rows=plan.n_rows, n_fin=plan.n_fin)
        has_dec = decode is not None and dec[0].size > 0
        return StepMeta(write, canary_rows, dviews[0] if has_dec else None, dviews[1] if has_dec else None,
                        dviews[2] if has_dec else None, self.num_splits, bps_dev)

    # -- canary (reference: EchoKVMetadataBuilder._run_canary, backend.py:314-333) --------------
    def stash_queries(self, layer: int, query: torch.Tensor, meta: StepMeta) -> None:
        """Keep the step's canary query rows (graph-capturable: indices come from device metadata)."""
        gather_rows(query, meta.canary_rows, self.stashes[layer])

    def measure_canary(self, nq: int, tp_group=None) -> torch.Tensor | None:
        """KL at 2/4/8 bits for every layer from the stashed queries and the K_ref rings, averaged
        over tensor-parallel ranks; float32 ``[L, 3]`` on the device, or None while the rings hold
        less than one K group.  Must run before the next ``plan_step`` moves the ring cursor."""
        pl = self.shared.planner
        if pl.kref_fill < self.layout.k_group:
            return None
        kref = self._kref_all if self._kref_all is not None else torch.stack(self.krefs)
        stash = self._stash_all if self._stash_all is not None else torch.stack(self.stashes)
        deltas = canary_kl_ring(stash[:, :nq], kref, pl.kref_pos, pl.kref_fill, self.layout.k_group, self.scale)
        deltas = tp_mean(deltas, tp_group)
        # Start the copy to pinned host memory now, so that `observe` (one measurement later) only waits for an
        # event that has long passed instead of synchronizing the stream.
        turn = self._canary_turn = (getattr(self, "_canary_turn", 0) + 1) % 2
        if not hasattr(self, "_canary_host"):
            self._canary_host = [torch.zeros(deltas.shape, dtype=torch.float32).pin_memory() for _ in range(2)]
            self._canary_done = [torch.cuda.Event() for _ in range(2)]
            self._canary_of = [None, None]
        self._canary_host[turn].copy_(deltas, non_blocking=True)
        self._canary_done[turn].record()
        self._canary_of[turn] = deltas
        return deltas

    def observe(self, deltas: torch.Tensor, ctx_len: float) -> None:
        """Feed a finished measurement to every layer's controller.  A measurement that came from
        `measure_canary` is read from its pinned host copy (the reference reads the previous measurement for
        the same reason, backend.py:316-326); anything else is read back from the device."""
        rows = None
        for k in range(2 if hasattr(self, "_canary_of") else 0):
            if self._canary_of[k] is deltas:
                self._canary_done[k].synchronize()
                rows = self._canary_host[k].tolist()
        if rows is None:
            rows = deltas.tolist()
        for ctl, row in zip(self.controllers, rows):
            ctl.observe(dict(zip(SUPPORTED_BITS, row)), ctx_len)

    # -- device side, per layer ---------------------------------------------------------------
    def write(self, layer: int, key: torch.Tensor, value: torch.Tensor, meta: StepMeta, capturing: bool = False,
              query: torch.Tensor | None = None) -> None:
        """Store the step's keys and values of one layer; with ``query`` also keep its canary rows (what
        ``stash_queries`` does) in the same launch."""
        stash = None if query is None else (query, meta.canary_rows, self.stashes[layer])
        self.stores[layer].apply(meta.write, key, value, self.krefs[layer], capturing=capturing, stash=stash)

    def decode(self, layer: int, query: torch.Tensor, block_table: torch.Tensor, out: torch.Tensor,
               meta: StepMeta) -> None:
        decode_attention(self.stores[layer], query, block_table, meta.decode_lens, self.scale, self.split_floor,
                         q_rows=meta.decode_rows, bt_rows=meta.decode_reqs, out=out, num_splits=meta.num_splits,
                         bps_dev=meta.bps_dev)
