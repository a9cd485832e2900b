"""Host-side plan of one step's KV writes (shared by all layers of a KV-cache group).

Mirrors the interface of the reference's ``echokv_vllm/write_plan.py``
(``WritePlanner.plan`` :98-240, ``SharedState`` :243-271, ``WriteMeta``
:274-282, ``stage_plan`` :285-315): everything a write needs that does not
depend on tensor values follows from the slot mapping alone, so it is decided
once per step on the host and uploaded as int64 arrays the CUDA kernels read.

Decisions (identical to the reference, including slot numbering):
  * a block *opens* when its offset 0 is written; its residual slot and sealed
    mask are dropped first;
  * a K group whose ``k_group`` tokens all arrive in this step is finalized
    straight from the step's key rows;
  * a group that reaches its last position with earlier tokens parked in a
    residual slot is finalized from both, and the slot is released;
  * any other group keeps (or gets) a residual slot; when none is free the
    least recently written unprotected slot is evicted and its group *sealed*
    (later tokens of a sealed group quantize against the stored stats);
  * the last ``kref_window`` keys of the step go to the K_ref ring in order.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from echokv_b200._util import to_device

_I64 = np.int64


def _none() -> np.ndarray:
    return np.zeros(0, dtype=_I64)


@dataclass
class Eviction:
    """A residual slot taken from (block, group) holding ``fill`` keys; sealed before reuse."""

    slot: int
    block: int
    group: int
    fill: int


@dataclass
class WritePlan:
    """One step's writes as host arrays (per token row unless noted).

    ``tok_slot`` -1 = row not stored; ``tok_res`` residual slot of keys whose
    group stays open, else -1; ``tok_sealed`` 1 = key of a sealed group;
    ``tok_kref`` K_ref ring row or -1.  ``fin`` is ``[n_fin, 3 + k_group]``:
    block, group, residual slot or -1, then the key row of every position
    (-1 = take it from the residual).
    """

    step: int
    n_rows: int
    tok_slot: np.ndarray
    tok_res: np.ndarray
    tok_sealed: np.ndarray
    tok_kref: np.ndarray
    fin: np.ndarray
    evictions: list = field(default_factory=list)
    open_np: np.ndarray = field(default_factory=_none)
    touched_np: np.ndarray = field(default_factory=_none)
    touched_fill: np.ndarray = field(default_factory=_none)
    touched_count: np.ndarray = field(default_factory=_none)
    res_map_block: np.ndarray = field(default_factory=_none)
    res_map_value: np.ndarray = field(default_factory=_none)
    res_group_slot: np.ndarray = field(default_factory=_none)
    res_group_value: np.ndarray = field(default_factory=_none)
    block_size: int = 0
    k_group: int = 0

    @property
    def n_fin(self) -> int:
        return int(self.fin.shape[0])


class _MapLog:
    """Ordered log of ``block_res`` / ``res_group`` updates; the last write to a key wins."""

    def __init__(self) -> None:
        self.block: dict[int, int] = {}
        self.group: dict[int, int] = {}

    def arrays(self):
        kb = np.fromiter(self.block.keys(), _I64, len(self.block))
        vb = np.fromiter(self.block.values(), _I64, len(self.block))
        ks = np.fromiter(self.group.keys(), _I64, len(self.group))
        vs = np.fromiter(self.group.values(), _I64, len(self.group))
        return kb, vb, ks, vs


class WritePlanner:
    """Residual-slot allocator + K_ref ring cursor + the per-step plan."""

    def __init__(self, block_size: int, k_group: int, residual_slots: int, kref_window: int = 64) -> None:
        self.bs = int(block_size)
        self.g = int(k_group)
        self.num_slots = int(residual_slots)
        self.free = list(range(self.num_slots - 1, -1, -1))  # popped from the end: 0, 1, 2, ...
        self.block_slot: dict[int, int] = {}
        self.slot_info: dict[int, list[int]] = {}  # slot -> [block, group, fill, last step]
        self.sealed: dict[int, int] = {}  # block -> bitmask of sealed groups
        self.step = 0
        self.kref_window = int(kref_window)
        self.kref_pos = 0
        self.kref_fill = 0

    # -- slot bookkeeping ---------------------------------------------------
    def _drop(self, slot: int, log: _MapLog) -> None:
        block = self.slot_info.pop(slot)[0]
        self.block_slot.pop(block, None)
        self.free.append(slot)
        log.block[block] = -1

    def _is_sealed(self, block: int, group: int) -> bool:
        return bool((self.sealed.get(block, 0) >> group) & 1)

    def _take_slot(self, block: int, group: int, protected: set, evictions: list, log: _MapLog) -> int:
        if not self.free:
            cands = [s for s in self.slot_info if s not in protected]
            if not cands:
                raise RuntimeError(f"more than {self.num_slots} open K groups in one step")
            victim = min(cands, key=lambda s: self.slot_info[s][3])
            vb, vg, vfill, _ = self.slot_info[victim]
            evictions.append(Eviction(victim, vb, vg, vfill))
            self.sealed[vb] = self.sealed.get(vb, 0) | (1 << vg)
            self._drop(victim, log)
        slot = self.free.pop()
        self.slot_info[slot] = [block, group, 0, 0]
        self.block_slot[block] = slot
        protected.add(slot)
        log.block[block] = slot
        log.group[slot] = group
        return slot

    # -- the plan -------------------------------------------------------------
    def plan(self, slot_mapping_cpu) -> WritePlan:
        self.step += 1
        bs, g = self.bs, self.g
        gpb = bs // g
        if torch.is_tensor(slot_mapping_cpu):
            slot_mapping_cpu = slot_mapping_cpu.numpy()
        sm = np.asarray(slot_mapping_cpu).astype(_I64).reshape(-1)
        n_rows = sm.size
        live = np.flatnonzero(sm >= 0)
        n = live.size
        blk, off = np.divmod(sm[live], bs)
        gid = blk * gpb + off // g  # global K-group id
        pos = off % g
        log = _MapLog()

        opened = np.unique(blk[off == 0])
        for b in opened.tolist():
            s = self.block_slot.get(b)
            if s is not None:
                self._drop(s, log)
            self.sealed.pop(b, None)

        # Tokens sorted by (group id, position); runs of equal group id are the step's K groups.
        order = np.lexsort((pos, gid))
        gsorted = gid[order]
        first = np.flatnonzero(np.r_[True, gsorted[1:] != gsorted[:-1]]) if n else _none()
        size = np.diff(np.r_[first, n])
        g_blk = gsorted[first] // gpb if n else _none()
        g_grp = gsorted[first] % gpb if n else _none()

        whole = size == g
        if self.sealed and whole.any():
            for u in np.flatnonzero(whole).tolist():
                if self._is_sealed(int(g_blk[u]), int(g_grp[u])):
                    whole[u] = False
        wi = np.flatnonzero(whole)
        fin_whole = np.empty((wi.size, 3 + g), dtype=_I64)
        if wi.size:
            fin_whole[:, 0], fin_whole[:, 1], fin_whole[:, 2] = g_blk[wi], g_grp[wi], -1
            fin_whole[:, 3:] = live[order[first[wi][:, None] + np.arange(g)]]
            if self.block_slot:  # a rewritten group that still owned a slot
                by_block: dict[int, set] = {}
                for b, gr in zip(g_blk[wi].tolist(), g_grp[wi].tolist()):
                    by_block.setdefault(b, set()).add(gr)
                for b in g_blk[wi].tolist():
                    s = self.block_slot.get(b)
                    if s is not None and self.slot_info[s][1] in by_block[b]:
                        self._drop(s, log)

        tok_res = np.full(n, -1, dtype=_I64)
        tok_sealed = np.zeros(n, dtype=_I64)
        fin_part: list[list[int]] = []
        evictions: list[Eviction] = []
        protected = {self.block_slot[b] for b in np.unique(blk).tolist() if b in self.block_slot}
        for u in np.flatnonzero(~whole).tolist():
            members = order[first[u]: first[u] + size[u]]
            b, gr = int(g_blk[u]), int(g_grp[u])
            if self._is_sealed(b, gr):
                tok_sealed[members] = 1
                continue
            top = int(pos[members].max())
            slot = self.block_slot.get(b)
            if slot is not None and self.slot_info[slot][1] != gr:
                slot = None
            if top == g - 1:  # the group completes in this step
                line = [b, gr, -1 if slot is None else slot] + [-1] * g
                for p, r in zip(pos[members].tolist(), live[members].tolist()):
                    line[3 + p] = r
                fin_part.append(line)
                if slot is not None:
                    self._drop(slot, log)
                continue
            if slot is None:
                slot = self._take_slot(b, gr, protected, evictions, log)
            tok_res[members] = slot
            info = self.slot_info[slot]
            info[2] = max(info[2], top + 1)
            info[3] = self.step

        fin = np.concatenate([fin_whole, np.asarray(fin_part, dtype=_I64).reshape(-1, 3 + g)])

        # Per touched block: highest offset written + 1, and how many tokens.
        if n:
            touched, inv = np.unique(blk, return_inverse=True)
            t_fill = np.zeros(touched.size, dtype=_I64)
            np.maximum.at(t_fill, inv, off + 1)
            t_count = np.bincount(inv, minlength=touched.size).astype(_I64)
        else:
            touched, t_fill, t_count = _none(), _none(), _none()

        kref = np.full(n, -1, dtype=_I64)
        k = min(n, self.kref_window)
        if k:
            kref[n - k:] = (self.kref_pos + np.arange(k)) % self.kref_window
            self.kref_pos = (self.kref_pos + k) % self.kref_window
            self.kref_fill = min(self.kref_window, self.kref_fill + k)

        def rows_of(vals: np.ndarray, fill: int) -> np.ndarray:
            full = np.full(n_rows, fill, dtype=_I64)
            full[live] = vals
            return full

        mb, mv, gs, gv = log.arrays()
        return WritePlan(
            step=self.step, n_rows=n_rows, tok_slot=sm, tok_res=rows_of(tok_res, -1),
            tok_sealed=rows_of(tok_sealed, 0), tok_kref=rows_of(kref, -1), fin=fin, evictions=evictions,
            open_np=opened, touched_np=touched, touched_fill=t_fill, touched_count=t_count,
            res_map_block=mb, res_map_value=mv, res_group_slot=gs, res_group_value=gv,
            block_size=bs, k_group=g,
        )


class _SealedView:
    """``planner.sealed.get(block, default)`` over the native planner's map."""

    def __init__(self, owner) -> None:
        self._owner = owner

    def get(self, block: int, default: int = 0) -> int:
        from echokv_b200 import _native as N

        return int(N.lib.echokv_planner_sealed_mask(self._owner._h, int(block), int(default)))


class NativeWritePlanner:
    """``WritePlanner`` with the state and ``plan`` in the C++ library (``csrc/planner.cu``): the same decisions, slot
    numbering and output order (``tests/test_host_plan.py`` compares the two on seeded traffic), a fraction of the
    host time per step.  Exposes what the stores read of a planner: ``plan``, ``free`` (its length), ``sealed.get``,
    ``num_slots``, ``kref_pos``, ``kref_fill``, ``step``."""

    def __init__(self, block_size: int, k_group: int, residual_slots: int, kref_window: int = 64) -> None:
        from echokv_b200 import _native as N

        self._N = N
        self.bs, self.g = int(block_size), int(k_group)
        self.num_slots, self.kref_window = int(residual_slots), int(kref_window)
        self._h = N.lib.echokv_planner_create(self.bs, self.g, self.num_slots, self.kref_window)
        if not self._h:
            raise ValueError(N.lib.echokv_last_error().decode())
        self.sealed = _SealedView(self)

    def __del__(self) -> None:
        h, self._h = getattr(self, "_h", None), None
        try:
            if h:
                self._N.lib.echokv_planner_destroy(h)
        except Exception:  # interpreter shutdown: the library may already be gone
            pass

    def _get(self, what: int) -> int:
        return int(self._N.lib.echokv_planner_get(self._h, what))

    free = property(lambda self: range(self._get(0)))
    kref_pos = property(lambda self: self._get(1))
    kref_fill = property(lambda self: self._get(2))
    step = property(lambda self: self._get(3))

    def plan(self, slot_mapping_cpu) -> WritePlan:
        if torch.is_tensor(slot_mapping_cpu):
            slot_mapping_cpu = slot_mapping_cpu.numpy()
        sm = np.ascontiguousarray(np.asarray(slot_mapping_cpu).astype(_I64).reshape(-1))
        n, w = sm.size, 3 + self.g
        tok = np.empty((4, max(n, 1)), dtype=_I64)
        fin = np.empty((max(n, 1), w), dtype=_I64)
        ev = np.empty((max(n, 1), 4), dtype=_I64)
        small = np.empty((4, max(n, 1)), dtype=_I64)  # opened, touched, touched fill, touched count
        maps = np.empty((4, 4 * n + 8), dtype=_I64)   # map block / value, group slot / value
        counts = np.zeros(8, dtype=_I64)
        tokv = tok[:, :n]
        rc = self._N.lib.echokv_planner_plan(
            self._h, sm.ctypes.data, n, tok.ctypes.data, fin.ctypes.data, ev.ctypes.data,
            small[0].ctypes.data, small[1].ctypes.data, small[2].ctypes.data, small[3].ctypes.data,
            maps[0].ctypes.data, maps[1].ctypes.data, maps[2].ctypes.data, maps[3].ctypes.data, counts.ctypes.data)
        if rc != 0:
            raise RuntimeError(self._N.lib.echokv_last_error().decode())
        n_fin, n_ev, n_open, n_touched, n_mb, n_mg, step = (int(x) for x in counts[:7])
        evictions = [Eviction(*(int(x) for x in row)) for row in ev[:n_ev]]
        return WritePlan(
            step=step, n_rows=n, tok_slot=sm, tok_res=tokv[1].copy(), tok_sealed=tokv[2].copy(), tok_kref=tokv[3].copy(),
            fin=fin[:n_fin].copy(), evictions=evictions, open_np=small[0, :n_open].copy(),
            touched_np=small[1, :n_touched].copy(), touched_fill=small[2, :n_touched].copy(),
            touched_count=small[3, :n_touched].copy(), res_map_block=maps[0, :n_mb].copy(),
            res_map_value=maps[1, :n_mb].copy(), res_group_slot=maps[2, :n_mg].copy(),
            res_group_value=maps[3, :n_mg].copy(), block_size=self.bs, k_group=self.g,
        )


class SharedState:
    """What all layers of one KV-cache group share: the planner, the device residual map read by
    the attention kernels, and per-block host bookkeeping (fill, recency, tokens written)."""

    def __init__(self, num_blocks: int, block_size: int, k_group: int, residual_slots: int,
                 kref_window: int, device) -> None:
        self.num_blocks = num_blocks
        self.planner = NativeWritePlanner(block_size, k_group, residual_slots, kref_window)
        self.fill_h = np.zeros(num_blocks, dtype=_I64)
        self.last_h = np.zeros(num_blocks, dtype=_I64)
        self.cum_h = np.zeros(num_blocks, dtype=_I64)
        self.block_res = torch.full((num_blocks,), -1, dtype=torch.long, device=device)
        self.res_group = torch.zeros(residual_slots + 1, dtype=torch.long, device=device)

    def commit(self, plan: WritePlan) -> None:
        t = plan.touched_np
        if t.size:
            self.fill_h[t] = np.maximum(self.fill_h[t], plan.touched_fill)
            self.last_h[t] = plan.step
            self.cum_h[t] += plan.touched_count

    def apply_res_map(self, blocks, values, slots, groups) -> None:
        """Scatter the step's residual-map updates (device int64 index/value tensors)."""
        from echokv_b200.kernels.write import scatter_i64

        scatter_i64(self.block_res, blocks, values)
        scatter_i64(self.res_group, slots, groups)


@dataclass
class WriteMeta:
    """A plan's device arrays as the write kernels read them."""

    tok: torch.Tensor  # [4, >= n_rows] int64: slot, residual slot, sealed, K_ref row
    fin: torch.Tensor  # [>= n_fin, 3 + k_group] int64
    fin_count: torch.Tensor  # [1] int64: masks a full-grid (graph-captured) finalize
    n_rows: int
    n_fin: int


def stage_plan(plan: WritePlan, device, opened=None):
    """Upload ``plan`` (and the ``opened`` page headers) with one host-to-device copy.

    Returns ``(WriteMeta, (res_blocks, res_values, grp_slots, grp_values, hdr_blocks, hdr_bytes))``;
    the last two are None without ``opened``.  Every region starts on a 16-byte boundary.
    """
    t, f, w = plan.n_rows, plan.n_fin, 3 + plan.k_group
    tp = t + (t & 1)  # even row pitch keeps every row of ``tok`` 16-byte aligned
    tok = np.full((4, tp), -1, dtype=_I64)
    tok[0, :t], tok[1, :t], tok[2, :t], tok[3, :t] = plan.tok_slot, plan.tok_res, plan.tok_sealed, plan.tok_kref
    parts = [np.array([f, 0], dtype=_I64), tok.reshape(-1), plan.fin.reshape(-1),
             plan.res_map_block, plan.res_map_value, plan.res_group_slot, plan.res_group_value]
    if opened is not None:
        parts += [np.asarray(opened[0], dtype=_I64), np.ascontiguousarray(opened[1]).view(_I64).reshape(-1)]
    offs, o = [], 0
    for p in parts:
        offs.append(o)
        o += p.size + (p.size & 1)
    host = np.zeros(max(o, 2), dtype=_I64)
    for p, s in zip(parts, offs):
        host[s: s + p.size] = p
    dev = to_device(torch.from_numpy(host), device)
    view = [dev[s: s + p.size] for p, s in zip(parts, offs)]
    meta = WriteMeta(tok=view[1].view(4, tp)[:, :t], fin=view[2].view(f, w), fin_count=view[0][:1], n_rows=t, n_fin=f)
    hdr = (None, None)
    if opened is not None:
        hdr = (view[7], view[8].view(torch.uint8).view(-1, 16))
    return meta, (view[3], view[4], view[5], view[6], *hdr)
