"""CPU restatement (numpy) of EchoKV's paged mixed-precision KV-cache hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this module;
only the tests, the smoke check and the benchmark's CPU-baseline leg do, and
there only as the checker / the timed baseline, never as the product.

Parity is PINNED: every function below is checked bit for bit (bytes, codes,
fp16 stats, slot maps) or to 1e-5 (attention, KL) against outputs of the
reference's own Python implementation, stored as fixtures under
``tests/golden`` (made by ``tests/golden/make_golden.py``, which imports the
reference unchanged).

Each function cites the reference file:line it restates (paths are relative
to the reference project's root).

Arithmetic contract (echokv_vllm/quant.py:26-45, :63-75):
  mn16    = fp16_rne(min(group))
  scale16 = fp16_rne(max((max(group) - fp32(mn16)) / (2**b - 1), 2**-14))   # IEEE fp32 divide
  code    = clamp(rne((x - fp32(mn16)) / fp32(scale16)), 0, 2**b - 1)
  recon   = code * fp32(scale16) + fp32(mn16)
V groups run along head_dim per token; K groups run along ``k_group``
consecutive tokens per channel.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

SUPPORTED_BITS = (2, 4, 8)
FP16_TINY = np.float32(6.103515625e-05)
NEXTRA = {2: 0, 4: 1, 8: 3}  # echokv_vllm/tiered_cache.py:73

try:  # bf16 inputs (as uint16 bit patterns) are widened with this helper
    import ml_dtypes  # noqa: F401
except Exception:  # pragma: no cover
    ml_dtypes = None


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    """uint16 bf16 bit patterns -> float32 (exact)."""
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns, round-to-nearest-even (as torch's .bfloat16())."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = u + (np.uint32(0x7FFF) + ((u >> 16) & np.uint32(1)))
    return (rounded >> 16).astype(np.uint16)


# --------------------------------------------------------------------------
# quant.py
# --------------------------------------------------------------------------


def _levels(bits: int) -> np.float32:
    if bits not in SUPPORTED_BITS:
        raise ValueError(f"unsupported bits: {bits}")
    return np.float32((1 << bits) - 1)


def quantize(x: np.ndarray, bits: int, group_size: int):
    """echokv_vllm/quant.py:26-45. Returns (codes u8 [...,D], scale f16 [...,G], min f16 [...,G])."""
    lv = _levels(bits)
    d = x.shape[-1]
    if d % group_size:
        raise ValueError(f"head dim {d} not divisible by group_size {group_size}")
    xg = np.asarray(x, dtype=np.float32).reshape(*x.shape[:-1], d // group_size, group_size)
    mn16 = xg.min(axis=-1).astype(np.float16)
    mn = mn16.astype(np.float32)
    scale16 = np.maximum((xg.max(axis=-1) - mn) / lv, FP16_TINY).astype(np.float16)
    q = np.rint((xg - mn[..., None]) / scale16.astype(np.float32)[..., None])
    q = np.clip(q, 0, lv)
    return q.reshape(x.shape).astype(np.uint8), scale16, mn16


def dequantize(codes: np.ndarray, scale: np.ndarray, mn: np.ndarray, group_size: int) -> np.ndarray:
    """echokv_vllm/quant.py:48-55."""
    d = codes.shape[-1]
    qg = codes.astype(np.float32).reshape(*codes.shape[:-1], d // group_size, group_size)
    out = qg * scale.astype(np.float32)[..., None] + mn.astype(np.float32)[..., None]
    return out.reshape(codes.shape)


def fake_quant(x: np.ndarray, bits: int, group_size: int) -> np.ndarray:
    """echokv_vllm/quant.py:58-60."""
    return dequantize(*quantize(x, bits, group_size), group_size)


def stats_along(x: np.ndarray, bits: int, axis: int):
    """echokv_vllm/quant.py:63-69. fp16 (scale, min) of x reduced over ``axis``."""
    lv = _levels(bits)
    xf = np.asarray(x, dtype=np.float32)
    mn16 = xf.min(axis=axis).astype(np.float16)
    scale16 = np.maximum((xf.max(axis=axis) - mn16.astype(np.float32)) / lv, FP16_TINY).astype(np.float16)
    return scale16, mn16


def quantize_with(x: np.ndarray, scale: np.ndarray, mn: np.ndarray, bits: int) -> np.ndarray:
    """echokv_vllm/quant.py:72-75."""
    lv = _levels(bits)
    q = np.rint((np.asarray(x, dtype=np.float32) - mn.astype(np.float32)) / scale.astype(np.float32))
    return np.clip(q, 0, lv).astype(np.uint8)


def dequantize_with(codes: np.ndarray, scale: np.ndarray, mn: np.ndarray) -> np.ndarray:
    """echokv_vllm/quant.py:78-79."""
    return codes.astype(np.float32) * scale.astype(np.float32) + mn.astype(np.float32)


def fake_quant_channels(k: np.ndarray, bits: int, group: int) -> np.ndarray:
    """echokv_vllm/quant.py:82-96. ``k`` is [..., T, H, D]; a trailing partial group stays exact."""
    t = k.shape[-3]
    full = (t // group) * group
    out = np.array(k, dtype=np.float32, copy=True)
    if full:
        lead = out.shape[:-3]
        kg = out[..., :full, :, :].reshape(*lead, full // group, group, *out.shape[-2:])
        scale, mn = stats_along(kg, bits, axis=-3)
        sc, m = np.expand_dims(scale, -3), np.expand_dims(mn, -3)
        rec = dequantize_with(quantize_with(kg, sc, m, bits), sc, m)
        out[..., :full, :, :] = rec.reshape(*lead, full, *out.shape[-2:])
    return out


def pack(codes: np.ndarray, bits: int) -> np.ndarray:
    """echokv_vllm/quant.py:99-110. Element i of a byte sits at bits [i*b, (i+1)*b)."""
    if bits == 8:
        return codes.astype(np.uint8)
    per = 8 // bits
    c = codes.reshape(*codes.shape[:-1], codes.shape[-1] // per, per).astype(np.uint32)
    sh = (np.arange(per, dtype=np.uint32) * bits)
    return (c << sh).sum(axis=-1).astype(np.uint8)


def unpack(packed: np.ndarray, bits: int) -> np.ndarray:
    """echokv_vllm/quant.py:113-120."""
    if bits == 8:
        return packed.astype(np.uint8)
    per = 8 // bits
    sh = (np.arange(per, dtype=np.uint32) * bits)
    c = (packed.astype(np.uint32)[..., None] >> sh) & ((1 << bits) - 1)
    return c.reshape(*packed.shape[:-1], packed.shape[-1] * per).astype(np.uint8)


# --------------------------------------------------------------------------
# tiered_cache.py: page layout
# --------------------------------------------------------------------------


@dataclass(frozen=True)
class Layout:
    """echokv_vllm/tiered_cache.py:76-147."""

    num_kv_heads: int
    head_size: int
    block_size: int
    mem_bits: int
    k_group: int = 32
    v_group: int = 32

    def __post_init__(self):
        if self.mem_bits not in (2, 4, 6, 8):
            raise ValueError("mem_bits must be one of 2/4/6/8")
        if self.block_size % 16:
            raise ValueError("block_size must be a multiple of 16")
        if self.block_size % self.k_group or self.block_size // self.k_group > 8:
            raise ValueError("block_size must be 1-8 multiples of k_group")
        if self.head_size % self.v_group or self.head_size % 4:
            raise ValueError("head_size must be divisible by v_group and by 4")

    @staticmethod
    def per_token_bytes(h: int, d: int, mem_bits: int, k_group: int = 32, v_group: int = 32) -> int:
        raw = 1 + 4 * h * (d // v_group) + 4 * h * d // k_group + (mem_bits // 2) * h * d // 2
        return -(-raw // 4) * 4

    @property
    def kgpb(self) -> int:
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
    def offsets(self) -> dict:
        bs, h, d = self.block_size, self.num_kv_heads, self.head_size
        o = {"v_scale": bs}
        o["v_min"] = o["v_scale"] + bs * h * self.v_groups * 2
        o["k_scale"] = o["v_min"] + bs * h * self.v_groups * 2
        o["k_min"] = o["k_scale"] + self.kgpb * h * d * 2
        o["data"] = o["k_min"] + self.kgpb * h * d * 2
        o["end"] = o["data"] + self.chunks_per_page * self.chunk_bytes
        return o

    @property
    def page_bytes(self) -> int:
        return self.offsets["end"]

    def side_bytes(self, bits: int) -> int:
        return self.num_kv_heads * self.head_size * bits // 8

    def row_bytes(self, bits: int) -> int:
        return 2 * self.side_bytes(bits)

    def tokens_per_chunk(self, bits: int) -> int:
        return 2 * self.block_size // bits


# --------------------------------------------------------------------------
# write_plan.py: the host planner, restated as a plain per-group loop
# --------------------------------------------------------------------------


@dataclass
class Eviction:
    slot: int
    block: int
    group: int
    fill: int


@dataclass
class Plan:
    step: int
    n_rows: int
    tok_slot: np.ndarray
    tok_res: np.ndarray
    tok_sealed: np.ndarray
    tok_kref: np.ndarray
    fin: np.ndarray  # [f, 3 + g]
    evictions: list
    open_blocks: np.ndarray
    touched: np.ndarray
    touched_fill: np.ndarray
    touched_count: np.ndarray
    res_map: dict = field(default_factory=dict)  # block -> slot or -1
    grp_map: dict = field(default_factory=dict)  # slot -> group


class Planner:
    """echokv_vllm/write_plan.py:77-240 (same decisions, in a token/group loop)."""

    def __init__(self, block_size: int, k_group: int, residual_slots: int, kref_window: int = 64):
        self.bs, self.g = block_size, k_group
        self.num_slots = residual_slots
        self.free = list(range(residual_slots - 1, -1, -1))
        self.block_slot: dict[int, int] = {}
        self.slot_info: dict[int, list[int]] = {}
        self.sealed: dict[int, int] = {}
        self.step = 0
        self.kref_window = kref_window
        self.kref_pos = 0
        self.kref_fill = 0

    def _release(self, slot: int, res_ops: list) -> None:
        b = self.slot_info.pop(slot)[0]
        self.block_slot.pop(b, None)
        self.free.append(slot)
        res_ops.append((b, -1))

    def plan(self, slot_mapping) -> Plan:
        self.step += 1
        bs, g = self.bs, self.g
        sm = np.asarray(slot_mapping, dtype=np.int64).reshape(-1)
        n_rows = sm.size
        rows = [int(r) for r in np.nonzero(sm >= 0)[0]]
        res_ops: list[tuple[int, int]] = []
        grp_ops: list[tuple[int, int]] = []

        # (block, group) -> [(pos, row)], tokens in position order (stable)
        groups: dict[tuple[int, int], list[tuple[int, int]]] = {}
        opens = set()
        blocks_seen: dict[int, list[int]] = {}
        for r in rows:
            s = int(sm[r])
            b, off = divmod(s, bs)
            if off == 0:
                opens.add(b)
            groups.setdefault((b, off // g), []).append((off % g, r))
            blocks_seen.setdefault(b, []).append(off)
        for v in groups.values():
            v.sort(key=lambda pr: pr[0])

        open_blocks = np.array(sorted(opens), dtype=np.int64)
        for b in open_blocks.tolist():
            s = self.block_slot.get(b)
            if s is not None:
                self._release(s, res_ops)
            self.sealed.pop(b, None)

        order = sorted(groups.keys(), key=lambda bg: bg[0] * (bs // g) + bg[1])
        is_fast = {}
        for bg in order:
            is_fast[bg] = len(groups[bg]) == g and not ((self.sealed.get(bg[0], 0) >> bg[1]) & 1)

        fin_rows: list[list[int]] = []
        # fast groups first (write_plan.py:135-148), in key order
        fast_groups_of: dict[int, set] = {}
        for bg in order:
            if is_fast[bg]:
                fin_rows.append([bg[0], bg[1], -1] + [r for _, r in groups[bg]])
                fast_groups_of.setdefault(bg[0], set()).add(bg[1])
        for bg in order:
            if is_fast[bg]:
                s_ = self.block_slot.get(bg[0])
                if s_ is not None and self.slot_info[s_][1] in fast_groups_of[bg[0]]:
                    self._release(s_, res_ops)

        n = len(rows)
        row_res = {}
        row_sealed = {}
        evictions: list[Eviction] = []
        protected = {self.block_slot[b] for b in sorted(blocks_seen) if b in self.block_slot}
        for bg in order:
            if is_fast[bg]:
                continue
            b, gr = bg
            toks = groups[bg]
            pmax = max(p for p, _ in toks)
            if (self.sealed.get(b, 0) >> gr) & 1:
                for _, r in toks:
                    row_sealed[r] = 1
                continue
            s = self.block_slot.get(b)
            if s is not None and self.slot_info[s][1] != gr:
                s = None
            if pmax == g - 1:
                line = [b, gr, -1 if s is None else s] + [-1] * g
                for p, r in toks:
                    line[3 + p] = r
                fin_rows.append(line)
                if s is not None:
                    self._release(s, res_ops)
                continue
            if s is None:
                if not self.free:
                    victims = [v for v in self.slot_info if v not in protected]
                    if not victims:
                        raise RuntimeError(f"more than {self.num_slots} open K groups in one step")
                    v = min(victims, key=lambda x: self.slot_info[x][3])
                    vb, vg, vf, _ = self.slot_info[v]
                    evictions.append(Eviction(v, vb, vg, vf))
                    self.sealed[vb] = self.sealed.get(vb, 0) | (1 << vg)
                    self._release(v, res_ops)
                s = self.free.pop()
                self.slot_info[s] = [b, gr, 0, 0]
                self.block_slot[b] = s
                protected.add(s)
                res_ops.append((b, s))
                grp_ops.append((s, gr))
            for _, r in toks:
                row_res[r] = s
            info = self.slot_info[s]
            info[2] = max(info[2], pmax + 1)
            info[3] = self.step

        tok_res = np.full(n_rows, -1, dtype=np.int64)
        tok_sealed = np.zeros(n_rows, dtype=np.int64)
        for r, s in row_res.items():
            tok_res[r] = s
        for r in row_sealed:
            tok_sealed[r] = 1

        touched = np.array(sorted(blocks_seen), dtype=np.int64)
        touched_fill = np.array([max(blocks_seen[b]) + 1 for b in touched.tolist()], dtype=np.int64)
        touched_count = np.array([len(blocks_seen[b]) for b in touched.tolist()], dtype=np.int64)

        tok_kref = np.full(n_rows, -1, dtype=np.int64)
        k = min(n, self.kref_window)
        if k:
            for i, r in enumerate(rows[n - k:]):
                tok_kref[r] = (self.kref_pos + i) % self.kref_window
            self.kref_pos = (self.kref_pos + k) % self.kref_window
            self.kref_fill = min(self.kref_window, self.kref_fill + k)

        fin = np.array(fin_rows, dtype=np.int64).reshape(-1, 3 + g)
        return Plan(
            step=self.step, n_rows=n_rows, tok_slot=sm.copy(), tok_res=tok_res, tok_sealed=tok_sealed,
            tok_kref=tok_kref, fin=fin, evictions=evictions, open_blocks=open_blocks, touched=touched,
            touched_fill=touched_fill, touched_count=touched_count,
            res_map=dict(res_ops), grp_map=dict(grp_ops),
        )


# --------------------------------------------------------------------------
# tiered_cache.py + kernels/write.py: the store
# --------------------------------------------------------------------------


class Store:
    """One layer's tiered store over a byte array of pages.

    Restates echokv_vllm/tiered_cache.py:150-478 (TieredKVCache) and the
    PyTorch write path echokv_vllm/kernels/write.py:61-121.  ``backing`` may be
    given to model strided pages (page_stride > page size), as the reference's
    ``make_cache(row_pad=...)`` test helper does.
    """

    def __init__(self, layout: Layout, num_blocks: int, page_bytes: int | None = None,
                 page_stride: int | None = None, residual_slots: int = 256,
                 residual_dtype=np.float32, kref_window: int | None = None, fill: int = 0,
                 planner: Planner | None = None):
        L = layout
        self.layout = L
        self.num_blocks = n = num_blocks
        pb = page_bytes if page_bytes is not None else L.page_bytes
        if pb < L.page_bytes:
            raise ValueError("page too small for layout")
        ps = page_stride if page_stride is not None else pb
        if ps % 16:
            raise ValueError("page stride must be 16-byte aligned")
        self.page_size, self.page_stride = pb, ps
        self.backing = np.full(n * ps + 64, fill, dtype=np.uint8)
        self.pages = np.lib.stride_tricks.as_strided(self.backing, (n, pb), (ps, 1))
        self.pages[:, : L.block_size] = 0  # tiered_cache.py:194
        k = L.chunks_per_page
        self.free = np.arange(n * k).reshape(n, k)[:, 1:].reshape(-1)[::-1].tolist()  # :200-202
        self.pool_size = len(self.free)
        self.tag_h = np.zeros(n, dtype=np.int64)
        self.table_h = np.zeros((n, 3), dtype=np.int64)
        r = residual_slots
        self.res_dtype = residual_dtype  # np.float32 / np.float16 / "bf16"
        self.res_k = np.zeros((r + 1, L.k_group, L.num_kv_heads, L.head_size), dtype=np.float32)
        self.planner = planner or Planner(L.block_size, L.k_group, r,
                                          kref_window if kref_window is not None else L.k_group)
        self.block_res = np.full(n, -1, dtype=np.int64)
        self.res_group = np.zeros(r + 1, dtype=np.int64)
        self.fill_h = np.zeros(n, dtype=np.int64)
        self.last_h = np.zeros(n, dtype=np.int64)
        self.cum_h = np.zeros(n, dtype=np.int64)
        self.blocks_opened = {b: 0 for b in SUPPORTED_BITS}
        self.downgraded_blocks = 0
        self.demoted_blocks = 0
        self.sealed_groups = 0

    # ---- typed views over the page bytes ---------------------------------
    def _f16(self, blk: int, name: str, nxt: str, *shape) -> np.ndarray:
        o = self.layout.offsets
        return self.pages[blk, o[name]:o[nxt]].view(np.float16).reshape(*shape)

    def v_scale(self, blk):
        L = self.layout
        return self._f16(blk, "v_scale", "v_min", L.block_size, L.num_kv_heads, L.v_groups)

    def v_min(self, blk):
        L = self.layout
        return self._f16(blk, "v_min", "k_scale", L.block_size, L.num_kv_heads, L.v_groups)

    def k_scale(self, blk):
        L = self.layout
        return self._f16(blk, "k_scale", "k_min", L.kgpb, L.num_kv_heads, L.head_size)

    def k_min(self, blk):
        L = self.layout
        return self._f16(blk, "k_min", "data", L.kgpb, L.num_kv_heads, L.head_size)

    def tag(self, blk: int) -> int:
        return int(self.pages[blk, 0])

    def table(self, blk: int) -> np.ndarray:
        return self.pages[blk, 4:16].view(np.int32)

    @property
    def pool_free(self) -> int:
        return len(self.free)

    @property
    def residual_free(self) -> int:
        return len(self.planner.free)

    def _res_round(self, x: np.ndarray) -> np.ndarray:
        """Round fp32 to the residual buffer's dtype and widen back (it stores K in model dtype)."""
        if self.res_dtype is np.float32 or self.res_dtype == np.float32:
            return np.asarray(x, dtype=np.float32)
        if self.res_dtype is np.float16 or self.res_dtype == np.float16:
            return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)
        return bf16_bits_to_f32(f32_to_bf16_bits(np.asarray(x, dtype=np.float32)))

    # ---- addressing: tiered_cache.py:350-359 -----------------------------
    def _row(self, blk: int, off: int, bits: int) -> np.ndarray:
        """Byte view of token ``off``'s K+V row of block ``blk`` stored at ``bits``."""
        L = self.layout
        tpc = L.tokens_per_chunk(bits)
        j = off // tpc
        if j > 0:
            cid = int(self.table(blk)[j - 1])
            page, slot = cid // L.chunks_per_page, cid % L.chunks_per_page
        else:
            page, slot = blk, 0
        base = L.offsets["data"] + slot * L.chunk_bytes + (off % tpc) * L.row_bytes(bits)
        return self.pages[page, base: base + L.row_bytes(bits)]

    def _put_side(self, blk: int, off: int, bits: int, codes_hd: np.ndarray, side: int) -> None:
        sb = self.layout.side_bytes(bits)
        self._row(blk, off, bits)[side * sb:(side + 1) * sb] = pack(codes_hd, bits).reshape(-1)

    def _get_side(self, blk: int, off: int, bits: int, side: int) -> np.ndarray:
        L = self.layout
        sb = L.side_bytes(bits)
        raw = self._row(blk, off, bits)[side * sb:(side + 1) * sb]
        return unpack(raw, bits).reshape(L.num_kv_heads, L.head_size)

    # ---- chunk pool: tiered_cache.py:258-346 -----------------------------
    def open_blocks(self, blocks, target_bits: int, protect=None):
        if target_bits not in SUPPORTED_BITS:
            raise ValueError(f"unsupported target bits {target_bits}")
        blocks = np.asarray(blocks, dtype=np.int64)
        for b in blocks.tolist():
            ne = NEXTRA.get(int(self.tag_h[b]), 0)
            self.free.extend(self.table_h[b, :ne].tolist())
            self.tag_h[b] = 0
        need = NEXTRA[target_bits] * blocks.size
        if need > len(self.free):
            keep = set(blocks.tolist()) | (set() if protect is None else set(np.asarray(protect).tolist()))
            self._demote_lru(need - len(self.free), keep)
        tiers = np.full(blocks.size, 2, dtype=np.int64)
        start = 0
        for bits in (x for x in (8, 4) if x <= target_bits):
            ne = NEXTRA[bits]
            take = min(blocks.size - start, len(self.free) // ne)
            if take:
                sel = blocks[start:start + take]
                ids = self.free[len(self.free) - take * ne:][::-1]
                del self.free[len(self.free) - take * ne:]
                self.table_h[sel, :ne] = np.asarray(ids, dtype=np.int64).reshape(take, ne)
                tiers[start:start + take] = bits
                start += take
        for bits in SUPPORTED_BITS:
            self.blocks_opened[bits] += int((tiers == bits).sum())
        self.downgraded_blocks += int((tiers < target_bits).sum())
        self.tag_h[blocks] = tiers
        headers = np.zeros((blocks.size, 16), dtype=np.uint8)
        headers[:, 0] = tiers
        headers[:, 4:] = np.ascontiguousarray(self.table_h[blocks].astype(np.int32)).view(np.uint8)
        return blocks, headers

    def _demote_lru(self, chunks_needed: int, keep: set) -> None:
        L = self.layout
        cand = np.nonzero((self.tag_h >= 4) & (self.fill_h == L.block_size))[0]
        cand = [b for b in cand[np.argsort(self.last_h[cand], kind="stable")].tolist() if b not in keep]
        victims, freed = [], 0
        for b in cand:
            if freed >= chunks_needed:
                break
            victims.append(b)
            freed += NEXTRA[int(self.tag_h[b])]
        if not victims:
            return
        bs, g = L.block_size, L.k_group
        for b in victims:
            k, v = self.gather(np.full(bs, b), np.arange(bs))  # at the current tier
            kg = k.reshape(bs // g, g, L.num_kv_heads, L.head_size)
            ks, km = stats_along(kg, 2, axis=1)
            kc = quantize_with(kg, ks[:, None], km[:, None], 2).reshape(bs, L.num_kv_heads, L.head_size)
            vc, vs, vm = quantize(v, 2, L.v_group)
            self.pages[b, 0] = 2
            self.k_scale(b)[...] = ks
            self.k_min(b)[...] = km
            self.v_scale(b)[...] = vs
            self.v_min(b)[...] = vm
            for t in range(bs):
                self._put_side(b, t, 2, kc[t], 0)
                self._put_side(b, t, 2, vc[t], 1)
        for b in victims:
            ne = NEXTRA[int(self.tag_h[b])]
            self.free.extend(self.table_h[b, :ne].tolist())
            self.tag_h[b] = 2
        self.demoted_blocks += len(victims)

    # ---- write: tiered_cache.py:379-447, kernels/write.py:61-121 ---------
    def _seal(self, ev: Eviction) -> None:
        if ev.fill <= 0:
            return
        g = self.layout.k_group
        bits = int(self.tag_h[ev.block]) or 2
        ks = self.res_k[ev.slot, :ev.fill]
        scale, mn = stats_along(ks, bits, axis=0)
        self.k_scale(ev.block)[ev.group] = scale
        self.k_min(ev.block)[ev.group] = mn
        codes = quantize_with(ks, scale, mn, bits)
        for i in range(ev.fill):
            self._put_side(ev.block, ev.group * g + i, bits, codes[i], 0)
        self.pages[ev.block, 1] = self.planner.sealed.get(ev.block, 1 << ev.group) & 0xFF
        self.sealed_groups += 1

    def prepare(self, plan: Plan, target_bits: int):
        for ev in plan.evictions:
            self._seal(ev)
        opens = plan.open_blocks
        if plan.touched.size:
            fresh = plan.touched[self.tag_h[plan.touched] == 0]
            if fresh.size:
                opens = np.union1d(opens, fresh)
        if not opens.size:
            return None
        return self.open_blocks(opens, target_bits, protect=plan.touched)

    def commit(self, plan: Plan) -> None:
        t = plan.touched
        if t.size:
            self.fill_h[t] = np.maximum(self.fill_h[t], plan.touched_fill)
            self.last_h[t] = plan.step
            self.cum_h[t] += plan.touched_count

    def apply_res_map(self, plan: Plan) -> None:
        for b, s in plan.res_map.items():
            self.block_res[b] = s
        for s, gr in plan.grp_map.items():
            self.res_group[s] = gr

    def write_headers(self, blocks, headers) -> None:
        for b, h in zip(np.asarray(blocks).tolist(), headers):
            self.pages[b, :16] = h

    def finalize_k(self, key: np.ndarray, fin: np.ndarray) -> None:
        """kernels/write.py:96-121. ``key`` float32 [n_rows, H, D]."""
        L = self.layout
        g = L.k_group
        for line in fin.tolist():
            b, gr, rslot = line[0], line[1], line[2]
            rows = line[3:]
            full = np.empty((g, L.num_kv_heads, L.head_size), dtype=np.float32)
            for p, r in enumerate(rows):
                full[p] = key[r] if r >= 0 else self.res_k[max(rslot, 0), p]
            bits = self.tag(b) or 2
            scale, mn = stats_along(full, bits, axis=0)
            self.k_scale(b)[gr] = scale
            self.k_min(b)[gr] = mn
            codes = quantize_with(full, scale, mn, bits)
            for p in range(g):
                self._put_side(b, gr * g + p, bits, codes[p], 0)

    def write_tokens(self, key, value, plan: Plan, kref: np.ndarray | None) -> None:
        """kernels/write.py:61-93."""
        L = self.layout
        bs, g = L.block_size, L.k_group
        for r in range(plan.n_rows):
            slot = int(plan.tok_slot[r])
            if slot < 0:
                continue
            b, off = divmod(slot, bs)
            bits = self.tag(b) or 2
            codes, scale, mn = quantize(value[r], bits, L.v_group)
            self.v_scale(b)[off] = scale
            self.v_min(b)[off] = mn
            self._put_side(b, off, bits, codes, 1)
            rs = int(plan.tok_res[r])
            if rs >= 0:
                self.res_k[rs, off % g] = self._res_round(key[r])
            if plan.tok_sealed[r]:
                kc = quantize_with(key[r], self.k_scale(b)[off // g], self.k_min(b)[off // g], bits)
                self._put_side(b, off, bits, kc, 0)
            if kref is not None and plan.tok_kref[r] >= 0:
                kref[int(plan.tok_kref[r])] = key[r]

    def write(self, key, value, slots, target_bits: int, kref: np.ndarray | None = None) -> Plan:
        """tiered_cache.py:434-447: plan, prepare, commit, stage, apply. key/value float32 [n,H,D]
        holding values already rounded to the model dtype."""
        key = np.asarray(key, dtype=np.float32)
        value = np.asarray(value, dtype=np.float32)
        plan = self.planner.plan(slots)
        opened = self.prepare(plan, target_bits)
        self.commit(plan)
        self.apply_res_map(plan)
        if opened is not None:
            self.write_headers(*opened)
        if plan.fin.shape[0]:
            self.finalize_k(key, plan.fin)
        self.write_tokens(key, value, plan, kref)
        return plan

    # ---- read: tiered_cache.py:451-478 -----------------------------------
    def gather(self, blk, off):
        """Dequantized K, V float32 [n, H, D] for tokens at (blk, off)."""
        L = self.layout
        blk = np.asarray(blk, dtype=np.int64).reshape(-1)
        off = np.asarray(off, dtype=np.int64).reshape(-1)
        n = blk.size
        h, d, g = L.num_kv_heads, L.head_size, L.k_group
        k_out = np.zeros((n, h, d), dtype=np.float32)
        v_out = np.zeros((n, h, d), dtype=np.float32)
        for i in range(n):
            b, o = int(blk[i]), int(off[i])
            bits = self.tag(b)
            if bits not in SUPPORTED_BITS:
                continue  # never opened: the reference returns zeros
            vc = self._get_side(b, o, bits, 1)
            v_out[i] = dequantize(vc, self.v_scale(b)[o], self.v_min(b)[o], L.v_group)
            slot = int(self.block_res[b])
            if slot >= 0 and int(self.res_group[slot]) == o // g:
                k_out[i] = self.res_k[slot, o % g]
            else:
                kc = self._get_side(b, o, bits, 0)
                k_out[i] = dequantize_with(kc, self.k_scale(b)[o // g], self.k_min(b)[o // g])
        return k_out, v_out

    def gather_seq(self, block_row: np.ndarray, n: int):
        """K, V of a sequence's first ``n`` tokens (block-vectorized gather)."""
        L = self.layout
        bs, g, h, d = L.block_size, L.k_group, L.num_kv_heads, L.head_size
        k_out = np.zeros((n, h, d), dtype=np.float32)
        v_out = np.zeros((n, h, d), dtype=np.float32)
        for bi in range(-(-n // bs)):
            b = int(block_row[bi])
            cnt = min(bs, n - bi * bs)
            bits = self.tag(b)
            if bits not in SUPPORTED_BITS:
                continue
            sb = L.side_bytes(bits)
            tpc = L.tokens_per_chunk(bits)
            rows = np.empty((cnt, 2 * sb), dtype=np.uint8)
            for c0 in range(0, cnt, tpc):
                c1 = min(cnt, c0 + tpc)
                first = self._row(b, c0, bits)
                page_off = first.__array_interface__["data"][0] - self.backing.__array_interface__["data"][0]
                rows[c0:c1] = self.backing[page_off: page_off + (c1 - c0) * 2 * sb].reshape(c1 - c0, 2 * sb)
            kc = unpack(rows[:, :sb], bits).reshape(cnt, h, d)
            vc = unpack(rows[:, sb:], bits).reshape(cnt, h, d)
            v_out[bi * bs: bi * bs + cnt] = dequantize(vc, self.v_scale(b)[:cnt], self.v_min(b)[:cnt], L.v_group)
            grp = np.arange(cnt) // g
            kd = dequantize_with(kc, self.k_scale(b)[grp], self.k_min(b)[grp])
            slot = int(self.block_res[b])
            if slot >= 0:
                rg = int(self.res_group[slot])
                m = grp == rg
                kd[m] = self.res_k[slot, np.arange(cnt)[m] % g]
            k_out[bi * bs: bi * bs + cnt] = kd
        return k_out, v_out


# --------------------------------------------------------------------------
# kernels/decode.py, kernels/prefill.py: attention over the store
# --------------------------------------------------------------------------


def _softmax_rows(s: np.ndarray) -> np.ndarray:
    m = s.max(axis=-1, keepdims=True)
    e = np.exp(s - m)
    return e / e.sum(axis=-1, keepdims=True)


def decode_attention(store: Store, query: np.ndarray, block_table: np.ndarray, seq_lens,
                     softmax_scale: float) -> np.ndarray:
    """echokv_vllm/kernels/decode.py:95-129 (decode_attention_torch): float32 [S, Hq, D]."""
    q = np.asarray(query, dtype=np.float32)
    s, hq, d = q.shape
    h = store.layout.num_kv_heads
    rep = hq // h
    out = np.zeros((s, hq, d), dtype=np.float32)
    for i in range(s):
        n = int(seq_lens[i])
        if n == 0:
            continue
        k, v = store.gather_seq(np.asarray(block_table[i]), n)  # [n, H, D]
        kh = np.repeat(k.transpose(1, 0, 2), rep, axis=0)  # [Hq, n, D]
        vh = np.repeat(v.transpose(1, 0, 2), rep, axis=0)
        sc = np.einsum("hd,hnd->hn", q[i], kh) * np.float32(softmax_scale)
        p = _softmax_rows(sc.astype(np.float32))
        out[i] = np.einsum("hn,hnd->hd", p, vh)
    return out


def prefill_attention(store: Store, query: np.ndarray, prefill, req_of, block_table: np.ndarray,
                      softmax_scale: float, round_kv=None) -> np.ndarray:
    """echokv_vllm/kernels/prefill.py:210-236 (prefill_attention_torch).

    ``prefill`` holds (q_start, q_end, ctx, _); bottom-right causal mask.  The
    reference casts the gathered K/V to the query dtype first; ``round_kv`` is
    that rounding (None = float32 queries).
    """
    q = np.asarray(query, dtype=np.float32)
    out = np.zeros_like(q)
    h = store.layout.num_kv_heads
    rep = q.shape[1] // h
    for (qs, qe, ctx, _), r in zip(prefill, req_of):
        nq = qe - qs
        k, v = store.gather_seq(np.asarray(block_table[r]), ctx)
        if round_kv is not None:
            k, v = round_kv(k), round_kv(v)
        kh = np.repeat(k.transpose(1, 0, 2), rep, axis=0)
        vh = np.repeat(v.transpose(1, 0, 2), rep, axis=0)
        sc = np.einsum("qhd,hnd->hqn", q[qs:qe], kh) * np.float32(softmax_scale)
        qpos = (ctx - nq) + np.arange(nq)
        mask = np.arange(ctx)[None, :] <= qpos[:, None]
        sc = np.where(mask[None], sc, -np.inf).astype(np.float32)
        p = _softmax_rows(sc)
        out[qs:qe] = np.einsum("hqn,hnd->qhd", p, vh)
    return out


# --------------------------------------------------------------------------
# canary.py, controller.py
# --------------------------------------------------------------------------


def ring_view(buf: np.ndarray, pos: int, fill: int, axis: int = 0) -> np.ndarray:
    """echokv_vllm/canary.py:19-23."""
    if fill < buf.shape[axis]:
        return np.take(buf, np.arange(fill), axis=axis)
    return np.roll(buf, -pos, axis=axis)


def _log_softmax(x: np.ndarray) -> np.ndarray:
    m = x.max(axis=-1, keepdims=True)
    z = x - m
    return z - np.log(np.exp(z).sum(axis=-1, keepdims=True))


def canary_kl(query: np.ndarray, kref: np.ndarray, bits=SUPPORTED_BITS, k_group: int = 32,
              softmax_scale: float = 1.0) -> np.ndarray:
    """echokv_vllm/canary.py:59-89. query [..., nq, Hq, D], kref [..., W, H, D] -> [..., len(bits)]."""
    w = (kref.shape[-3] // k_group) * k_group
    if w == 0:
        raise ValueError("K_ref has fewer keys than k_group")
    kref = np.asarray(kref, dtype=np.float32)[..., kref.shape[-3] - w:, :, :]
    q = np.swapaxes(np.asarray(query, dtype=np.float32), -3, -2)  # [..., Hq, nq, D]
    rep = q.shape[-3] // kref.shape[-2]

    def logw(k):
        kh = np.repeat(np.swapaxes(k, -3, -2), rep, axis=-3)  # [..., Hq, W, D]
        s = np.matmul(q, np.swapaxes(kh, -1, -2)) * np.float32(softmax_scale)
        return _log_softmax(s.astype(np.float32))

    ref = logw(kref)
    out = []
    for b in bits:
        lq = logw(fake_quant_channels(kref, b, k_group))
        out.append((np.exp(lq) * (lq - ref)).sum(-1).mean(axis=(-2, -1)))
    return np.maximum(np.stack(out, -1), 0.0).astype(np.float32)


class Controller:
    """echokv_vllm/controller.py:22-68: EMA per tier, lowest tier under tau."""

    def __init__(self, tau0=0.01, l0=4096, tau_scaling="none", alpha=0.1, init_bits=8,
                 fixed_bits=None, frozen=False):
        self.tau0, self.l0, self.tau_scaling, self.alpha = tau0, l0, tau_scaling, alpha
        self.fixed_bits, self.frozen = fixed_bits, frozen
        self.bits = fixed_bits or init_bits
        self.ema = {b: None for b in SUPPORTED_BITS}
        self.fires = 0
        self.transitions = 0

    def tau(self, ctx_len: float) -> float:
        if self.tau_scaling == "sqrt":
            return self.tau0 * (max(ctx_len, self.l0) / self.l0) ** 0.5
        return self.tau0

    def observe(self, deltas: dict, ctx_len: float) -> None:
        for b, d in deltas.items():
            prev = self.ema[b]
            self.ema[b] = d if prev is None else self.alpha * d + (1.0 - self.alpha) * prev
        self.fires += 1
        if self.frozen or self.fixed_bits is not None:
            return
        tau = self.tau(ctx_len)
        new = max(SUPPORTED_BITS)
        for b in sorted(SUPPORTED_BITS):
            e = self.ema[b]
            if e is not None and e < tau:
                new = b
                break
        if new != self.bits:
            self.transitions += 1
            self.bits = new
