"""Seeded scenarios shared by the fixture generator, the oracle tests and the GPU parity tests.

A scenario is a store configuration plus a sequence of write steps
``(key, value, slots, target_bits)`` and, optionally, attention queries.  All
values come from ``numpy.random.default_rng(seed)`` (PCG64, stable across
numpy versions) as float32 and are rounded to the scenario's model dtype, so
the reference, the oracle and the CUDA path all see identical bits.

The scenarios mirror the reference's own tests:
tests/echokv_vllm/test_tiered_cache.py, test_step_path.py,
test_decode_kernel.py (CASES :69-75), test_prefill_kernel.py (CASES :9-14),
plus the benchmark's CPU-runnable configuration (batch 4, 8 query heads, 2 KV
heads, head_dim 128, block 16, INT4, 160 physical blocks).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np


def round_to(x: np.ndarray, dtype: str) -> np.ndarray:
    """float32 values representable in ``dtype`` ('f32' | 'f16' | 'bf16')."""
    x = np.asarray(x, dtype=np.float32)
    if dtype == "f32":
        return x
    if dtype == "f16":
        return x.astype(np.float16).astype(np.float32)
    u = np.ascontiguousarray(x).view(np.uint32)
    r = (u + (np.uint32(0x7FFF) + ((u >> 16) & np.uint32(1)))) & np.uint32(0xFFFF0000)
    return r.view(np.float32)


@dataclass
class StoreSpec:
    h: int
    d: int
    bs: int
    mem_bits: int
    kg: int = 32
    vg: int = 32
    num_blocks: int = 8
    row_pad: int = 0  # bytes between consecutive pages (layer-interleaved pools)
    page_extra: int = 0  # bytes of the page beyond per_token_bytes * bs that belong to the page
    residual_slots: int = 16
    dtype: str = "f32"  # model dtype of K/V and of the residual buffer
    fill: int = 0  # initial byte value of the backing buffer
    kref_window: int | None = None  # None: k_group (standalone store default)

    @property
    def per_token(self) -> int:
        h, d = self.h, self.d
        raw = 1 + 4 * h * (d // self.vg) + 4 * h * d // self.kg + (self.mem_bits // 2) * h * d // 2
        return -(-raw // 4) * 4

    @property
    def page_size(self) -> int:
        return self.bs * self.per_token + self.page_extra

    @property
    def page_stride(self) -> int:
        return self.page_size + self.row_pad


@dataclass
class Scenario:
    name: str
    spec: StoreSpec
    steps: list = field(default_factory=list)  # (key, value, slots, bits)
    use_kref: bool = False
    # attention part (optional)
    block_table: np.ndarray | None = None
    seq_lens: list | None = None
    query: np.ndarray | None = None  # decode: [S, Hq, D]; prefill: [T, Hq, D]
    scale: float = 1.0
    prefill: list | None = None  # (q_start, q_end, ctx, 0)
    req_of: list | None = None
    # gather checks: list of (blk array, off array)
    gathers: list = field(default_factory=list)


def _tokens(rng, n, h, d, dtype, outlier_ch=3, outlier=40.0):
    k = rng.standard_normal((n, h, d), dtype=np.float32)
    v = rng.standard_normal((n, h, d), dtype=np.float32)
    if outlier:
        k[..., outlier_ch] += np.float32(outlier)
    return round_to(k, dtype), round_to(v, dtype)


# ---------------------------------------------------------------- store scenarios
# tests/echokv_vllm/test_tiered_cache.py: H, D, BS, KG, VG = 2, 64, 64, 32, 32

_TC = dict(h=2, d=64, bs=64, kg=32, vg=32)
BS = 64


def store_scenarios() -> list[Scenario]:
    out = []
    for bits in (2, 4, 8):  # test_uniform_roundtrip
        rng = np.random.default_rng(100 + bits)
        sp = StoreSpec(**_TC, mem_bits=8, num_blocks=6)
        k, v = _tokens(rng, 6 * BS, 2, 64, "f32")
        sc = Scenario(f"uniform_{bits}", sp, [(k, v, np.arange(6 * BS), bits)])
        sc.gathers = [(np.repeat(np.arange(6), BS), np.tile(np.arange(BS), 6))]
        out.append(sc)

    rng = np.random.default_rng(1)  # test_tier_change_is_forward_only
    sp = StoreSpec(**_TC, mem_bits=8, num_blocks=6)
    k, v = _tokens(rng, 6 * BS, 2, 64, "f32")
    steps = []
    for b, bits in enumerate([8, 2, 4, 8, 2, 4]):
        sl = slice(b * BS, (b + 1) * BS)
        steps.append((k[sl], v[sl], np.arange(b * BS, (b + 1) * BS), bits))
    sc = Scenario("forward_only", sp, steps)
    sc.gathers = [(np.repeat(np.arange(6), BS), np.tile(np.arange(BS), 6))]
    out.append(sc)

    for dt in ("f32", "bf16"):  # test_decode_one_token_at_a_time (+ a bf16 residual variant)
        rng = np.random.default_rng(2)
        sp = StoreSpec(**_TC, mem_bits=8, num_blocks=3, dtype=dt)
        k, v = _tokens(rng, 3 * BS, 2, 64, dt)
        n = 2 * BS + 40
        steps = [(k[t:t + 1], v[t:t + 1], np.array([t]), [4, 8, 2][t % 3]) for t in range(n)]
        sc = Scenario(f"one_token_{dt}", sp, steps)
        pos = np.arange(n)
        sc.gathers = [(pos // BS, pos % BS)]
        out.append(sc)

    rng = np.random.default_rng(3)  # test_prefill_then_decode_completes_group_from_residual
    sp = StoreSpec(**_TC, mem_bits=8, num_blocks=2, dtype="f16")
    k, v = _tokens(rng, BS, 2, 64, "f16")
    sc = Scenario("prefill_then_decode", sp, [
        (k[:20], v[:20], np.arange(20), 4),
        (k[20:50], v[20:50], np.arange(20, 50), 4),
        (k[50:], v[50:], np.arange(50, BS), 4),
    ])
    sc.gathers = [(np.zeros(BS, dtype=np.int64), np.arange(BS))]
    out.append(sc)

    rng = np.random.default_rng(4)  # test_pool_exhaustion_downgrades_without_overlap
    n = 12
    sp = StoreSpec(**_TC, mem_bits=4, num_blocks=n, row_pad=48, fill=0xAB)
    k, v = _tokens(rng, n * BS, 2, 64, "f32")
    sc = Scenario("pool_exhaustion", sp, [(k, v, np.arange(n * BS), 8)])
    sc.gathers = [(np.repeat(np.arange(n), BS), np.tile(np.arange(BS), n))]
    out.append(sc)

    sp = StoreSpec(**_TC, mem_bits=4, num_blocks=4)  # test_pool_pressure_demotes_lru_full_block
    k0, v0 = _tokens(np.random.default_rng(5), BS, 2, 64, "f32")
    k1, v1 = _tokens(np.random.default_rng(6), BS, 2, 64, "f32")
    sc = Scenario("demote_lru", sp, [(k0, v0, np.arange(BS), 8), (k1, v1, np.arange(BS, 2 * BS), 8)])
    sc.gathers = [(np.repeat(np.arange(2), BS), np.tile(np.arange(BS), 2))]
    out.append(sc)

    sp = StoreSpec(**_TC, mem_bits=4, num_blocks=4)  # test_pool_pressure_without_victims_opens_lower
    k0, v0 = _tokens(np.random.default_rng(5), 40, 2, 64, "f32")
    k1, v1 = _tokens(np.random.default_rng(6), BS, 2, 64, "f32")
    sc = Scenario("no_victims", sp, [(k0, v0, np.arange(40), 8), (k1, v1, np.arange(BS, 2 * BS), 8)])
    sc.gathers = [(np.r_[np.zeros(40, dtype=np.int64), np.ones(BS, dtype=np.int64)], np.r_[np.arange(40), np.arange(BS)])]
    out.append(sc)

    sp = StoreSpec(**_TC, mem_bits=8, num_blocks=4)  # test_reopen_returns_chunks_and_residual
    k, v = _tokens(np.random.default_rng(7), 4 * BS, 2, 64, "f32")
    k2, v2 = _tokens(np.random.default_rng(8), BS, 2, 64, "f32")
    sc = Scenario("reopen", sp, [
        (k[:3 * BS + 10], v[:3 * BS + 10], np.arange(3 * BS + 10), 8),
        (k2, v2, np.arange(3 * BS, 4 * BS), 2),
        (k2, v2, np.arange(0, BS), 2),
    ])
    sc.gathers = [(np.repeat(np.arange(4), BS), np.tile(np.arange(BS), 4))]
    out.append(sc)

    sp = StoreSpec(**_TC, mem_bits=6, num_blocks=10)  # test_interleaved_requests_partial_blocks
    a = np.arange(3 * BS, 3 * BS + 21)
    b = np.arange(7 * BS, 7 * BS + 37)
    rng = np.random.default_rng(9)
    k, v = _tokens(rng, a.size + b.size, 2, 64, "f32")
    order = np.random.default_rng(0).permutation(a.size + b.size)
    slots = np.r_[a, b]
    sc = Scenario("interleaved", sp, [(k[order], v[order], slots[order], 4)])
    sc.gathers = [(np.r_[np.full(21, 3), np.full(37, 7)], np.r_[np.arange(21), np.arange(37)])]
    out.append(sc)

    sp = StoreSpec(**_TC, mem_bits=8, num_blocks=6, residual_slots=2)  # test_residual_eviction_seals_lru_group
    k, v = _tokens(np.random.default_rng(10), 6 * BS, 2, 64, "f32")
    steps = [(k[b * BS:b * BS + 5], v[b * BS:b * BS + 5], np.arange(b * BS, b * BS + 5), 8) for b in range(3)]
    steps.append((k[5:BS], v[5:BS], np.arange(5, BS), 8))
    sc = Scenario("eviction_seal", sp, steps)
    sc.gathers = [(np.r_[np.zeros(BS, dtype=np.int64), np.full(5, 1), np.full(5, 2)],
                   np.r_[np.arange(BS), np.arange(5), np.arange(5)])]
    out.append(sc)

    # test_step_path.py: prefill of two requests, then 60 decode steps with padding rows (slot -1)
    H, D = 2, 64
    sp = StoreSpec(h=H, d=D, bs=BS, kg=32, vg=32, mem_bits=8, num_blocks=8, residual_slots=8, dtype="bf16")
    rng = np.random.default_rng(11)
    steps = []

    def sl_iter():
        yield np.r_[np.arange(40), 3 * BS + np.arange(10)]
        for i in range(60):
            a_, b_ = 40 + i, 10 + i
            yield np.array([[0, 5][a_ // BS] * BS + a_ % BS, [3, 6][b_ // BS] * BS + b_ % BS])

    for i, sl in enumerate(sl_iter()):
        bits = (8, 4, 2)[(i // 7) % 3]
        k, v = _tokens(rng, sl.size + 3, H, D, "bf16", outlier_ch=1, outlier=30.0)
        steps.append((k, v, np.r_[sl, np.full(3, -1)], bits))
    sc = Scenario("step_path_padded", sp, steps, use_kref=True)
    out.append(sc)
    return out


# ---------------------------------------------------------------- attention scenarios


def build_attention(name, h, d, bs, mem_bits, seq_lens, tier_plan, seed, kg=32, vg=32, dtype="f32",
                    num_blocks=None, gqa=4, outlier_ch=(1,), outlier_add=30.0, outlier_mul=None,
                    chunks=None) -> Scenario:
    """test_decode_kernel.py:20-50 ``build``: block i of sequence s opens at tier_plan[(i+s) % n],
    written block by block with sequences interleaved.  ``chunks`` makes it a prefill scenario."""
    rng = np.random.default_rng(seed)
    bps = [-(-n // bs) for n in seq_lens]
    num_blocks = num_blocks or sum(bps) + 3
    sp = StoreSpec(h=h, d=d, bs=bs, mem_bits=mem_bits, kg=kg, vg=vg, num_blocks=num_blocks,
                   residual_slots=len(seq_lens) + 2, dtype=dtype, row_pad=32)
    perm = rng.permutation(num_blocks)
    table = np.zeros((len(seq_lens), max(bps)), dtype=np.int32)
    nxt = 0
    for s, nb in enumerate(bps):
        table[s, :nb] = perm[nxt:nxt + nb]
        nxt += nb
    steps = []
    for bi in range(max(bps)):
        for s, n in enumerate(seq_lens):
            lo, hi = bi * bs, min((bi + 1) * bs, n)
            if lo >= hi:
                continue
            k = rng.standard_normal((hi - lo, h, d), dtype=np.float32)
            v = rng.standard_normal((hi - lo, h, d), dtype=np.float32)
            for c in outlier_ch:
                if outlier_mul is not None:
                    k[..., c] *= np.float32(outlier_mul)
                else:
                    k[..., c] += np.float32(outlier_add)
            slots = int(table[s, bi]) * bs + np.arange(hi - lo)
            steps.append((round_to(k, dtype), round_to(v, dtype), slots, tier_plan[(bi + s) % len(tier_plan)]))
    sc = Scenario(name, sp, steps)
    sc.block_table = table
    sc.seq_lens = list(seq_lens)
    sc.scale = float(d) ** -0.5
    hq = gqa * h
    if chunks is None:
        sc.query = round_to(rng.standard_normal((len(seq_lens), hq, d), dtype=np.float32), dtype)
    else:
        prefill, req_of, row = [], [], 0
        for r, (ctx, nq) in enumerate(zip(seq_lens, chunks)):
            prefill.append((row, row + nq, ctx, 0))
            req_of.append(r)
            row += nq
        sc.prefill, sc.req_of = prefill, req_of
        sc.query = round_to(rng.standard_normal((row, hq, d), dtype=np.float32), dtype)
    return sc


DECODE_CASES = [  # test_decode_kernel.py:69-75
    (2, 64, 64, 8, [1, 40, 64, 65, 200], [8, 4, 2]),
    (1, 128, 32, 4, [33, 97, 128], [8, 8, 4]),
    (4, 64, 64, 6, [500, 3], [2, 4]),
    (8, 128, 64, 8, [200, 70], [8, 4, 2]),
]

PREFILL_CASES = [  # test_prefill_kernel.py:9-14
    (2, 64, 64, 8, [70, 200, 33], [70, 40, 1], [8, 4, 2]),
    (8, 128, 64, 8, [300, 130], [17, 130], [4, 8]),
    (1, 128, 32, 4, [97], [50], [8, 8, 4]),
]


def decode_scenarios() -> list[Scenario]:
    out = []
    for i, (h, d, bs, mem, lens, plan) in enumerate(DECODE_CASES):
        for gqa in (1, 4):
            out.append(build_attention(f"decode_case{i}_gqa{gqa}", h, d, bs, mem, lens, plan, seed=20 + i, gqa=gqa))
    # block_size 16 / k_group 16 (the benchmark's geometry), mixed tiers, bf16
    out.append(build_attention("decode_bs16_bf16", 8, 128, 16, 8, [77, 16, 250, 33], [4, 8, 2, 4], seed=30,
                               kg=16, dtype="bf16", gqa=4))
    out.append(build_attention("decode_bs16_gqa8", 1, 128, 16, 4, [300, 45], [4, 4, 2], seed=31,
                               kg=16, dtype="bf16", gqa=8))
    out.append(config1())
    return out


def config1() -> Scenario:
    """The benchmark's CPU-runnable configuration: batch 4, Hq 8, H 2, D 128, block 16, INT4,
    160 physical blocks, lens uniform in [32, 512], fp16, 4 K channels scaled x8."""
    rng = np.random.default_rng(0)
    lens = rng.integers(32, 513, size=4).tolist()
    return build_attention("config1", 2, 128, 16, 4, lens, [4], seed=1, kg=16, dtype="f16", num_blocks=160,
                           gqa=4, outlier_ch=(3, 17, 64, 101), outlier_mul=8.0)


def prefill_scenarios() -> list[Scenario]:
    out = []
    for i, (h, d, bs, mem, ctxs, chunks, plan) in enumerate(PREFILL_CASES):
        for gqa in (1, 4, 7):
            out.append(build_attention(f"prefill_case{i}_gqa{gqa}", h, d, bs, mem, ctxs, plan, seed=40 + i,
                                       gqa=gqa, chunks=chunks))
    out.append(build_attention("prefill_bs16_bf16", 8, 128, 16, 8, [200, 90], [4, 8], seed=50, kg=16,
                               dtype="bf16", gqa=4, chunks=[136, 90]))
    return out


def canary_inputs():
    """test_step_path.py:87-97 / test_canary_controller.py:20-41 shapes."""
    rng = np.random.default_rng(60)
    cases = []
    q = rng.standard_normal((3, 5, 8, 64), dtype=np.float32) * 3
    kref = rng.standard_normal((3, 70, 2, 64), dtype=np.float32) * 3
    cases.append(("layers3_w70", q, kref, 32, 64 ** -0.5))
    q = rng.standard_normal((4, 8, 64), dtype=np.float32) * 3
    kref = rng.standard_normal((64, 2, 64), dtype=np.float32) * 3
    cases.append(("single_w64", q, kref, 32, 64 ** -0.5))
    q = rng.standard_normal((32, 8, 32, 128), dtype=np.float32)
    kref = rng.standard_normal((32, 64, 8, 128), dtype=np.float32)
    kref[..., 5] *= 10.0
    cases.append(("llama8b_l32", q, kref, 16, 128 ** -0.5))
    return cases


def all_scenarios() -> list[Scenario]:
    return store_scenarios() + decode_scenarios() + prefill_scenarios()
