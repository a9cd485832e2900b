"""Host logic without a GPU: the write planner and the chunk pool against the oracle's plain
restatement (itself pinned to the reference) on seeded request traffic, the layout arithmetic
through the C ABI, and that the shared library exports every declared symbol."""

import ctypes
import re
from pathlib import Path

import numpy as np
import pytest

from oracle import echokv_oracle as O

ROOT = Path(__file__).resolve().parent.parent


def traffic(seed, bs, n_blocks, n_req, steps):
    """Slot mappings of a continuous-batching run: requests prefill in chunks, decode one token
    per step, finish and hand their blocks back; rows arrive in shuffled order with padding."""
    rng = np.random.default_rng(seed)
    free = list(rng.permutation(n_blocks))
    reqs = {}
    nxt = 0
    for _ in range(steps):
        while len(reqs) < n_req and len(free) > 6:
            reqs[nxt] = dict(blocks=[], pos=0, prompt=int(rng.integers(1, 3 * bs)), total=int(rng.integers(2, 5 * bs)))
            nxt += 1
        slots = []
        for rid in list(reqs):
            r = reqs[rid]
            n = int(min(r["prompt"] - r["pos"], rng.integers(1, 2 * bs))) if r["pos"] < r["prompt"] else 1
            for _ in range(n):
                if r["pos"] % bs == 0:
                    if not free:
                        break
                    r["blocks"].append(free.pop())
                if r["pos"] // bs >= len(r["blocks"]):
                    break
                slots.append(int(r["blocks"][r["pos"] // bs]) * bs + r["pos"] % bs)
                r["pos"] += 1
            if r["pos"] >= max(r["total"], r["prompt"]) or rng.random() < 0.03:
                free.extend(r["blocks"])
                del reqs[rid]
        slots = np.array(slots + [-1] * int(rng.integers(0, 4)), dtype=np.int64)
        yield slots[rng.permutation(slots.size)] if rng.random() < 0.5 else slots


@pytest.mark.parametrize("seed,bs,g,slots", [(0, 64, 32, 6), (1, 16, 16, 5), (2, 32, 16, 40), (3, 128, 32, 3)])
def test_planner_matches_oracle(seed, bs, g, slots):
    from echokv_b200.write_plan import WritePlanner

    mine, ref = WritePlanner(bs, g, slots, 8), O.Planner(bs, g, slots, 8)
    for sm in traffic(seed, bs, 48, 6, 150):
        try:
            b = ref.plan(sm)
        except RuntimeError:
            with pytest.raises(RuntimeError):
                mine.plan(sm)
            return
        a = mine.plan(sm)
        assert a.n_rows == b.n_rows and a.step == b.step
        for x, y in ((a.tok_slot, b.tok_slot), (a.tok_res, b.tok_res), (a.tok_sealed, b.tok_sealed),
                     (a.tok_kref, b.tok_kref), (a.fin, b.fin), (a.open_np, b.open_blocks),
                     (a.touched_np, b.touched), (a.touched_fill, b.touched_fill), (a.touched_count, b.touched_count)):
            assert np.array_equal(x, y)
        assert [(e.slot, e.block, e.group, e.fill) for e in a.evictions] == \
               [(e.slot, e.block, e.group, e.fill) for e in b.evictions]
        assert dict(zip(a.res_map_block.tolist(), a.res_map_value.tolist())) == b.res_map
        assert dict(zip(a.res_group_slot.tolist(), a.res_group_value.tolist())) == b.grp_map
        assert (mine.kref_pos, mine.kref_fill, mine.free, mine.sealed) == (ref.kref_pos, ref.kref_fill, ref.free, ref.sealed)


def test_chunk_pool_matches_oracle_order():
    from echokv_b200.tiered_cache import ChunkPool

    rng = np.random.default_rng(5)
    n, kc = 40, 4
    pool = ChunkPool(n, kc)
    ost = O.Store(O.Layout(2, 64, 64, 8), n, residual_slots=2)
    assert pool.free == ost.free
    for _ in range(60):
        blocks = np.unique(rng.integers(0, n, size=int(rng.integers(1, 6))))
        target = int(rng.choice([2, 4, 8]))
        for b in blocks.tolist():
            pool.release(b, 0)
        tiers = pool.allot(blocks, target)
        _, hdr = ost.open_blocks(blocks, target)  # no full blocks: nothing to demote
        assert np.array_equal(pool.headers(blocks), hdr) and np.array_equal(tiers, ost.tag_h[blocks])
        assert pool.free == ost.free


def test_layout_matches_oracle_and_c_abi():
    from echokv_b200 import _native as N
    from echokv_b200.tiered_cache import TieredLayout

    for h, d, bs, mem, kg, vg in [(8, 128, 32, 4, 32, 32), (2, 64, 64, 8, 32, 32), (1, 128, 256, 2, 32, 32),
                                  (4, 96, 32, 6, 32, 32), (8, 128, 16, 8, 16, 32), (2, 128, 16, 4, 16, 32)]:
        L, Lo = TieredLayout(h, d, bs, mem, kg, vg), O.Layout(h, d, bs, mem, kg, vg)
        info = N.describe(h, d, bs, mem, kg, vg)
        assert L.offsets == Lo.offsets and L.page_bytes == Lo.page_bytes == info.page_bytes
        assert (info.o_v_scale, info.o_v_min, info.o_k_scale, info.o_k_min, info.o_data) == tuple(
            Lo.offsets[k] for k in ("v_scale", "v_min", "k_scale", "k_min", "data"))
        assert TieredLayout.per_token_bytes(h, d, mem, kg, vg) == O.Layout.per_token_bytes(h, d, mem, kg, vg) \
            == info.per_token_bytes
        assert bs * info.per_token_bytes >= info.page_bytes
        assert L.chunk_bytes == info.chunk_bytes and L.chunks_per_page == info.chunks_per_page
    for bad in (dict(block_size=8, mem_bits=4), dict(block_size=32, mem_bits=5), dict(block_size=48, mem_bits=4)):
        with pytest.raises(ValueError):
            TieredLayout(num_kv_heads=2, head_size=64, **bad)
        with pytest.raises(ValueError):
            N.describe(2, 64, bad["block_size"], bad["mem_bits"], 32, 32)


def test_library_exports_every_declared_symbol():
    from echokv_b200 import _native as N

    header = (ROOT / "include" / "echokv_b200.h").read_text()
    declared = set(re.findall(r"\b(echokv_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    lib = ctypes.CDLL(str(N.LIB_PATH))
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in include/echokv_b200.h but not exported"
    assert declared == set(N.EXPORTS)
    assert lib.echokv_abi_version() == 1


def test_product_has_no_cpu_path():
    import torch

    from echokv_b200._util import to_device
    from echokv_b200.tiered_cache import TieredKVCache, TieredLayout

    L = TieredLayout(num_kv_heads=2, head_size=64, block_size=64, mem_bits=4)
    with pytest.raises(RuntimeError):
        TieredKVCache(L, torch.zeros(4, 64 * TieredLayout.per_token_bytes(2, 64, 4), dtype=torch.uint8))
    with pytest.raises(RuntimeError):
        to_device(torch.zeros(1), "cpu")


def test_product_controller_follows_the_reference_trace(golden):
    """echokv_b200.controller.LayerController on the reference's recorded trace (controller.py:45-68 of the
    reference: EMA per tier, lowest tier under tau, optional sqrt scaling of tau with the context length)."""
    from echokv_b200.controller import ControllerParams, LayerController

    z = golden("canary_controller")
    for mode in ("none", "sqrt"):
        c = LayerController(ControllerParams(tau0=0.01, l0=4096, tau_scaling=mode, alpha=0.3, init_bits=8))
        trace = []
        for d, ctx in zip(z["ctl_obs"], z["ctl_ctx"]):
            c.observe(dict(zip((2, 4, 8), d.tolist())), float(ctx))
            trace.append(c.bits)
        assert trace == z[f"ctl_bits_{mode}"].tolist()
        assert c.fires == len(trace)
    pinned = LayerController(ControllerParams(fixed_bits=4))
    pinned.observe({2: 0.0, 4: 0.0, 8: 0.0}, 4096.0)
    assert pinned.bits == 4 and pinned.transitions == 0


def test_blocks_per_split_fill_whole_waves_of_the_kernels_team_slots():
    """The per-step split size: never below 64 tokens, an even number of 16-token tiles, never more splits than the
    grid holds, and items that fill the split kernel's slots in whole waves at the benchmark's shapes."""
    from echokv_b200.kernels.decode import BLOCKS_PER_SPLIT, choose_blocks_per_split

    lens = np.full(64, 4097)
    for slots, want_waves in ((296, 2), (592, 1), (888, 1), (1480, 1)):
        b = choose_blocks_per_split(lens, 16, 64, slots)
        used = -(-257 // b)
        assert b >= 4 and b % 2 == 0 and used <= 64
        assert -(-(64 * used) // slots) == want_waves, (slots, b)
    # a long context at block size 64 (four tiles per block): any block count is an even number of tiles
    b = choose_blocks_per_split(np.full(128, 32768), 64, 64, 296)
    assert 1 <= b <= 512 and -(-512 // b) <= 64
    # the grid's capacity wins over the minimum, padding rows (length 0) are ignored, no live row: the default
    assert choose_blocks_per_split(np.array([0, 0, 100000]), 16, 8, 296) >= -(-6250 // 8)
    assert choose_blocks_per_split(np.zeros(4, dtype=np.int64), 16, 64, 296) == BLOCKS_PER_SPLIT
    assert choose_blocks_per_split(lens, 16, 64, 0) == BLOCKS_PER_SPLIT


def test_native_planner_makes_the_same_plans_as_the_python_planner():
    """`csrc/planner.cu` against `WritePlanner` on seeded traffic: prefill chunks and decode steps of several
    sequences, padding rows, shuffled rows, blocks rewritten from their start, and so few residual slots that groups
    are evicted and sealed -- every array of every plan, the eviction list, the K_ref cursor and the free-slot count."""
    import dataclasses

    from echokv_b200.write_plan import NativeWritePlanner, WritePlanner

    rng = np.random.default_rng(42)
    evictions = finalized = errors = 0
    for trial in range(60):
        bs = int(rng.choice([16, 32, 64]))
        g = int(rng.choice([x for x in (16, 32) if bs % x == 0]))
        n_slots, window = int(rng.choice([2, 3, 5, 16])), int(rng.choice([0, 8, 64]))
        py, cc = WritePlanner(bs, g, n_slots, window), NativeWritePlanner(bs, g, n_slots, window)
        n_seq = int(rng.integers(1, 5))
        blocks = [list(rng.permutation(12)[:3]) for _ in range(n_seq)]
        lens = [0] * n_seq
        for step in range(40):
            rows = []
            for sq in range(n_seq):
                for _ in range(int(rng.choice([0, 1, 1, 1, 2, 7, g, bs + 3]))):
                    if lens[sq] >= 3 * bs:
                        lens[sq] = 0  # the sequence starts over: its blocks are reopened
                    rows.append(blocks[sq][lens[sq] // bs] * bs + lens[sq] % bs)
                    lens[sq] += 1
                if rng.random() < 0.2:
                    rows.append(-1)
            sm = np.array(rows, dtype=np.int64)
            if rng.random() < 0.3:
                rng.shuffle(sm)
            msgs = []
            plans = []
            for pl in (py, cc):
                try:
                    plans.append(pl.plan(sm))
                    msgs.append(None)
                except RuntimeError as e:
                    msgs.append(str(e))
            assert msgs[0] == msgs[1]
            if msgs[0] is not None:
                errors += 1
                break
            a, b = plans
            for f in dataclasses.fields(a):
                x, y = getattr(a, f.name), getattr(b, f.name)
                if isinstance(x, np.ndarray):
                    assert x.shape == y.shape and np.array_equal(x, y), (trial, step, f.name)
                else:
                    assert x == y, (trial, step, f.name)
            assert (py.kref_pos, py.kref_fill, len(py.free), py.step) == (cc.kref_pos, cc.kref_fill, len(cc.free), cc.step)
            for blk in range(12):
                assert py.sealed.get(blk, 7) == cc.sealed.get(blk, 7)
            evictions += len(a.evictions)
            finalized += a.n_fin
    assert evictions > 20 and finalized > 200  # the traffic does reach those paths
    empty = NativeWritePlanner(16, 16, 4, 8).plan(np.zeros(0, dtype=np.int64))
    assert empty.n_rows == 0 and empty.fin.shape == (0, 19) and empty.step == 1
