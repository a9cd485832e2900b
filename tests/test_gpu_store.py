"""GPU parity of the quantize-on-write path: page bytes, slot maps, residual rows and the K_ref
ring written by the CUDA kernels (through the C ABI) against the numpy oracle AND the fixtures the
reference produced -- bit for bit."""

import numpy as np
import pytest

import scenarios as S
from conftest import load_golden
from runners import run_oracle, sha

pytestmark = pytest.mark.gpu

ALL = S.store_scenarios() + S.decode_scenarios() + S.prefill_scenarios()[::3]


def compare_store(sc, got, want, ref=None):
    assert np.array_equal(got["backing"], want["backing"]), "page bytes differ from the oracle"
    for key in ("block_res", "res_group", "tag_h", "pool_free", "residual_free", "downgraded", "demoted",
                "sealed_groups", "kref", "kref_pos", "kref_fill"):
        if key in want:
            assert np.array_equal(got[key], want[key]), key
    live = want["block_res"][want["block_res"] >= 0]
    assert np.array_equal(got["res_k"][live], want["res_k"][live]), "live residual rows differ"
    for i in range(len(sc.gathers)):
        for side in "kv":
            assert np.array_equal(got[f"gather{i}_{side}"], want[f"gather{i}_{side}"]), f"gather {side}"
    if ref is not None:
        assert sha(got["backing"]) == str(ref["backing_sha256"]), "page bytes differ from the reference fixture"
        assert np.array_equal(got["tokens_written"], ref["tokens_written"])


@pytest.mark.parametrize("sc", ALL, ids=lambda s: s.name)
def test_written_bytes_match(sc):
    from cuda_runner import run_cuda

    got = run_cuda(sc)
    compare_store(sc, got, run_oracle(sc), load_golden(sc.name))


@pytest.mark.parametrize("name", ["step_path_padded", "one_token_bf16", "eviction_seal", "interleaved"])
def test_full_grid_masked_launch_stores_same_bytes(name):
    """tests/echokv_vllm/test_step_path.py:35-71: padding rows and full-grid launches masked by the
    device-side count (CUDA-graph semantics) store exactly the same bytes."""
    from cuda_runner import run_cuda

    sc = next(s for s in S.store_scenarios() if s.name == name)
    got = run_cuda(sc, graph_semantics=True)
    compare_store(sc, got, run_oracle(sc), load_golden(sc.name))


def test_bulk_write_over_1024_rows_takes_the_warp_per_row_kernel():
    """Steps of more than 1,024 rows use the warp-per-row shape of the token kernel, smaller ones the
    CTA-per-row shape: both must store the bytes the oracle stores (mixed tiers, a partial last group)."""
    from cuda_runner import run_cuda

    rng = np.random.default_rng(77)
    h, d, bs, n = 2, 128, 32, 1100
    blocks = -(-n // bs)
    sp = S.StoreSpec(h=h, d=d, bs=bs, mem_bits=8, kg=32, vg=32, num_blocks=blocks + 2, residual_slots=4, dtype="bf16",
                     kref_window=32)
    k = S.round_to(rng.standard_normal((n, h, d), dtype=np.float32), "bf16")
    v = S.round_to(rng.standard_normal((n, h, d), dtype=np.float32) * 3, "bf16")
    perm = rng.permutation(blocks + 2)[:blocks]
    pos = np.arange(n)
    slots = perm[pos // bs].astype(np.int64) * bs + pos % bs
    pad = np.full(1500, -1, dtype=np.int64)  # a second step of padding rows only: nothing is stored
    sc = S.Scenario("bulk_1100", sp, [(k, v, slots, 4), (np.tile(k[:1], (1500, 1, 1)), np.tile(v[:1], (1500, 1, 1)), pad, 8)])
    sc.use_kref = True
    got = run_cuda(sc)
    compare_store(sc, got, run_oracle(sc))


def _takeover_scenario(dtype):
    """Two sequences, one residual slot in play: in the second step sequence A's group completes out of slot 0
    while sequence B's first key of a new group takes slot 0 over; in the third step B's group completes from
    that key in the slot plus fifteen new ones."""
    rng = np.random.default_rng(5)
    h, d, bs = 2, 128, 16
    sp = S.StoreSpec(h=h, d=d, bs=bs, mem_bits=8, kg=16, vg=32, num_blocks=4, residual_slots=2, dtype=dtype)

    def kv(n):
        return (S.round_to(rng.standard_normal((n, h, d), dtype=np.float32) * 2, dtype),
                S.round_to(rng.standard_normal((n, h, d), dtype=np.float32), dtype))

    a, b = 1 * bs, 3 * bs  # first slots of A's block 1 and B's block 3: A's group has the lower id, so it is planned first
    steps = [(*kv(15), a + np.arange(15), 4),
             (*kv(2), np.array([a + 15, b + 0]), 4),
             (*kv(15), b + 1 + np.arange(15), 8)]
    sc = S.Scenario(f"takeover_{dtype}", sp, steps)
    sc.gathers = [(np.array([1] * 16 + [3] * 16), np.array(list(range(16)) * 2))]
    return sc


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_slot_given_up_and_taken_over_in_one_step(dtype):
    """tiered_cache.py:415-432 runs the group pass before the token pass because a slot a completing group gives
    up may be reused in the same step; the one-launch kernel must store the same bytes with both running at once."""
    from cuda_runner import run_cuda
    from echokv_b200.write_plan import WritePlanner

    sc = _takeover_scenario(dtype)
    pl = WritePlanner(sc.spec.bs, sc.spec.kg, sc.spec.residual_slots)
    plans = [pl.plan(np.asarray(st[2], dtype=np.int64)) for st in sc.steps]
    second = plans[1]
    given_up = second.fin[:, 2]
    assert (given_up >= 0).any() and np.isin(second.tok_res[second.tok_res >= 0], given_up).any(), \
        "the scenario no longer reuses a slot inside one step"
    want = run_oracle(sc)
    for graph_semantics in (False, True):
        compare_store(sc, run_cuda(sc, graph_semantics=graph_semantics), want)


def test_write_step_equals_the_three_launches():
    """echokv_write_step against echokv_finalize_k + echokv_write_tokens + echokv_gather_rows on the same step:
    identical page bytes, residual rows, K_ref ring and stashed query rows."""
    import torch
    from cuda_runner import make_cuda_store
    from echokv_b200.kernels.write import finalize_k, gather_rows, write_step, write_tokens
    from echokv_b200.write_plan import stage_plan

    rng = np.random.default_rng(9)
    h, d, bs, hq = 4, 128, 16, 8
    sp = S.StoreSpec(h=h, d=d, bs=bs, mem_bits=8, kg=16, vg=32, num_blocks=12, residual_slots=6, dtype="bf16", kref_window=32)
    results = []
    for fused in (False, True):
        store, backing = make_cuda_store(sp)
        kref = torch.zeros(32, h, d, device="cuda")
        stash = torch.zeros(4, hq, d, device="cuda", dtype=torch.bfloat16)
        g = np.random.default_rng(10)
        lens = [0, 0, 0, 0, 0]
        for step in range(40):  # five sequences one token at a time, with padding rows: groups complete at different steps
            rows = [s for s in range(5) if (step + s) % 7]
            slots = np.full(8, -1, dtype=np.int64)
            for i, sq in enumerate(rows):
                slots[i] = (2 * sq + lens[sq] // bs) * bs + lens[sq] % bs
                lens[sq] += 1
            k = torch.from_numpy(S.round_to(g.standard_normal((8, h, d), dtype=np.float32), "bf16")).cuda().bfloat16()
            v = torch.from_numpy(S.round_to(g.standard_normal((8, h, d), dtype=np.float32) * 3, "bf16")).cuda().bfloat16()
            q = torch.from_numpy(g.standard_normal((8, hq, d), dtype=np.float32)).cuda().bfloat16()
            qrows = torch.tensor([0, 2, 1, 3], device="cuda")
            plan = store.planner.plan(slots)
            opened = store.prepare(plan, (4, 8, 2)[step % 3])
            store.shared.commit(plan)
            meta, extra = stage_plan(plan, "cuda", opened)
            store.shared.apply_res_map(*extra[:4])
            if opened is not None:
                store.write_headers(extra[4], extra[5])
            if fused:
                write_step(store, k, v, meta, kref, full_grid=True, stash=(q, qrows, stash))
            else:
                finalize_k(store, k, meta, full_grid=True)
                write_tokens(store, k, v, meta, kref)
                gather_rows(q, qrows, stash)
        torch.cuda.synchronize()
        live = store.block_res.cpu().numpy()
        live = live[live >= 0]
        results.append((backing.cpu().numpy(), store.res_k.float().cpu().numpy()[live], kref.cpu().numpy(),
                        stash.float().cpu().numpy(), live))
    for x, y in zip(*results):
        assert np.array_equal(x, y)
    assert results[0][4].size > 0 and results[0][3].any()


def test_layout_errors_and_cpu_tensors_rejected():
    import torch

    from echokv_b200.tiered_cache import TieredKVCache, TieredLayout

    L = TieredLayout(num_kv_heads=2, head_size=64, block_size=64, mem_bits=4)
    with pytest.raises(RuntimeError):
        TieredKVCache(L, torch.zeros(4, 64 * TieredLayout.per_token_bytes(2, 64, 4), dtype=torch.uint8))
    with pytest.raises(ValueError):
        TieredKVCache(L, torch.zeros(4, 100, dtype=torch.uint8, device="cuda"))
