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


def test_layout_errors_and_cpu_tensors_rejected():
    import torch

    from echokv_b200.tiered_cache import TieredKVCache, TieredLayout

    L = TieredLayout(num_kv_heads=2, head_size=64, block_size=64, mem_bits=4)
    with pytest.raises(RuntimeError):
        TieredKVCache(L, torch.zeros(4, 64 * TieredLayout.per_token_bytes(2, 64, 4), dtype=torch.uint8))
    with pytest.raises(ValueError):
        TieredKVCache(L, torch.zeros(4, 100, dtype=torch.uint8, device="cuda"))
