"""GPU parity at the sizes the benchmark runs, against the numpy oracle on the same seeded inputs.

The small scenarios elsewhere stop at 1,000 tokens; these cover the geometry of the benchmark's
configurations at their real lengths: configuration 2 (8 KV / 32 query heads, block 16, k_group 16,
~4,100-token sequences, all three tiers, the runner's 17 splits and a 32-split grid), configuration 5
per tensor-parallel rank (1 KV head, 8 query heads per KV head, one 32,768-token sequence of INT4 /
INT2 blocks over 32 splits of 64 blocks) and configuration 3 (a 512-token chunk over an 8,192-token
INT4 / INT8 prefix through the dense-dequantization + tcgen05 attention path).
Tolerances as in tests/echokv_vllm/test_decode_kernel.py:100,136 and test_prefill_kernel.py:100-103 of
the reference: float32 out 5e-3 / 2e-3 (max-abs / relative L2), bf16 prefill out 3e-2.
"""

import numpy as np
import pytest

import scenarios as S
from runners import run_oracle

pytestmark = pytest.mark.gpu


def rel_l2(a, b):
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-12))


def _decode(sc, splits_and_bps):
    import torch
    from cuda_runner import run_cuda
    from echokv_b200.kernels.decode import decode_attention

    res = run_cuda(sc)
    want = run_oracle(sc)
    assert np.array_equal(res["backing"], want["backing"]), "page bytes differ from the oracle"
    store = res["_store"]
    q = torch.from_numpy(sc.query).to("cuda", dtype=torch.bfloat16)
    table = torch.from_numpy(sc.block_table).cuda()
    lens = torch.tensor(sc.seq_lens, device="cuda")
    outs = []
    for num_splits, bps in splits_and_bps:
        got = decode_attention(store, q, table, lens, sc.scale, bps, num_splits=num_splits)
        g = got.cpu().numpy()
        assert np.isfinite(g).all()
        assert np.abs(g - want["attn_out"]).max() <= 5e-3 and rel_l2(g, want["attn_out"]) <= 2e-3, (num_splits, bps)
        outs.append(got)
    return store, q, table, lens, outs


def test_decode_configuration2_geometry_at_length():
    import torch
    from echokv_b200.kernels.decode import decode_attention

    sc = S.build_attention("cfg2_len", 8, 128, 16, 8, [4100, 4173, 4097], [4, 8, 2], seed=201, kg=16, dtype="bf16", gqa=4)
    store, q, table, lens, outs = _decode(sc, [(17, 16), (32, 16)])
    # batch invariance at length: a sequence alone gives the same bits as inside the batch
    alone = decode_attention(store, q[1:2], table[1:2].contiguous(), lens[1:2], sc.scale, 16, num_splits=17)
    assert torch.equal(alone[0], outs[0][1])


def test_decode_configuration2_uniform_int4_layer():
    """Every block INT4, as in the layers the benchmark's roofline figure is taken from."""
    sc = S.build_attention("cfg2_int4", 8, 128, 16, 8, [4097, 4112], [4], seed=203, kg=16, dtype="bf16", gqa=4)
    _decode(sc, [(17, 16)])


def test_decode_configuration5_rank_geometry_at_length():
    """One KV head with 8 query heads (tensor parallelism 8 of a 64 / 8-head model), 32,768 tokens:
    32 splits of 64 blocks, more blocks per split than `blocks_per_split` (kernels/decode.py:166-172)."""
    sc = S.build_attention("cfg5_len", 1, 128, 16, 4, [32768, 32700], [4, 2], seed=202, kg=16, dtype="bf16", gqa=8)
    _decode(sc, [(32, 16)])


def test_decode_serving_geometry_block64_kgroup32():
    """Block 64 / k_group 32 (the reference's serving default, evaluation/serving/echokv_throughput.py:85)."""
    sc = S.build_attention("serve_len", 8, 128, 64, 4, [4100, 2050], [4, 2], seed=204, kg=32, dtype="bf16", gqa=4)
    _decode(sc, [(5, 16), (32, 2)])


def test_prefill_configuration3_at_size():
    """One 512-token chunk at the end of 8,704 stored tokens (INT4 / INT8 blocks): dense dequantization +
    the tcgen05 attention kernel against the oracle's prefill attention."""
    import torch
    from cuda_runner import run_cuda

    sc = S.build_attention("cfg3_len", 8, 128, 16, 8, [8704], [4, 8], seed=205, kg=16, dtype="bf16", gqa=4, chunks=[512])
    got = run_cuda(sc)
    want = run_oracle(sc)
    assert np.array_equal(got["backing"], want["backing"])
    g, w = got["attn_out"], want["attn_out"]
    assert np.isfinite(g).all()
    assert np.abs(g - w).max() <= 3e-2 and rel_l2(g, w) <= 1e-2
