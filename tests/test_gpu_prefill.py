"""GPU parity of the dense chunked-prefill path: dense dequantization is bit-identical to the
token gather, and the attention kernel over it matches the oracle (tests/echokv_vllm/
test_prefill_kernel.py:74-103: 5e-3 for float16, 3e-2 for bfloat16) and the row path."""

import numpy as np
import pytest

import scenarios as S
from runners import run_oracle

pytestmark = pytest.mark.gpu

DT = {"f16": "float16", "bf16": "bfloat16"}


def _setup(sc):
    import torch
    from cuda_runner import run_cuda

    store = run_cuda(sc)["_store"]
    q = torch.from_numpy(sc.query).to("cuda", dtype=getattr(torch, DT[sc.spec.dtype]))
    return store, q, torch.from_numpy(sc.block_table).cuda()


CASES = [
    S.build_attention("dense_f16_gqa4", 2, 128, 32, 8, [300, 130, 64], [8, 4, 2], seed=90, dtype="f16", gqa=4,
                      chunks=[170, 130, 1]),
    S.build_attention("dense_bf16_gqa7", 1, 128, 16, 8, [411, 97], [4, 8], seed=91, kg=16, dtype="bf16", gqa=7,
                      chunks=[200, 97]),
    S.build_attention("dense_bf16_d64", 4, 64, 64, 4, [500, 77], [4, 2, 4], seed=92, dtype="bf16", gqa=2,
                      chunks=[333, 5]),
    S.build_attention("dense_f16_gqa1", 8, 128, 16, 8, [129, 1000], [2, 8, 4, 4], seed=93, kg=16, dtype="f16", gqa=1,
                      chunks=[129, 400]),
    S.build_attention("dense_bf16_h3", 3, 128, 16, 8, [150, 45], [4, 8], seed=94, kg=16, dtype="bf16", gqa=2,
                      chunks=[90, 45]),
]


@pytest.mark.parametrize("kernel", ["tcgen05", "mma_sync", "tcgen05_plain", "tcgen05_row_copies", "tcgen05_64key_tiles"])
@pytest.mark.parametrize("sc", CASES, ids=lambda s: s.name)
def test_dense_path_matches_oracle_and_row_path(sc, kernel):
    """Both attention kernels of the dense path (head size 128 takes the tcgen05 kernel unless told otherwise)."""
    import torch
    from echokv_b200 import _native as N
    from echokv_b200.kernels.prefill import build_dense, build_rows, prefill_attention

    old = N.lib.echokv_set_prefill_path({"tcgen05": 0, "mma_sync": 1, "tcgen05_plain": 2, "tcgen05_row_copies": 3, "tcgen05_64key_tiles": 4}[kernel])
    try:
        _dense_case(sc)
    finally:
        N.lib.echokv_set_prefill_path(old)


def _dense_case(sc):
    import torch
    from echokv_b200.kernels.prefill import build_dense, build_rows, prefill_attention

    store, q, table = _setup(sc)
    want = run_oracle(sc)["attn_out"]
    tol = 5e-3 if sc.spec.dtype == "f16" else 3e-2
    dense = build_dense(sc.prefill, sc.req_of, sc.spec.bs, "cuda")
    out = torch.full(q.shape, 7.0, dtype=torch.float32, device="cuda")  # float32 output of 16-bit inputs
    prefill_attention(store, q, out, sc.prefill, sc.req_of, table, sc.scale, dense=dense)
    live = np.concatenate([np.arange(qs, qe) for qs, qe, _, _ in sc.prefill])
    got = out.cpu().numpy()
    assert np.isfinite(got).all() and np.abs(got[live] - want[live]).max() <= tol
    rest = np.setdiff1d(np.arange(q.shape[0]), live)
    assert (got[rest] == 7.0).all()
    rows = torch.zeros_like(out)
    prefill_attention(store, q, rows, sc.prefill, sc.req_of, table, sc.scale,
                      rows=build_rows(sc.prefill, sc.req_of, "cuda"))
    assert np.abs(rows.cpu().numpy()[live] - got[live]).max() <= tol
    same = torch.zeros_like(q)  # model-dtype output, written in place
    prefill_attention(store, q, same, sc.prefill, sc.req_of, table, sc.scale, dense=dense)
    assert np.abs(same.float().cpu().numpy()[live] - got[live]).max() <= 2e-2


@pytest.mark.parametrize("sc", CASES, ids=lambda s: s.name)
def test_dense_dequant_equals_gather(sc):
    """kernels/prefill.py:90-115 against tiered_cache.py:451-478: the same values, token by token."""
    import torch
    from echokv_b200.kernels.prefill import build_dense, dequant_dense

    store, q, table = _setup(sc)
    bs = sc.spec.bs
    work, total, chunks, _ = build_dense(sc.prefill, sc.req_of, bs, "cuda")
    k, v = dequant_dense(store, work, total, table, torch.float32)
    assert total == sum(ctx for _, _, ctx, _ in sc.prefill)
    for (_, _, ctx, at), r in zip(chunks.tolist(), sc.req_of):
        pos = torch.arange(ctx, device="cuda")
        gk, gv = store.gather(table[r, pos // bs].long(), pos % bs)
        assert torch.equal(k[at:at + ctx], gk) and torch.equal(v[at:at + ctx], gv)
    half = dequant_dense(store, work, total, table, q.dtype)
    assert torch.equal(half[0], k.to(q.dtype)) and torch.equal(half[1], v.to(q.dtype))


def test_dense_rejects_what_it_cannot_run():
    import torch
    from echokv_b200.kernels.prefill import dense_attention

    q = torch.zeros(4, 4, 128, device="cuda")
    kv = torch.zeros(8, 2, 128, device="cuda")
    chunks = torch.tensor([[0, 4, 8, 0]], dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="float16 or bfloat16"):
        dense_attention(q, kv, kv, chunks, 4, torch.zeros_like(q), 0.1)
    with pytest.raises(ValueError):
        dense_attention(q.half(), kv.half(), kv.bfloat16(), chunks, 4, torch.zeros_like(q), 0.1)


@pytest.mark.parametrize("path", [0, 4, 3, 2, 1], ids=["tcgen05", "64key_tiles", "row_copies", "plain", "mma_sync"])
def test_dense_attention_long_context_matches_sdpa(path):
    """Contexts of dozens of key tiles (the K / V rings wrap many times) whose scores grow along the context, so the
    softmax reference moves and rows of O are rescaled; against torch's fp32 attention, tolerance 2e-2 (bf16)."""
    import torch
    import torch.nn.functional as F
    from echokv_b200 import _native as N
    from echokv_b200.kernels.prefill import dense_attention

    torch.manual_seed(5)
    Hq, H, D, dt = 8, 2, 128, torch.bfloat16
    shapes = [(300, 3000), (77, 2500), (130, 130)]  # (chunk length, context)
    T, total = sum(nq for nq, _ in shapes), sum(ctx for _, ctx in shapes)
    q = torch.randn(T, Hq, D, device="cuda", dtype=dt)
    k = torch.randn(total, H, D, device="cuda", dtype=dt)
    v = torch.randn(total, H, D, device="cuda", dtype=dt)
    rows, at_q, at_k = [], 0, 0
    for nq, ctx in shapes:
        ramp = torch.linspace(0.2, 3.0, ctx, device="cuda")[:, None, None]  # later keys score higher
        k[at_k:at_k + ctx] = (k[at_k:at_k + ctx].float() * ramp).to(dt)
        rows.append([at_q, at_q + nq, ctx, at_k])
        at_q, at_k = at_q + nq, at_k + ctx
    chunks = torch.tensor(rows, dtype=torch.int32, device="cuda")
    out = torch.zeros(T, Hq, D, device="cuda", dtype=torch.float32)
    old = N.lib.echokv_set_prefill_path(path)
    try:
        dense_attention(q, k, v, chunks, max(nq for nq, _ in shapes), out, D ** -0.5)
    finally:
        N.lib.echokv_set_prefill_path(old)
    for qs, qe, ctx, ks in rows:
        nq = qe - qs
        qf = q[qs:qe].transpose(0, 1).float()
        kf = k[ks:ks + ctx].transpose(0, 1).repeat_interleave(Hq // H, 0).float()
        vf = v[ks:ks + ctx].transpose(0, 1).repeat_interleave(Hq // H, 0).float()
        mask = torch.arange(ctx, device="cuda")[None, :] <= (ctx - nq + torch.arange(nq, device="cuda"))[:, None]
        want = F.scaled_dot_product_attention(qf, kf, vf, attn_mask=mask, scale=D ** -0.5).transpose(0, 1)
        assert (out[qs:qe] - want).abs().max().item() <= 2e-2
