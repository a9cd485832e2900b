"""GPU parity of split-K paged decode attention (through the C ABI) against the numpy oracle and
the reference fixtures.  Tolerances (tests/echokv_vllm/test_decode_kernel.py:100,136): float32
output max-abs 5e-3 and relative-L2 2e-3; bf16 output max-abs 2e-2 and relative-L2 1e-2.
Batch invariance is bit-exact (test_decode_kernel.py:106-114)."""

import numpy as np
import pytest

import scenarios as S
from conftest import load_golden
from runners import run_oracle

pytestmark = pytest.mark.gpu

DEC = S.decode_scenarios()


def rel_l2(a, b):
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-12))


@pytest.mark.parametrize("sc", DEC, ids=lambda s: s.name)
def test_decode_matches_oracle_and_fixture(sc):
    from cuda_runner import run_cuda

    got = run_cuda(sc)["attn_out"]
    want = run_oracle(sc)["attn_out"]
    assert np.abs(got - want).max() <= 5e-3 and rel_l2(got, want) <= 2e-3
    ref = load_golden(sc.name)
    assert np.abs(got[ref["attn_rows"]] - ref["attn_out"]).max() <= 5e-3


def _store_and_inputs(sc):
    import torch
    from cuda_runner import run_cuda

    res = run_cuda(sc)
    store = res["_store"]
    q = torch.from_numpy(sc.query).to("cuda", dtype={"f32": torch.float32, "f16": torch.float16,
                                                       "bf16": torch.bfloat16}[sc.spec.dtype])
    table = torch.from_numpy(sc.block_table).cuda()
    lens = torch.tensor(sc.seq_lens, device="cuda")
    return store, q, table, lens, res


@pytest.mark.parametrize("bps", [1, 2, 3])
def test_split_sizes_and_batch_invariance(bps):
    import torch
    from echokv_b200.kernels.decode import decode_attention

    sc = DEC[1]  # case 0, gqa 4: lens 1, 40, 64, 65, 200
    store, q, table, lens, res = _store_and_inputs(sc)
    full = decode_attention(store, q, table, lens, sc.scale, bps)
    want = run_oracle(sc)["attn_out"]
    assert np.abs(full.cpu().numpy() - want).max() <= 5e-3
    bs = sc.spec.bs
    for i, n in enumerate(sc.seq_lens):  # each sequence alone, with a narrower block table
        nb = -(-n // bs)
        alone = decode_attention(store, q[i:i + 1], table[i:i + 1, :nb].contiguous(), lens[i:i + 1], sc.scale, bps)
        assert torch.equal(alone[0], full[i])


def test_indexed_rows_padding_and_fixed_grid():
    """test_decode_kernel.py:117-142, :166-190: rows by index, bf16 output written in place,
    untouched rows stay, length-0 padding entries are skipped, a fixed split grid."""
    import torch
    from echokv_b200.kernels.decode import decode_attention

    sc = DEC[1]
    store, q, table, lens, _ = _store_and_inputs(sc)
    hq, d = q.shape[1], q.shape[2]
    q_all = torch.randn(7, hq, d, device="cuda", generator=torch.Generator("cuda").manual_seed(3))
    q_rows = torch.tensor([6, 1, 3, 0], device="cuda")
    bt_rows = torch.tensor([4, 0, 2, 0], device="cuda")
    sel = torch.tensor([sc.seq_lens[4], sc.seq_lens[0], sc.seq_lens[2], 0], device="cuda")
    out = torch.full((7, hq, d), 7.0, device="cuda", dtype=torch.bfloat16)
    decode_attention(store, q_all, table, sel, sc.scale, 2, q_rows=q_rows, bt_rows=bt_rows, out=out, num_splits=3)
    # oracle on the selected rows
    from oracle import echokv_oracle as O
    from runners import make_oracle_store

    ost = make_oracle_store(sc.spec)
    for k, v, slots, bits in sc.steps:
        ost.write(k, v, slots, bits)
    want = O.decode_attention(ost, q_all[q_rows[:3]].cpu().numpy(), sc.block_table[[4, 0, 2]],
                              [sc.seq_lens[4], sc.seq_lens[0], sc.seq_lens[2]], sc.scale)
    got = out[q_rows[:3]].float().cpu().numpy()
    assert np.abs(got - want).max() <= 2e-2 and rel_l2(got, want) <= 1e-2
    untouched = [0, 2, 4, 5]
    assert (out[untouched] == 7.0).all()
    wide = torch.zeros_like(out)  # a wider grid must not change any bit
    decode_attention(store, q_all, table, sel, sc.scale, 2, q_rows=q_rows, bt_rows=bt_rows, out=wide, num_splits=9)
    assert torch.equal(wide[q_rows[:3]], out[q_rows[:3]])


def test_never_opened_blocks_are_safe():
    """test_decode_kernel.py:145-163: reads of blocks nothing wrote (tier 0) stay finite and in
    bounds; a mid-block write into such a block opens it."""
    import torch
    from echokv_b200.kernels.decode import decode_attention

    sc = S.build_attention("fresh", 2, 64, 64, 8, [70], [8], seed=5, gqa=2)
    store, q, table, lens, _ = _store_and_inputs(sc)
    used = set(sc.block_table[0, :2].tolist())
    unused = [x for x in range(store.num_blocks) if x not in used][:2]
    fresh = torch.tensor([unused], dtype=torch.int32, device="cuda")
    out = decode_attention(store, q, fresh, torch.tensor([100], device="cuda"), sc.scale, 4)
    assert torch.isfinite(out).all()
    b = unused[0]
    k = torch.randn(3, 2, 64, device="cuda")
    store.write(k, k, b * 64 + 5 + torch.arange(3), 4)
    assert int(store.tag[b]) == 4


@pytest.mark.parametrize("sc", S.prefill_scenarios(), ids=lambda s: s.name)
def test_prefill_matches_oracle_and_fixture(sc):
    """tests/echokv_vllm/test_prefill_kernel.py:40,100-103: 5e-3 for float32, 3e-2 for bf16."""
    from cuda_runner import run_cuda

    got = run_cuda(sc)["attn_out"]
    want = run_oracle(sc)["attn_out"]
    tol = 5e-3 if sc.spec.dtype == "f32" else 3e-2
    assert np.abs(got - want).max() <= tol
    ref = load_golden(sc.name)
    assert np.abs(got[ref["attn_rows"]] - ref["attn_out"]).max() <= tol


MMA_SHAPES = [s for s in DEC if s.spec.d == 128 and s.spec.vg == 32 and s.spec.h in (1, 2, 4, 8)]


@pytest.mark.parametrize("sc", MMA_SHAPES, ids=lambda s: s.name)
def test_tensor_core_and_generic_kernels_agree(sc):
    """Both decode kernels on the same store: each within tolerance of the oracle, and within
    2e-3 of each other (they differ only in fp16 operand rounding)."""
    import torch
    from echokv_b200 import _native as N
    from echokv_b200.kernels.decode import decode_attention

    store, q, table, lens, _ = _store_and_inputs(sc)
    want = run_oracle(sc)["attn_out"]
    old = N.lib.echokv_set_decode_path(1)
    try:
        gen = decode_attention(store, q, table, lens, sc.scale).cpu().numpy()
    finally:
        N.lib.echokv_set_decode_path(old)
    mma = decode_attention(store, q, table, lens, sc.scale).cpu().numpy()
    assert np.isfinite(mma).all()
    assert np.abs(gen - want).max() <= 5e-3 and np.abs(mma - want).max() <= 5e-3
    assert np.abs(mma - gen).max() <= 5e-3 and rel_l2(mma, want) <= 2e-3


def test_mixed_tiers_inside_one_split_remap_accumulators():
    """Blocks of all three tiers alternate inside every split of a long sequence (the tensor-core
    kernel re-maps its accumulators at every tier change) with 1, 3 and 7 splits."""
    import torch
    from echokv_b200.kernels.decode import decode_attention

    sc = S.build_attention("alternating", 8, 128, 16, 8, [1000, 517, 31], [8, 4, 2, 4, 2, 8, 2], seed=77, kg=16,
                           dtype="bf16", gqa=4)
    store, q, table, lens, _ = _store_and_inputs(sc)
    want = run_oracle(sc)["attn_out"]
    for num_splits, bps in ((1, 1), (3, 4), (7, 2), (32, 1)):
        got = decode_attention(store, q, table, lens, sc.scale, bps, num_splits=num_splits).cpu().numpy()
        assert np.abs(got - want).max() <= 5e-3 and rel_l2(got, want) <= 2e-3, (num_splits, bps)


def test_decode_events_hook_times_the_split_kernel():
    """echokv_set_decode_events: two caller-provided CUDA events are recorded around the split kernel."""
    import torch
    from cuda_runner import run_cuda
    from echokv_b200 import _native as N
    from echokv_b200.kernels.decode import decode_attention

    sc = next(s for s in S.decode_scenarios() if s.name == "decode_bs16_bf16")
    res = run_cuda(sc)
    store = res["_store"]
    q = torch.from_numpy(sc.query).to("cuda", dtype=torch.bfloat16)
    table = torch.from_numpy(sc.block_table).cuda()
    lens = torch.tensor(sc.seq_lens, device="cuda")
    want = decode_attention(store, q, table, lens, sc.scale)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(); e1.record()
    torch.cuda.synchronize()
    N.lib.echokv_set_decode_events(e0.cuda_event, e1.cuda_event)
    try:
        got = decode_attention(store, q, table, lens, sc.scale)
        torch.cuda.synchronize()
        assert 0.0 < e0.elapsed_time(e1) < 50.0
    finally:
        N.lib.echokv_set_decode_events(None, None)
    assert torch.equal(got, want)


def test_captured_graph_keeps_its_scratch_when_a_larger_eager_call_follows():
    """A CUDA graph holds the address of the split-partials buffer it was captured with.  A later eager call
    that needs more scratch (more sequences or splits than the captured grid) must not take that buffer
    away from under the graph: the replay still gives the eager result bit for bit."""
    import torch
    from echokv_b200.kernels import decode as KD
    from echokv_b200.kernels.decode import decode_attention

    sc = DEC[1]
    store, q, table, lens, _ = _store_and_inputs(sc)
    dev = q.device
    want = decode_attention(store, q, table, lens, sc.scale, 1, num_splits=4)
    out = torch.zeros_like(want)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        decode_attention(store, q, table, lens, sc.scale, 1, num_splits=4, out=out)  # warm on the side stream
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        decode_attention(store, q, table, lens, sc.scale, 1, num_splits=4, out=out)
    held = KD._scratch.buf[dev]
    # an eager call whose partials cannot fit the held buffer: many sequences x the widest split grid
    reps = max(1, held.numel() // (q.shape[1] * 32 * (q.shape[2] + 2) * 4 * len(sc.seq_lens))) + 1
    big_q, big_t, big_l = q.repeat(reps, 1, 1), table.repeat(reps, 1), lens.repeat(reps)
    big = decode_attention(store, big_q, big_t, big_l, sc.scale, 1, num_splits=32)
    assert KD._scratch.buf[dev] is not held and any(t is held for t in KD._scratch.retired)  # kept alive for the graph
    junk = torch.full((held.numel() // 4,), 3.0e38, device=dev)  # whatever the allocator hands out next is not the held buffer
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, want)
    assert torch.isfinite(big).all() and junk.numel() > 0


def test_a_wait_that_runs_out_raises_the_status_word_and_the_next_launch_is_fine():
    """The give-up path of the bounded waits: with the producer warps idle (a test hook) nothing is ever staged, every
    consumer's first wait runs out after the (shortened) limit, the kernel returns by itself with no copy in flight and
    the status word reports it once; the following ordinary launch gives the ordinary result."""
    import torch
    from echokv_b200 import _native as N
    from echokv_b200.kernels.decode import decode_attention

    sc = next(s for s in DEC if s.name == "decode_bs16_bf16")
    store, q, table, lens, _ = _store_and_inputs(sc)
    want = decode_attention(store, q, table, lens, sc.scale)
    torch.cuda.synchronize()
    assert N.lib.echokv_kernel_status(1) == 0
    N.lib.echokv_set_decode_wait_limit(20_000_000, 1)  # 20 ms, idle producer
    try:
        decode_attention(store, q, table, lens, sc.scale)
        torch.cuda.synchronize()
    finally:
        N.lib.echokv_set_decode_wait_limit(0, 0)
    assert N.lib.echokv_kernel_status(1) & 1  # raised ...
    assert N.lib.echokv_kernel_status(1) == 0  # ... and cleared by the read
    got = decode_attention(store, q, table, lens, sc.scale)
    torch.cuda.synchronize()
    assert torch.equal(got, want) and N.lib.echokv_kernel_status(1) == 0
