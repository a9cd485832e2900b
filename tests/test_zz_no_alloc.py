"""The allocation-free decode entry point (``echokv_decode_static``) against ``echokv_decode``.

Some hosts of this library may not allocate device memory at the point where they run attention --
a plugin living inside another framework's frozen memory pool, or a C program with no CUDA
allocator -- so ``echokv_decode_static`` keeps the split partials in an 8 MiB array that is part
of the library.  This test calls it through the C ABI twice in a row (the array is shared by all
calls and keeps the previous call's contents) and compares with the ordinary entry point: both run
the same kernels on the same inputs, so the outputs must be identical bit for bit (which is inside
the decode tolerance used everywhere else, max-abs 5e-3); the second call must leave the amount of
device memory in use unchanged; oversized or malformed requests must be refused.
It is collected last so that a failure here cannot hide any other test.
"""

import numpy as np
import pytest

import scenarios as S

pytestmark = pytest.mark.gpu


def _call(fn_static, store, q, table, lens, scale, num_splits, bps, out, scratch=None):
    from echokv_b200 import _native as N

    args_head = (store.c_layout, store.c_pages, store.c_res, q.data_ptr(), q.stride(0), q.stride(1),
                 N.dtype_code(q.dtype), None, table.data_ptr(), table.stride(0), None, lens.data_ptr())
    args_tail = (out.data_ptr(), out.stride(0), out.stride(1), N.dtype_code(out.dtype), float(scale), num_splits, bps,
                 lens.numel(), q.shape[1], N.stream_ptr(q.device))
    if fn_static:
        return N.lib.echokv_decode_static(*args_head, *args_tail)
    return N.lib.echokv_decode(*args_head, scratch.data_ptr(), scratch.numel(), *args_tail)


def test_static_scratch_decode_matches_regular_entry_point():
    import torch
    from cuda_runner import run_cuda
    from echokv_b200 import _native as N

    for sc in (S.build_attention("na_h8", 8, 128, 16, 8, [300, 45, 1000], [4, 8, 2, 4], seed=91, kg=16, dtype="bf16", gqa=4),
               S.build_attention("na_h2", 2, 64, 64, 8, [130, 7], [8, 4, 2], seed=92, gqa=2)):
        store = run_cuda(sc)["_store"]
        dt = {"f32": torch.float32, "bf16": torch.bfloat16}[sc.spec.dtype]
        table = torch.from_numpy(sc.block_table).cuda()
        lens = torch.tensor(sc.seq_lens, device="cuda", dtype=torch.long)
        num_splits, bps = 4, 2
        hq, d = sc.query.shape[1], sc.query.shape[2]
        nbytes = N.lib.echokv_decode_scratch_bytes(len(sc.seq_lens), hq, d, num_splits)
        assert 0 < nbytes <= N.lib.echokv_decode_static_scratch_bytes()
        scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        gen = torch.Generator("cuda").manual_seed(5)
        for rep in range(2):  # two calls in a row share the built-in array
            q = torch.randn(len(sc.seq_lens), hq, d, device="cuda", generator=gen).to(dt)
            want = torch.zeros(q.shape, device="cuda", dtype=torch.float32)
            got = torch.zeros_like(want)
            N.check(_call(False, store, q, table, lens, sc.scale, num_splits, bps, want, scratch))
            torch.cuda.synchronize()
            free0, used0 = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
            N.check(_call(True, store, q, table, lens, sc.scale, num_splits, bps, got))
            torch.cuda.synchronize()
            if rep:  # the first call on a device may load the module and looks up the array's address
                assert torch.cuda.mem_get_info()[0] == free0 and torch.cuda.memory_allocated() == used0
            assert torch.isfinite(got).all()
            assert float((got - want).abs().max()) <= 5e-3, (sc.name, rep)
            assert torch.equal(got, want), (sc.name, rep)


def test_static_scratch_decode_refuses_oversized_requests():
    import torch
    from cuda_runner import run_cuda
    from echokv_b200 import _native as N

    sc = S.build_attention("na_big", 2, 64, 64, 8, [130, 7], [8], seed=93, gqa=2)
    store = run_cuda(sc)["_store"]
    s = 4096  # 4096 sequences x 4 query heads x 32 splits x (64 + 2) floats > 8 MiB
    assert N.lib.echokv_decode_scratch_bytes(s, 4, 64, 32) > N.lib.echokv_decode_static_scratch_bytes()
    q = torch.zeros(s, 4, 64, device="cuda")
    out = torch.zeros_like(q)
    table = torch.zeros(s, 4, dtype=torch.int32, device="cuda")
    lens = torch.zeros(s, dtype=torch.long, device="cuda")
    rc = _call(True, store, q, table, lens, 1.0, 32, 1, out)
    assert rc == -2 and b"built-in scratch" in N.lib.echokv_last_error()
    rc = N.lib.echokv_decode_static(store.c_layout, store.c_pages, store.c_res, q.data_ptr(), q.stride(0), q.stride(1), 0, None,
                                    table.data_ptr(), table.stride(0), None, lens.data_ptr(), out.data_ptr(), out.stride(0),
                                    out.stride(1), 0, 1.0, 4, 1, 2, 0, N.stream_ptr(q.device))
    assert rc == -3  # no query heads: an argument error, not a size refusal
