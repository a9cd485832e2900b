"""GPU parity of the canary KL kernel (through the C ABI) against the oracle and the reference
fixtures: absolute error <= 1e-5 (relative 1e-4 for large values)."""

import numpy as np
import pytest

import scenarios as S
from conftest import load_golden
from oracle import echokv_oracle as O

pytestmark = pytest.mark.gpu


def test_canary_matches_oracle_and_fixture():
    import torch
    from echokv_b200.canary import canary_kl

    z = load_golden("canary_controller")
    for name, q, kref, kg, scale in S.canary_inputs():
        got = canary_kl(torch.from_numpy(q).cuda(), torch.from_numpy(kref).cuda(), (2, 4, 8), kg, scale).cpu().numpy()
        want = O.canary_kl(q, kref, (2, 4, 8), kg, scale)
        np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-5)
        np.testing.assert_allclose(got, z[name], rtol=1e-4, atol=1e-5)
        assert got.shape == z[name].shape
        assert (got[..., 0] >= got[..., 1]).all() and (got[..., 1] >= got[..., 2]).all() and (got >= 0).all()


def test_ring_cursor_equals_unrolled_view_and_bf16_inputs():
    import torch
    from echokv_b200.canary import canary_kl, canary_kl_ring, ring_view

    rng = np.random.default_rng(3)
    q = torch.from_numpy(rng.standard_normal((4, 5, 8, 128), dtype=np.float32)).cuda()
    ring = torch.from_numpy(rng.standard_normal((4, 48, 2, 128), dtype=np.float32) * 2).cuda()
    for pos, fill in ((0, 48), (17, 48), (20, 20), (40, 40)):
        got = canary_kl_ring(q, ring, pos, fill, 16, 0.1)
        view = ring_view(ring, pos, fill, dim=1)
        want = O.canary_kl(q.cpu().numpy(), view.cpu().numpy(), (2, 4, 8), 16, 0.1)
        np.testing.assert_allclose(got.cpu().numpy(), want, rtol=1e-4, atol=1e-5)
    sub = canary_kl(q[0].bfloat16(), ring[0], (4,), 16, 0.1)  # a subset of tiers, model-dtype queries
    assert sub.shape == (1,) and sub.dtype == torch.float32
    with pytest.raises(ValueError):
        canary_kl_ring(q, ring, 0, 10, 16, 0.1)


def test_gather_rows_equals_index_select():
    """The canary's query stash (backend.py:632-634 in the reference is an index_select)."""
    import torch
    from echokv_b200.kernels.write import gather_rows

    g = torch.Generator("cuda").manual_seed(5)
    q = torch.randn(70, 32, 128, device="cuda", generator=g).bfloat16()
    rows = torch.tensor([69, 0, 3, 3, 41, 7, 0, 0], device="cuda")
    out = torch.zeros(8, 32, 128, device="cuda", dtype=torch.bfloat16)
    gather_rows(q, rows, out)
    assert torch.equal(out, q[rows])
    part = q[:, :6, :]  # a view with a larger row stride than the row itself
    out2 = torch.zeros(5, 6, 128, device="cuda", dtype=torch.bfloat16)
    gather_rows(part, rows, out2)
    assert torch.equal(out2, part[rows[:5]])
    odd = torch.randn(9, 3, 5, device="cuda", generator=g)  # rows that are not a multiple of 16 bytes
    out3 = torch.zeros(2, 3, 5, device="cuda")
    gather_rows(odd, rows[1:3], out3)
    assert torch.equal(out3, odd[rows[1:3]])
