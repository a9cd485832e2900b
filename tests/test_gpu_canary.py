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
