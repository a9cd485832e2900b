"""The numpy oracle against the fixtures produced by the reference implementation.

Bytes (pages, slot maps, residual rows, K_ref ring) must be identical;
attention outputs agree to 2e-5 (float32) -- the reference's own test
tolerance between two float32 formulations is 1e-5.
"""

import numpy as np
import pytest

import scenarios as S
from conftest import load_golden
from oracle import echokv_oracle as O
from runners import run_oracle, sha

STORE = S.store_scenarios()
ATTN = S.decode_scenarios() + S.prefill_scenarios()


def check(sc, got, ref):
    assert sha(got["backing"]) == str(ref["backing_sha256"]), "page bytes differ"
    if "backing" in ref:
        assert np.array_equal(got["backing"], ref["backing"])
    for key in ("block_res", "res_group", "tag_h", "pool_free", "residual_free", "downgraded", "demoted",
                "sealed_groups", "kref", "kref_pos", "kref_fill"):
        if key in ref:
            assert np.array_equal(got[key], ref[key]), key
    live = ref["block_res"][ref["block_res"] >= 0]
    assert np.array_equal(got["res_k"][live], ref["res_k"][live])
    for i in range(len(sc.gathers)):
        for side in "kv":
            key = f"gather{i}_{side}"
            assert sha(got[key]) == str(ref[key + "_sha256"]), key
    if "attn_out" in ref:
        tol = 2e-5 if sc.spec.dtype == "f32" or sc.prefill is None else 3e-2
        np.testing.assert_allclose(got["attn_out"][ref["attn_rows"]], ref["attn_out"], rtol=0, atol=tol)


@pytest.mark.parametrize("sc", STORE, ids=lambda s: s.name)
def test_store_scenarios(sc):
    check(sc, run_oracle(sc), load_golden(sc.name))


@pytest.mark.parametrize("sc", ATTN, ids=lambda s: s.name)
def test_attention_scenarios(sc):
    check(sc, run_oracle(sc), load_golden(sc.name))


def test_quantizer_known_answers():
    z = load_golden("quant")
    for bits in (2, 4, 8):
        for shift in (0, 40, -40):
            tag = f"b{bits}_s{shift}"
            c, s, m = O.quantize(z[f"x_{tag}"], bits, 32)
            assert np.array_equal(O.pack(c, bits), z[f"packed_{tag}"])
            assert np.array_equal(s, z[f"scale_{tag}"]) and np.array_equal(m, z[f"min_{tag}"])
            assert np.array_equal(O.unpack(z[f"packed_{tag}"], bits), c)
        assert np.array_equal(O.fake_quant_channels(z[f"kch_{bits}"], bits, 32), z[f"kch_fq_{bits}"])


def test_pack_layout_is_little_endian_within_a_byte():
    # echokv_vllm/quant.py:99-110: element i of a byte at bits [i*b, (i+1)*b)
    assert O.pack(np.array([1, 2], dtype=np.uint8), 4).tolist() == [0x21]
    assert O.pack(np.array([1, 2, 3, 0], dtype=np.uint8), 2).tolist() == [0b00111001]


def test_canary_and_controller():
    z = load_golden("canary_controller")
    for name, q, kref, kg, scale in S.canary_inputs():
        got = O.canary_kl(q, kref, (2, 4, 8), kg, scale)
        np.testing.assert_allclose(got, z[name], rtol=1e-4, atol=1e-6)
    for mode in ("none", "sqrt"):
        c = O.Controller(tau0=0.01, l0=4096, tau_scaling=mode, alpha=0.3, init_bits=8)
        trace = []
        for d, ctx in zip(z["ctl_obs"], z["ctl_ctx"]):
            c.observe(dict(zip((2, 4, 8), d.tolist())), float(ctx))
            trace.append(c.bits)
        assert trace == z[f"ctl_bits_{mode}"].tolist()


def test_layout_known_offsets():
    # the benchmark's CPU-runnable geometry: H2 D128 BS16 KG16 mem4
    L = O.Layout(2, 128, 16, 4, 16, 32)
    assert L.offsets == {"v_scale": 16, "v_min": 272, "k_scale": 528, "k_min": 1040, "data": 1552, "end": 5648}
    assert O.Layout.per_token_bytes(2, 128, 4, 16, 32) == 356
    assert O.Layout.per_token_bytes(8, 128, 4, 16, 32) == 1412
    assert O.Layout.per_token_bytes(8, 128, 8, 16, 32) == 2436
    assert O.Layout.per_token_bytes(8, 128, 4, 32, 32) == 1284
    for bad in (dict(block_size=8, mem_bits=4), dict(block_size=32, mem_bits=5), dict(block_size=48, mem_bits=4)):
        with pytest.raises(ValueError):
            O.Layout(2, 64, k_group=32, **bad)


def test_reciprocal_quantizer_rule_equals_division():
    """The write kernels quantize with d * (1 / scale) and fall back to the exact division when the
    product lies within 2^-12 of a half-integer (csrc/common.cuh, quant_code_r).  In float32 arithmetic
    that rule must give the code of the reference's divide-then-round (quant.py:39-45) for every input,
    also for quotients crowded around the rounding ties."""
    rng = np.random.default_rng(0)
    n = 1_000_000
    for levels in (3.0, 15.0, 255.0):
        s = (np.float32(2.0) ** rng.uniform(-14, 4, n).astype(np.float32) * rng.uniform(1, 2, n).astype(np.float32))
        s = np.maximum(s, np.float32(6.103515625e-05)).astype(np.float16).astype(np.float32)
        k = rng.integers(0, int(levels) + 1, n).astype(np.float32)
        off = np.where(rng.random(n) < 0.5, np.float32(0.5) + rng.uniform(-3e-4, 3e-4, n).astype(np.float32),
                       rng.uniform(-0.2, 1.2, n).astype(np.float32))
        d = ((k + off) * s).astype(np.float32)
        fast = (d * (np.float32(1) / s).astype(np.float32)).astype(np.float32)
        exact = (d / s).astype(np.float32)
        tie = (np.abs(fast - np.floor(fast) - np.float32(0.5)) < np.float32(2.0 ** -12)) | ~(np.abs(fast) < 512)
        got = np.clip(np.rint(np.where(tie, exact, fast)), 0, levels)
        assert np.array_equal(got, np.clip(np.rint(exact), 0, levels))
