"""Generate the golden fixtures in this directory from the reference implementation.

Run in a container that has the reference checkout (it is imported unchanged,
CPU torch path, Triton disabled) -- not needed at test time:

    python tests/golden/make_golden.py /path/to/reference

For every scenario in ``scenarios.py`` the reference's TieredKVCache /
decode_attention_torch / prefill_attention_torch / canary_kl / LayerController
are run on the seeded inputs and their results are stored as ``*.npz``.  The
numpy oracle (``oracle/echokv_oracle.py``) is run on the same inputs and must
agree (bytes exactly, attention to 1e-5) or the script fails: this is what
pins the oracle.
"""

from __future__ import annotations

import hashlib
import os
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(HERE))
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("ECHOKV_REFERENCE", "")
if not REF:
    sys.exit("usage: make_golden.py <path of a checkout of the reference> (or set ECHOKV_REFERENCE)")
os.environ["ECHOKV_DISABLE_TRITON"] = "1"
sys.path.insert(0, REF)

import torch  # noqa: E402

from echokv_vllm.canary import canary_kl as ref_canary_kl, ring_view as ref_ring_view  # noqa: E402
from echokv_vllm.controller import ControllerParams, LayerController  # noqa: E402
from echokv_vllm.kernels.decode import decode_attention_torch  # noqa: E402
from echokv_vllm.kernels.prefill import prefill_attention_torch  # noqa: E402
from echokv_vllm import quant as ref_quant  # noqa: E402
from echokv_vllm.tiered_cache import TieredKVCache, TieredLayout  # noqa: E402

import scenarios as S  # noqa: E402
from oracle import echokv_oracle as O  # noqa: E402
from runners import run_oracle  # noqa: E402

TDT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
PAGES_INLINE_LIMIT = 160_000  # larger page sets are pinned by sha256 only
GATHER_INLINE_LIMIT = 40_000  # elements; larger gathers are pinned by sha256 only
ATTN_ROWS_MAX = 24  # attention outputs keep at most this many (evenly spaced) rows


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def run_reference(sc: S.Scenario) -> dict:
    sp = sc.spec
    layout = TieredLayout(num_kv_heads=sp.h, head_size=sp.d, block_size=sp.bs, mem_bits=sp.mem_bits,
                          k_group=sp.kg, v_group=sp.vg)
    backing = torch.full((sp.num_blocks * sp.page_stride + 64,), sp.fill, dtype=torch.uint8)
    pages = torch.as_strided(backing, (sp.num_blocks, sp.page_size), (sp.page_stride, 1))
    store = TieredKVCache(layout, pages, residual_slots=sp.residual_slots, residual_dtype=TDT[sp.dtype])
    kw = sp.kref_window or sp.kg
    kref = torch.zeros(kw, sp.h, sp.d) if sc.use_kref else None
    for k, v, slots, bits in sc.steps:
        store.write(torch.from_numpy(k).to(TDT[sp.dtype]), torch.from_numpy(v).to(TDT[sp.dtype]),
                    torch.from_numpy(np.asarray(slots, dtype=np.int64)), bits, kref=kref)
    res = {
        "backing": backing.numpy().copy(),
        "block_res": store.block_res.numpy().copy(),
        "res_group": store.res_group.numpy().copy(),
        "res_k": store.res_k.float().numpy().copy(),
        "tag_h": store._tag_h.copy(),
        "pool_free": np.int64(store.pool_free),
        "residual_free": np.int64(store.residual_free),
        "downgraded": np.int64(store.downgraded_blocks),
        "demoted": np.int64(store.demoted_blocks),
        "sealed_groups": np.int64(store.sealed_groups),
        "tokens_written": np.array([store.tokens_written[b] for b in (2, 4, 8)], dtype=np.int64),
    }
    if kref is not None:
        res["kref"] = kref.numpy().copy()
        res["kref_pos"] = np.int64(store.planner.kref_pos)
        res["kref_fill"] = np.int64(store.planner.kref_fill)
    for i, (blk, off) in enumerate(sc.gathers):
        kg, vg = store.gather(torch.from_numpy(np.asarray(blk, dtype=np.int64)),
                              torch.from_numpy(np.asarray(off, dtype=np.int64)))
        res[f"gather{i}_k"], res[f"gather{i}_v"] = kg.numpy(), vg.numpy()
    if sc.query is not None:
        q = torch.from_numpy(sc.query).to(TDT[sp.dtype])
        table = torch.from_numpy(sc.block_table)
        if sc.prefill is None:
            out = decode_attention_torch(store, q, table, torch.tensor(sc.seq_lens), sc.scale)
        else:
            out = torch.zeros_like(q)
            prefill_attention_torch(store, q, out, sc.prefill, table, sc.scale, req_of=sc.req_of)
        res["attn_out"] = out.float().numpy()
    return res


def compare(name: str, ref: dict, ora: dict, attn_tol: float) -> None:
    for key, val in ora.items():
        r = ref[key]
        if key == "attn_out":
            err = float(np.abs(r - val).max())
            assert err <= attn_tol, f"{name}: attention differs by {err}"
        elif key == "res_k":
            # only slots the map points at are defined contents
            live = ref["block_res"][ref["block_res"] >= 0]
            assert np.array_equal(r[live], val[live]), f"{name}: live residual rows differ"
        else:
            assert np.array_equal(r, val), f"{name}: {key} differs"


def main() -> None:
    out_dir = HERE
    n = 0
    for sc in S.all_scenarios():
        ref = run_reference(sc)
        ora = run_oracle(sc)
        tol = 2e-5 if sc.spec.dtype == "f32" or sc.prefill is None else 3e-2
        compare(sc.name, ref, ora, tol)
        save = dict(ref)
        save["backing_sha256"] = np.array(sha(ref["backing"]))
        if ref["backing"].size > PAGES_INLINE_LIMIT:
            del save["backing"]
        for key in [k for k in save if k.startswith("gather")]:
            save[key + "_sha256"] = np.array(sha(save[key]))
            if save[key].size > GATHER_INLINE_LIMIT:
                del save[key]
        if "attn_out" in save:
            rows = np.unique(np.linspace(0, save["attn_out"].shape[0] - 1, ATTN_ROWS_MAX).astype(np.int64))
            save["attn_rows"] = rows
            save["attn_out"] = save["attn_out"][rows]
        np.savez_compressed(out_dir / f"{sc.name}.npz", **save)
        n += 1
        print(f"ok {sc.name}: backing {ref['backing'].size} B")

    # quantizer known answers (quant.py)
    rng = np.random.default_rng(70)
    qz = {}
    for bits in (2, 4, 8):
        for shift in (0.0, 40.0, -40.0):
            x = rng.standard_normal((7, 4, 128), dtype=np.float32) + np.float32(shift)
            c, s, m = ref_quant.quantize(torch.from_numpy(x), bits, 32)
            oc, os_, om = O.quantize(x, bits, 32)
            assert np.array_equal(c.numpy(), oc) and np.array_equal(s.numpy(), os_) and np.array_equal(m.numpy(), om)
            p = ref_quant.pack(c, bits).numpy()
            assert np.array_equal(p, O.pack(oc, bits)) and np.array_equal(O.unpack(p, bits), oc)
            tag = f"b{bits}_s{int(shift)}"
            qz[f"x_{tag}"], qz[f"packed_{tag}"], qz[f"scale_{tag}"], qz[f"min_{tag}"] = x, p, s.numpy(), m.numpy()
        k = rng.standard_normal((70, 2, 64), dtype=np.float32)
        k[:, :, 5] += 25.0
        fk = ref_quant.fake_quant_channels(torch.from_numpy(k), bits, 32).numpy()
        assert np.array_equal(fk, O.fake_quant_channels(k, bits, 32))
        qz[f"kch_{bits}"], qz[f"kch_fq_{bits}"] = k, fk
    np.savez_compressed(out_dir / "quant.npz", **qz)

    # canary + controller
    cz = {}
    for name, q, kref, kg, scale in S.canary_inputs():
        r = ref_canary_kl(torch.from_numpy(q), torch.from_numpy(kref), (2, 4, 8), kg, scale).numpy()
        o = O.canary_kl(q, kref, (2, 4, 8), kg, scale)
        assert np.abs(r - o).max() <= 1e-5 * max(1.0, np.abs(r).max()), (name, r, o)
        cz[name] = r
    buf = np.arange(8.0).reshape(2, 4)
    assert ref_ring_view(torch.from_numpy(buf), 1, 4, dim=1).numpy().tolist() == O.ring_view(buf, 1, 4, axis=1).tolist()
    rng = np.random.default_rng(80)
    obs = np.abs(rng.standard_normal((40, 3))).astype(np.float64) * np.array([0.05, 0.01, 0.001])
    ctxs = rng.integers(100, 100000, size=40)
    for mode in ("none", "sqrt"):
        rc = LayerController(ControllerParams(tau0=0.01, l0=4096, tau_scaling=mode, alpha=0.3, init_bits=8))
        oc = O.Controller(tau0=0.01, l0=4096, tau_scaling=mode, alpha=0.3, init_bits=8)
        trace = []
        for d, c in zip(obs, ctxs):
            rc.observe(dict(zip((2, 4, 8), d.tolist())), float(c))
            oc.observe(dict(zip((2, 4, 8), d.tolist())), float(c))
            assert rc.bits == oc.bits and rc.ema == oc.ema
            trace.append(rc.bits)
        cz[f"ctl_bits_{mode}"] = np.array(trace)
    cz["ctl_obs"], cz["ctl_ctx"] = obs, ctxs
    np.savez_compressed(out_dir / "canary_controller.npz", **cz)
    print(f"wrote {n} scenario fixtures + quant.npz + canary_controller.npz")


if __name__ == "__main__":
    main()
