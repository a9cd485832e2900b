"""Run a scenario (see ``scenarios.py``) through the numpy oracle and collect what the fixtures hold."""

from __future__ import annotations

import hashlib

import numpy as np

import scenarios as S
from oracle import echokv_oracle as O


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def make_oracle_store(sp: S.StoreSpec) -> O.Store:
    layout = O.Layout(sp.h, sp.d, sp.bs, sp.mem_bits, sp.kg, sp.vg)
    rdt = {"f32": np.float32, "f16": np.float16, "bf16": "bf16"}[sp.dtype]
    return O.Store(layout, sp.num_blocks, page_bytes=sp.page_size, page_stride=sp.page_stride,
                   residual_slots=sp.residual_slots, residual_dtype=rdt, fill=sp.fill,
                   kref_window=sp.kref_window)


def run_oracle(sc: S.Scenario) -> dict:
    sp = sc.spec
    store = make_oracle_store(sp)
    kw = sp.kref_window or sp.kg
    kref = np.zeros((kw, sp.h, sp.d), dtype=np.float32) if sc.use_kref else None
    for k, v, slots, bits in sc.steps:
        store.write(k, v, slots, bits, kref=kref)
    res = {
        "backing": store.backing.copy(), "block_res": store.block_res.copy(),
        "res_group": store.res_group.copy(), "res_k": store.res_k.copy(), "tag_h": store.tag_h.copy(),
        "pool_free": np.int64(store.pool_free), "residual_free": np.int64(store.residual_free),
        "downgraded": np.int64(store.downgraded_blocks), "demoted": np.int64(store.demoted_blocks),
        "sealed_groups": np.int64(store.sealed_groups),
    }
    if kref is not None:
        res["kref"] = kref
        res["kref_pos"] = np.int64(store.planner.kref_pos)
        res["kref_fill"] = np.int64(store.planner.kref_fill)
    for i, (blk, off) in enumerate(sc.gathers):
        res[f"gather{i}_k"], res[f"gather{i}_v"] = store.gather(blk, off)
    if sc.query is not None:
        if sc.prefill is None:
            res["attn_out"] = O.decode_attention(store, sc.query, sc.block_table, sc.seq_lens, sc.scale)
        else:
            rk = None if sp.dtype == "f32" else (lambda x: S.round_to(x, sp.dtype))
            res["attn_out"] = O.prefill_attention(store, sc.query, sc.prefill, sc.req_of, sc.block_table,
                                                  sc.scale, round_kv=rk)
    return res
