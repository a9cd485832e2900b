"""Run a scenario (see ``scenarios.py``) through the CUDA store and collect what the fixtures hold."""

from __future__ import annotations

import numpy as np
import torch

import scenarios as S

TDT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def make_cuda_store(sp: S.StoreSpec, device="cuda"):
    from echokv_b200.tiered_cache import TieredKVCache, TieredLayout

    layout = TieredLayout(num_kv_heads=sp.h, head_size=sp.d, block_size=sp.bs, mem_bits=sp.mem_bits,
                          k_group=sp.kg, v_group=sp.vg)
    backing = torch.full((sp.num_blocks * sp.page_stride + 64,), sp.fill, dtype=torch.uint8, device=device)
    pages = torch.as_strided(backing, (sp.num_blocks, sp.page_size), (sp.page_stride, 1))
    store = TieredKVCache(layout, pages, residual_slots=sp.residual_slots, residual_dtype=TDT[sp.dtype])
    return store, backing


def run_cuda(sc: S.Scenario, device="cuda", graph_semantics=False) -> dict:
    from echokv_b200.kernels.decode import decode_attention
    from echokv_b200.kernels.prefill import prefill_attention
    from echokv_b200.write_plan import stage_plan

    sp = sc.spec
    dt = TDT[sp.dtype]
    store, backing = make_cuda_store(sp, device)
    kw = sp.kref_window or sp.kg
    kref = torch.zeros(kw, sp.h, sp.d, device=device) if sc.use_kref else None
    for k, v, slots, bits in sc.steps:
        kt = torch.from_numpy(k).to(device=device, dtype=dt)
        vt = torch.from_numpy(v).to(device=device, dtype=dt)
        st = torch.from_numpy(np.asarray(slots, dtype=np.int64))
        if not graph_semantics:
            store.write(kt, vt, st, bits, kref=kref)
        else:  # full-grid launches masked by the device-side counts, as a captured graph replays them
            plan = store.planner.plan(st)
            opened = store.prepare(plan, bits)
            store.shared.commit(plan)
            meta, extra = stage_plan(plan, device, opened)
            store.shared.apply_res_map(*extra[:4])
            if opened is not None:
                store.write_headers(extra[4], extra[5])
            store.apply(meta, kt, vt, kref=kref, capturing=True)
    torch.cuda.synchronize()
    res = {
        "backing": backing.cpu().numpy(), "block_res": store.block_res.cpu().numpy(),
        "res_group": store.res_group.cpu().numpy(), "res_k": store.res_k.float().cpu().numpy(),
        "tag_h": store._tag_h.copy(), "pool_free": np.int64(store.pool_free),
        "residual_free": np.int64(store.residual_free), "downgraded": np.int64(store.downgraded_blocks),
        "demoted": np.int64(store.demoted_blocks), "sealed_groups": np.int64(store.sealed_groups),
        "tokens_written": np.array([store.tokens_written[b] for b in (2, 4, 8)], dtype=np.int64),
    }
    if kref is not None:
        res["kref"] = kref.cpu().numpy()
        res["kref_pos"] = np.int64(store.planner.kref_pos)
        res["kref_fill"] = np.int64(store.planner.kref_fill)
    for i, (blk, off) in enumerate(sc.gathers):
        kg, vg = store.gather(torch.from_numpy(np.asarray(blk, dtype=np.int64)),
                              torch.from_numpy(np.asarray(off, dtype=np.int64)))
        res[f"gather{i}_k"], res[f"gather{i}_v"] = kg.cpu().numpy(), vg.cpu().numpy()
    if sc.query is not None:
        q = torch.from_numpy(sc.query).to(device=device, dtype=dt)
        table = torch.from_numpy(sc.block_table).to(device)
        if sc.prefill is None:
            lens = torch.tensor(sc.seq_lens, device=device)
            res["attn_out"] = decode_attention(store, q, table, lens, sc.scale).float().cpu().numpy()
        else:
            out = torch.zeros_like(q)
            prefill_attention(store, q, out, sc.prefill, sc.req_of, table, sc.scale)
            res["attn_out"] = out.float().cpu().numpy()
    res["_store"] = store
    return res
