#!/usr/bin/env python
"""Benchmark of the hot path: quantize-on-write + mixed-precision paged decode attention.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

Workload (one GPU): 32 layers of Llama-3.1-8B attention shape (32 query heads, 8 KV heads,
head_dim 128), bf16, block_size 16, k_group 16, v_group 32, mem_bits 8, a per-layer tier drawn
from {8, 4, 2} with probabilities {0.25, 0.5, 0.25} by seed, batch 64, context 4096 per sequence,
K/V ~ N(0, 1) with 1 % of channels scaled x10.  Data is synthetic (seeded) and stands in for
real model activations.  A *step* is one decode step of the whole stack: the host plans the
step's writes, then every layer stores its 64 new K/V rows (quantize-on-write) and runs paged
decode attention over its cache.  ``value`` is decode tokens/s (batch / step time) with q, k, v
resident in HBM; ``e2e`` adds the pinned host->device copy of the step's q/k/v and the
device->host copy of the attention output.  With N > 1 the KV heads are sharded over the ranks
(tensor parallelism: H/N KV heads and Hq/N query heads per rank, same batch), so total work is
fixed ("strong" scaling); no data-path collective is needed.

One JSON line is printed by rank 0.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

HQ, H, D, BS, KG, VG, MEM_BITS = 32, 8, 128, 16, 16, 32, 8
METRIC = "decode tokens/s/GPU at INT4 KV; paged-decode attention HBM GB/s vs peak"
# dram__bytes_read.sum + dram__bytes_write.sum of one INT4 decode launch at batch 64 x ctx 4096 from the
# ncu capture summarised under profiles/ (reads 376 MB of pages, writes 14 MB of split partials)
DRAM_TRAFFIC_INT4 = 390_500_000


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel eagerly instead of replaying a CUDA graph")
    ap.add_argument("--cpu-seqs", type=int, default=4, help="sequences in the CPU-baseline sample")
    ap.add_argument("--canary-interval", type=int, default=8, help="measure the canary KL every N steps (0 = never)")
    ap.add_argument("--stock", action="store_true", help="also time the image's flash-attention library over a bf16 KV cache "
                                                         "of the same shape (off by default: third-party kernels)")
    ap.add_argument("--no-prefill", action="store_true", help="skip the chunked-prefill probe (configuration 3 shape)")
    ap.add_argument("--tiers", default="", help="comma list of tiers cycled over the layers instead of the seeded draw "
                                                "(small profiling cases, e.g. --layers 2 --tiers 4)")
    return ap.parse_args()


def tier_vector(layers: int, seed: int, fixed: str = "") -> list[int]:
    if fixed:
        cyc = [int(x) for x in fixed.split(",")]
        return [cyc[i % len(cyc)] for i in range(layers)]
    rng = np.random.default_rng(seed)
    return [int(b) for b in rng.choice([8, 4, 2], size=layers, p=[0.25, 0.5, 0.25])]


def bytes_per_token(bits: int, h: int) -> int:
    """Algorithmic bytes one stored token costs a decode read: K+V codes, V stats, amortized K stats."""
    return h * D * bits // 4 + 4 * h * D // VG + 4 * h * D // KG


def decode_bytes(lens: np.ndarray, bits: int, h: int, hq: int, elt: int = 2) -> int:
    """Algorithmic bytes of one decode-attention launch over sequences of ``lens`` tokens at ``bits``."""
    total = 0
    for n in lens.tolist():
        blocks = -(-n // BS)
        open_tok = n % KG  # keys of the open group come from the residual instead of codes
        total += blocks * 20 + n * bytes_per_token(bits, h) + open_tok * (h * D * elt - h * D * bits // 8)
        total += 2 * hq * D * elt
    return total


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.rows: list[list[str]] = []
        self.proc = None
        self.index = index

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self) -> None:
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [r for r in self.rows if len(r) == 7 and r[0].replace(".", "").isdigit()]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = sorted(float(r[0]) for r in rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(rows[0][1]), "reasons": reasons, "samples": len(rows),
                "power_w_max": max(float(r[2]) for r in rows if r[2].replace(".", "").isdigit())}


# ----------------------------------------------------------------------------------------------
# CPU baseline: the numpy oracle on a bounded sample of the same workload
# ----------------------------------------------------------------------------------------------

def _cpu_seq_layer(args):
    """One (sequence, layer) of the workload through the oracle: returns seconds for the decode
    step (one-token write + attention); the context build is setup and untimed."""
    sys.path.insert(0, str(ROOT))
    from oracle import echokv_oracle as O

    seed, ctx, bits = args
    rng = np.random.default_rng(seed)
    layout = O.Layout(H, D, BS, MEM_BITS, KG, VG)
    nb = -(-(ctx + 1) // BS) + 1
    st = O.Store(layout, nb, residual_slots=4, residual_dtype="bf16")
    k = rng.standard_normal((ctx + 1, H, D), dtype=np.float32)
    v = rng.standard_normal((ctx + 1, H, D), dtype=np.float32)
    k[..., rng.integers(0, D, size=max(1, D // 100))] *= 10.0
    k, v = O.bf16_bits_to_f32(O.f32_to_bf16_bits(k)), O.bf16_bits_to_f32(O.f32_to_bf16_bits(v))
    table = np.arange(nb, dtype=np.int32)[None]
    for c0 in range(0, ctx, 1024):
        c1 = min(ctx, c0 + 1024)
        st.write(k[c0:c1], v[c0:c1], np.arange(c0, c1), bits)
    q = O.bf16_bits_to_f32(O.f32_to_bf16_bits(rng.standard_normal((1, HQ, D), dtype=np.float32)))
    t0 = time.perf_counter()
    st.write(k[ctx:], v[ctx:], np.array([ctx]), bits)
    O.decode_attention(st, q, table, [ctx + 1], D ** -0.5)
    return time.perf_counter() - t0


def cpu_baseline(a, tiers, workers: int, n_seqs: int, layers_sample: int) -> dict:
    """Times ``n_seqs`` sequences x ``layers_sample`` layers of the decode step on the host and
    scales to the full step (batch x layers); ``workers`` processes run in parallel."""
    from concurrent.futures import ProcessPoolExecutor

    jobs = [(1000 + 17 * s + l, a.ctx, tiers[l % len(tiers)]) for l in range(layers_sample) for s in range(n_seqs)]
    t0 = time.perf_counter()
    if workers > 1:
        with ProcessPoolExecutor(workers) as ex:
            per = list(ex.map(_cpu_seq_layer, jobs))
    else:
        per = [_cpu_seq_layer(j) for j in jobs]
    wall = time.perf_counter() - t0
    # throughput of the pool: seq-layers per second of timed work, all workers busy
    busy = sum(per) / max(1, min(workers, len(jobs)))
    step_seconds = busy / len(jobs) * (a.batch * a.layers)
    return {"value": a.batch / step_seconds, "unit": "tokens/s", "cores": workers, "kind": "port",
            "sample": f"{n_seqs} sequences x {layers_sample} layers of ctx {a.ctx} (one-token write + decode attention, "
                      f"numpy oracle), scaled to batch {a.batch} x {a.layers} layers; context build untimed; wall {wall:.1f}s"}


def prefill_probe(dev, peaks: dict, seed: int) -> dict:
    """Chunked prefill at the shape of configuration 3 (8 sequences, a 512-token chunk at the end of a context of
    8,704 stored tokens, layers at INT4 and INT8): dense dequantization + the attention kernel, timed with CUDA
    events; the tensor-pipe figure counts the attention kernel's FLOPs only."""
    import torch

    from echokv_b200.controller import ControllerParams, LayerController
    from echokv_b200.kernels.prefill import build_dense, dense_attention, dequant_dense
    from echokv_b200.step import GroupRunner
    from echokv_b200.tiered_cache import TieredLayout

    S, nq, prefix = 8, 512, 8192
    ctx = prefix + nq
    tiers = [4, 8]
    layout = TieredLayout(num_kv_heads=H, head_size=D, block_size=BS, mem_bits=MEM_BITS, k_group=KG, v_group=VG)
    bps = -(-ctx // BS)
    nb = S * bps + 8
    page = BS * TieredLayout.per_token_bytes(H, D, MEM_BITS, KG, VG)
    caches = [torch.zeros(nb, page, dtype=torch.uint8, device=dev) for _ in tiers]
    ctl = [LayerController(ControllerParams(fixed_bits=b)) for b in tiers]
    runner = GroupRunner(layout, caches, HQ, D ** -0.5, ctl, residual_slots=S + 16, model_dtype=torch.bfloat16,
                         cap=64, max_model_len=bps * BS)
    table_np = np.random.default_rng(seed + 7).permutation(nb)[: S * bps].reshape(S, bps).astype(np.int32)
    table = torch.from_numpy(table_np).to(dev)
    gen = torch.Generator(device=dev).manual_seed(seed + 300)
    for c0 in range(0, ctx, 512):
        pos = np.arange(c0, min(ctx, c0 + 512))
        slots = (table_np[:, pos // BS].astype(np.int64) * BS + pos % BS).reshape(-1)
        meta = runner.plan_step(slots)
        for l in range(len(tiers)):
            k = torch.randn(slots.size, H, D, device=dev, generator=gen).bfloat16()
            v = torch.randn(slots.size, H, D, device=dev, generator=gen).bfloat16()
            runner.write(l, k, v, meta)
    q = torch.randn(S * nq, HQ, D, device=dev, generator=gen).bfloat16()
    out = torch.empty_like(q)
    prefill = [(i * nq, (i + 1) * nq, ctx, 0) for i in range(S)]
    work, total, chunks, max_chunk = build_dense(prefill, list(range(S)), BS, dev)

    def timed(fn, reps=3):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    dq_ms, at_ms = [], []
    for st in runner.stores:
        kv = dequant_dense(st, work, total, table, torch.bfloat16)
        dq_ms.append(timed(lambda: dequant_dense(st, work, total, table, torch.bfloat16)))
        at_ms.append(timed(lambda: dense_attention(q, kv[0], kv[1], chunks, max_chunk, out, D ** -0.5)))
    flops = 4 * HQ * D * S * sum(ctx - nq + i + 1 for i in range(nq))
    peak = float(peaks.get("bf16_tflops", 1590.0))
    t = float(np.mean(at_ms))
    return {"workload": f"{S} sequences x {nq}-token chunk over {ctx} stored tokens, layers INT4 / INT8 (configuration 3 shape)",
            "attention_ms_per_layer": t, "dequant_ms_per_layer": float(np.mean(dq_ms)), "tflops": flops / t / 1e9,
            "peak_tflops": peak, "frac": flops / t / 1e9 / peak,
            "peak_source": "measured" if "bf16_tflops" in peaks else "fallback", "bound": "tensor"}


def stock_bf16_probe(dev, S: int, ctx: int, seed: int):
    """The "stock" bar: the same decode step's attention over an uncompressed bf16 KV cache with the
    flash-attention library that ships with the image (a library call, not part of this package).  Returns
    None when the library is missing or has no kernel for this GPU."""
    import torch

    try:
        from flash_attn import flash_attn_with_kvcache
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"flash_attn import failed: {type(e).__name__}"}
    try:
        gen = torch.Generator(device=dev).manual_seed(seed + 500)
        layers = 2  # alternate so that nothing is served from L2 (1.08 GB of K+V per layer)
        kc = [torch.randn(S, ctx + 16, H, D, device=dev, generator=gen).bfloat16() for _ in range(layers)]
        vc = [torch.randn(S, ctx + 16, H, D, device=dev, generator=gen).bfloat16() for _ in range(layers)]
        q = torch.randn(S, 1, HQ, D, device=dev, generator=gen).bfloat16()
        lens = torch.full((S,), ctx + 1, dtype=torch.int32, device=dev)

        def run():
            for l in range(layers):
                flash_attn_with_kvcache(q, kc[l], vc[l], cache_seqlens=lens, softmax_scale=D ** -0.5, causal=True)

        run()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            run()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / (3 * layers)
        nbytes = S * (ctx + 1) * H * D * 2 * 2
        return {"what": "flash_attn_with_kvcache over a contiguous bf16 KV cache, same batch / context / heads",
                "ms_per_layer": ms, "gbs": nbytes / ms / 1e6, "bytes_per_layer": nbytes}
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"{type(e).__name__}: {str(e)[:120]}"}


def run_reference(a) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    tiers = tier_vector(a.layers, a.seed, a.tiers)
    cores = os.cpu_count() or 1
    vals = []
    base = None
    for _ in range(max(1, min(a.steps, 3))):
        base = cpu_baseline(a, tiers, cores, n_seqs=max(cores // 2, 2), layers_sample=2)
        vals.append(base["value"])
    v = float(np.median(vals))
    base["value"] = v
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": "tokens/s", "n_gpus": a.gpus, "steps": a.steps,
        "warmup": a.warmup, "ms_per_step": 1e3 * a.batch / v, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{a.layers}-layer Llama-3.1-8B-shape mixed-tier decode step, batch {a.batch}, ctx {a.ctx}, "
                               f"block 16 (CPU port of the reference's torch path, bounded sample)"},
        "cpu_baseline": base,
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ----------------------------------------------------------------------------------------------
# The B200 arm
# ----------------------------------------------------------------------------------------------

def run_b200(a) -> None:
    import torch
    import torch.distributed as dist

    from echokv_b200.controller import ControllerParams, LayerController
    from echokv_b200.step import GroupRunner
    from echokv_b200.tiered_cache import TieredLayout

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU implementation")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if H % world:
        raise SystemExit(f"{H} KV heads cannot be sharded over {world} ranks")
    h, hq = H // world, HQ // world

    tiers = tier_vector(a.layers, a.seed, a.tiers)
    layout = TieredLayout(num_kv_heads=h, head_size=D, block_size=BS, mem_bits=MEM_BITS, k_group=KG, v_group=VG)
    S, ctx, Lr = a.batch, a.ctx, a.layers
    total_steps = a.warmup + a.steps + 4
    blocks_per_seq = -(-(ctx + 2 * total_steps + 8) // BS)
    num_blocks = S * blocks_per_seq + 8
    page = BS * TieredLayout.per_token_bytes(h, D, MEM_BITS, KG, VG)
    caches = [torch.zeros(num_blocks, page, dtype=torch.uint8, device=dev) for _ in range(Lr)]
    ctl = [LayerController(ControllerParams(fixed_bits=b)) for b in tiers]
    runner = GroupRunner(layout, caches, hq, D ** -0.5, ctl, residual_slots=S + 16, model_dtype=torch.bfloat16,
                         cap=max(64, S), max_model_len=blocks_per_seq * BS)
    # block table: a seeded permutation of the physical blocks
    perm = np.random.default_rng(a.seed + 1).permutation(num_blocks)[: S * blocks_per_seq]
    table_np = perm.reshape(S, blocks_per_seq).astype(np.int32)
    table = torch.from_numpy(table_np).to(dev)

    gen = torch.Generator(device=dev).manual_seed(a.seed + 100 + rank)
    out_ch = torch.from_numpy(np.random.default_rng(a.seed + 2).permutation(D)[: max(1, D // 100)]).to(dev)

    def kv_rows(n):
        k = torch.randn(n, h, D, device=dev, generator=gen)
        k[..., out_ch] *= 10.0
        v = torch.randn(n, h, D, device=dev, generator=gen)
        return k.bfloat16(), v.bfloat16()

    # ---- build the context: bulk quantize-on-write of S x ctx tokens per layer (untimed setup,
    # but its device time is recorded as the write kernels' throughput)
    chunk = 512
    write_ms, write_bytes = 0.0, 0
    for c0 in range(0, ctx, chunk):
        c1 = min(ctx, c0 + chunk)
        pos = np.arange(c0, c1)
        slots = (table_np[:, pos // BS].astype(np.int64) * BS + pos % BS).reshape(-1)
        meta = runner.plan_step(slots)
        for l in range(Lr):
            k, v = kv_rows(slots.size)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            runner.write(l, k, v, meta)
            e1.record()
            torch.cuda.synchronize()
            write_ms += e0.elapsed_time(e1)
            write_bytes += slots.size * (4 * h * D + bytes_per_token(tiers[l], h))

    # ---- per-step inputs, resident on the device (and a pinned host copy for the e2e leg)
    q_dev = torch.randn(Lr, S, hq, D, device=dev, generator=gen).bfloat16()
    k_dev = torch.randn(Lr, S, h, D, device=dev, generator=gen).bfloat16()
    k_dev[..., out_ch] *= 10.0
    v_dev = torch.randn(Lr, S, h, D, device=dev, generator=gen).bfloat16()
    out_dev = torch.zeros(Lr, S, hq, D, device=dev, dtype=torch.bfloat16)
    q_host, k_host, v_host = (t.cpu().pin_memory() for t in (q_dev, k_dev, v_dev))
    out_host = torch.zeros_like(out_dev, device="cpu").pin_memory()
    rows = np.arange(S)
    state = {"len": ctx}

    def host_plan():
        n = state["len"]
        slots = table_np[:, n // BS].astype(np.int64) * BS + n % BS
        state["len"] = n + 1
        return runner.plan_step(slots, decode=(rows, rows, np.full(S, n + 1)), canary=rows[:8].astype(np.int64))

    def device_step(meta, capturing=False):
        for l in range(Lr):
            runner.write(l, k_dev[l], v_dev[l], meta, capturing=capturing)
            runner.decode(l, q_dev[l], table, out_dev[l], meta)
            runner.stash_queries(l, q_dev[l], meta)  # the canary's query rows (captured unconditionally)

    launches_per_step = 4 * Lr  # finalize, write_tokens, decode, merge per layer (+ host-plan scatters)
    graph = None
    meta = host_plan()
    device_step(meta)  # eager step: sizes the decode scratch, touches every kernel
    torch.cuda.synchronize()
    if not a.no_graph:
        meta = host_plan()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            device_step(meta, capturing=True)
        graph.replay()
        torch.cuda.synchronize()

    canary = {"n": 0, "pending": None, "fires": 0}
    tp_group = None  # the default process group is the tensor-parallel group here

    def canary_tick():
        """Every --canary-interval steps: KL of every layer at 2/4/8 bits from the K_ref rings and the
        stashed queries (one kernel), mean over TP ranks (one small NCCL all-reduce), and the previous
        measurement goes to the controllers (so nothing waits on the GPU)."""
        canary["n"] += 1
        if not a.canary_interval or canary["n"] % a.canary_interval:
            return
        if canary["pending"] is not None:
            runner.observe(canary["pending"], float(state["len"]))
        canary["pending"] = runner.measure_canary(8, tp_group)
        canary["fires"] += 1

    def step(e2e: bool):
        canary_tick()  # before this step's plan moves the K_ref ring
        if e2e:
            q_dev.copy_(q_host, non_blocking=True)
            k_dev.copy_(k_host, non_blocking=True)
            v_dev.copy_(v_host, non_blocking=True)
        m = host_plan()
        if graph is not None:
            graph.replay()
        else:
            device_step(m)
        if e2e:
            out_host.copy_(out_dev, non_blocking=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(n_steps: int, e2e: bool) -> float:
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n_steps):
            step(e2e)
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(a.warmup):
        step(False)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms = timed(a.steps, False)
    clocks = sampler.stop() if rank == 0 else {}
    ms_e2e = timed(max(2, a.steps // 2), True) / max(2, a.steps // 2)

    # ---- roofline of the dominant kernel: paged decode attention (split kernel + merge), timed with
    # CUDA events on the launching stream over back-to-back launches: all layers of one tier, three
    # passes, no host synchronisation in between (consecutive launches read different layers' pools,
    # ~640 MB each, so nothing is served from L2)
    lens_now = np.full(S, state["len"])
    meta = host_plan()
    per_tier: dict[int, list[float]] = {2: [], 4: [], 8: []}
    kernel_ms: dict[int, float] = {}
    from echokv_b200 import _native as N

    for b in (2, 4, 8):
        layers_b = [l for l in range(Lr) if tiers[l] == b]
        if not layers_b:
            continue
        for l in layers_b:  # warm
            runner.decode(l, q_dev[l], table, out_dev[l], meta)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 3
        e0.record()
        for _ in range(reps):
            for l in layers_b:
                runner.decode(l, q_dev[l], table, out_dev[l], meta)
        e1.record()
        torch.cuda.synchronize()
        per_tier[b].append(e0.elapsed_time(e1) / (reps * len(layers_b)))
        # the split kernel alone: the library records these two events on the launching stream right around it
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        k0.record(); k1.record()  # creates the underlying CUDA events
        torch.cuda.synchronize()
        ks = []
        N.lib.echokv_set_decode_events(k0.cuda_event, k1.cuda_event)
        try:
            for _ in range(reps):
                for l in layers_b:
                    runner.decode(l, q_dev[l], table, out_dev[l], meta)
                    torch.cuda.synchronize()
                    ks.append(k0.elapsed_time(k1))
        finally:
            N.lib.echokv_set_decode_events(None, None)
        kernel_ms[b] = float(np.mean(ks))
    peaks = {}
    try:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    except OSError:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    peak_src = "measured" if "hbm_gbs" in peaks else "fallback"
    tier_stats = {}
    for b, ts in per_tier.items():
        if ts:
            nbytes = decode_bytes(lens_now + 1, b, h, hq)
            t = float(np.mean(ts))
            tk = kernel_ms.get(b, t)
            tier_stats[f"int{b}"] = {"kernel_ms": tk, "gbs": nbytes / tk / 1e6, "frac": nbytes / tk / 1e6 / peak, "bytes": nbytes,
                                     "call_ms": t, "call_gbs": nbytes / t / 1e6, "call_frac": nbytes / t / 1e6 / peak}
    main = tier_stats.get("int4") or next(iter(tier_stats.values()))
    prefill = None
    if rank == 0 and world == 1 and not a.no_prefill:
        prefill = prefill_probe(dev, peaks, a.seed)
    stock = stock_bf16_probe(dev, S, ctx, a.seed) if (rank == 0 and world == 1 and a.stock) else None

    if rank == 0:
        cores = os.cpu_count() or 1
        base = cpu_baseline(a, tiers, 1, n_seqs=a.cpu_seqs, layers_sample=2) if a.cpu_seqs > 0 else None
        value = S * a.steps / (ms / 1e3)
        h2d = sum(t.numel() * t.element_size() for t in (q_host, k_host, v_host))
        d2h = out_host.numel() * out_host.element_size()
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": ms / a.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"quantize-on-write + mixed-tier paged decode, {Lr} layers Llama-3.1-8B shape "
                                   f"(32 q / 8 kv heads, d128), batch {S}, ctx {ctx}, block 16, k_group 16, mem_bits 8",
                       "tiers": {str(b): tiers.count(b) for b in (8, 4, 2)}, "parallelism": f"tp{world} by KV head",
                       "cuda_graph": graph is not None, "l2": "each layer's pool is larger than L2; layers alternate",
                       "host_cores": cores},
            "roofline": {"bound": "hbm", "achieved": main["gbs"], "peak": peak, "unit": "GB/s", "frac": main["frac"],
                         "traffic": DRAM_TRAFFIC_INT4 if (S, ctx, world) == (64, 4096, 1) else None,
                         "kernel": "decode_mma_kernel (the split kernel of paged decode attention), INT4 layers; call_* = whole "
                                   "decode call (counter memset + split kernel + merge), back to back",
                         "peak_source": peak_src,
                         "algorithmic_bytes_per_launch": main["bytes"], "per_tier": tier_stats},
            "cpu_baseline": base,
            "e2e": {"value": S / (ms_e2e / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches_per_step * a.steps + canary["fires"],
            "canary": {"interval": a.canary_interval, "fires": canary["fires"],
                       "last": None if canary["pending"] is None else [round(x, 6) for x in canary["pending"][0].tolist()]},
            "clocks": clocks,
            "kernel_status": int(N.lib.echokv_kernel_status(0)),  # 0: no kernel gave up on a bounded wait
            "prefill": prefill,
            "stock_bf16_decode": stock,
            "write": {"gbs": write_bytes / write_ms / 1e6, "ms_total": write_ms, "what": "bulk quantize-on-write of the context"},
        }))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)
