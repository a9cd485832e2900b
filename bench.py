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
fixed ("strong" scaling); the only exchange is the all-reduce of the canary statistic.

The line also carries: the roofline of the split-K decode kernel, a parity check of the GPU output
against the CPU oracle on the sequences the CPU baseline rebuilds, the CPU baseline itself, the
chunked-prefill probe (configuration 3 shape), a bf16-KV decode of a stock attention library on the
same shape, and ``config5``: the Llama-3.1-70B attention shape (64 query / 8 KV heads, batch 128,
context 32,768) under the same tensor parallelism with the precision controller live.

One JSON line is printed by rank 0.
"""

from __future__ import annotations

import argparse
import json
import multiprocessing as mp
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
CPU_LAYERS = 2  # layers of the workload the CPU legs run (the step has --layers of them)
# dram__bytes_read.sum + dram__bytes_write.sum of one INT4 decode launch at batch 64 x ctx 4096 from the ncu capture
# summarised under profiles/ (reads 373.5 MB of pages, writes 7.3 MB of split partials)
DRAM_TRAFFIC_INT4 = 380_700_000


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
    ap.add_argument("--windows", type=int, default=5, help="timed windows of --steps steps each; the median is reported")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel eagerly instead of replaying a CUDA graph")
    ap.add_argument("--cpu-seqs", type=int, default=4, help="sequences in the CPU-baseline / parity sample (0 = skip both)")
    ap.add_argument("--canary-interval", type=int, default=8, help="measure the canary KL every N steps (0 = never)")
    ap.add_argument("--no-stock", action="store_true", help="skip the stock bf16-KV attention library on the same shape")
    ap.add_argument("--no-prefill", action="store_true", help="skip the chunked-prefill probe (configuration 3 shape)")
    ap.add_argument("--no-config5", action="store_true", help="skip the 70B-shape run with the live controller")
    ap.add_argument("--no-serving-geometry", action="store_true",
                    help="skip the split kernel's probe at block 64 / k_group 32 (the reference's serving geometry)")
    ap.add_argument("--config5-layers", type=int, default=4, help="resident layers cycled to stand for the 80 of the 70B shape")
    ap.add_argument("--config5-steps", type=int, default=4)
    ap.add_argument("--one-rank-of", type=int, default=1, metavar="N",
                    help="diagnostic: run the share of one rank of an N-times larger tensor-parallel job (KV heads / N); "
                         "the line it prints is not a whole-job figure")
    ap.add_argument("--tiers", default="", help="comma list of tiers cycled over the layers instead of the seeded draw "
                                                "(small profiling cases, e.g. --layers 2 --tiers 4)")
    return ap.parse_args()


def workload_string(a) -> str:
    """The same words in both arms, so that their configurations can be compared as text."""
    return (f"quantize-on-write + mixed-tier paged decode, {a.layers} layers Llama-3.1-8B shape "
            f"(32 q / 8 kv heads, d128), batch {a.batch}, ctx {a.ctx}, block 16, k_group 16, mem_bits 8")


def tier_vector(layers: int, seed: int, fixed: str = "") -> list[int]:
    if fixed:
        cyc = [int(x) for x in fixed.split(",")]
        return [cyc[i % len(cyc)] for i in range(layers)]
    rng = np.random.default_rng(seed)
    return [int(b) for b in rng.choice([8, 4, 2], size=layers, p=[0.25, 0.5, 0.25])]


def outlier_channels(seed: int) -> np.ndarray:
    return np.random.default_rng(seed + 2).permutation(D)[: max(1, D // 100)]


def bytes_per_token(bits: int, h: int, kg: int = KG) -> int:
    """Algorithmic bytes one stored token costs a decode read: K+V codes, V stats, amortized K stats."""
    return h * D * bits // 4 + 4 * h * D // VG + 4 * h * D // kg


def decode_bytes(lens: np.ndarray, bits, h: int, hq: int, elt: int = 2, bs: int = BS, kg: int = KG) -> int:
    """Algorithmic bytes of one decode-attention launch over sequences of ``lens`` tokens stored at ``bits``
    (an int, or one average figure of bytes per token for mixed tiers via ``bits=None`` is not supported)."""
    total = 0
    for n in np.asarray(lens).tolist():
        blocks = -(-n // bs)
        open_tok = n % kg  # keys of the open group come from the residual instead of codes
        total += blocks * 20 + n * bytes_per_token(bits, h, kg) + open_tok * (h * D * elt - h * D * bits // 8)
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
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50"],
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
        busy = [r for r in rows if r[2].replace(".", "").isdigit() and float(r[2]) > 250.0] or rows  # samples under load
        sm = sorted(float(r[0]) for r in busy)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(rows[0][1]), "reasons": reasons, "samples": len(rows),
                "samples_under_load": len(busy) if busy is not rows else 0,
                "power_w_max": max(float(r[2]) for r in rows if r[2].replace(".", "").isdigit())}


# ----------------------------------------------------------------------------------------------
# The CPU arm: the numpy oracle (a restatement of the reference's torch path) on every host core
# ----------------------------------------------------------------------------------------------

def cpu_job_inputs(seed: int, ctx: int, out_ch: np.ndarray):
    """Inputs of one (sequence, layer) of the workload: ctx + 1 K/V rows and the query of the decode step, rounded
    to bf16.  The B200 arm feeds the same values to the same (sequence, layer), so the outputs can be compared."""
    from oracle import echokv_oracle as O

    rng = np.random.default_rng(seed)
    k = rng.standard_normal((ctx + 1, H, D), dtype=np.float32)
    k[..., out_ch] *= 10.0
    v = rng.standard_normal((ctx + 1, H, D), dtype=np.float32)
    q = rng.standard_normal((1, HQ, D), dtype=np.float32)
    rb = lambda x: O.bf16_bits_to_f32(O.f32_to_bf16_bits(x))  # noqa: E731
    return rb(k), rb(v), rb(q)


def job_seed(seed: int, s: int, layer: int) -> int:
    return seed + 1000 + 17 * s + 7919 * layer


def _cpu_worker(conn, jobs, ctx, out_ch):
    """Owns the oracle stores of its (sequence, layer) jobs: builds their contexts (untimed), then runs one decode
    step (one-token write + attention) of all of them per "go" and reports the seconds and the first step's output."""
    sys.path.insert(0, str(ROOT))
    from oracle import echokv_oracle as O

    layout = O.Layout(H, D, BS, MEM_BITS, KG, VG)
    state = []
    for seed, bits in jobs:
        k, v, q = cpu_job_inputs(seed, ctx, out_ch)
        nb = -(-(ctx + 64) // BS) + 1
        st = O.Store(layout, nb, residual_slots=4, residual_dtype="bf16")
        for c0 in range(0, ctx, 1024):
            c1 = min(ctx, c0 + 1024)
            st.write(k[c0:c1], v[c0:c1], np.arange(c0, c1), bits)
        state.append([st, k[ctx:], v[ctx:], q, bits, ctx, np.arange(nb, dtype=np.int32)[None]])
    conn.send("ready")
    first = True
    while True:
        msg = conn.recv()
        if msg == "stop":
            return
        t0 = time.perf_counter()
        outs = []
        for job in state:
            st, k1, v1, q, bits, n, table = job
            st.write(k1, v1, np.array([n]), bits)
            o = O.decode_attention(st, q, table, [n + 1], D ** -0.5)
            job[5] = n + 1
            if first:
                outs.append(o[0])
        first = False
        conn.send((time.perf_counter() - t0, outs))


class CpuSteps:
    """The decode step of `n_seqs` sequences x CPU_LAYERS layers on `workers` host processes."""

    def __init__(self, a, tiers, n_seqs: int, workers: int) -> None:
        self.jobs = [(job_seed(a.seed, s, l), tiers[l % len(tiers)]) for l in range(min(CPU_LAYERS, a.layers)) for s in range(n_seqs)]
        self.workers = max(1, min(workers, len(self.jobs)))
        self.n_seqs, self.layers = n_seqs, min(CPU_LAYERS, a.layers)
        ctxm = mp.get_context("spawn")
        out_ch = outlier_channels(a.seed)
        self.conns, self.procs, self.owner = [], [], []
        t0 = time.perf_counter()
        for w in range(self.workers):
            mine = list(range(w, len(self.jobs), self.workers))
            parent, child = ctxm.Pipe()
            p = ctxm.Process(target=_cpu_worker, args=(child, [self.jobs[i] for i in mine], a.ctx, out_ch), daemon=True)
            p.start()
            self.conns.append(parent)
            self.procs.append(p)
            self.owner.append(mine)
        for c in self.conns:
            assert c.recv() == "ready"
        self.build_s = time.perf_counter() - t0

    def step(self):
        """One decode step of every job, all workers in parallel; wall seconds and (first call) the outputs by job."""
        t0 = time.perf_counter()
        for c in self.conns:
            c.send("go")
        replies = [c.recv() for c in self.conns]
        wall = time.perf_counter() - t0
        outs = {}
        for mine, (_, o) in zip(self.owner, replies):
            for i, x in zip(mine, o):
                outs[i] = x
        return wall, outs

    def close(self) -> None:
        for c in self.conns:
            c.send("stop")
        for p in self.procs:
            p.join(timeout=5)


def cpu_record(a, steps_s: list[float], pool: CpuSteps, kind_note: str) -> dict:
    """tokens/s of the full step from the wall time of the sampled step (batch x layers = factor x sample)."""
    factor = (a.batch * a.layers) / (pool.n_seqs * pool.layers)
    t = float(np.median(steps_s))
    return {"value": a.batch / (t * factor), "unit": "tokens/s", "cores": pool.workers, "kind": "port",
            "sample": f"{pool.n_seqs} sequences x {pool.layers} layers of ctx {a.ctx} per step (one-token write + decode attention, "
                      f"numpy oracle, {pool.workers} processes, {len(steps_s)} steps, {t:.3f} s each); "
                      f"extrapolated x{factor:g} to batch {a.batch} x {a.layers} layers; context build untimed ({pool.build_s:.0f} s). {kind_note}",
            "extrapolated": True, "factor": factor, "sample_step_s": t}


def run_reference(a) -> None:
    """The reference arm: the reference's CPU path (its torch code, restated in numpy: the reference is Python and
    does not travel to the GPU box) over the full batch x CPU_LAYERS layers per step on every host core."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    tiers = tier_vector(a.layers, a.seed, a.tiers)
    cores = os.cpu_count() or 1
    pool = CpuSteps(a, tiers, a.batch, cores)
    try:
        for _ in range(min(a.warmup, 1)):
            pool.step()
        steps = [pool.step()[0] for _ in range(a.steps)]
    finally:
        pool.close()
    base = cpu_record(a, steps, pool, "")
    t = float(np.median(steps))
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": "tokens/s", "n_gpus": a.gpus, "steps": a.steps,
        "warmup": a.warmup, "ms_per_step": 1e3 * t, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_string(a), "extrapolated": True, "factor": base["factor"],
                   "step": f"a timed step covers the full batch over {pool.layers} of the {a.layers} layers; value = batch / "
                           f"(ms_per_step x factor)", "host_cores": cores},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ----------------------------------------------------------------------------------------------
# Probes that ride along with the B200 arm
# ----------------------------------------------------------------------------------------------

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
    t, tq = float(np.mean(at_ms)), float(np.mean(dq_ms))
    return {"workload": f"{S} sequences x {nq}-token chunk over {ctx} stored tokens, layers INT4 / INT8 (configuration 3 shape)",
            "attention_ms_per_layer": t, "dequant_ms_per_layer": tq, "tflops": flops / t / 1e9,
            "peak_tflops": peak, "frac": flops / t / 1e9 / peak, "op_frac": flops / (t + tq) / 1e9 / peak,
            "peak_source": "measured" if "bf16_tflops" in peaks else "fallback", "bound": "tensor"}


def stock_bf16_probe(dev, S: int, ctx: int, seed: int):
    """The "stock" bar: the same decode step's attention over an uncompressed bf16 KV cache with an attention library
    of the image (library calls, not part of this package): FlashInfer's paged decode if it can be brought up here,
    else flash-attn's kv-cache kernel; whichever is fastest is reported with every attempt listed."""
    import torch

    layers = 2  # alternate so that nothing is served from L2 (1.07 GB of K+V per layer)
    gen = torch.Generator(device=dev).manual_seed(seed + 500)
    nbytes = S * (ctx + 1) * H * D * 2 * 2
    tried = {}

    def time_it(run):
        run()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            run()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (3 * layers)

    q = torch.randn(S, HQ, D, device=dev, generator=gen).bfloat16()
    try:  # FlashInfer: paged bf16 KV, page size 16, tensor-core decode
        import flashinfer

        page = 16
        ppr = -(-(ctx + 1) // page)
        kv = [torch.randn(S * ppr, 2, page, H, D, device=dev, generator=gen).bfloat16() for _ in range(layers)]
        indptr = torch.arange(0, S + 1, dtype=torch.int32, device=dev) * ppr
        indices = torch.arange(S * ppr, dtype=torch.int32, device=dev)
        last = torch.full((S,), (ctx + 1) - (ppr - 1) * page, dtype=torch.int32, device=dev)
        ws = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        wrap = flashinfer.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD", use_tensor_cores=True)
        wrap.plan(indptr, indices, last, HQ, H, D, page, q_data_type=torch.bfloat16, kv_data_type=torch.bfloat16)
        ms = time_it(lambda: [wrap.run(q, kv[l]) for l in range(layers)])
        tried["flashinfer BatchDecodeWithPagedKVCacheWrapper (bf16 pages of 16, tensor cores)"] = ms
        del kv, ws
    except Exception as e:  # noqa: BLE001
        tried["flashinfer"] = f"unavailable: {type(e).__name__}: {str(e)[:100]}"
    try:
        from flash_attn import flash_attn_with_kvcache

        kc = [torch.randn(S, ctx + 16, H, D, device=dev, generator=gen).bfloat16() for _ in range(layers)]
        vc = [torch.randn(S, ctx + 16, H, D, device=dev, generator=gen).bfloat16() for _ in range(layers)]
        lens = torch.full((S,), ctx + 1, dtype=torch.int32, device=dev)
        q4 = q.view(S, 1, HQ, D)
        ms = time_it(lambda: [flash_attn_with_kvcache(q4, kc[l], vc[l], cache_seqlens=lens, softmax_scale=D ** -0.5, causal=True)
                              for l in range(layers)])
        tried["flash_attn_with_kvcache (contiguous bf16 KV)"] = ms
        del kc, vc
    except Exception as e:  # noqa: BLE001
        tried["flash_attn"] = f"unavailable: {type(e).__name__}: {str(e)[:100]}"
    timed = {k: v for k, v in tried.items() if isinstance(v, float)}
    if not timed:
        return {"unavailable": tried}
    best = min(timed, key=timed.get)
    return {"what": best + ", same batch / context / heads", "ms_per_layer": timed[best], "gbs": nbytes / timed[best] / 1e6,
            "bytes_per_layer": nbytes, "tried": tried}


def serving_geometry_probe(a, dev, peaks: dict, S: int, ctx: int) -> dict:
    """The split kernel at the reference's serving geometry (block 64, k_group 32, mem_bits 4: 1,280 bytes per
    token at INT4, evaluation/serving/echokv_throughput.py:85 and echokv_vllm/config.py:43) on the benchmark's batch
    and context: two resident INT4 layers alternate (each pool larger than L2), CUDA events right around the kernel."""
    import torch

    from echokv_b200 import _native as N
    from echokv_b200.controller import ControllerParams, LayerController
    from echokv_b200.step import GroupRunner
    from echokv_b200.tiered_cache import TieredLayout

    bs, kg, mem, R = 64, 32, 4, 2
    layout = TieredLayout(num_kv_heads=H, head_size=D, block_size=bs, mem_bits=mem, k_group=kg, v_group=VG)
    bpseq = -(-(ctx + 64) // bs)
    nb = S * bpseq + 8
    page = bs * TieredLayout.per_token_bytes(H, D, mem, kg, VG)
    caches = [torch.zeros(nb, page, dtype=torch.uint8, device=dev) for _ in range(R)]
    ctl = [LayerController(ControllerParams(fixed_bits=4)) for _ in range(R)]
    runner = GroupRunner(layout, caches, HQ, D ** -0.5, ctl, residual_slots=S + 16, model_dtype=torch.bfloat16, cap=S,
                         max_model_len=bpseq * bs)
    table_np = np.random.default_rng(a.seed + 23).permutation(nb)[: S * bpseq].reshape(S, bpseq).astype(np.int32)
    table = torch.from_numpy(table_np).to(dev)
    gen = torch.Generator(device=dev).manual_seed(a.seed + 900)
    for c0 in range(0, ctx, 512):
        pos = np.arange(c0, min(ctx, c0 + 512))
        slots = (table_np[:, pos // bs].astype(np.int64) * bs + pos % bs).reshape(-1)
        meta = runner.plan_step(slots)
        for l in range(R):
            runner.write(l, torch.randn(slots.size, H, D, device=dev, generator=gen).bfloat16(),
                         torch.randn(slots.size, H, D, device=dev, generator=gen).bfloat16(), meta)
    rows = np.arange(S)
    slots = table_np[:, ctx // bs].astype(np.int64) * bs + ctx % bs
    meta = runner.plan_step(slots, decode=(rows, rows, np.full(S, ctx + 1)))
    q = torch.randn(R, S, HQ, D, device=dev, generator=gen).bfloat16()
    out = torch.zeros_like(q)
    for l in range(R):
        runner.write(l, torch.randn(S, H, D, device=dev, generator=gen).bfloat16(),
                     torch.randn(S, H, D, device=dev, generator=gen).bfloat16(), meta)
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    k0.record(); k1.record()
    torch.cuda.synchronize()
    ts = []
    N.lib.echokv_set_decode_events(k0.cuda_event, k1.cuda_event)
    try:
        for i in range(8):
            runner.decode(i % R, q[i % R], table, out[i % R], meta)
            torch.cuda.synchronize()
            ts.append(k0.elapsed_time(k1))
    finally:
        N.lib.echokv_set_decode_events(None, None)
    t = float(np.median(ts[2:]))
    nbytes = decode_bytes(np.full(S, ctx + 1), 4, H, HQ, bs=bs, kg=kg)
    peak = float(peaks.get("hbm_gbs", 6650.0))
    return {"what": "decode_mma_kernel, INT4, block 64 / k_group 32 / mem_bits 4 (the reference's serving geometry)",
            "kernel_ms": t, "bytes": nbytes, "bytes_per_token": bytes_per_token(4, H, kg), "gbs": nbytes / t / 1e6,
            "frac": nbytes / t / 1e6 / peak, "status": int(N.lib.echokv_kernel_status(0))}


def config5_probe(a, dev, world: int, rank: int, peaks: dict) -> dict | None:
    """Configuration 5: Llama-3.1-70B attention shape (64 query / 8 KV heads, d 128, 80 layers) sharded by KV head over
    the ranks, decode batch 128 at context 32,768, mem_bits 4, every layer's tier chosen by its controller from the
    canary (starting at INT4), the canary measured and all-reduced EVERY step.  80 layers of that size do not fit one
    GPU, so `--config5-layers` resident layers are cycled 80 times per step (every layer-step reads a pool far larger
    than L2).  Returns step time, the decode kernel's per-rank throughput against the HBM peak, and the tiers in use."""
    import torch
    import torch.distributed as dist

    from echokv_b200 import _native as N
    from echokv_b200.controller import ControllerParams, LayerController
    from echokv_b200.step import GroupRunner
    from echokv_b200.tiered_cache import TieredLayout

    HQ5, H5, L5, S, ctx, mem = 64, 8, 80, 128, 32768, 4
    h, hq = H5 // world, HQ5 // world
    R = max(1, a.config5_layers)
    layout = TieredLayout(num_kv_heads=h, head_size=D, block_size=BS, mem_bits=mem, k_group=KG, v_group=VG)
    steps_total = 3 + a.config5_steps + 2
    bps = -(-(ctx + steps_total + 8) // BS)
    nb = S * bps + 8
    page = BS * TieredLayout.per_token_bytes(h, D, mem, KG, VG)
    free = torch.cuda.mem_get_info(dev)[0]
    if R * nb * page > 0.8 * free:
        return {"skipped": f"{R} resident layers need {R * nb * page / 2**30:.1f} GiB, {free / 2**30:.1f} GiB free"}
    caches = [torch.zeros(nb, page, dtype=torch.uint8, device=dev) for _ in range(R)]
    ctl = [LayerController(ControllerParams(init_bits=4)) for _ in range(R)]
    runner = GroupRunner(layout, caches, hq, D ** -0.5, ctl, residual_slots=S + 16, model_dtype=torch.bfloat16,
                         cap=S, max_model_len=bps * BS)
    table_np = np.random.default_rng(a.seed + 11).permutation(nb)[: S * bps].reshape(S, bps).astype(np.int32)
    table = torch.from_numpy(table_np).to(dev)
    gen = torch.Generator(device=dev).manual_seed(a.seed + 700 + rank)
    out_ch = torch.from_numpy(outlier_channels(a.seed)).to(dev)
    chunk = 512
    for c0 in range(0, ctx, chunk):
        pos = np.arange(c0, min(ctx, c0 + chunk))
        slots = (table_np[:, pos // BS].astype(np.int64) * BS + pos % BS).reshape(-1)
        meta = runner.plan_step(slots)
        k = torch.randn(slots.size, h, D, device=dev, generator=gen)
        k[..., out_ch] *= 10.0
        k, v = k.bfloat16(), torch.randn(slots.size, h, D, device=dev, generator=gen).bfloat16()
        for l in range(R):
            runner.write(l, k, v, meta)
    torch.cuda.synchronize()
    q = torch.randn(R, S, hq, D, device=dev, generator=gen).bfloat16()
    kn = torch.randn(R, S, h, D, device=dev, generator=gen).bfloat16()
    vn = torch.randn(R, S, h, D, device=dev, generator=gen).bfloat16()
    out = torch.zeros(R, S, hq, D, device=dev, dtype=torch.bfloat16)
    rows = np.arange(S)
    state = {"len": ctx, "pending": None, "fires": 0}

    def host_plan():
        n = state["len"]
        slots = table_np[:, n // BS].astype(np.int64) * BS + n % BS
        state["len"] = n + 1
        return runner.plan_step(slots, decode=(rows, rows, np.full(S, n + 1)), canary=rows[:8].astype(np.int64))

    def device_step(meta, capturing=False):
        for it in range(L5):
            l = it % R
            runner.write(l, kn[l], vn[l], meta, capturing=capturing, query=q[l])  # + the canary's query rows
            runner.decode(l, q[l], table, out[l], meta)

    meta = host_plan()
    device_step(meta)
    torch.cuda.synchronize()
    graph = None
    if not a.no_graph:
        meta = host_plan()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            device_step(meta, capturing=True)

    def step():
        # canary interval 1: measure (and all-reduce over the ranks) every step; the controllers get the previous one
        if state["pending"] is not None:
            runner.observe(state["pending"], float(state["len"]))
        state["pending"] = runner.measure_canary(8, None)
        state["fires"] += 1
        m = host_plan()
        if graph is not None:
            graph.replay()
        else:
            device_step(m)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(3):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.config5_steps):
        step()
    e1.record()
    barrier()
    ms = torch.tensor([e0.elapsed_time(e1) / a.config5_steps], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    # the decode calls alone, back to back over the resident layers (every pool is far larger than L2)
    meta = host_plan()
    for l in range(R):
        runner.decode(l, q[l], table, out[l], meta)
    torch.cuda.synchronize()
    e0.record()
    reps = 2
    for _ in range(reps):
        for l in range(R):
            runner.decode(l, q[l], table, out[l], meta)
    e1.record()
    torch.cuda.synchronize()
    call_ms = e0.elapsed_time(e1) / (reps * R)
    # bytes: the blocks of every tier actually present in layer 0's pool
    st0 = runner.stores[0]
    tag = np.asarray(st0._tag_h)
    lens_now = np.full(S, state["len"])
    blocks_used = table_np[:, : -(-state["len"] // BS)].reshape(-1)
    hist = {str(b): int((tag[blocks_used] == b).sum()) for b in (2, 4, 8)}
    nbytes = sum(cnt * BS * bytes_per_token(int(b), h) for b, cnt in hist.items()) + S * (bps * 20 + 2 * hq * D * 2)
    peak = float(peaks.get("hbm_gbs", 6650.0))
    status = int(N.lib.echokv_kernel_status(0))
    del caches, runner, graph
    torch.cuda.empty_cache()
    return {"workload": f"Llama-3.1-70B attention shape, 80 layer-steps per decode step over {R} resident layers, batch {S}, ctx {ctx}, "
                        f"tp{world} by KV head ({h} KV / {hq} query heads per rank), mem_bits 4, controller live from INT4, canary interval 1",
            "ms_per_step": float(ms.item()), "tokens_per_s": S / (float(ms.item()) / 1e3), "steps": a.config5_steps,
            "decode_call_ms": call_ms, "decode_gbs_per_rank": nbytes / call_ms / 1e6, "frac": nbytes / call_ms / 1e6 / peak,
            "bytes_per_call_per_rank": nbytes, "peak": peak, "canary_fires": state["fires"],
            "tiers_of_layers": [c.bits for c in ctl], "blocks_by_tier_layer0": hist, "cuda_graph": not a.no_graph,
            "kernel_status": status, "rank0_lens": int(lens_now[0])}


# ----------------------------------------------------------------------------------------------
# The B200 arm
# ----------------------------------------------------------------------------------------------

def run_b200(a) -> None:
    import torch
    import torch.distributed as dist

    from echokv_b200 import _native as N
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
    shards = world * max(1, a.one_rank_of)
    if H % shards:
        raise SystemExit(f"{H} KV heads cannot be sharded over {shards} ranks")
    h, hq = H // shards, HQ // shards
    peaks = {}
    try:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    except OSError:
        pass

    tiers = tier_vector(a.layers, a.seed, a.tiers)
    layout = TieredLayout(num_kv_heads=h, head_size=D, block_size=BS, mem_bits=MEM_BITS, k_group=KG, v_group=VG)
    S, ctx, Lr = a.batch, a.ctx, a.layers
    total_steps = a.warmup + a.steps * (a.windows + 1) + 8
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
    out_ch_np = outlier_channels(a.seed)
    out_ch = torch.from_numpy(out_ch_np).to(dev)

    # the sequences and layers the CPU legs rebuild get the CPU legs' inputs, so the outputs can be compared
    n_par = min(a.cpu_seqs, S) if (world == 1 and rank == 0 and shards == 1) else 0
    par_layers = min(CPU_LAYERS, Lr) if n_par else 0
    par = {(s, l): cpu_job_inputs(job_seed(a.seed, s, l), ctx, out_ch_np) for s in range(n_par) for l in range(par_layers)}

    def kv_rows(n):
        k = torch.randn(n, h, D, device=dev, generator=gen)
        k[..., out_ch] *= 10.0
        v = torch.randn(n, h, D, device=dev, generator=gen)
        return k.bfloat16(), v.bfloat16()

    # ---- build the context: bulk quantize-on-write of S x ctx tokens per layer (untimed setup,
    # but its device time is recorded as the write kernels' throughput: events around each layer's
    # launches, read after the whole chunk, no host synchronisation between launches)
    chunk = 512
    write_ms, write_bytes = 0.0, 0
    # ~100 us of device work enqueued right before the first event: the host gets ahead of the device while it
    # runs, so the window between the events holds the write kernels' device time and not Python's launch time
    filler = torch.zeros(64 << 20, dtype=torch.float32, device=dev)
    for c0 in range(0, ctx, chunk):
        c1 = min(ctx, c0 + chunk)
        pos = np.arange(c0, c1)
        slots = (table_np[:, pos // BS].astype(np.int64) * BS + pos % BS).reshape(-1)
        meta = runner.plan_step(slots)
        evs = []
        for l in range(Lr):
            k, v = kv_rows(slots.size)
            for s in range(n_par if l < par_layers else 0):
                k[s * (c1 - c0):(s + 1) * (c1 - c0)] = torch.from_numpy(par[(s, l)][0][c0:c1]).to(dev).bfloat16()
                v[s * (c1 - c0):(s + 1) * (c1 - c0)] = torch.from_numpy(par[(s, l)][1][c0:c1]).to(dev).bfloat16()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            filler.add_(1.0)
            e0.record()
            runner.write(l, k, v, meta)
            e1.record()
            evs.append((e0, e1))
            write_bytes += slots.size * (4 * h * D + bytes_per_token(tiers[l], h))
        torch.cuda.synchronize()
        write_ms += sum(x.elapsed_time(y) for x, y in evs)
    del filler

    # ---- per-step inputs, resident on the device (and a pinned host copy for the e2e leg)
    q_dev = torch.randn(Lr, S, hq, D, device=dev, generator=gen).bfloat16()
    k_dev = torch.randn(Lr, S, h, D, device=dev, generator=gen).bfloat16()
    k_dev[..., out_ch] *= 10.0
    v_dev = torch.randn(Lr, S, h, D, device=dev, generator=gen).bfloat16()
    for (s, l), (pk, pv, pq) in par.items():
        k_dev[l, s] = torch.from_numpy(pk[ctx]).to(dev).bfloat16()
        v_dev[l, s] = torch.from_numpy(pv[ctx]).to(dev).bfloat16()
        q_dev[l, s] = torch.from_numpy(pq[0]).to(dev).bfloat16()
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
            # quantize-on-write + the canary's query rows (captured unconditionally) in one launch, then decode
            runner.write(l, k_dev[l], v_dev[l], meta, capturing=capturing, query=q_dev[l])
            runner.decode(l, q_dev[l], table, out_dev[l], meta)

    # kernels launched per step and layer: write_step (completed K groups + token rows + canary stash), the decode
    # split kernel and its merge (a memset node zeroes the split kernel's work counter before it)
    launches_per_step = 3 * Lr
    graph = None
    meta = host_plan()
    device_step(meta)  # eager step: sizes the decode scratch, touches every kernel
    torch.cuda.synchronize()
    first_out = out_dev[:par_layers, :n_par].float().cpu().numpy() if n_par else None
    if not a.no_graph:
        meta = host_plan()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            device_step(meta, capturing=True)
        graph.replay()
        torch.cuda.synchronize()

    canary = {"n": 0, "pending": None, "fires": 0}
    tp_group = None  # the default process group is the tensor-parallel group here

    def canary_fire():
        if canary["pending"] is not None:
            runner.observe(canary["pending"], float(state["len"]))  # reads a pinned copy made one measurement ago
        canary["pending"] = runner.measure_canary(8, tp_group)
        canary["fires"] += 1

    def canary_tick():
        """Every --canary-interval steps: KL of every layer at 2/4/8 bits from the K_ref rings and the
        stashed queries (one kernel), mean over TP ranks (one small NCCL all-reduce), and the previous
        measurement goes to the controllers (so nothing waits on the GPU)."""
        canary["n"] += 1
        if a.canary_interval and canary["n"] % a.canary_interval == 0:
            canary_fire()

    # The end-to-end leg moves every step's q / k / v from pinned host memory and its output back, as a serving
    # engine would: on two copy streams, so that step k + 1's inputs and step k - 1's output cross PCIe while step k
    # computes.  Landing buffers on the device decouple the copies from the buffers the graph was captured with.
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    q_land, k_land, v_land = (torch.empty_like(t) for t in (q_dev, k_dev, v_dev))
    out_land = torch.empty_like(out_dev)
    ev_in_ready, ev_in_taken, ev_out_ready, ev_out_done = (torch.cuda.Event() for _ in range(4))
    ev_in_taken.record()
    ev_out_done.record()

    def step(e2e: bool):
        canary_tick()  # before this step's plan moves the K_ref ring
        cur = torch.cuda.current_stream(dev)
        if e2e:
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_in_taken)  # the previous step has taken its inputs out of the landing buffers
                q_land.copy_(q_host, non_blocking=True)
                k_land.copy_(k_host, non_blocking=True)
                v_land.copy_(v_host, non_blocking=True)
                ev_in_ready.record(s_in)
            cur.wait_event(ev_in_ready)
            q_dev.copy_(q_land, non_blocking=True)
            k_dev.copy_(k_land, non_blocking=True)
            v_dev.copy_(v_land, non_blocking=True)
            ev_in_taken.record(cur)
        m = host_plan()
        if graph is not None:
            graph.replay()
        else:
            device_step(m)
        if e2e:
            cur.wait_event(ev_out_done)  # the previous step's output has left the landing buffer
            out_land.copy_(out_dev, non_blocking=True)
            ev_out_ready.record(cur)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_out_ready)
                out_host.copy_(out_land, non_blocking=True)
                ev_out_done.record(s_out)

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
        if e2e:
            torch.cuda.current_stream(dev).wait_event(ev_out_done)  # the last step's output is on the host
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    # warm-up: W steps, and the canary with its all-reduce fired twice (so that neither the communicator's set-up
    # nor the first read-back lands in a timed window)
    for i in range(a.warmup):
        step(False)
        if a.canary_interval and i < 2:
            canary_fire()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    windows = [timed(a.steps, False) for _ in range(max(1, a.windows))]
    clocks = sampler.stop() if rank == 0 else {}
    ms = float(np.median(windows))
    n_e2e = max(2, a.steps)  # windows of K steps like the device-timed ones: the pipeline's fill and drain are in the window
    step(True)  # touch the copies once
    ms_e2e = float(np.median([timed(n_e2e, True) / n_e2e for _ in range(3)]))

    # host share of a step: wall time of plan + upload + graph launch for three steps issued onto an idle GPU (the
    # staging ring holds four steps, so the host never waits for the device here)
    host_ms = []
    for _ in range(3):
        barrier()
        t0 = time.perf_counter()
        for _ in range(3):
            step(False)
        host_ms.append((time.perf_counter() - t0) / 3 * 1e3)
    barrier()
    host_ms_per_step = float(np.median(host_ms))

    # ---- roofline of the dominant kernel: paged decode attention (split kernel + merge), timed with
    # CUDA events on the launching stream over back-to-back launches: all layers of one tier, three
    # passes, no host synchronisation in between (consecutive launches read different layers' pools,
    # ~640 MB each, so nothing is served from L2)
    lens_now = np.full(S, state["len"])
    meta = host_plan()
    per_tier: dict[int, list[float]] = {2: [], 4: [], 8: []}
    kernel_ms: dict[int, float] = {}
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
    status = int(N.lib.echokv_kernel_status(0))  # 0: no kernel gave up on a bounded wait
    # free the main workload before the probes that need room of their own
    del graph, caches, runner
    torch.cuda.empty_cache()
    prefill = prefill_probe(dev, peaks, a.seed) if (rank == 0 and world == 1 and not a.no_prefill) else None
    torch.cuda.empty_cache()
    stock = stock_bf16_probe(dev, S, ctx, a.seed) if (rank == 0 and world == 1 and not a.no_stock) else None
    torch.cuda.empty_cache()
    cfg5 = None if a.no_config5 else config5_probe(a, dev, world, rank, peaks)
    serving = serving_geometry_probe(a, dev, peaks, S, ctx) if (rank == 0 and world == 1 and shards == 1 and not a.no_serving_geometry) else None

    if rank == 0:
        cores = os.cpu_count() or 1
        base, parity = None, None
        if n_par:
            pool = CpuSteps(a, tiers, n_par, cores)
            try:
                w0, outs = pool.step()
                steps_s = [w0] + [pool.step()[0] for _ in range(2)]
            finally:
                pool.close()
            base = cpu_record(a, steps_s, pool, "The same sequences and layers carry the same inputs on the GPU (see parity).")
            want = np.stack([np.stack([outs[l * n_par + s] for s in range(n_par)]) for l in range(par_layers)])
            diff = first_out - want
            parity = {"what": f"GPU decode output (bf16) of the first {n_par} sequences x {par_layers} layers of the step vs the CPU "
                              f"oracle on the same inputs (tiers {[tiers[l] for l in range(par_layers)]}); tolerance max_abs 2e-2, rel_l2 1e-2",
                      "max_abs": float(np.abs(diff).max()), "rel_l2": float(np.linalg.norm(diff) / max(np.linalg.norm(want), 1e-12)),
                      "ok": bool(np.abs(diff).max() <= 2e-2 and np.linalg.norm(diff) / max(np.linalg.norm(want), 1e-12) <= 1e-2)}
        value = S * a.steps / (ms / 1e3)
        h2d = sum(t.numel() * t.element_size() for t in (q_host, k_host, v_host))
        d2h = out_host.numel() * out_host.element_size()
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": ms / a.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload_string(a),
                       "tiers": {str(b): tiers.count(b) for b in (8, 4, 2)}, "parallelism": f"tp{world} by KV head" + (f" (one rank of tp{shards} only)" if shards != world else ""),
                       "cuda_graph": not a.no_graph, "l2": "each layer's pool is larger than L2; layers alternate",
                       "host_cores": cores, "timing": f"median of {len(windows)} windows of {a.steps} steps",
                       "e2e_transfers": "every step's q / k / v (pinned host -> device) and output (device -> pinned host) on two "
                                        "copy streams, overlapped with the neighbouring steps' compute",
                       "window_ms": [round(w, 3) for w in windows]},
            "roofline": {"bound": "hbm", "achieved": main["gbs"], "peak": peak, "unit": "GB/s", "frac": main["frac"],
                         "traffic": DRAM_TRAFFIC_INT4 if (S, ctx, world) == (64, 4096, 1) else None,
                         "kernel": "decode_mma_kernel (the split kernel of paged decode attention), INT4 layers; call_* = whole "
                                   "decode call (counter memset + split kernel + merge), back to back",
                         "peak_source": peak_src,
                         "algorithmic_bytes_per_launch": main["bytes"], "per_tier": tier_stats},
            "parity": parity,
            "cpu_baseline": base,
            "e2e": {"value": S / (ms_e2e / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "host_ms_per_step": host_ms_per_step,
            "gpu_launches": launches_per_step * a.steps + canary["fires"],
            "canary": {"interval": a.canary_interval, "fires": canary["fires"],
                       "last": None if canary["pending"] is None else [round(x, 6) for x in canary["pending"][0].tolist()]},
            "clocks": clocks,
            "kernel_status": status,
            "prefill": prefill,
            "stock_bf16_decode": stock,
            "config5": cfg5,
            "serving_geometry": serving,
            "write": {"gbs": write_bytes / write_ms / 1e6, "frac": write_bytes / write_ms / 1e6 / peak, "ms_total": write_ms,
                      "what": "bulk quantize-on-write of the context (finalize_k + write_tokens per layer and 512-position chunk, "
                              "events around each layer's launches, no host synchronisation between them)"},
        }))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)
