"""Closed-loop serving latency inside a vLLM engine: stock bf16 KV cache vs this package's tiered cache at the same
KV memory.

Counterpart of the reference's ``evaluation/serving/echokv_latency.py`` (:65-145): for each configuration and each
concurrency level a fixed number of requests is kept in flight (a new request enters when one finishes), prompts are
``--input-len`` random token ids with ``--output-len`` greedy output tokens (``ignore_eos``), and time to first token,
time per output token, inter-token latency and end-to-end latency are reported as mean / median / p99 next to the
output throughput.  Past the point where the stock cache runs out of KV memory its requests queue and its time to
first token grows; the tiered cache holds about three times the tokens.  Differences from the reference: it drives
the engine in-process (``LLMEngine.add_request`` / ``step``) instead of an HTTP server and ``vllm bench serve``, the
plugin is ``echokv_b200``, and ``--random-init`` builds the model from a configuration alone (no weights can be
downloaded where this runs).

    python -m echokv_b200.harness.latency --random-init --input-len 8192 --output-len 256 --concurrency 16 32 \\
        --kv-cache-gib 16 --configs stock echokv-int4
"""

from __future__ import annotations

import argparse
import json
import os
import random
import subprocess
import sys
import time

from echokv_b200.harness.throughput import CONFIGS, random_init_dir

METRICS = ("ttft", "tpot", "itl", "e2el")  # the reference's columns (echokv_latency.py:36)


def percentiles(xs: list[float]) -> dict:
    """mean / median / p99 in milliseconds of a list of seconds."""
    if not xs:
        return {"mean_ms": None, "median_ms": None, "p99_ms": None}
    s = sorted(xs)

    def at(q: float) -> float:
        return s[min(len(s) - 1, int(round(q * (len(s) - 1))))]

    return {"mean_ms": 1e3 * sum(s) / len(s), "median_ms": 1e3 * at(0.5), "p99_ms": 1e3 * at(0.99)}


def summarize_requests(reqs: list[dict], wall: float) -> dict:
    """``reqs``: per request the arrival time and the time of every output token (seconds)."""
    ttft, tpot, itl, e2el, out_tokens = [], [], [], [], 0
    for r in reqs:
        ts = r["token_times"]
        if not ts:
            continue
        out_tokens += len(ts)
        ttft.append(ts[0] - r["arrival"])
        e2el.append(ts[-1] - r["arrival"])
        if len(ts) > 1:
            tpot.append((ts[-1] - ts[0]) / (len(ts) - 1))
            itl.extend(b - a for a, b in zip(ts, ts[1:]))
    res = {m: percentiles(v) for m, v in zip(METRICS, (ttft, tpot, itl, e2el))}
    res.update(completed=len(e2el), wall_s=wall, output_tok_s=out_tokens / wall if wall > 0 else 0.0)
    return res


def closed_loop(engine, prompts: list[dict], sampling, concurrency: int, delta: bool = False) -> dict:
    """Keep ``concurrency`` requests in flight until every prompt has been served.  ``delta``: the engine's outputs
    carry only the tokens produced since the previous step (otherwise all tokens so far)."""
    pending = list(enumerate(prompts))
    reqs: dict[str, dict] = {}
    seen: dict[str, int] = {}

    def admit() -> None:
        i, p = pending.pop(0)
        rid = f"r{concurrency}-{i}"
        reqs[rid] = {"arrival": time.perf_counter(), "token_times": []}
        seen[rid] = 0
        engine.add_request(rid, p, sampling)

    t0 = time.perf_counter()
    while pending and len(reqs) < concurrency:
        admit()
    running = len(reqs)
    while running:
        outs = engine.step()
        now = time.perf_counter()
        for o in outs:
            n = len(o.outputs[0].token_ids) + (seen[o.request_id] if delta else 0)
            if n > seen[o.request_id]:
                reqs[o.request_id]["token_times"].extend([now] * (n - seen[o.request_id]))
                seen[o.request_id] = n
            if o.finished:
                running -= 1
                if pending:
                    admit()
                    running += 1
    return summarize_requests(list(reqs.values()), time.perf_counter() - t0)


def child(args) -> None:
    import torch
    from vllm import LLM, SamplingParams

    echokv = os.environ.get("ECHOKV_ENABLE") == "1"
    kw = dict(
        model=args.model, dtype=args.dtype, max_model_len=args.input_len + args.output_len + 64,
        kv_cache_memory_bytes=int(args.kv_cache_gib * 2**30), tensor_parallel_size=args.tp, block_size=args.block_size,
        enable_prefix_caching=False, enforce_eager=args.enforce_eager, max_num_seqs=max(args.concurrency),
        gpu_memory_utilization=float(os.environ.get("ECHOKV_GPU_UTIL", "0.7")),
    )
    if args.random_init:
        kw.update(load_format="dummy", skip_tokenizer_init=True)
    if echokv and torch.cuda.is_available():
        kw["attention_config"] = {"backend": "CUSTOM"}
    llm = LLM(**kw)
    cfg = llm.llm_engine.vllm_config.cache_config
    rng = random.Random(0)
    vocab = llm.llm_engine.vllm_config.model_config.get_vocab_size()
    from vllm.sampling_params import RequestOutputKind

    def sampling(kind):
        return SamplingParams(temperature=0.0, max_tokens=args.output_len, ignore_eos=True,
                              detokenize=not args.random_init, output_kind=kind)

    def make(n: int) -> list[dict]:
        return [{"prompt_token_ids": [rng.randrange(100, vocab - 100) for _ in range(args.input_len)]} for _ in range(n)]

    llm.generate(make(2), sampling(RequestOutputKind.FINAL_ONLY))  # warm up (`generate` reports a request once, at its end)
    res = {"kv_capacity_tokens": (cfg.num_gpu_blocks or 0) * cfg.block_size, "levels": {}}
    for c in args.concurrency:
        # DELTA: every engine step reports the tokens it produced; parameters of their own, `generate` rewrites its
        sp = sampling(RequestOutputKind.DELTA)
        res["levels"][str(c)] = closed_loop(llm.llm_engine, make(args.requests_per_user * c), sp, c, delta=True)
    with open(args.child_out, "w") as f:
        json.dump(res, f)


def main() -> None:
    p = argparse.ArgumentParser()
    p.add_argument("--model", default="")
    p.add_argument("--random-init", action="store_true", help="Llama-3.1-8B architecture with dummy weights, no tokenizer")
    p.add_argument("--layers", type=int, default=0, help="with --random-init: number of layers (0 = the architecture's 32)")
    p.add_argument("--dtype", default="auto")
    p.add_argument("--tp", type=int, default=1)
    p.add_argument("--block-size", type=int, default=64)
    p.add_argument("--kv-cache-gib", type=float, default=16.0)
    p.add_argument("--input-len", type=int, default=8192)
    p.add_argument("--output-len", type=int, default=256)
    p.add_argument("--concurrency", type=int, nargs="+", default=[16, 32])
    p.add_argument("--requests-per-user", type=int, default=2, help="requests served per concurrency slot")
    p.add_argument("--enforce-eager", action="store_true")
    p.add_argument("--configs", nargs="*", default=["stock", "echokv-int4"])
    p.add_argument("--out", default="echokv_latency.json")
    p.add_argument("--child-out")
    args = p.parse_args()
    if args.child_out:
        child(args)
        return
    argv = list(sys.argv[1:])
    if args.random_init and not args.model:
        argv += ["--model", random_init_dir(args.layers)]
    elif not args.model:
        p.error("give --model or --random-init")
    results = {}
    for name in args.configs:
        tmp = f"{args.out}.{name}.tmp"
        env = dict(os.environ, VLLM_ALLOW_INSECURE_SERIALIZATION="1", **CONFIGS[name])
        proc = subprocess.run([sys.executable, "-m", "echokv_b200.harness.latency", "--child-out", tmp] + argv, env=env)
        if not os.path.exists(tmp):  # vLLM can abort during teardown after finishing: the result file is the success signal
            print(f"[{name}] FAILED (exit {proc.returncode})")
            results[name] = {"error": f"exit {proc.returncode}"}
            continue
        with open(tmp) as f:
            results[name] = json.load(f)
        os.remove(tmp)
    with open(args.out, "w") as f:
        json.dump({"rows": results, "args": {k: v for k, v in vars(args).items() if k != "child_out"}}, f, indent=1)
    for name, r in results.items():
        if "error" in r:
            print(name, r["error"])
            continue
        for c, lv in r["levels"].items():
            print(name, f"users={c}", f"capacity={r['kv_capacity_tokens']}", f"out_tok_s={lv['output_tok_s']:.0f}",
                  *(f"{m}_ms(mean/p99)={lv[m]['mean_ms']:.1f}/{lv[m]['p99_ms']:.1f}" for m in METRICS if lv[m]["mean_ms"] is not None))
    if any("error" in r for r in results.values()):
        sys.exit(1)


if __name__ == "__main__":
    main()
