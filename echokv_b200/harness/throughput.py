"""Throughput and KV capacity inside a vLLM engine: stock bf16 KV cache vs this package's tiered cache at the same
memory budget.

Counterpart of the reference's ``evaluation/serving/echokv_throughput.py`` (:30-79 the child run, :82-140 the driver):
each configuration boots its own engine in a subprocess, runs ``--num-prompts`` requests of ``--input-len`` random
token ids with ``--output-len`` greedy output tokens (``ignore_eos``), and reports the KV capacity in tokens (from
vLLM's allocator), the wall time and output tokens/s.  Differences: the plugin is ``echokv_b200`` and, since model
weights cannot be downloaded where this runs, ``--random-init`` builds the model from a configuration alone
(Llama-3.1-8B architecture by default, vLLM's ``load_format="dummy"`` weights, no tokenizer).

    python -m echokv_b200.harness.throughput --random-init --num-prompts 256 --input-len 1024 --output-len 256 \\
        --kv-cache-gib 16 --configs stock echokv-int4
"""

from __future__ import annotations

import argparse
import json
import os
import random
import subprocess
import sys
import tempfile
import time

CONFIGS = {  # same names and variables as the reference harness
    "stock": {"ECHOKV_ENABLE": "0"},
    "echokv-int8": {"ECHOKV_ENABLE": "1", "ECHOKV_MEM_BITS": "8", "ECHOKV_FIXED_BITS": "8"},
    "echokv-int4": {"ECHOKV_ENABLE": "1", "ECHOKV_MEM_BITS": "4", "ECHOKV_FIXED_BITS": "4"},
    "echokv-live-mem6": {"ECHOKV_ENABLE": "1", "ECHOKV_MEM_BITS": "6"},
    "echokv-live-mem4": {"ECHOKV_ENABLE": "1", "ECHOKV_MEM_BITS": "4"},
}

LLAMA_31_8B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 4096, "intermediate_size": 14336,
    "num_hidden_layers": 32, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 128256,
    "max_position_embeddings": 131072, "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "hidden_act": "silu",
    "tie_word_embeddings": False, "torch_dtype": "bfloat16", "bos_token_id": 128000, "eos_token_id": 128001,
    "attention_bias": False, "mlp_bias": False,
}


def random_init_dir(layers: int | None) -> str:
    """A model directory holding only ``config.json`` (the architecture); the weights come from the dummy loader."""
    cfg = dict(LLAMA_31_8B)
    if layers:
        cfg["num_hidden_layers"] = layers
    d = tempfile.mkdtemp(prefix="echokv_llama_")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    return d


def child(args) -> None:
    import torch
    from vllm import LLM, SamplingParams

    echokv = os.environ.get("ECHOKV_ENABLE") == "1"
    kw = dict(
        model=args.model, dtype=args.dtype, max_model_len=args.input_len + args.output_len + 64,
        kv_cache_memory_bytes=int(args.kv_cache_gib * 2**30), tensor_parallel_size=args.tp, block_size=args.block_size,
        enable_prefix_caching=False, enforce_eager=args.enforce_eager, max_num_seqs=args.num_prompts,
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
    prompts = [{"prompt_token_ids": [rng.randrange(100, vocab - 100) for _ in range(args.input_len)]}
               for _ in range(args.num_prompts)]
    sp = SamplingParams(temperature=0.0, max_tokens=args.output_len, ignore_eos=True, detokenize=not args.random_init)
    llm.generate(prompts[: min(4, len(prompts))], sp)  # warm up
    t = time.perf_counter()
    outs = llm.generate(prompts, sp)
    wall = time.perf_counter() - t
    out_tokens = sum(len(o.outputs[0].token_ids) for o in outs)
    res = {
        "kv_capacity_tokens": (cfg.num_gpu_blocks or 0) * cfg.block_size,
        "wall_s": wall,
        "output_tok_s": out_tokens / wall,
        "total_tok_s": (out_tokens + args.input_len * len(prompts)) / wall,
    }
    if echokv:
        from echokv_b200 import control

        st = llm.apply_model(control.get_state)[0]
        res["avg_stored_bits"] = st["avg_stored_bits"]
        res["tier_vector"] = st["tier_vector"]
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
    p.add_argument("--kv-cache-gib", type=float, default=1.0)
    p.add_argument("--num-prompts", type=int, default=64)
    p.add_argument("--input-len", type=int, default=512)
    p.add_argument("--output-len", type=int, default=128)
    p.add_argument("--enforce-eager", action="store_true")
    p.add_argument("--configs", nargs="*", default=list(CONFIGS))
    p.add_argument("--out", default="echokv_throughput.json")
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
        proc = subprocess.run([sys.executable, "-m", "echokv_b200.harness.throughput", "--child-out", tmp] + argv, env=env)
        # vLLM can abort during teardown after finishing: the result file is the success signal.
        if not os.path.exists(tmp):
            print(f"[{name}] FAILED (exit {proc.returncode})")
            results[name] = {"error": f"exit {proc.returncode}"}
            continue
        with open(tmp) as f:
            results[name] = json.load(f)
        os.remove(tmp)
    report = summarize(results)
    report["args"] = {k: v for k, v in vars(args).items() if k != "child_out"}
    with open(args.out, "w") as f:
        json.dump(report, f, indent=1)
    for name, row in report["rows"].items():
        print(name, json.dumps(row))
    if report["failed"]:
        sys.exit(1)


def summarize(results: dict) -> dict:
    """Per configuration: what the child measured plus, against the stock run when there is one, the KV-capacity
    ratio (the reference's target is >= 3x at INT4) and the output-throughput ratio."""
    stock = results.get("stock")
    if stock is not None and "error" in stock:
        stock = None
    rows, failed = {}, []
    for name, r in results.items():
        if "error" in r:
            failed.append(name)
            rows[name] = r
            continue
        row = dict(r)
        if stock:
            row["capacity_vs_stock"] = r["kv_capacity_tokens"] / max(stock["kv_capacity_tokens"], 1)
            row["output_tok_s_vs_stock"] = r["output_tok_s"] / stock["output_tok_s"]
        rows[name] = row
    return {"rows": rows, "failed": failed}


if __name__ == "__main__":
    main()
