"""Look into, and steer, the EchoKV layers of a running engine.

Each function takes the model as its first argument and returns something picklable, so
``llm.apply_model(fn)`` (with ``functools.partial`` for further arguments and
``VLLM_ALLOW_INSECURE_SERIALIZATION=1``) runs it in every worker.  Function names, arguments and
the fields of ``get_state`` follow the reference's ``echokv_vllm/control.py:27-117``.
"""

from __future__ import annotations

import re

import torch

from echokv_b200.quant import SUPPORTED_BITS

_STORE_COUNTERS = ("downgraded_blocks", "demoted_blocks", "sealed_groups", "pool_free", "pool_size")


def iter_layers(model: torch.nn.Module):
    """Yield ``(layer_name, impl)`` for every attention layer served by this backend, by layer number."""
    from echokv_b200.backend import EchoKVAttentionImpl

    def number(name: str, fallback: int) -> int:
        hit = re.search(r"layers\.(\d+)\.", name)
        return int(hit.group(1)) if hit else fallback

    ours = [(getattr(m, "layer_name", path), m.impl) for path, m in model.named_modules()
            if isinstance(getattr(m, "impl", None), EchoKVAttentionImpl)]
    keyed = [(number(name, i), name, impl) for i, (name, impl) in enumerate(ours)]
    for _, name, impl in sorted(keyed, key=lambda item: item[0]):
        yield name, impl


def _apply(model: torch.nn.Module, action) -> int:
    """Run ``action(impl)`` on every layer; the number of layers touched."""
    count = 0
    for _, impl in iter_layers(model):
        action(impl)
        count += 1
    return count


def _by_tier(counts: dict) -> dict:
    return {str(bits): n for bits, n in counts.items()}


def get_state(model: torch.nn.Module) -> dict:
    """Tier, EMAs and storage counters of each layer, and totals over the model."""
    per_layer = []
    totals = dict.fromkeys(SUPPORTED_BITS, 0)
    for name, impl in iter_layers(model):
        ctl = impl.controller
        row = dict(layer=name, bits=ctl.bits, ema=_by_tier(ctl.ema), fires=ctl.fires, transitions=ctl.transitions,
                   forward_calls=impl.forward_calls)
        if impl.store is not None:
            written = impl.store.tokens_written
            row["tokens_written"] = _by_tier(written)
            row["blocks_opened"] = _by_tier(impl.store.blocks_opened)
            row.update({key: getattr(impl.store, key) for key in _STORE_COUNTERS})
            for bits, n in written.items():
                totals[bits] += n
        per_layer.append(row)
    stored = sum(totals.values())
    return {
        "tier_vector": [row["bits"] for row in per_layer],
        "tokens_written": _by_tier(totals),
        "avg_stored_bits": sum(bits * n for bits, n in totals.items()) / stored if stored else None,
        "layers": per_layer,
    }


def get_tier_vector(model: torch.nn.Module) -> list[int]:
    return [impl.controller.bits for _, impl in iter_layers(model)]


def set_frozen(model: torch.nn.Module, frozen: bool) -> int:
    """Hold every layer at its tier (or let go again); the canary still feeds the EMAs."""
    return _apply(model, lambda impl: setattr(impl.controller.params, "frozen", frozen))


def set_tau0(model: torch.nn.Module, tau0: float) -> int:
    return _apply(model, lambda impl: setattr(impl.controller.params, "tau0", tau0))


def set_tier_vector(model: torch.nn.Module, bits) -> int:
    """Give each layer a tier (one int for all, or one per layer); blocks opened from now on use it."""
    impls = [impl for _, impl in iter_layers(model)]
    wanted = [bits] * len(impls) if isinstance(bits, int) else list(bits)
    if len(wanted) != len(impls):
        raise ValueError(f"got {len(wanted)} tiers for {len(impls)} layers")
    for b in wanted:
        if b not in SUPPORTED_BITS:
            raise ValueError(f"unsupported tier {b}")
    for impl, b in zip(impls, wanted):
        impl.controller.bits = b
    return len(impls)


def reset_counters(model: torch.nn.Module) -> int:
    """Zero the storage counters and forward-call counts, e.g. between warmup and measurement."""

    def clear(impl) -> None:
        if impl.store is not None:
            impl.store.reset_counters()
        impl.forward_calls = 0

    return _apply(model, clear)
