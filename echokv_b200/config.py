"""Settings from ``ECHOKV_*`` environment variables (same names, defaults and checks as the
reference's ``echokv_vllm/config.py:6-28, :62-99``).  Environment variables reach every worker
process, so the backend can read them wherever it is constructed.

    ECHOKV_ENABLE           1 installs the backend (plugin.py)
    ECHOKV_MEM_BITS         memory budget in bits/element: 2, 4, 6 or 8 (default 4, or
                            ECHOKV_FIXED_BITS when that is set)
    ECHOKV_INIT_BITS        starting tier of every layer (default: the highest tier the budget
                            gives every block: 8, 4, 4, 2 for budgets 8, 6, 4, 2)
    ECHOKV_FIXED_BITS       pin every layer to this tier (controller off)
    ECHOKV_FROZEN           1 keeps tiers fixed while the canary keeps measuring
    ECHOKV_TAU0             per-layer KL budget (default 0.01)
    ECHOKV_L0               reference context length for tau scaling (default 4096)
    ECHOKV_TAU_SCALING      none (default) or sqrt
    ECHOKV_ALPHA            EMA weight of the newest sample (default 0.1)
    ECHOKV_CANARY_INTERVAL  measure every N model steps (default 64)
    ECHOKV_KREF_WINDOW      K_ref ring size in tokens (default 64)
    ECHOKV_CANARY_MAX_Q     decode queries sampled per measurement (default 8)
    ECHOKV_K_GROUP          tokens per per-channel K group (default 32; power of 2, >= 16)
    ECHOKV_V_GROUP          head_dim elements per per-token V group (default 32)
    ECHOKV_RESIDUAL_SLOTS   open-K-group slots per layer (default max_num_seqs + 16)
    ECHOKV_CUDAGRAPH        0 keeps attention out of full CUDA graphs (backend.py)
    ECHOKV_CHECK_HOST_SLOTS 1 checks the host slot mapping against the device's every step
"""

from __future__ import annotations

import os
from dataclasses import dataclass, field

from echokv_b200.controller import ControllerParams
from echokv_b200.quant import SUPPORTED_BITS


@dataclass(frozen=True)
class EchoKVConfig:
    mem_bits: int = 4
    k_group: int = 32
    v_group: int = 32
    residual_slots: int | None = None
    canary_interval: int = 64
    kref_window: int = 64
    canary_max_q: int = 8
    controller: ControllerParams = field(default_factory=ControllerParams)


def _env(name: str, default, cast):
    raw = os.environ.get(name, "")
    return cast(raw) if raw != "" else default


def default_init_bits(mem_bits: int) -> int:
    """The highest tier every block can hold under the budget."""
    fitting = [b for b in SUPPORTED_BITS if b <= mem_bits]
    return max(fitting) if fitting else 2


def load_config() -> EchoKVConfig:
    fixed = _env("ECHOKV_FIXED_BITS", None, int)
    mem_bits = _env("ECHOKV_MEM_BITS", 4 if fixed is None else max(fixed, 2), int)  # a pinned tier gets its budget
    init = _env("ECHOKV_INIT_BITS", default_init_bits(mem_bits), int)
    for name, b in (("ECHOKV_INIT_BITS", init), ("ECHOKV_FIXED_BITS", fixed)):
        if b is not None and b not in SUPPORTED_BITS:
            raise ValueError(f"{name} must be one of {SUPPORTED_BITS}, got {b}")
    scaling = _env("ECHOKV_TAU_SCALING", "none", str)
    if scaling not in ("none", "sqrt"):
        raise ValueError("ECHOKV_TAU_SCALING must be none or sqrt")
    if mem_bits not in (2, 4, 6, 8):
        raise ValueError(f"ECHOKV_MEM_BITS must be 2, 4, 6 or 8, got {mem_bits}")
    cfg = EchoKVConfig(
        mem_bits=mem_bits,
        k_group=_env("ECHOKV_K_GROUP", 32, int),
        v_group=_env("ECHOKV_V_GROUP", 32, int),
        residual_slots=_env("ECHOKV_RESIDUAL_SLOTS", None, int),
        canary_interval=_env("ECHOKV_CANARY_INTERVAL", 64, int),
        kref_window=_env("ECHOKV_KREF_WINDOW", 64, int),
        canary_max_q=_env("ECHOKV_CANARY_MAX_Q", 8, int),
        controller=ControllerParams(
            tau0=_env("ECHOKV_TAU0", 0.01, float), l0=_env("ECHOKV_L0", 4096, int), tau_scaling=scaling,
            alpha=_env("ECHOKV_ALPHA", 0.1, float), init_bits=init, fixed_bits=fixed,
            frozen=_env("ECHOKV_FROZEN", "0", str) == "1"),
    )
    if cfg.canary_interval < 1:
        raise ValueError("ECHOKV_CANARY_INTERVAL must be >= 1")
    if cfg.k_group < 16 or cfg.k_group & (cfg.k_group - 1):
        raise ValueError(f"ECHOKV_K_GROUP must be a power of 2 and >= 16, got {cfg.k_group}")
    if cfg.kref_window < cfg.k_group:
        raise ValueError("ECHOKV_KREF_WINDOW must be >= ECHOKV_K_GROUP")
    return cfg
