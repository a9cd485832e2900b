"""Per-layer tier controller: an EMA of the canary's KL per tier, lowest tier under the budget.

Behaviour of the reference's ``echokv_vllm/controller.py`` (``ControllerParams``
:11-19, ``LayerController`` :22-68): every canary measurement updates
``ema[b]`` for all tiers; unless frozen or pinned, the layer then moves to the
lowest tier whose EMA is below tau (the highest tier if none is).  With
``tau_scaling="sqrt"`` the budget is ``tau0 * sqrt(max(L, L0) / L0)``.  A tier
change only affects blocks opened afterwards.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

from echokv_b200.quant import SUPPORTED_BITS


@dataclass
class ControllerParams:
    tau0: float = 0.01
    l0: int = 4096
    tau_scaling: str = "none"  # "none" | "sqrt"
    alpha: float = 0.1
    init_bits: int = 8
    fixed_bits: int | None = None
    frozen: bool = False


def _no_ema() -> dict:
    return dict.fromkeys(SUPPORTED_BITS)


@dataclass
class LayerController:
    params: ControllerParams
    bits: int = 0
    ema: dict = field(default_factory=_no_ema)
    fires: int = 0
    transitions: int = 0

    def __post_init__(self) -> None:
        if not self.bits:
            self.bits = self.params.fixed_bits or self.params.init_bits

    def tau(self, ctx_len: float) -> float:
        p = self.params
        if p.tau_scaling != "sqrt":
            return p.tau0
        return p.tau0 * math.sqrt(max(ctx_len, p.l0) / p.l0)

    def observe(self, deltas: dict, ctx_len: float) -> None:
        """Fold one measurement ``{bits: KL}`` into the EMAs and re-evaluate the tier."""
        w = self.params.alpha
        for b, value in deltas.items():
            old = self.ema[b]
            self.ema[b] = value if old is None else w * value + (1.0 - w) * old
        self.fires += 1
        if self.params.frozen or self.params.fixed_bits is not None:
            return
        budget = self.tau(ctx_len)
        under = [b for b in sorted(SUPPORTED_BITS) if self.ema[b] is not None and self.ema[b] < budget]
        choice = under[0] if under else max(SUPPORTED_BITS)
        if choice != self.bits:
            self.bits = choice
            self.transitions += 1
