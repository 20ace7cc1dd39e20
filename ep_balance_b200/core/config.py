"""Solver knobs.

Every decision knob is an integer so that all ranks, solving the same load
matrix independently, take identical branches (no float compare ever decides a
placement).  Field names and defaults follow the reference's frozen dataclass
(eplb/config.py:8-42) so existing call sites keep working.
"""

from __future__ import annotations

from dataclasses import dataclass, fields

_POSITIVE = (
    "alpha",
    "beta",
    "gamma",
    "eta_milli",
    "u_min",
    "max_stage2_iters",
    "max_fast_stage2_iters",
    "stage2_stagnation_patience",
    "theta_bisect_iters",
)


@dataclass(frozen=True)
class EPLBConfig:
    """Objective weights and iteration budgets of ``min a*theta + b*phi_token + g*phi_weight``."""

    alpha: int = 1
    beta: int = 1
    gamma: int = 1
    eta_milli: int = 1000
    u_min: int = 1
    allow_cross_domain: bool = True
    max_stage2_iters: int = 4096
    max_fast_stage2_iters: int = 64
    stage2_stagnation_patience: int = 8
    stage2_patience_all_scales: bool = False
    theta_bisect_iters: int = 24

    def __post_init__(self) -> None:
        for name in _POSITIVE:
            if int(getattr(self, name)) <= 0:
                raise ValueError(f"EPLBConfig.{name} must be a positive integer")

    @property
    def eta(self) -> float:
        """``eta_milli`` as a float; reporting only."""
        return self.eta_milli / 1000.0

    @property
    def device_stage2_iters(self) -> int:
        """Repair budget per domain used by the on-device solver."""
        return min(int(self.max_stage2_iters), int(self.max_fast_stage2_iters))

    def as_dict(self) -> dict:
        return {f.name: getattr(self, f.name) for f in fields(self)}
