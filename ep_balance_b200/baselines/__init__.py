"""Comparison strategies and the common benchmark harness (``python -m ep_balance_b200.baselines.benchmark``)."""

from .adapters import (BaselineResult, LPLBBaseline, LPLBUnavailableError, run_deepseek_eplb, run_fastermoe,
                       run_flexmoe, run_scale_eplb, slot_budget)
from .deepseek_eplb import balanced_packing, rebalance_experts, replicate_experts
from .fastermoe import ShadowCostModel, select_shadow_experts
from .flexmoe import FlexMoECostModel, flexmoe_schedule

__all__ = [n for n in dir() if not n.startswith("_")]
