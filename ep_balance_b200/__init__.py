"""ep_balance_b200: per-micro-batch expert-parallel load balancing for MoE training on B200.

Public surface mirrors the reference package ``eplb`` (eplb/__init__.py:3-24).
"""

from .core.config import EPLBConfig
from .core.loads import Loads
from .core.metrics import ConstraintReport, Metrics, check_constraints, compute_metrics
from .core.plan import Plan
from .core.problem import ProblemSpec
from .core.topology import Topology
from .parallel.rebalancer import EPLBRebalancer
from .solver.api import solve

__all__ = ["EPLBConfig", "Topology", "ProblemSpec", "Loads", "Plan", "solve", "compute_metrics",
           "check_constraints", "Metrics", "ConstraintReport", "EPLBRebalancer"]
__version__ = "0.1.0"
