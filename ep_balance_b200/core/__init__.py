from .config import EPLBConfig
from .loads import Loads
from .metrics import ConstraintReport, Metrics, check_constraints, compute_metrics
from .plan import Plan
from .problem import ProblemSpec
from .topology import Topology

__all__ = ["EPLBConfig", "Topology", "ProblemSpec", "Loads", "Plan", "Metrics", "ConstraintReport",
           "compute_metrics", "check_constraints"]
