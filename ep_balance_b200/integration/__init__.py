"""Framework bindings (Megatron-Core by duck typing) and the apply/observe public surface.

Reference: eplb/integration/__init__.py:3-50.
"""

from ..parallel.comm import a2a_raw, all_to_all_single, broadcast_from_main
from ..parallel.grouped_mlp import (check_row_budget, grouped_expert_mlp, make_batched_gated_mlp, make_grouped_gated_mlp,
                                    row_budget_status)
from ..parallel.hooks import Dispatcher, NullWeightMaterializer, RebalanceResult, WeightMaterializer
from ..parallel.library_path import (AllToAllAdapter, BroadcastReplicaTransport, CommAdapter, PaddedAllToAllAdapter,
                                     ReplicaTransport, sync_free_moe_forward)
from ..parallel.physical import assign_physical, build_phys_slot_table
from ..parallel.rebalancer import EPLBRebalancer
from ..parallel.symm_weights import SymmReplicaTransport, SymmWeightReplicator, symm_weights_enabled
from .megatron import (MegatronEPLBHook, assert_plan_replicated, attach_router_observers, build_spec_for_megatron,
                       omega_row_from_routing_map, omega_row_from_topk_indices, reduce_router_counts_tp_cp,
                       setup_eplb_observer)
from .megatron_moe import (bind_eplb_to_moe_layer, bind_fused_moe_layer, eplb_moe_forward,
                           extract_local_expert_weights, find_moe_layers)
from .megatron_timing import NativeMoETimingBinding, bind_native_moe_timing

__all__ = [n for n in dir() if not n.startswith("_")]
