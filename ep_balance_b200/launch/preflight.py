"""Pre-launch validation of a training configuration: reject knob combinations that cannot work BEFORE any
process group, heap or kernel exists, with a message that names the knob.

    python -m ep_balance_b200.launch.preflight --nproc 8        # reads the same environment as run_train.sh

This is the counterpart of the launcher-side checks of the reference (scripts/run_real_moe.sh:148-154
knob export list, 167-203 zero-sync preflight, 240-263 router balancing / skew switches).  What differs:
the zero-sync transport here is ``EPLB_ADAPTER=fused`` (own kernels), so its preconditions are shape
divisibility rules of those kernels instead of DeepEP/NCCL version probes.
"""

from __future__ import annotations

import argparse
import os
import sys
from dataclasses import dataclass, field
from typing import Dict, List, Mapping, Optional

from .recipes import RECIPES, recipe

KNOWN_MODES = ("off", "observe", "apply")
KNOWN_ADAPTERS = ("alltoall", "padded", "fused")
KNOWN_WEIGHT_COMM = ("broadcast", "symm")
KNOWN_ROUTER_BALANCING = ("none", "aux_loss")
# reference knobs that have no meaning in this build; setting them is an error rather than a silent no-op
REMOVED_KNOBS = {
    "EPLB_DEEPEP_HYBRID": "DeepEP is not part of this build (EPLB_ADAPTER=fused is the zero-sync transport)",
    "EPLB_DEEPEP_MAX_TOKENS_PER_RANK": "DeepEP is not part of this build",
    "EPLB_DEEPEP_NUM_SMS": "DeepEP is not part of this build",
    "EPLB_GIN_FENCE": "the symmetric weight channel always fences on the device (EPLB_WEIGHT_COMM=symm)",
    "EPLB_GIN_LSA": "every peer of one NVSwitch box is load/store reachable; there is no NIC path to select",
}


@dataclass
class Preflight:
    errors: List[str] = field(default_factory=list)
    warnings: List[str] = field(default_factory=list)
    resolved: Dict[str, object] = field(default_factory=dict)

    @property
    def ok(self) -> bool:
        return not self.errors

    def report(self) -> str:
        lines = [f"[preflight] {k}={v}" for k, v in self.resolved.items()]
        lines += [f"[preflight] WARNING: {w}" for w in self.warnings]
        lines += [f"[preflight] ERROR: {e}" for e in self.errors]
        return "\n".join(lines)


def _int(env: Mapping[str, str], key: str, default: int, out: Preflight, minimum: Optional[int] = None) -> int:
    raw = env.get(key, "")
    if raw == "":
        return default
    try:
        value = int(raw)
    except ValueError:
        out.errors.append(f"{key}={raw!r} is not an integer")
        return default
    if minimum is not None and value < minimum:
        out.errors.append(f"{key}={value} must be >= {minimum}")
    return value


def check(env: Mapping[str, str], nproc: int, *, shape: Optional[Dict[str, int]] = None) -> Preflight:
    """Validate ``env`` for ``nproc`` expert-parallel ranks.  ``shape``: model shape (keys of launch/recipes.py);
    default: the recipe named by ``MODEL`` (``gpt_moe_1b``)."""
    out = Preflight()
    model = env.get("MODEL", "") or "gpt_moe_1b"
    if shape is None:
        if model not in RECIPES:
            out.errors.append(f"MODEL={model!r} is not a known recipe ({', '.join(sorted(RECIPES))})")
            return out
        shape = recipe(model, _int(env, "NUM_LAYERS", 0, out, 0))
    E, H, F, K = shape["experts"], shape["hidden"], shape["ffn"], shape["top_k"]
    out.resolved.update(model=model, layers=shape["layers"], experts=E, hidden=H, ffn=F, top_k=K, nproc=nproc)

    mode = env.get("EPLB_MODE", "apply").strip().lower()
    if mode not in KNOWN_MODES:
        out.errors.append(f"EPLB_MODE={mode!r} must be one of {', '.join(KNOWN_MODES)}")
    adapter = env.get("EPLB_ADAPTER", "fused").strip().lower() or "fused"
    if adapter in ("deepep", "deep_ep"):
        out.errors.append("EPLB_ADAPTER=deepep: DeepEP is not part of this build; EPLB_ADAPTER=fused is the zero-sync transport")
    elif adapter not in KNOWN_ADAPTERS:
        out.errors.append(f"EPLB_ADAPTER={adapter!r} must be one of {', '.join(KNOWN_ADAPTERS)}")
    for knob, why in REMOVED_KNOBS.items():
        if env.get(knob, "") != "":
            out.errors.append(f"{knob} is set, but {why}")

    if nproc < 1:
        out.errors.append(f"NPROC={nproc} must be >= 1")
        return out
    if E % nproc:
        out.errors.append(f"NPROC={nproc} does not divide the {E} experts of {model}: every rank owns the same number of experts")
        return out
    home = E // nproc
    gpn = _int(env, "GPUS_PER_NODE", nproc, out, 1)
    if gpn > 0 and nproc % gpn:
        out.errors.append(f"GPUS_PER_NODE={gpn} does not divide NPROC={nproc}: logical domains must have equal size")
    n_slot = _int(env, "EPLB_N_SLOT", home + 2, out, 1)
    if n_slot < home:
        out.errors.append(f"EPLB_N_SLOT={n_slot} is below the {home} experts every rank owns "
                          f"(EPLB_N_SLOT counts ALL slots of a rank, owned experts included)")
    elif n_slot == home and mode == "apply" and nproc > 1:
        out.warnings.append(f"EPLB_N_SLOT={n_slot} leaves no replica slot: apply mode can only re-route, not replicate")
    out.resolved.update(mode=mode, adapter=adapter, domains=nproc // gpn if gpn and nproc % gpn == 0 else 1,
                        n_slot=n_slot, replica_slots=max(0, n_slot - home))

    if _int(env, "NNODES", 1, out, 1) > 1 and adapter == "fused":
        out.errors.append("NNODES > 1: the fused transport maps every rank's symmetric heap through CUDA IPC, which spans "
                          "one node (one NVLink domain); use EPLB_ADAPTER=alltoall or padded across nodes")
    if mode == "apply" and adapter == "fused":
        if H % 64:
            out.errors.append(f"EPLB_ADAPTER=fused needs hidden % 64 == 0 (hidden={H}): the grouped GEMM moves 64-element k-blocks")
        if F % 128:
            out.errors.append(f"EPLB_ADAPTER=fused needs ffn % 128 == 0 (ffn={F}): GEMM1 pairs 128 gate and 128 up columns per tile")
        if nproc > 64:
            out.errors.append(f"EPLB_ADAPTER=fused supports at most 64 expert-parallel ranks (NPROC={nproc})")
        if n_slot > 320:
            out.errors.append(f"EPLB_ADAPTER=fused supports at most 320 expert slots per rank (EPLB_N_SLOT={n_slot})")
        for knob in ("EPLB_CHUNKS", "EPLB_OVERLAP", "EPLB_REMATERIALIZE", "EPLB_MANUAL_BWD", "EPLB_CAP", "EPLB_MAX_RECV_ROWS"):
            if env.get(knob, "") not in ("", "0"):
                out.warnings.append(f"{knob} only affects EPLB_ADAPTER=alltoall; the fused transport overlaps transfer "
                                    "and GEMM tiles inside its kernels and sizes its buffers from MoEConfig.capacity_factor")
    if mode == "apply" and adapter == "padded" and _int(env, "EPLB_PAIR_ROWS", 0, out, 0) <= 0:
        out.errors.append("EPLB_ADAPTER=padded needs EPLB_PAIR_ROWS: the rows every pair of ranks exchanges per chunk "
                          "(blocks are fixed-size so that no split size is read back from the device)")
    if mode == "apply" and adapter in ("alltoall", "padded"):
        wc = env.get("EPLB_WEIGHT_COMM", "broadcast").strip().lower() or "broadcast"
        if wc in ("gin", "nccl_gin", "devnccl"):
            wc = "symm"  # the reference's names for its device-initiated channel select ours
        if wc not in KNOWN_WEIGHT_COMM:
            out.errors.append(f"EPLB_WEIGHT_COMM={wc!r} must be one of {', '.join(KNOWN_WEIGHT_COMM)}")
        chunks = _int(env, "EPLB_CHUNKS", 1, out, 1)
        if chunks > 2:
            out.errors.append(f"EPLB_CHUNKS={chunks}: the token-chunk pipeline has one or two chunks")
        if env.get("EPLB_REMATERIALIZE", "0") not in ("", "0") and wc != "broadcast":
            out.errors.append("EPLB_REMATERIALIZE=1 re-broadcasts replica weights in backward and needs EPLB_WEIGHT_COMM=broadcast")
        if env.get("EPLB_OVERLAP", "0") not in ("", "0") and env.get("EPLB_REMATERIALIZE", "0") not in ("", "0"):
            out.errors.append("EPLB_OVERLAP=1 and EPLB_REMATERIALIZE=1 are alternatives; set one")
        out.resolved.update(weight_comm=wc, chunks=chunks)

    balancing = env.get("ROUTER_BALANCING", "none").strip().lower() or "none"
    if balancing not in KNOWN_ROUTER_BALANCING:
        out.errors.append(f"ROUTER_BALANCING={balancing!r} must be one of {', '.join(KNOWN_ROUTER_BALANCING)}")
    elif balancing != "none" and env.get("ROUTER_SKEW", "") != "":
        out.warnings.append("ROUTER_BALANCING=aux_loss flattens the routing skew that ROUTER_SKEW injects; "
                            "the balancer is then measured on an easier problem")
    out.resolved["router_balancing"] = balancing
    if env.get("ROUTER_SKEW", "") != "":
        try:
            out.resolved["router_skew"] = float(env["ROUTER_SKEW"])
            out.warnings.append("ROUTER_SKEW biases the router logits: use the run for step time and imbalance, not for the loss curve")
        except ValueError:
            out.errors.append(f"ROUTER_SKEW={env['ROUTER_SKEW']!r} is not a number")
    if env.get("EPLB_DEBUG_TIMING", "0") not in ("", "0"):
        out.warnings.append("EPLB_DEBUG_TIMING=1 synchronises once per MoE invocation: phase times are diagnostic, "
                            "throughput is perturbed")
    trace_out = env.get("EPLB_TRACE_OUT", "")
    if trace_out:
        parent = os.path.dirname(os.path.abspath(trace_out))
        if not os.path.isdir(parent):
            out.errors.append(f"EPLB_TRACE_OUT={trace_out!r}: directory {parent!r} does not exist")
    micro, seq = _int(env, "MICRO_BATCH", 4, out, 1), _int(env, "SEQ_LEN", 2048, out, 1)
    out.resolved.update(tokens_per_rank=micro * seq)
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--nproc", type=int, default=int(os.environ.get("NPROC", "1") or 1))
    a = ap.parse_args(argv)
    result = check(os.environ, a.nproc)
    print(result.report(), file=sys.stderr if not result.ok else sys.stdout, flush=True)
    return 0 if result.ok else 2


if __name__ == "__main__":
    raise SystemExit(main())
