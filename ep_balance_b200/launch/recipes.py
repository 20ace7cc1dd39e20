"""Named model shapes (reference: scripts/model_recipes.sh:36-137) as plain data."""

from __future__ import annotations

from typing import Dict

RECIPES: Dict[str, Dict[str, int]] = {
    # name: layers, hidden, heads, moe ffn, experts, top-k, shared experts
    "qwen3_30b_a3b": dict(layers=48, hidden=2048, heads=32, ffn=768, experts=128, top_k=8, shared=0),
    "deepseek_v2_160e": dict(layers=60, hidden=5120, heads=128, ffn=1536, experts=160, top_k=6, shared=2),
    "glm45_air": dict(layers=46, hidden=4096, heads=96, ffn=1408, experts=128, top_k=8, shared=1),
    "gpt_moe_1b": dict(layers=16, hidden=2048, heads=16, ffn=1024, experts=64, top_k=8, shared=0),
    "dsv3_stack": dict(layers=4, hidden=7168, heads=128, ffn=2048, experts=256, top_k=8, shared=1),
    # the reference's bring-up model (scripts/run_phaseB.sh, run_phaseC.sh: 4 layers, hidden 512, 8 experts, top-2)
    "tiny": dict(layers=4, hidden=512, heads=8, ffn=512, experts=8, top_k=2, shared=0),
}


def recipe(name: str, num_layers: int = 0) -> Dict[str, int]:
    """Shape of ``name``; ``num_layers`` > 0 overrides the depth (``NUM_LAYERS`` in the reference)."""
    if name not in RECIPES:
        raise KeyError(f"unknown model recipe {name!r}; known: {sorted(RECIPES)}")
    out = dict(RECIPES[name])
    if num_layers > 0:
        out["layers"] = int(num_layers)
    return out


def expert_param_bytes(hidden: int, ffn: int, dtype_bytes: int = 2) -> int:
    """Bytes of one gated expert: gate, up and down projections."""
    return 3 * hidden * ffn * dtype_bytes


def default_n_slot(num_experts: int, ep_size: int, env_value: str = "") -> int:
    """TOTAL slots per rank: ``EPLB_N_SLOT`` when set, else ``max(2, 2 * owned experts)``."""
    if env_value:
        v = int(env_value)
        if v <= 0:
            raise ValueError("EPLB_N_SLOT must be a positive integer")
        return v
    return max(2, 2 * (num_experts // ep_size))
