"""DeepSeek-V3-shaped MoE layer stack: group-limited top-k routing, one shared expert per layer.

Routing (DeepSeek-V3): sigmoid affinities; experts are split into ``n_groups`` groups, a group's
score is the sum of its two best affinities, only the best ``topk_groups`` groups stay eligible, the
top-k experts among them are selected and their affinities normalised to sum to one.
Expert GEMMs run in bf16 on the native grouped GEMM; the block-scaled fp8 variant of the
reference's target configuration is not built in this version.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..core.config import EPLBConfig
from ..parallel.symm import SymmetricHeap
from ..utils.status import StatusBoard
from .moe_layer import FusedMoE, MoEConfig, heap_layout


def group_limited_topk(logits: torch.Tensor, n_groups: int, topk_groups: int, top_k: int,
                       routed_scale: float = 1.0):
    """``logits`` [N, E] -> ``(top_idx int64 [N, K], weights fp32 [N, K])``."""
    N, E = logits.shape
    scores = torch.sigmoid(logits.float())
    per_group = scores.view(N, n_groups, E // n_groups)
    group_score = per_group.topk(2, dim=-1).values.sum(-1)  # [N, G]
    keep = torch.zeros_like(group_score, dtype=torch.bool).scatter_(1, group_score.topk(topk_groups, dim=-1).indices, True)
    masked = torch.where(keep[:, :, None].expand_as(per_group), per_group, torch.zeros_like(per_group)).reshape(N, E)
    top_val, top_idx = masked.topk(top_k, dim=-1)
    weights = top_val / top_val.sum(-1, keepdim=True).clamp_min(1e-20) * routed_scale
    return top_idx, weights


@dataclass
class DSv3Config:
    layers: int = 4
    hidden: int = 7168
    ffn: int = 2048
    experts: int = 256
    top_k: int = 8
    n_groups: int = 8
    topk_groups: int = 4
    shared_ffn: int = 2048
    max_tokens: int = 4096
    extra_slots: int = 2
    capacity_factor: float = 2.0
    num_domains: int = 2
    fp8_inference: bool = False  # forwards without autograd use block-scaled fp8 expert GEMMs


class SharedExpert(nn.Module):
    """Dense SwiGLU MLP applied to every token (library GEMMs)."""

    def __init__(self, hidden: int, ffn: int) -> None:
        super().__init__()
        self.up = nn.Linear(hidden, 2 * ffn, bias=False)
        self.down = nn.Linear(ffn, hidden, bias=False)

    def forward(self, x):
        gate, up = self.up(x).chunk(2, dim=-1)
        return self.down(F.silu(gate) * up)


class DSv3Block(nn.Module):
    def __init__(self, cfg: DSv3Config, moe: FusedMoE) -> None:
        super().__init__()
        self.norm = nn.RMSNorm(cfg.hidden)
        self.moe = moe
        self.shared = SharedExpert(cfg.hidden, cfg.shared_ffn)
        moe.route_fn = lambda logits: group_limited_topk(logits, cfg.n_groups, cfg.topk_groups, cfg.top_k)
        moe.fused_router = dict(mode=2, n_groups=cfg.n_groups, topk_groups=cfg.topk_groups, scale=1.0)

    def forward(self, x):
        h = self.norm(x)
        return x + self.moe(h) + self.shared(h)


class DSv3Stack(nn.Module):
    """``layers`` residual MoE blocks over a flat token batch ``[tokens, hidden]`` (bf16)."""

    def __init__(self, cfg: DSv3Config, device, *, rank: int = 0, world: int = 1, group=None,
                 solver_cfg: Optional[EPLBConfig] = None) -> None:
        super().__init__()
        self.cfg, self.rank, self.world, self.group = cfg, rank, world, group
        domains = cfg.num_domains if world % max(cfg.num_domains, 1) == 0 and world >= cfg.num_domains else 1
        mcfg = MoEConfig(hidden=cfg.hidden, ffn=cfg.ffn, num_experts=cfg.experts, top_k=cfg.top_k,
                         max_tokens=cfg.max_tokens, extra_slots=cfg.extra_slots,
                         capacity_factor=cfg.capacity_factor, num_domains=domains,
                         fp8_inference=cfg.fp8_inference)
        # one symmetric allocation for the stack: per-layer state + one set of per-step scratch buffers
        self.heap = SymmetricHeap(heap_layout(mcfg, world, layers=cfg.layers), device, group=group)
        self.status = StatusBoard(cfg.layers, device)
        self._scratch: dict = {}
        blocks = []
        for layer in range(cfg.layers):
            blk = DSv3Block(cfg, FusedMoE(mcfg, self.heap, rank, world, solver_cfg=solver_cfg, seed=layer,
                                          layer_index=layer, scratch=self._scratch, status=self.status.row(layer)))
            blk.norm.to(device=device, dtype=torch.bfloat16)
            blk.shared.to(device=device, dtype=torch.bfloat16)
            blocks.append(blk)
        self.blocks = nn.ModuleList(blocks)

    def expert_parameters(self):
        for b in self.blocks:
            yield b.moe.w1
            yield b.moe.w2

    def dense_parameters(self):
        skip = {id(p) for p in self.expert_parameters()}
        return [p for p in self.parameters() if id(p) not in skip]

    def set_router_bias(self, bias: Optional[torch.Tensor]) -> None:
        for i, b in enumerate(self.blocks):
            b.moe.router_bias = None if bias is None else bias[i]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        for b in self.blocks:
            x = b(x)
        return x

    def check_status(self) -> None:
        self.status.check_now()

    def quantize_weights(self) -> None:
        """Refresh the fp8 copies of every layer's own experts (``DSv3Config.fp8_inference``); collective:
        every rank calls it, and the ranks are synchronised before the next forward reads peers' copies."""
        for b in self.blocks:
            b.moe.quantize_weights()
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(group=self.group)
