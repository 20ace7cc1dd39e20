"""Decoder-only GPT with MoE feed-forward blocks balanced per layer and per step.

Dense parts (embedding, RMSNorm, RoPE causal attention via PyTorch SDPA, LM head) are ordinary
PyTorch modules replicated on every rank (data parallel); every block's FFN is a
:class:`~ep_balance_b200.models.moe_layer.FusedMoE` sharded over the same ranks (expert parallel).
Shape of the reference's Megatron recipes (scripts/model_recipes.sh:36-137), without Megatron.
"""

from __future__ import annotations

import math
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


@dataclass
class GPTMoEConfig:
    vocab: int = 32000
    layers: int = 16
    hidden: int = 2048
    heads: int = 16
    ffn: int = 1024
    experts: int = 64
    top_k: int = 8
    seq_len: int = 2048
    micro_batch: int = 4
    extra_slots: int = 2
    capacity_factor: float = 2.0
    num_domains: int = 1
    rope_base: float = 10000.0
    grad_accum_dtype: Optional[torch.dtype] = None  # set for steps made of several micro-batches
    aux_loss_coeff: float = 0.0  # > 0: router load-balancing auxiliary loss (ROUTER_BALANCING=aux_loss)

    @property
    def tokens_per_rank(self) -> int:
        return self.seq_len * self.micro_batch


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        return F.rms_norm(x, (x.shape[-1],), self.weight, self.eps)


def rope_tables(seq: int, dim: int, base: float, device, dtype):
    inv = 1.0 / (base ** (torch.arange(0, dim, 2, device=device, dtype=torch.float32) / dim))
    ang = torch.outer(torch.arange(seq, device=device, dtype=torch.float32), inv)
    return ang.cos().to(dtype), ang.sin().to(dtype)


def apply_rope(x, cos, sin):
    """x [B, heads, S, D]; rotates interleaved halves."""
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat([x1 * cos - x2 * sin, x1 * sin + x2 * cos], dim=-1)


class Attention(nn.Module):
    def __init__(self, cfg: GPTMoEConfig) -> None:
        super().__init__()
        self.heads, self.dim = cfg.heads, cfg.hidden // cfg.heads
        self.qkv = nn.Linear(cfg.hidden, 3 * cfg.hidden, bias=False)
        self.proj = nn.Linear(cfg.hidden, cfg.hidden, bias=False)

    def forward(self, x, cos, sin):
        B, S, H = x.shape
        q, k, v = self.qkv(x).view(B, S, 3, self.heads, self.dim).permute(2, 0, 3, 1, 4)
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        out = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        return self.proj(out.transpose(1, 2).reshape(B, S, H))


class Block(nn.Module):
    def __init__(self, cfg: GPTMoEConfig, moe: FusedMoE) -> None:
        super().__init__()
        self.norm1, self.norm2 = RMSNorm(cfg.hidden), RMSNorm(cfg.hidden)
        self.attn, self.moe = Attention(cfg), moe

    def forward(self, x, cos, sin):
        x = x + self.attn(self.norm1(x), cos, sin)
        B, S, H = x.shape
        return x + self.moe(self.norm2(x).reshape(B * S, H)).view(B, S, H)


class GPTMoE(nn.Module):
    def __init__(self, cfg: GPTMoEConfig, device, *, rank: int = 0, world: int = 1, group=None,
                 solver_cfg: Optional[EPLBConfig] = None) -> None:
        super().__init__()
        self.cfg, self.rank, self.world, self.group = cfg, rank, world, group
        mcfg = MoEConfig(hidden=cfg.hidden, ffn=cfg.ffn, num_experts=cfg.experts, top_k=cfg.top_k,
                         max_tokens=cfg.tokens_per_rank, extra_slots=cfg.extra_slots,
                         capacity_factor=cfg.capacity_factor, num_domains=cfg.num_domains,
                         grad_accum_dtype=cfg.grad_accum_dtype, aux_loss_coeff=cfg.aux_loss_coeff)
        # one symmetric allocation (and one handle exchange) for the whole model: per-layer state plus a single
        # set of per-step scratch buffers shared by all layers; one status board for every layer's status word
        self.heap = SymmetricHeap(heap_layout(mcfg, world, layers=cfg.layers), device, group=group)
        self.status = StatusBoard(cfg.layers, device)
        self._scratch: dict = {}
        blocks = []
        for layer in range(cfg.layers):
            blocks.append(Block(cfg, FusedMoE(mcfg, self.heap, rank, world, solver_cfg=solver_cfg, seed=layer,
                                              layer_index=layer, scratch=self._scratch, status=self.status.row(layer))))
        self.embed = nn.Embedding(cfg.vocab, cfg.hidden)
        self.blocks = nn.ModuleList(blocks)
        self.norm = RMSNorm(cfg.hidden)
        self.head = nn.Linear(cfg.hidden, cfg.vocab, bias=False)
        for m in (self.embed, self.norm, self.head, *[b.norm1 for b in blocks], *[b.norm2 for b in blocks],
                  *[b.attn for b in blocks]):
            m.to(device=device, dtype=torch.bfloat16)
        for p in self.dense_parameters():
            if p.dim() > 1:
                nn.init.normal_(p, std=0.02)
        self.cos, self.sin = rope_tables(cfg.seq_len, cfg.hidden // cfg.heads, cfg.rope_base, device, torch.bfloat16)

    # ---- parameter groups ----------------------------------------------------
    def expert_parameters(self):
        for b in self.blocks:
            yield b.moe.w1
            yield b.moe.w2

    def dense_parameters(self):
        skip = {id(p) for p in self.expert_parameters()}
        return [p for p in self.parameters() if id(p) not in skip]

    def sync_dense_parameters(self) -> None:
        """Make the replicated (data-parallel) parameters identical on every rank."""
        if self.world > 1:
            for p in self.dense_parameters():
                dist.broadcast(p.data, src=0, group=self.group)

    def allreduce_dense_grads(self) -> None:
        """Average data-parallel gradients with one flat NCCL all-reduce per dtype."""
        if self.world <= 1:
            return
        by_dtype = {}
        for p in self.dense_parameters():
            if p.grad is not None:
                by_dtype.setdefault(p.grad.dtype, []).append(p.grad)
        for grads in by_dtype.values():
            flat = torch.cat([g.reshape(-1) for g in grads])
            dist.all_reduce(flat, group=self.group)
            flat /= self.world
            off = 0
            for g in grads:
                g.copy_(flat[off:off + g.numel()].view_as(g))
                off += g.numel()

    def set_router_bias(self, bias: Optional[torch.Tensor]) -> None:
        """``bias`` [layers, experts] additive router-logit skew (synthetic drift), or None."""
        for i, b in enumerate(self.blocks):
            b.moe.router_bias = None if bias is None else bias[i]

    def forward(self, ids: torch.Tensor, targets: Optional[torch.Tensor] = None):
        x = self.embed(ids)
        S = ids.shape[1]
        cos, sin = self.cos[:S], self.sin[:S]
        for b in self.blocks:
            x = b(x, cos, sin)
        logits = self.head(self.norm(x))
        if targets is None:
            return logits
        loss = F.cross_entropy(logits.float().view(-1, logits.shape[-1]), targets.reshape(-1))
        for b in self.blocks:  # router balancing pressure, when switched on
            if b.moe.aux_loss is not None:
                loss = loss + b.moe.aux_loss
        return loss

    def check_status(self) -> None:
        """Synchronous read of every layer's status word; raises :class:`MoEStatusError` if one is set."""
        self.status.check_now()

    def zero_expert_grad_accum(self) -> None:
        for b in self.blocks:
            b.moe.zero_grad_accum()

    # ---- checkpoint state ------------------------------------------------------
    def replicated_state(self) -> dict:
        """Parameters that are identical on every rank (everything but the experts), by name."""
        skip = {id(p) for p in self.expert_parameters()}
        return {n: p.detach().cpu() for n, p in self.named_parameters() if id(p) not in skip}

    def expert_state(self) -> dict:
        """This rank's own experts (the owners' copies; replica slots are transient and not saved)."""
        return {f"blocks.{i}.moe.{n}": getattr(b.moe, n).detach().cpu() for i, b in enumerate(self.blocks)
                for n in ("w1", "w2")}

    @torch.no_grad()
    def load_states(self, replicated: dict, experts: dict) -> None:
        named = dict(self.named_parameters())
        for n, t in {**replicated, **experts}.items():
            named[n].copy_(t.to(named[n].device, named[n].dtype))
