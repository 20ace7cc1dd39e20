"""R logical expert-parallel ranks on ONE GPU, for validating the multi-rank kernels.

Kernels of different ranks must never wait on one another when they share a GPU, so the cluster is
stepped phase by phase: every rank's kernel of a phase is enqueued before any kernel of the next
phase, and the stream's order stands in for the cross-rank barriers (which are skipped).  All
"peer" pointers are plain local buffers of the same process.
"""

from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from ..core.config import EPLBConfig
from ..parallel.symm import SymmetricHeap
from ..utils.status import StatusBoard
from .moe_layer import FusedMoE, MoEConfig, heap_layout


class EmulatedCluster:
    def __init__(self, cfg: MoEConfig, world: int, device="cuda:0", solver_cfg: Optional[EPLBConfig] = None,
                 seed: int = 0) -> None:
        self.cfg, self.world = cfg, world
        self.heap = SymmetricHeap(heap_layout(cfg, world), torch.device(device), backend="local",
                                  num_local_ranks=world)
        self.status = StatusBoard(world, torch.device(device))  # row r: status word of logical rank r
        self.layers: List[FusedMoE] = [
            FusedMoE(cfg, self.heap, r, world, solver_cfg=solver_cfg, multi_rank_sync=False, seed=seed,
                     status=self.status.row(r))
            for r in range(world)
        ]
        for l in self.layers[1:]:  # one router for the whole group
            l.router.data.copy_(self.layers[0].router.data)

    def full_weights(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """All experts' weights in expert order, gathered from their owners."""
        w1 = torch.cat([l.w1.detach() for l in self.layers])
        w2 = torch.cat([l.w2.detach() for l in self.layers])
        return w1, w2

    def full_grads(self) -> Tuple[torch.Tensor, torch.Tensor]:
        return (torch.cat([l.w1.grad for l in self.layers]), torch.cat([l.w2.grad for l in self.layers]))

    @torch.no_grad()
    def step(self, tokens: List[torch.Tensor], douts: List[torch.Tensor], routing=None):
        """One forward+backward of every rank.  Returns per-rank (out, dtokens, dprob, top_idx, prob)."""
        L, K = self.layers, self.cfg.top_k
        if routing is None:
            routing = [l.route_tokens(t) for l, t in zip(L, tokens)]
        n = [t.shape[0] for t in tokens]
        outs = [torch.empty_like(t) for t in tokens]
        dtok = [torch.empty_like(t) for t in tokens]
        dprob = [torch.empty_like(p) for _, p in routing]
        for l, (idx, _) , m in zip(L, routing, n):
            l.rt.publish(idx.data_ptr(), m * K)
        for l in L:
            l.rt.solve()
        for l, (idx, _), m in zip(L, routing, n):
            l.rt.route(idx.data_ptr(), m * K)
        for l, t, (_, p), m in zip(L, tokens, routing, n):
            l.rt.dispatch_tokens(t.data_ptr(), p.data_ptr(), m * K)
        for l in L:
            l.rt.pull_weights()
        for l in L:
            l.rt.gemm1()
        for l in L:
            l.rt.gemm2()
        for l, o, m in zip(L, outs, n):
            l.rt.reduce_out(o.data_ptr(), m)
        for l, d, m in zip(L, douts, n):
            l.rt.dispatch_grads(d.data_ptr(), m * K)
        for l in L:
            l.rt.dgrad2()
            l.rt.wgrad2()
            l.rt.wgrad1()
            l.rt.dgrad1()
        for l, dt, dp, m in zip(L, dtok, dprob, n):
            l.rt.reduce_dtokens(dt.data_ptr(), dp.data_ptr(), m)
        for l in L:
            l.rt.reduce_weight_grads()
        return [(outs[r], dtok[r], dprob[r], routing[r][0], routing[r][1]) for r in range(self.world)]

    @torch.no_grad()
    def forward_fp8(self, tokens: List[torch.Tensor], routing=None):
        """Inference forward of every rank with block-scaled fp8 expert GEMMs (``MoEConfig.fp8_inference``;
        call ``quantize_weights()`` on every layer first).  Returns (outputs, routing)."""
        L, K = self.layers, self.cfg.top_k
        if routing is None:
            routing = [l.route_tokens(t) for l, t in zip(L, tokens)]
        n = [t.shape[0] for t in tokens]
        outs = [torch.empty_like(t) for t in tokens]
        for l, (idx, _), m in zip(L, routing, n):
            l.rt.publish(idx.data_ptr(), m * K)
        for l in L:
            l.rt.solve()
        for l, (idx, _), m in zip(L, routing, n):
            l.rt.route(idx.data_ptr(), m * K)
        for l, t, m in zip(L, tokens, n):
            l.rt.dispatch_fp8(t.data_ptr(), m * K)
        for l in L:
            l.rt.pull_weights_fp8()
        for l in L:
            l.rt.gemm1_fp8()
            l.rt.act_fp8()
        for l in L:
            l.rt.gemm2_fp8()
        for l, (_, p), o, m in zip(L, routing, outs, n):
            l.rt.reduce_out(o.data_ptr(), m, False, p.data_ptr())
        return outs, routing
