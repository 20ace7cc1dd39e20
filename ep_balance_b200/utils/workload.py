"""Synthetic load matrices.

* :func:`make_loads` -- Zipf popularity with hotspot ranks (reference: sim/workload.py:10-57).
* :func:`softmax_router_loads` -- top-k without replacement from ``softmax(g/tau)`` with a
  per-rank Dirichlet perturbation (the CPU plan benchmark's generator).
* :class:`DriftingRouterSkew` -- ``g_t = 0.9 g_{t-1} + 0.1 N(0,1)`` logit bias per layer.
* :func:`tune_tau_for_imbalance` -- bisection on ``tau`` for a target expert max/mean.
"""

from __future__ import annotations

from typing import Optional

import torch

from ..core.loads import Loads


def make_loads(num_ranks: int, num_experts: int, tokens_per_rank: int = 4096, top_k: int = 8,
               skew: float = 1.2, hotspot_ranks: float = 0.25, seed: int = 0,
               device="cpu") -> Loads:
    """Zipf ``1/(i+1)^skew`` over a seeded expert permutation; non-hot ranks blend 50% uniform."""
    g = torch.Generator().manual_seed(int(seed))
    base = 1.0 / torch.arange(1, num_experts + 1, dtype=torch.float64) ** float(skew)
    base = base[torch.randperm(num_experts, generator=g)]
    base = base / base.sum()
    uniform = torch.full_like(base, 1.0 / num_experts)
    n_hot = max(1, int(round(num_ranks * float(hotspot_ranks))))
    hot = set(torch.randperm(num_ranks, generator=g)[:n_hot].tolist())
    rows = []
    for r in range(num_ranks):
        p = base if r in hot else 0.5 * base + 0.5 * uniform
        draws = torch.multinomial(p, tokens_per_rank * top_k, replacement=True, generator=g)
        rows.append(torch.bincount(draws, minlength=num_experts))
    return Loads(torch.stack(rows).to(torch.int64).to(device))


def softmax_router_loads(num_ranks: int, num_experts: int, tokens_per_rank: int = 4096, top_k: int = 6,
                         tau: float = 0.5, dirichlet_alpha: float = 5.0, seed: int = 0,
                         logits: Optional[torch.Tensor] = None, device="cpu") -> Loads:
    g = torch.Generator().manual_seed(int(seed))
    if logits is None:
        logits = torch.randn(num_experts, generator=g, dtype=torch.float64)
    p = torch.softmax(logits.to(torch.float64) / float(tau), 0)
    conc = torch.full((num_experts,), float(dirichlet_alpha), dtype=torch.float64)
    rows = []
    for _ in range(num_ranks):
        # Dirichlet via normalised Gamma draws (seeded generator)
        gam = torch._standard_gamma(conc, generator=g)
        pr = p * (gam / gam.sum()) * num_experts
        pr = pr / pr.sum()
        pick = torch.multinomial(pr.expand(tokens_per_rank, -1), top_k, replacement=False, generator=g)
        rows.append(torch.bincount(pick.flatten(), minlength=num_experts))
    return Loads(torch.stack(rows).to(torch.int64).to(device))


def expert_max_mean(omega: torch.Tensor) -> float:
    c = omega.sum(0).to(torch.float64)
    return float(c.max() / c.mean()) if float(c.mean()) > 0 else 0.0


def rank_max_mean(omega: torch.Tensor, main_rank: torch.Tensor, num_ranks: int) -> float:
    load = torch.zeros(num_ranks, dtype=torch.float64)
    load.index_add_(0, main_rank.cpu(), omega.sum(0).to(torch.float64).cpu())
    return float(load.max() / load.mean()) if float(load.mean()) > 0 else 0.0


def tune_tau_for_imbalance(target: float, num_experts: int, top_k: int, seed: int = 0,
                           samples: int = 16384, iters: int = 30) -> float:
    """Bisect ``tau`` so that top-k sampling from softmax(g/tau) has expert max/mean ~= target."""
    g = torch.Generator().manual_seed(int(seed))
    logits = torch.randn(num_experts, generator=g, dtype=torch.float64)

    def ratio(tau: float) -> float:
        gg = torch.Generator().manual_seed(int(seed) + 1)
        p = torch.softmax(logits / tau, 0)
        pick = torch.multinomial(p.expand(samples, -1), top_k, replacement=False, generator=gg)
        c = torch.bincount(pick.flatten(), minlength=num_experts).to(torch.float64)
        return float(c.max() / c.mean())

    lo, hi = 0.02, 50.0  # small tau = sharp = more imbalance
    for _ in range(iters):
        mid = (lo * hi) ** 0.5
        if ratio(mid) > target:
            lo = mid
        else:
            hi = mid
    return (lo * hi) ** 0.5


class DriftingRouterSkew:
    """Per-layer AR(1) logit bias ``g_t = rho*g_{t-1} + (1-rho)*N(0,1)`` added to router logits."""

    def __init__(self, num_layers: int, num_experts: int, rho: float = 0.9, scale: float = 1.0,
                 seed: int = 0, device="cpu") -> None:
        self.rho, self.scale = float(rho), float(scale)
        self.gen = torch.Generator().manual_seed(int(seed))
        self.device = device
        self.g = torch.randn(num_layers, num_experts, generator=self.gen)

    def step(self) -> torch.Tensor:
        self.g = self.rho * self.g + (1.0 - self.rho) * torch.randn(self.g.shape, generator=self.gen)
        return self.bias()

    def bias(self) -> torch.Tensor:
        return (self.scale * self.g).to(self.device)


def router_bias_for_imbalance(num_experts: int, top_k: int, logit_std: float, target: float = 3.5,
                              seed: int = 2024, samples: int = 32768, iters: int = 24) -> torch.Tensor:
    """Per-expert additive logit bias ``beta * g`` (``g ~ N(0,1)`` seeded) such that top-k routing of
    logits ``N(0, logit_std^2) + bias`` has expert max/mean load ~= ``target``.  Runs on the CPU and is
    deterministic, so every rank and every implementation under comparison gets the same skew."""
    g = torch.Generator().manual_seed(int(seed))
    direction = torch.randn(num_experts, generator=g)
    noise = torch.randn(samples, num_experts, generator=torch.Generator().manual_seed(int(seed) + 1)) * logit_std

    def ratio(beta: float) -> float:
        idx = (noise + beta * direction).topk(top_k, dim=-1).indices
        c = torch.bincount(idx.flatten(), minlength=num_experts).double()
        return float(c.max() / c.mean())

    lo, hi = 0.0, 8.0
    for _ in range(iters):
        mid = 0.5 * (lo + hi)
        if ratio(mid) < target:
            lo = mid
        else:
            hi = mid
    return (0.5 * (lo + hi)) * direction
