"""AdamW whose update is one native kernel launch per parameter tensor.

Expert weights of :class:`~ep_balance_b200.models.moe_layer.FusedMoE` are two flat bf16 tensors
per layer, so the whole expert update is two launches.  Moments are kept in the parameter's dtype
(the convention of ``torch.optim.AdamW(fused=True)``).  No host synchronisation: the step count
lives on the host and enters the kernel as two bias-correction scalars.  With ``capturable=True`` the step
count lives on the device instead and the kernel derives the bias corrections itself, so ``step()`` can be
captured in a CUDA graph and replayed.

``guard`` (an int32 ``[n, 4]`` tensor of device status words, e.g. ``StatusBoard.words``) contains a damaged
step: while any word is set the kernel leaves parameter and moments untouched, so a step in which rows
were dropped or a peer's data did not arrive never reaches the weights; the host raises a step or two
later (``ep_balance_b200.utils.status.StatusMonitor``).
"""

from __future__ import annotations

from typing import Iterable, Optional

import torch

from ..ops.extension import load


class FusedAdamW(torch.optim.Optimizer):
    def __init__(self, params: Iterable[torch.nn.Parameter], lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 1e-2, capturable: bool = False, guard: Optional[torch.Tensor] = None) -> None:
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self._ext = load()
        self.capturable = bool(capturable)
        self.guard = guard

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                # Megatron convention: an fp32 ``main_grad`` accumulated over micro-batches wins over ``.grad``
                grad = getattr(p, "main_grad", None)
                if grad is None:
                    grad = p.grad
                if grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"] = torch.zeros((), dtype=torch.int64, device=p.device) if self.capturable else 0
                    st["exp_avg"] = torch.zeros_like(p, memory_format=torch.contiguous_format)
                    st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.contiguous_format)
                st["step"] += 1
                if self.capturable:
                    self._ext.adamw_step(p.data, grad.contiguous(), st["exp_avg"], st["exp_avg_sq"], group["lr"], b1, b2,
                                         group["eps"], group["weight_decay"], 1, st["step"], self.guard)
                else:
                    self._ext.adamw_step(p.data, grad.contiguous(), st["exp_avg"], st["exp_avg_sq"], group["lr"], b1, b2,
                                         group["eps"], group["weight_decay"], st["step"], None, self.guard)
        return loss
