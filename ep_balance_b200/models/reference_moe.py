"""Plain PyTorch statement of the MoE layer math: the oracle the native kernels are tested against.

``out[t] = sum_k prob[t,k] * W2[e] @ (silu(W1g[e] x_t) * (W1u[e] x_t))`` with ``e = idx[t,k]``
(reference: tests/test_sync_free.py:45-58 single-process ground truth, grouped_mlp.py:117-137).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F_


def expert_mlp(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor) -> torch.Tensor:
    """Gated MLP with ``[out, in]`` weights: ``w1`` [2F, H] (gate rows, then up rows), ``w2`` [H, F]."""
    h = x @ w1.t()
    gate, up = h.chunk(2, dim=-1)
    return (F_.silu(gate) * up) @ w2.t()


def moe_reference(tokens: torch.Tensor, top_idx: torch.Tensor, prob: torch.Tensor, w1: torch.Tensor,
                  w2: torch.Tensor, *, compute_dtype=torch.float32) -> torch.Tensor:
    """``tokens`` [N, H]; ``top_idx``/``prob`` [N, K]; ``w1`` [E, 2F, H]; ``w2`` [E, H, F]."""
    N, K = top_idx.shape
    x = tokens.to(compute_dtype)
    out = torch.zeros_like(x)
    flat_e = top_idx.reshape(-1)
    flat_t = torch.arange(N, device=tokens.device).repeat_interleave(K)
    flat_p = prob.reshape(-1).to(compute_dtype)
    for e in torch.unique(flat_e).tolist():
        sel = (flat_e == e).nonzero(as_tuple=False).flatten()
        t = flat_t[sel]
        y = expert_mlp(x[t], w1[e].to(compute_dtype), w2[e].to(compute_dtype))
        out = out.index_add(0, t, flat_p[sel, None] * y)
    return out
