"""Block-scaled fp8 (e4m3) operands and the grouped GEMM that consumes them.

DeepSeek-V3 recipe: activations carry one scale per 1 x 128 block, weights one per 128 x 128 block.
Scales are powers of two kept as biased exponent bytes (UE8M0), the format the Blackwell tensor core
applies by itself (``tcgen05.mma.kind::mxf8f6f4.block_scale``), in the 512-byte chunk layout described
in ``csrc/grouped_gemm_fp8.h``.  The reference has no fp8 path; its expert GEMMs are bf16
``torch._grouped_mm`` (eplb/integration/grouped_mlp.py:88-114).

``dequantize_*`` restate the formats in plain PyTorch; the tests use them as the fp32 oracle.
"""

from __future__ import annotations

from typing import Tuple

import torch

from .extension import load


def _kgroups(K: int) -> int:
    return (K // 128 + 3) // 4


def quantize_rows(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 ``[rows, K]`` -> (e4m3 bytes ``[rows, K]``, scales ``[rows/128, kgroups, 512]``)."""
    rows, K = x.shape
    q = torch.empty((rows, K), dtype=torch.uint8, device=x.device)
    sfa = torch.zeros((rows // 128, _kgroups(K), 512), dtype=torch.uint8, device=x.device)
    load().quantize_rows(x.contiguous(), q, sfa)
    return q, sfa


def quantize_weights(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 ``[slots, N, K]`` -> (e4m3 bytes, scales ``[slots, N/128, kgroups, 512]``)."""
    S, N, K = w.shape
    q = torch.empty((S, N, K), dtype=torch.uint8, device=w.device)
    sfb = torch.zeros((S, N // 128, _kgroups(K), 512), dtype=torch.uint8, device=w.device)
    load().quantize_weights(w.contiguous(), q, sfb)
    return q, sfb


def grouped_gemm_fp8(aq, sfa, bq, sfb, out, group_off, group_rows, group_wslot, totals, status, num_sms=None,
                     ctas: int = 1) -> None:
    """``out[rows of group g] = dequant(aq) @ dequant(bq[group_wslot[g]])^T`` (bf16 out, fp32 accumulate).
    ``ctas=2`` runs the CTA-pair kernel (256 x 128 tiles; groups must start on multiples of 256 rows)."""
    if num_sms is None:
        num_sms = torch.cuda.get_device_properties(aq.device).multi_processor_count
    load().grouped_gemm_fp8(aq, sfa, bq, sfb, out, group_off, group_rows, group_wslot, totals, status, int(num_sms),
                            int(ctas))


# ---------------------------------------------------------------------- plain PyTorch restatement
def _chunk_index(r: torch.Tensor, kb: torch.Tensor) -> torch.Tensor:
    return (r % 32) * 16 + (r // 32) * 4 + kb % 4


def row_scale_exponents(sfa: torch.Tensor, rows: int, K: int) -> torch.Tensor:
    """Biased exponent bytes ``[rows, K/128]`` read out of the chunk layout."""
    kblocks = K // 128
    r = torch.arange(rows, device=sfa.device).view(-1, 1)
    kb = torch.arange(kblocks, device=sfa.device).view(1, -1)
    flat = sfa.reshape(-1)
    idx = ((r // 128) * sfa.shape[1] + kb // 4) * 512 + _chunk_index(r % 128, kb)
    return flat[idx]


def dequantize_rows(q: torch.Tensor, sfa: torch.Tensor) -> torch.Tensor:
    rows, K = q.shape
    e = row_scale_exponents(sfa, rows, K).to(torch.float32) - 127.0
    vals = q.view(torch.float8_e4m3fn).to(torch.float32).view(rows, K // 128, 128)
    return (vals * torch.exp2(e).unsqueeze(-1)).view(rows, K)


def dequantize_weights(q: torch.Tensor, sfb: torch.Tensor) -> torch.Tensor:
    S, N, K = q.shape
    kblocks = K // 128
    n = torch.arange(N, device=q.device).view(-1, 1)
    kb = torch.arange(kblocks, device=q.device).view(1, -1)
    idx = ((n // 128) * sfb.shape[2] + kb // 4) * 512 + _chunk_index(n % 128, kb)          # [N, kblocks]
    per_slot = sfb.shape[1] * sfb.shape[2] * 512
    flat = sfb.reshape(S, per_slot)
    e = flat[:, idx.reshape(-1)].view(S, N, kblocks).to(torch.float32) - 127.0
    vals = q.view(torch.float8_e4m3fn).to(torch.float32).view(S, N, kblocks, 128)
    return (vals * torch.exp2(e).unsqueeze(-1)).view(S, N, K)
