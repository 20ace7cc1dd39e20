"""DeepSeek-EPLB placement heuristic (hierarchical: groups -> nodes, replicate, pack onto GPUs).

Re-statement of the published algorithm (github.com/deepseek-ai/EPLB, MIT) on NumPy, used only as a
comparison baseline; the reference project vendors the same policy (baseline/deepseek_eplb.py:15-173).
All three public functions keep DeepSeek's names and return conventions.
"""

from __future__ import annotations

from typing import Tuple

import numpy as np
import torch


def _as_np(weight) -> np.ndarray:
    if isinstance(weight, torch.Tensor):
        return weight.detach().to("cpu", torch.float32).numpy()
    return np.asarray(weight, dtype=np.float32)  # single precision, like the published implementation


def balanced_packing(weight, num_packs: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Heaviest-first packing of ``n`` items into ``num_packs`` packs of exactly ``n/num_packs`` items.

    Returns ``(pack_index, rank_in_pack)``, both int64 ``[layers, n]``."""
    w = _as_np(weight)
    layers, n = w.shape
    if n % num_packs:
        raise ValueError("the number of objects must be divisible by num_packs")
    per = n // num_packs
    if per == 1:
        idx = np.broadcast_to(np.arange(n), (layers, n)).copy()
        return torch.from_numpy(idx), torch.zeros((layers, n), dtype=torch.int64)
    pack_index = np.full((layers, n), -1, dtype=np.int64)
    rank_in_pack = np.full((layers, n), -1, dtype=np.int64)
    for l in range(layers):
        load = [0.0] * num_packs
        used = [0] * num_packs
        for item in np.argsort(-w[l], kind="stable"):
            p = min((q for q in range(num_packs) if used[q] < per), key=load.__getitem__)
            pack_index[l, item], rank_in_pack[l, item] = p, used[p]
            load[p] += w[l, item]
            used[p] += 1
    return torch.from_numpy(pack_index), torch.from_numpy(rank_in_pack)


def replicate_experts(weight, num_physical: int):
    """Give the next replica to the expert with the largest load per replica, until ``num_physical``.

    Returns ``(phy2log [layers, P], replica_rank [layers, P], logcnt [layers, E])``."""
    w = _as_np(weight)
    layers, E = w.shape
    if num_physical < E:
        raise ValueError("num_physical must be at least num_logical")
    phy2log = np.tile(np.arange(num_physical), (layers, 1))
    rank = np.zeros((layers, num_physical), dtype=np.int64)
    cnt = np.ones((layers, E), dtype=np.int64)
    rows = np.arange(layers)
    for p in range(E, num_physical):
        e = np.argmax(w / cnt.astype(np.float32), axis=1)
        phy2log[:, p] = e
        rank[:, p] = cnt[rows, e]
        cnt[rows, e] += 1
    return torch.from_numpy(phy2log), torch.from_numpy(rank), torch.from_numpy(cnt)


def _inverse(perm: np.ndarray) -> np.ndarray:
    inv = np.empty_like(perm)
    np.put_along_axis(inv, perm, np.broadcast_to(np.arange(perm.shape[1]), perm.shape), axis=1)
    return inv


def rebalance_experts_hierarchical(weight, num_physical: int, num_groups: int, num_nodes: int, num_gpus: int):
    w = _as_np(weight)
    layers, E = w.shape
    if E % num_groups:
        raise ValueError("num_logical must be divisible by num_groups")
    if num_groups % num_nodes:
        raise ValueError("num_groups must be divisible by num_nodes")
    if num_gpus % num_nodes:
        raise ValueError("num_gpus must be divisible by num_nodes")
    if num_physical % num_gpus:
        raise ValueError("num_physical must be divisible by num_gpus")
    gsize, g_per_node, phy_per_gpu = E // num_groups, num_groups // num_nodes, num_physical // num_gpus

    # 1. expert groups -> nodes
    group_pack, group_rank = (t.numpy() for t in balanced_packing(w.reshape(layers, num_groups, gsize).sum(-1), num_nodes))
    log2mid = (((group_pack * g_per_node + group_rank) * gsize)[..., None] + np.arange(gsize)).reshape(layers, -1)
    mid2log = _inverse(log2mid)
    # 2. replicate inside each node
    per_node = np.take_along_axis(w, mid2log, axis=1).reshape(-1, E // num_nodes)
    phy2mid, rep_rank, mid_cnt = (t.numpy() for t in replicate_experts(per_node, num_physical // num_nodes))
    # 3. physical experts -> GPUs of the node
    per_phys = np.take_along_axis(per_node / mid_cnt.astype(np.float32), phy2mid, axis=1)
    gpu_pack, rank_in_gpu = (t.numpy() for t in balanced_packing(per_phys, num_gpus // num_nodes))
    packed2phy = _inverse(gpu_pack * phy_per_gpu + rank_in_gpu)
    packed2mid = np.take_along_axis(phy2mid, packed2phy, axis=1)
    packed2mid = (packed2mid.reshape(layers, num_nodes, -1)
                  + (np.arange(num_nodes) * (E // num_nodes))[None, :, None]).reshape(layers, -1)
    packed2log = np.take_along_axis(mid2log, packed2mid, axis=1)
    packed_rank = np.take_along_axis(rep_rank, packed2phy, axis=1).reshape(layers, -1)
    logcnt = np.take_along_axis(mid_cnt.reshape(layers, -1), log2mid, axis=1)
    return torch.from_numpy(packed2log), torch.from_numpy(packed_rank), torch.from_numpy(logcnt)


def rebalance_experts(weight, num_replicas: int, num_groups: int, num_nodes: int, num_gpus: int):
    """``(phy2log [L, P], log2phy [L, E, max_count] (-1 padded), logcnt [L, E])``."""
    w = _as_np(weight)
    layers, E = w.shape
    if num_groups % num_nodes == 0:
        phy2log, rank, logcnt = rebalance_experts_hierarchical(w, num_replicas, num_groups, num_nodes, num_gpus)
    else:
        phy2log, rank, logcnt = rebalance_experts_hierarchical(w, num_replicas, 1, 1, num_gpus)
    mx = int(logcnt.max())
    log2phy = torch.full((layers, E, mx), -1, dtype=torch.int64)
    log2phy.view(layers, -1).scatter_(-1, phy2log * mx + rank, torch.arange(num_replicas).expand(layers, -1))
    return phy2log, log2phy, logcnt


__all__ = ["balanced_packing", "replicate_experts", "rebalance_experts", "rebalance_experts_hierarchical"]
