"""Portable apply path on 4 gloo ranks (CPU): outputs, token/gate gradients and the owners' weight
gradients must equal a single-process loop over experts, for every execution mode
(reference strategy: tests/test_sync_free.py:177-232)."""

import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

W, E, H, F, T = 4, 8, 8, 16, 32


def _data():
    g = torch.Generator().manual_seed(1234)
    probs = torch.tensor([0.55, 0.15, 0.05, 0.05, 0.05, 0.05, 0.05, 0.05], dtype=torch.float64)
    unit_expert = torch.multinomial(probs, W * T, replacement=True, generator=g).reshape(W, T)
    unit_prob = 0.5 + torch.rand(W, T, generator=g)
    tokens = torch.randn(W, T, H, generator=g)
    w1 = torch.randn(E, 2 * F, H, generator=g) * 0.1  # [out, in], gate rows then up rows
    w2 = torch.randn(E, H, F, generator=g) * 0.1
    return unit_expert, unit_prob, tokens, w1, w2


def _truth():
    from ep_balance_b200.models.reference_moe import expert_mlp

    unit_expert, unit_prob, tokens, w1, w2 = _data()
    w1 = w1.clone().requires_grad_(True)
    w2 = w2.clone().requires_grad_(True)
    tok = tokens.clone().requires_grad_(True)
    pr = unit_prob.clone().requires_grad_(True)
    outs = []
    for r in range(W):
        res = torch.zeros(T, H)
        for t in range(T):
            e = int(unit_expert[r, t])
            res = res.index_add(0, torch.tensor([t]), pr[r, t] * expert_mlp(tok[r, t:t + 1], w1[e], w2[e]))
        outs.append(res)
    sum(o.sum() for o in outs).backward()
    return torch.stack(outs).detach(), tok.grad, pr.grad, w1.grad, w2.grad


def _worker(rank, port, mode):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.pop("EPLB_CHUNKS", None)
    dist.init_process_group("gloo", rank=rank, world_size=W)
    import torch.nn.functional as Fn

    from ep_balance_b200 import EPLBConfig, Loads, ProblemSpec, Topology, solve
    from ep_balance_b200.parallel.grouped_mlp import make_batched_gated_mlp, make_grouped_gated_mlp
    from ep_balance_b200.parallel.library_path import sync_free_moe_forward

    unit_expert, unit_prob, tokens, w1, w2 = _data()
    topo = Topology.from_nvlink_rdma(2, 2, 1, 8)
    spec = ProblemSpec.contiguous_main_placement(E, W, weight_bytes_each=100, s_tok=16, n_slot=4)
    omega = torch.stack([torch.bincount(unit_expert[r], minlength=E) for r in range(W)])
    plan = solve(Loads(omega), topo, spec, EPLBConfig())
    assert int(plan.x.sum()) > E, "test needs at least one replica"
    mine = [e for e in range(E) if int(spec.main_rank[e]) == rank]
    weights_local = {e: (w1[e].clone().requires_grad_(True), w2[e].clone().requires_grad_(True)) for e in mine}
    tok = tokens[rank].clone().requires_grad_(True)
    pr = unit_prob[rank].clone().requires_grad_(True)
    leases = []
    if mode == "overlap_chunks":       # count what the lease does: the chunks must share it
        import ep_balance_b200.parallel.library_path as lp

        class CountingLease(lp.WeightLease):
            def __init__(self, *a, **k):
                super().__init__(*a, **k)
                leases.append(self)

        lp.WeightLease = CountingLease
    adapter = None
    if mode.startswith("padded_transport"):
        from ep_balance_b200.parallel.library_path import PaddedAllToAllAdapter

        adapter = PaddedAllToAllAdapter(rows_per_pair=T)       # T units per rank: no pair can exceed it
        assert adapter.uses_padded_layout() and adapter.cap % PaddedAllToAllAdapter.ALIGN == 0
    kw = dict(rematerialize=mode == "remat", overlap=mode in ("overlap", "overlap_chunks"), adapter=adapter,
              num_chunks=2 if mode in ("chunks", "overlap_chunks", "padded_transport_chunks") else None,
              grouped_mlp_fn=None if mode in ("padded", "padded_transport_padded_experts")
              else make_grouped_gated_mlp(True, Fn.silu))
    out = sync_free_moe_forward(tokens=tok, unit_token_idx=torch.arange(T), unit_expert=unit_expert[rank],
                                unit_prob=pr, plan=plan, spec=spec, weights_local=weights_local,
                                weight_shapes=[(2 * F, H), (H, F)],
                                batched_mlp_fn=make_batched_gated_mlp(True, Fn.silu), gated=True, act=Fn.silu,
                                transpose_w=True, **kw)
    if leases:
        assert (leases[0].acquisitions, leases[0]._stacks) == (1, None), "replicas must not outlive the forward"
    out.sum().backward()
    if leases:   # one pull per pass for both chunks, one gradient return per layer call
        assert (len(leases), leases[0].acquisitions, leases[0].returns) == (1, 2, 1)
    t_out, t_tok, t_pr, t_w1, t_w2 = _truth()
    tol = dict(atol=1e-4, rtol=1e-3)
    assert torch.allclose(out.detach(), t_out[rank], **tol), float((out.detach() - t_out[rank]).abs().max())
    assert torch.allclose(tok.grad, t_tok[rank], **tol)
    assert torch.allclose(pr.grad, t_pr[rank], **tol)
    for e in mine:
        assert torch.allclose(weights_local[e][0].grad, t_w1[e], **tol), (mode, e)
        assert torch.allclose(weights_local[e][1].grad, t_w2[e], **tol), (mode, e)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("mode,port", [("plain", 6121), ("padded", 6122), ("remat", 6123), ("overlap", 6124),
                                       ("chunks", 6125), ("overlap_chunks", 6126), ("padded_transport", 6127),
                                       ("padded_transport_chunks", 6128), ("padded_transport_padded_experts", 6129)])
def test_library_path_matches_single_process_truth(mode, port):
    mp.spawn(_worker, args=(port, mode), nprocs=W, join=True)


def test_slot_tables_and_split_sizes():
    from ep_balance_b200 import Loads, ProblemSpec, Topology, solve
    from ep_balance_b200.parallel.library_path import group_sizes_by_slot, slot_tables, split_sizes
    from ep_balance_b200.utils.workload import make_loads

    topo = Topology.from_nvlink_rdma(2, 2)
    spec = ProblemSpec.contiguous_main_placement(8, 4, 100, 16, 4)
    loads = make_loads(4, 8, 64, 2, 1.5, 0.25, 3)
    plan = solve(loads, topo, spec)
    total_recv = 0
    for me in range(4):
        sent, recv, per_e = split_sizes(plan, me)
        assert int(sent.sum()) == int(loads.omega[me].sum())
        s2e, s_of_e, hosted = slot_tables(plan.x, me, 4)
        hosted_ids = [e for e in range(8) if int(plan.x[e, me])]
        assert s2e.tolist()[: len(hosted_ids)] == hosted_ids and set(s2e.tolist()[len(hosted_ids):]) <= {-1}
        assert all(int(s_of_e[e]) == i for i, e in enumerate(hosted_ids)) and hosted.tolist() == [e in hosted_ids for e in range(8)]
        gs = group_sizes_by_slot(s2e, per_e)
        assert int(gs.sum()) == int(recv.sum())
        total_recv += int(recv.sum())
    assert total_recv == int(loads.omega.sum())
