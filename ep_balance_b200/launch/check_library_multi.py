"""Multi-GPU check of the portable apply path (NCCL collectives) under both replica weight channels.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29519 -m ep_balance_b200.launch.check_library_multi

For ``EPLB_WEIGHT_COMM`` in {broadcast, symm} every rank runs ``sync_free_moe_forward`` +
backward on a skewed synthetic routing and compares outputs, token gradients, gate gradients and the
owners' weight gradients with a single-device loop over experts (fp32).  The symm channel moves the
replica weights and their gradients with this package's one-sided get/put kernels over the
symmetric heap; it also reports the achieved bandwidth of a large batched get.
Mirrors the reference's tests/test_gin_weights.py (two transports, same numbers).
"""

from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist
import torch.nn.functional as Fn


def _data(world: int, E: int, H: int, F: int, T: int):
    g = torch.Generator().manual_seed(4321)
    probs = torch.full((E,), 0.5 / (E - 1), dtype=torch.float64)
    probs[0] = 0.5
    unit_expert = torch.multinomial(probs, world * T, replacement=True, generator=g).reshape(world, T)
    unit_prob = 0.5 + torch.rand(world, T, generator=g)
    tokens = torch.randn(world, T, H, generator=g)
    w1 = torch.randn(E, 2 * F, H, generator=g) * 0.1
    w2 = torch.randn(E, H, F, generator=g) * 0.1
    return unit_expert, unit_prob, tokens, w1, w2


def _truth(rank_tokens, rank_expert, rank_prob, w1, w2, dev):
    """Loop over experts on one device, fp32."""
    from ..models.reference_moe import expert_mlp

    w1 = w1.to(dev).requires_grad_(True)
    w2 = w2.to(dev).requires_grad_(True)
    outs, toks, prs = [], [], []
    for r in range(rank_tokens.shape[0]):
        tok = rank_tokens[r].to(dev).requires_grad_(True)
        pr = rank_prob[r].to(dev).requires_grad_(True)
        res = torch.zeros_like(tok)
        for e in rank_expert[r].unique().tolist():
            sel = (rank_expert[r] == e).nonzero().flatten().to(dev)
            res = res.index_add(0, sel, pr[sel].unsqueeze(1) * expert_mlp(tok[sel], w1[e], w2[e]))
        outs.append(res)
        toks.append(tok)
        prs.append(pr)
    sum(o.sum() for o in outs).backward()
    return [o.detach() for o in outs], [t.grad for t in toks], [p.grad for p in prs], w1.grad, w2.grad


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--hidden", type=int, default=64)
    ap.add_argument("--ffn", type=int, default=128)
    ap.add_argument("--tokens", type=int, default=256)
    ap.add_argument("--bandwidth-mb", type=int, default=256, help="size of the batched-get bandwidth probe (0: skip)")
    a = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    from .. import EPLBConfig, Loads, ProblemSpec, Topology, solve
    from ..parallel.grouped_mlp import make_batched_gated_mlp, make_grouped_gated_mlp
    from ..parallel.library_path import sync_free_moe_forward
    from ..parallel.overlap import close_channels
    from ..parallel.symm_weights import clear_replicators

    E, H, F, T = a.experts, a.hidden, a.ffn, a.tokens
    unit_expert, unit_prob, tokens, w1, w2 = _data(world, E, H, F, T)
    topo = Topology.from_nvlink_rdma(1, world, 1, 8)
    n_slot = E // world + 2
    spec = ProblemSpec.contiguous_main_placement(E, world, weight_bytes_each=3 * H * F * 4, s_tok=H * 4, n_slot=n_slot)
    omega = torch.stack([torch.bincount(unit_expert[r], minlength=E) for r in range(world)])
    plan = solve(Loads(omega), topo, spec, EPLBConfig()).to(dev)
    spec = spec.to(dev)
    replicas = int(plan.x.sum()) - E
    t_out, t_tok, t_pr, t_w1, t_w2 = _truth(tokens, unit_expert, unit_prob, w1, w2, dev)
    mine = [e for e in range(E) if int(spec.main_rank[e]) == rank]

    ok = replicas > 0
    # every weight channel x every way of holding the replicas; on GPUs the token all-to-alls run on a comm
    # stream and the weight traffic on a stream (and, for broadcasts, a communicator) of its own
    from ..parallel.library_path import PaddedAllToAllAdapter

    modes = {"held": dict(), "held, 2 chunks": dict(num_chunks=2), "leased, 2 chunks": dict(overlap=True, num_chunks=2),
             "recomputed": dict(rematerialize=True),
             # fixed-size blocks per rank pair: no split size is read back from the device
             "held, padded transport": dict(adapter=PaddedAllToAllAdapter(rows_per_pair=T)),
             "leased, 2 chunks, padded transport": dict(overlap=True, num_chunks=2, adapter=PaddedAllToAllAdapter(rows_per_pair=T))}
    for channel in ("broadcast", "symm"):
        os.environ["EPLB_WEIGHT_COMM"] = channel
        for mode, kw in modes.items():
            weights_local = {e: (w1[e].to(dev).requires_grad_(True), w2[e].to(dev).requires_grad_(True)) for e in mine}
            tok = tokens[rank].to(dev).requires_grad_(True)
            pr = unit_prob[rank].to(dev).requires_grad_(True)
            out = sync_free_moe_forward(tokens=tok, unit_token_idx=torch.arange(T, device=dev),
                                        unit_expert=unit_expert[rank].to(dev), unit_prob=pr, plan=plan, spec=spec,
                                        weights_local=weights_local, weight_shapes=[(2 * F, H), (H, F)],
                                        batched_mlp_fn=make_batched_gated_mlp(True, Fn.silu),
                                        grouped_mlp_fn=None, gated=True, act=Fn.silu, transpose_w=True, **kw)
            out.sum().backward()
            torch.cuda.synchronize()
            tol = dict(atol=2e-4, rtol=2e-3)
            good = torch.allclose(out.detach(), t_out[rank], **tol) and torch.allclose(tok.grad, t_tok[rank], **tol) \
                and torch.allclose(pr.grad, t_pr[rank], **tol)
            for e in mine:
                good = good and torch.allclose(weights_local[e][0].grad, t_w1[e], **tol) \
                    and torch.allclose(weights_local[e][1].grad, t_w2[e], **tol)
            print(f"[rank {rank}] weight channel {channel}, replicas {mode}: {'PASS' if good else 'FAIL'} "
                  f"replicas={replicas}", flush=True)
            ok = ok and good

    if a.bandwidth_mb > 0 and world > 1:
        from ..parallel.onesided import SymmetricWorld

        nbytes = a.bandwidth_mb << 20
        sw = SymmetricWorld(nbytes + 4096, dev)
        src = sw.create_tensor((nbytes,), torch.uint8)
        src.fill_(rank + 1)
        dst = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
        peer = (rank + 1) % world
        chunk = nbytes // 16
        desc = torch.tensor([[peer, sw.offset_of(src) + i * chunk, i * chunk, chunk] for i in range(16)],
                            dtype=torch.int64, device=dev)
        sw.world_fence(0)
        for bulk in (True, False):
            sw.use_bulk = bulk
            for _ in range(3):
                sw.get_batched(dst, desc, blocks=16)
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            for _ in range(5):
                sw.get_batched(dst, desc, blocks=16)
            end.record()
            torch.cuda.synchronize()
            ms = torch.tensor([start.elapsed_time(end) / 5], device=dev)
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            right = bool((dst == peer + 1).all())
            ok = ok and right
            if rank == 0:
                print(f"batched get of {a.bandwidth_mb} MiB from the next rank, {'bulk-async' if bulk else 'vector'} "
                      f"copies: {float(ms):.3f} ms (max over ranks) = {nbytes / float(ms) / 1e6:.1f} GB/s "
                      f"per GPU, data {'ok' if right else 'WRONG'}", flush=True)
        sw.check_status()
        sw.world_fence(1)
        torch.cuda.synchronize()
        dist.barrier()
        sw.destroy()

    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("CHECK_LIBRARY_MULTI " + ("PASS" if int(flag) else "FAIL"), flush=True)
    torch.cuda.synchronize()
    dist.barrier()
    clear_replicators()
    close_channels()
    dist.destroy_process_group()
    return 0 if int(flag) else 1


if __name__ == "__main__":
    raise SystemExit(main())
