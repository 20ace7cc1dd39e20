"""Replica weight broadcast and gradient return bandwidth: one-sided kernels vs per-expert NCCL collectives.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29527 -m ep_balance_b200.launch.transport_bench --slots 1 2 4

Every rank owns ``--home`` experts (default weights 3 x 7168 x 2048 bf16 = 88 MB each, stored as a
``[2F, H]`` and an ``[H, F]`` tensor) and hosts ``slots`` replicas of experts owned by the next ranks
(rank r hosts one expert of each of ranks r+1 .. r+slots).  Timed with CUDA events, max over ranks:

* ``pull``      device-initiated get of the replica weights (this package's batched-get kernel)
* ``return``    gradient return: hosts stage their slot gradients, owners sum their replicas' rows with
                peer loads (``return_inbox_protocol`` = the reference's put-into-inbox + sum protocol)
* ``nccl``      what the reference's default transport does: one ``dist.broadcast`` per replicated
                expert and tensor, and one ``dist.reduce`` per expert and tensor for the gradients
                (eplb/integration/overlap.py:113-148, 203-232)

GB/s = bytes that one GPU must receive (pull) or send (return) divided by the time; the NVLink
figure to compare with is the per-direction peer bandwidth of one GPU.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def _time(fn, iters, warmup, dev):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if dist.is_initialized():
        dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    ms = torch.tensor([s.elapsed_time(e) / iters], device=dev)
    if dist.is_initialized():
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--ffn", type=int, default=2048)
    ap.add_argument("--home", type=int, default=2, help="experts owned per rank")
    ap.add_argument("--slots", type=int, nargs="*", default=[1, 2, 4])
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--skip-nccl", action="store_true")
    ap.add_argument("--json", default="")
    a = ap.parse_args(argv)
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world < 2:
        print("transport_bench needs at least two ranks")
        return 0
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    from ..parallel.onesided import SymmetricWorld
    from ..parallel.symm_weights import SymmReplicaTransport, SymmWeightReplicator

    H, F, home = a.hidden, a.ffn, a.home
    E = world * home
    shapes = [(2 * F, H), (H, F)]
    dtype = torch.bfloat16
    main_rank = torch.arange(E) // home
    per_expert = sum(torch.Size(s).numel() for s in shapes) * 2
    sw = SymmetricWorld(SymmWeightReplicator.arena_bytes(E, world, shapes, dtype, home_cap=home,
                                                            n_slot=sum(home + s for s in a.slots)), dev)
    rep = SymmWeightReplicator(sw, main_rank, shapes, dtype)
    weights_local = {rank * home + i: tuple(torch.randn(s, device=dev).to(dtype) for s in shapes) for i in range(home)}
    rows = []
    for slots in a.slots:
        if slots >= world:
            continue
        x = torch.zeros((E, world), dtype=torch.int8)
        x[torch.arange(E), main_rank] = 1
        for r in range(world):
            for k in range(1, slots + 1):
                x[((r + k) % world) * home + (k % home), r] = 1      # rank r hosts one expert of rank r+k
        n_slot = home + slots
        tr = SymmReplicaTransport(rep, x.to(dev), n_slot, weights_local)
        tr.publish()
        sw.world_fence(0)
        remote_bytes = slots * per_expert
        grads = [torch.randn((n_slot,) + s, device=dev).to(dtype) for s in shapes]

        def grad_return_inbox():
            tr.clear_inbox()
            sw.world_fence(2)
            tr.push(grads)
            sw.world_fence(3)
            tr.collect()

        def grad_return():
            tr.reduce_grads(grads)

        row = {"ranks": world, "slots": slots, "expert_mb": per_expert / 2 ** 20,
               "pull_ms": _time(lambda: tr.pull(), a.iters, a.warmup, dev),
               "pull_with_publish_and_fences_ms": _time(lambda: tr.materialize_replicas(), a.iters, a.warmup, dev),
               "return_ms": _time(grad_return, a.iters, a.warmup, dev),
               "return_inbox_protocol_ms": _time(grad_return_inbox, a.iters, a.warmup, dev)}
        row["pull_gbs"] = remote_bytes / row["pull_ms"] / 1e6
        row["return_gbs"] = remote_bytes / row["return_ms"] / 1e6
        sw.check_status()
        if not a.skip_nccl:
            replicated = [(e, int(main_rank[e])) for e in range(E) if int(x[e].sum()) > 1]
            bufs = [torch.empty(s, dtype=dtype, device=dev) for s in shapes]

            def nccl_broadcast():
                for _e, owner in replicated:
                    for b in bufs:
                        dist.broadcast(b, src=owner)

            def nccl_reduce():
                for _e, owner in replicated:
                    for b in bufs:
                        dist.reduce(b, dst=owner, op=dist.ReduceOp.SUM)

            row["nccl_broadcast_ms"] = _time(nccl_broadcast, max(a.iters // 2, 1), 1, dev)
            row["nccl_reduce_ms"] = _time(nccl_reduce, max(a.iters // 2, 1), 1, dev)
            row["nccl_broadcast_gbs"] = remote_bytes / row["nccl_broadcast_ms"] / 1e6
            row["nccl_reduce_gbs"] = remote_bytes / row["nccl_reduce_ms"] / 1e6
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
    if rank == 0 and a.json:
        with open(a.json, "w") as f:
            json.dump(rows, f, indent=1)
    torch.cuda.synchronize()
    dist.barrier()
    sw.destroy()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
