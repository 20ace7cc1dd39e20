"""Headline benchmark: one MoE FFN layer training step (forward + backward + optimizer) with
per-step expert load balancing, bf16, expert-parallel over N GPUs of one node.

Config (fixed per GPU, i.e. weak scaling): hidden 2048, 64 experts, SwiGLU intermediate 1408, top-6
fp32 router, 8192 tokens per rank, router skew tuned to expert max/mean ~= 3.5, 2 replica slots per
rank, replica weight transfer and gradient return every step.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 20 --warmup 5
    python bench.py --impl reference ...      # the unmodified upstream package from baseline/_ref

Prints ONE JSON line on rank 0.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CFG = dict(hidden=2048, ffn=1408, num_experts=64, top_k=6, tokens_per_rank=8192, extra_slots=2,
           imbalance_target=3.5, router_std=0.02)
DOMAINS = {1: 1, 2: 1, 4: 2, 8: 2}


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--tokens", type=int, default=CFG["tokens_per_rank"])
    p.add_argument("--gemm-ctas", type=int, default=2, choices=[1, 2], help="grouped GEMM: CTA pairs (2) or single CTAs (1)")
    p.add_argument("--no-graph", action="store_true",
                   help="end-to-end loop: launch every step eagerly instead of replaying it from a CUDA graph")
    p.add_argument("--phases", action="store_true", help="also print a per-phase device-time table (stderr)")
    p.add_argument("--check", action="store_true",
                   help="before timing, run one forward+backward through the native path and compare outputs, token, "
                        "gate and the owners' weight gradients with the plain PyTorch fp32 oracle (stderr; aborts on mismatch)")
    return p.parse_args()


# ---------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []
        self.first = 0
        self.thread = None

    def mark(self) -> None:
        """Samples taken before this call (warm-up) are not reported."""
        self.first = len(self.lines)

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return

        def pump():
            for line in self.proc.stdout:
                self.lines.append(line.strip())

        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines[self.first:]:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------- shared set-up
def init_dist(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    return world, rank, local


def host_batches(tokens: int, hidden: int, rank: int, count: int = 4):
    """Pinned host batches of synthetic N(0,1) activations (bf16); cycled by the end-to-end loop."""
    import torch

    g = torch.Generator().manual_seed(777 + rank)
    return [torch.randn(tokens, hidden, generator=g).to(torch.bfloat16).pin_memory() for _ in range(count)]


def timed_loop(step_fn, steps: int, world: int, finish=None):
    """Barrier + sync, K steps between CUDA events on the current stream, sync + barrier.
    ``finish`` (optional) runs after the last step and before the closing event (drains reads that
    the loop defers by one step, so that every step's result is read inside the timed region)."""
    import torch
    import torch.distributed as dist

    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for i in range(steps):
        step_fn(i)
    if finish is not None:
        finish()
    t1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = torch.tensor([t0.elapsed_time(t1)], device="cuda")
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms) / steps


def emit(args, world, impl, ms_dev, ms_e2e, launches, clocks, h2d, d2h, quality, notes):
    """One JSON line.  ``config`` has the same keys and values in both arms; what is specific to an arm goes to
    ``quality`` (plan quality of the last step: rank load max/mean, replicas, plan digest) and ``notes``."""
    tokens_total = args.tokens * world
    line = {
        "metric": "moe_layer_train_tokens_per_s", "value": tokens_total / (ms_dev * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_dev,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": impl,
        "config": {"model": "single MoE FFN layer: hidden 2048, 64 experts, SwiGLU 1408, top-6, fp32 router",
                   "global_batch": tokens_total, "seq_len": args.tokens, "parallelism": f"ep{world}",
                   "domains": DOMAINS.get(world, 1), "replica_slots_per_rank": CFG["extra_slots"] if world > 1 else 0,
                   "step": "forward + backward + fused AdamW, plan solved every step",
                   "l2": "per-step working set (activations + expert weights) is several hundred MB, far above the 126 MB L2"},
        "quality": quality,
        "notes": notes,
        "clocks": clocks,
        "e2e": {"value": tokens_total / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------- our implementation
def run_ours(args):
    import torch
    import torch.distributed as dist

    world, rank, local = init_dist(args)
    from ep_balance_b200.models.moe_layer import FusedMoE, MoEConfig, heap_layout
    from ep_balance_b200.parallel.symm import SymmetricHeap
    from ep_balance_b200.utils.workload import router_bias_for_imbalance

    dev = torch.device("cuda", local)
    cfg = MoEConfig(hidden=CFG["hidden"], ffn=CFG["ffn"], num_experts=CFG["num_experts"], top_k=CFG["top_k"],
                    max_tokens=args.tokens, extra_slots=CFG["extra_slots"], num_domains=DOMAINS.get(world, 1),
                    gemm_ctas=args.gemm_ctas)
    heap = SymmetricHeap(heap_layout(cfg, world), dev)
    layer = FusedMoE(cfg, heap, rank, world)
    # same router on every rank
    if world > 1:
        dist.broadcast(layer.router.data, src=0)
    logit_std = CFG["router_std"] * CFG["hidden"] ** 0.5
    layer.router_bias = router_bias_for_imbalance(CFG["num_experts"], CFG["top_k"], logit_std,
                                                  CFG["imbalance_target"]).to(dev)
    from ep_balance_b200.utils.optim import FusedAdamW

    opt = FusedAdamW(layer.parameters(), lr=1e-5, capturable=True)
    batches = host_batches(args.tokens, CFG["hidden"], rank)
    dev_batches = [b.to(dev) for b in batches]
    losses_read = []

    def train_step(x):
        out = layer(x)
        loss = out.float().square().mean()
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    def step_device(i):
        x = dev_batches[i % len(dev_batches)].detach().requires_grad_(True)
        train_step(x)

    # End-to-end loop.  Inputs: the batch of step i+1 is copied host->device on a side stream while step i
    # computes (ring of DEPTH device staging buffers).  Results: the loss of every step is copied
    # device->host into pinned memory asynchronously and read by the host LAG steps later, so the host can
    # enqueue ahead of the GPU (with device-side cross-rank barriers in every step, a host that waits for
    # its own GPU each step stalls every other rank too).  The losses still outstanding at the end are
    # read before the closing event of the timed loop.
    DEPTH, LAG = 6, 4   # DEPTH >= LAG + 2: a staging slot is long consumed when its next copy is enqueued
    copy_stream = torch.cuda.Stream(device=dev)
    staging = [torch.empty_like(dev_batches[0]) for _ in range(DEPTH)]
    ready = [torch.cuda.Event() for _ in range(DEPTH)]
    consumed = [torch.cuda.Event() for _ in range(DEPTH)]
    loss_host = torch.zeros(DEPTH, dtype=torch.float32).pin_memory()
    loss_ready = [torch.cuda.Event() for _ in range(DEPTH)]
    pending = []

    def prefetch(i):
        slot = i % DEPTH
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[slot])
            staging[slot].copy_(batches[i % len(batches)], non_blocking=True)
            ready[slot].record(copy_stream)

    def read_loss(i):
        loss_ready[i % DEPTH].synchronize()
        losses_read.append(float(loss_host[i % DEPTH]))

    graphed = {"step": None}

    e2e_count = [0]

    def step_e2e(_):
        # steps are numbered across the warm-up and the timed loop: the pipeline is in its steady state when the
        # clock starts (each timed step waits for a copy issued one step earlier and issues the next one)
        i = e2e_count[0]
        e2e_count[0] += 1
        slot = i % DEPTH
        if i == 0:
            prefetch(0)
        prefetch(i + 1)
        torch.cuda.current_stream().wait_event(ready[slot])
        if graphed["step"] is not None:
            loss = graphed["step"](staging[slot])   # copies the batch into the graph's input buffer, then replays
        else:
            loss = train_step(staging[slot].detach().requires_grad_(True))
        consumed[slot].record()
        loss_host[slot:slot + 1].copy_(loss.detach().reshape(1), non_blocking=True)  # device->host, 4 bytes
        loss_ready[slot].record()
        pending.append(i)
        while len(pending) > LAG:
            read_loss(pending.pop(0))

    def finish_e2e():
        while pending:
            read_loss(pending.pop(0))

    if args.check:
        from ep_balance_b200.launch.check_multi import oracle_errors

        x = dev_batches[0]
        g = torch.Generator(device="cpu").manual_seed(4242 + rank)
        dout = torch.randn(x.shape, generator=g).to(dev, torch.bfloat16)
        with torch.no_grad():
            idx, prob = layer.route_tokens(x)
        out, dtok, dprob = torch.empty_like(x), torch.empty_like(x), torch.empty_like(prob)
        layer.rt.forward(x.data_ptr(), idx.data_ptr(), prob.data_ptr(), out.data_ptr(), x.shape[0])
        layer.rt.backward(dout.data_ptr(), dtok.data_ptr(), dprob.data_ptr(), x.shape[0])
        torch.cuda.synchronize()
        layer.check_status()
        errs = oracle_errors(layer, x, idx, prob, dout, out, dtok, dprob, rank, world)
        digests = [layer.last_plan().digest()]
        if world > 1:
            digests = [None] * world
            dist.all_gather_object(digests, layer.last_plan().digest())
        line = f"[check rank {rank}/{world}] plan_identical={len(set(digests)) == 1} " + " ".join(f"{k}={v:.2e}" for k, v in errs.items())
        print(line, file=sys.stderr, flush=True)
        if max(errs.values()) > 3e-2 or len(set(digests)) != 1:
            raise SystemExit("bench --check: the native step disagrees with the fp32 oracle: " + line)
    for ev in consumed:
        ev.record()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()  # started before the warm-up so that it is already sampling when the timed region begins
    layer.rt.reset_launches()
    for i in range(args.warmup):
        step_device(i)
    torch.cuda.synchronize()
    launches_per_step = layer.rt.launches() // max(args.warmup, 1)   # native launches of one step, counted eagerly
    layer.check_status()
    sampler.mark()
    # The end-to-end loop (the headline) is timed first and the device-only loop second: under a sustained GEMM load
    # the GPU settles at lower clocks within seconds (sw_power_cap), so whichever loop runs second reads 2-5 % slower.
    e2e_mode = "eager launches"
    if not args.no_graph:
        # The whole step (router, native forward/backward, loss, AdamW) is a fixed launch sequence: capture it
        # once and replay it, so the host cost per step is one graph launch.
        try:
            from ep_balance_b200.utils.graphs import GraphedStep

            graphed["step"] = GraphedStep(lambda x: train_step(x.detach().requires_grad_(True)), dev_batches[0])
            e2e_mode = "CUDA-graph replay of the whole step"
        except Exception as exc:  # capture is an optimisation: fall back to eager launches
            graphed["step"] = None
            torch.cuda.synchronize()
            print(f"[bench] graph capture failed, running the end-to-end loop eagerly: {exc}", file=sys.stderr)
    for i in range(max(args.warmup, 2 * DEPTH)):   # untimed: fills the staging ring twice and settles the replay
        step_e2e(i)
    finish_e2e()
    losses_read.clear()
    ms_e2e = timed_loop(step_e2e, args.steps, world, finish=finish_e2e)
    if len(losses_read) != args.steps or not all(v == v and v > 0 for v in losses_read):
        raise RuntimeError(f"end-to-end loop read {len(losses_read)} losses for {args.steps} steps: {losses_read[:4]}")
    # device-only loop: the same step on device-resident inputs, no host traffic.  It replays the captured step too
    # (eager launches after a capture would pay cross-stream synchronisation in autograd's gradient accumulation);
    # a replay launches exactly the kernels of the eager step counted above.
    if graphed["step"] is not None and launches_per_step > 0:
        ms_dev = timed_loop(lambda i: graphed["step"](dev_batches[i % len(dev_batches)]), args.steps, world)
        launches = launches_per_step * args.steps
    else:
        layer.rt.reset_launches()
        ms_dev = timed_loop(step_device, args.steps, world)
        launches = layer.rt.launches()
    clocks = sampler.stop() if rank == 0 else {}
    layer.check_status()

    if args.phases:
        if world == 1:
            phase_table(layer, dev_batches[0])
        else:
            # multi-rank: events around every phase of whole steps (barrier waits included)
            layer.rt.enable_timing(True)
            acc = {}
            for i in range(5):
                torch.cuda.synchronize()
                dist.barrier()  # start the step together: otherwise `solve` also counts the host skew between ranks
                torch.cuda.synchronize()
                layer.fused_trace_reset()
                step_device(i)
                for name, ms in layer.rt.phase_times():
                    acc.setdefault(name, []).append(ms)
                for name, us in layer.fused_trace().items():   # EPLB_TRACE_FUSED=1: inside the fused kernels
                    acc.setdefault("  " + name, []).append(us * 1e-3)
            layer.rt.enable_timing(False)
            table = torch.tensor([[sum(v) / len(v)] for v in acc.values()], device=dev)
            worst = table.clone()
            dist.all_reduce(worst, op=dist.ReduceOp.MAX)
            dist.all_reduce(table, op=dist.ReduceOp.SUM)
            if rank == 0:
                for (name, _), mean, mx in zip(acc.items(), (table / world).flatten().tolist(), worst.flatten().tolist()):
                    print(f"[phase] {name:<20} mean {mean:8.3f} ms   max over ranks {mx:8.3f} ms", file=sys.stderr)
    plan = layer.last_plan()
    loads = layer.rank_loads().float()
    quality = {"rank_load_max_over_mean": float(loads.max() / loads.mean()),
               "replicas": int(plan.x.sum()) - CFG["num_experts"], "plan_digest": plan.digest()[:16]}
    notes = {"gemm_ctas": args.gemm_ctas, "fused_transport": bool(layer.rt_config["fused_comm"]),
             "e2e_step": e2e_mode, "device_step": e2e_mode, "timed_order": "end-to-end loop first, device-only loop second",
             "e2e_loop": "input H2D prefetched on a side stream (ring of 6 staging buffers); loss D2H copied "
                         "asynchronously and read by the host four steps later, the outstanding ones before the closing event",
             "kernels": "tcgen05 grouped GEMM with transport warps (dispatch + replica pull inside GEMM1, gradient dispatch "
                        "inside Dgrad2), per-tile arrival counters, device solver, peer-load grad return, fused AdamW"}
    if rank == 0:
        emit(args, world, "ours", ms_dev, ms_e2e, launches, clocks, batches[0].numel() * 2, 4, quality, notes)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def phase_table(layer, x):
    """Device time of each native phase, measured one by one (not part of the headline number)."""
    import torch

    rt, K = layer.rt, layer.cfg.top_k
    n = x.shape[0]
    idx, prob = layer.route_tokens(x)
    out = torch.empty_like(x)
    dprob = torch.empty_like(prob)
    def psr():  # every transport draws its blocks from a ticket that publish clears: re-run it before each one
        rt.publish(idx.data_ptr(), n * K)
        rt.solve()
        rt.route(idx.data_ptr(), n * K)

    phases = [
        ("publish", lambda: rt.publish(idx.data_ptr(), n * K)), ("solve", rt.solve),
        ("route", lambda: rt.route(idx.data_ptr(), n * K)),
        ("publish+solve+route (psr)", psr),
        ("psr + dispatch", lambda: (psr(), rt.dispatch_tokens(x.data_ptr(), prob.data_ptr(), n * K))),
        ("gemm1", rt.gemm1), ("gemm2", rt.gemm2),
        ("reduce_out", lambda: rt.reduce_out(out.data_ptr(), n)),
        ("psr + dispatch_grads", lambda: (psr(), rt.dispatch_grads(out.data_ptr(), n * K))),
        ("dgrad2 + swiglu pass", rt.dgrad2), ("wgrad2", rt.wgrad2), ("wgrad1", rt.wgrad1), ("dgrad1", rt.dgrad1),
        ("reduce_dtokens", lambda: rt.reduce_dtokens(out.data_ptr(), dprob.data_ptr(), n)),
        # the one-kernel forms the step itself uses
        ("psr + dispatch+gemm1 fused", lambda: (psr(), rt.gemm1_fused(x.data_ptr(), prob.data_ptr(), n * K))),
        ("psr + dispatch_grads+dgrad2 fused", lambda: (psr(), rt.dgrad2_fused(out.data_ptr(), n * K))),
    ]
    if layer.world > 1:
        return  # phases that wait on peers cannot be timed one rank at a time
    rows = []
    for name, fn in phases:
        fn()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        fn()
        t1.record()
        torch.cuda.synchronize()
        rows.append((name, t0.elapsed_time(t1)))
    for name, ms in rows:
        print(f"[phase] {name:<16} {ms:8.3f} ms", file=sys.stderr)


# ---------------------------------------------------------------- the reference
def run_reference(args):
    from ep_balance_b200.baselines.reference_install import use_reference  # path lookup only

    ref_root = use_reference(ROOT)
    if ref_root is None:
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed (pip --target install of the reference)"}))
        return
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    world, rank, local = init_dist(args)
    if world == 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", local))
    try:
        import eplb
        from eplb.integration.eplb_manager import AllToAllAdapter, sync_free_moe_forward
        from eplb.integration.grouped_mlp import make_batched_gated_mlp, make_grouped_gated_mlp
        from eplb.integration.rebalancer import EPLBRebalancer
    except Exception as exc:  # pragma: no cover
        print(json.dumps({"impl": "reference", "unavailable": f"import failed: {type(exc).__name__}: {exc}"[:300]}))
        return
    from ep_balance_b200.utils.workload import router_bias_for_imbalance  # input generator only

    dev = torch.device("cuda", local)
    E, H, Fd, K = CFG["num_experts"], CFG["hidden"], CFG["ffn"], CFG["top_k"]
    nd = DOMAINS.get(world, 1)
    local_e = E // world
    n_slot = local_e + (CFG["extra_slots"] if world > 1 else 0)
    topo = eplb.Topology.from_nvlink_rdma(nd, world // nd, 1, 8, device=dev)
    main_rank = torch.arange(E, device=dev, dtype=torch.int64) // local_e
    spec = eplb.ProblemSpec(E, main_rank, torch.full((E,), 3 * H * Fd * 2, dtype=torch.int64, device=dev), H * 2, n_slot)
    reb = EPLBRebalancer(topo, spec, eplb.EPLBConfig(), ring_size=0)
    g = torch.Generator(device="cpu").manual_seed(1234)
    router = torch.nn.Parameter((torch.randn(E, H, generator=g) * 0.02).to(dev, torch.float32))
    ge = torch.Generator(device="cpu")
    weights_local, params = {}, [router]
    for i in range(local_e):
        e = rank * local_e + i
        ge.manual_seed(10_000 + e)
        w1 = torch.nn.Parameter((torch.randn(2 * Fd, H, generator=ge) * 0.02).to(dev, torch.bfloat16))
        w2 = torch.nn.Parameter((torch.randn(H, Fd, generator=ge) * 0.02).to(dev, torch.bfloat16))
        weights_local[e] = (w1, w2)
        params += [w1, w2]
    weight_shapes = [torch.Size((2 * Fd, H)), torch.Size((H, Fd))]
    last = {"plan": None}
    bias = router_bias_for_imbalance(E, K, CFG["router_std"] * H ** 0.5, CFG["imbalance_target"]).to(dev)
    opt = torch.optim.AdamW(params, lr=1e-5, fused=True)
    batched = make_batched_gated_mlp(True, F.silu)
    grouped = make_grouped_gated_mlp(True, F.silu)
    adapter = AllToAllAdapter()
    batches = host_batches(args.tokens, H, rank)
    dev_batches = [b.to(dev) for b in batches]
    loss_host = torch.zeros(1, dtype=torch.float32).pin_memory()
    tok_idx = torch.arange(args.tokens, device=dev, dtype=torch.int64).view(-1, 1).expand(-1, K).reshape(-1).contiguous()
    state = {"mb": 0}

    def train_step(x):
        logits = x.to(torch.float32) @ router.t() + bias
        top_val, top_idx = torch.topk(logits, K, dim=-1)
        prob = torch.softmax(top_val, dim=-1)
        unit_expert = top_idx.reshape(-1).contiguous()
        local_row = torch.bincount(unit_expert, minlength=E).to(torch.int64)
        plan = reb.rebalance(local_row, 0, state["mb"], group=None).plan
        last["plan"] = plan
        state["mb"] += 1
        out = sync_free_moe_forward(
            tokens=x, unit_token_idx=tok_idx, unit_expert=unit_expert, unit_prob=prob.reshape(-1).to(x.dtype),
            plan=plan, spec=spec, weights_local=weights_local, weight_shapes=weight_shapes,
            batched_mlp_fn=batched, grouped_mlp_fn=grouped, group=None, adapter=adapter,
            gated=True, act=F.silu, transpose_w=True)
        loss = out.float().square().mean()
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    def step_device(i):
        train_step(dev_batches[i % len(dev_batches)].detach().requires_grad_(True))

    def step_e2e(i):
        x = batches[i % len(batches)].to(dev, non_blocking=True).requires_grad_(True)
        loss = train_step(x)
        loss_host.copy_(loss.detach().reshape(1), non_blocking=False)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    try:
        for i in range(args.warmup):
            step_device(i)
        torch.cuda.synchronize()
    except Exception as exc:
        sampler.stop()
        print(json.dumps({"impl": "reference", "unavailable": f"reference step failed: {type(exc).__name__}: {exc}"[:400]}))
        return
    sampler.mark()
    # same order as the other arm: the end-to-end loop first, the device-only loop second
    for i in range(min(3, args.warmup)):
        step_e2e(i)
    ms_e2e = timed_loop(step_e2e, args.steps, world)
    ms_dev = timed_loop(step_device, args.steps, world)
    clocks = sampler.stop() if rank == 0 else {}
    if rank == 0:
        from ep_balance_b200.core.plan import Plan  # digest of the reference's plan in this repo's plan format

        rp = last["plan"]
        loads = rp.q.sum((0, 1)).float()
        quality = {"rank_load_max_over_mean": float(loads.max() / loads.mean()), "replicas": int(rp.x.sum()) - E,
                   "plan_digest": Plan(rp.x.clone(), rp.q.to(torch.int64), rp.theta).digest()[:16]}
        emit(args, world, "reference", ms_dev, ms_e2e, 0, clocks, batches[0].numel() * 2, 4, quality,
             {"path": "eplb.EPLBRebalancer.rebalance + eplb.integration.sync_free_moe_forward (AllToAllAdapter, "
                      "dist.broadcast replicas, torch._grouped_mm), unmodified from baseline/_ref; stock knobs",
              "knobs": {k: os.environ[k] for k in ("EPLB_CHUNKS", "EPLB_OVERLAP", "EPLB_MANUAL_BWD") if k in os.environ}})
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
