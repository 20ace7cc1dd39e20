"""Training entry point: GPT-MoE on synthetic tokens with per-layer drifting router skew.

    python -m ep_balance_b200.launch.train_gpt_moe --layers 2 --steps 5                    # one GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29521 -m ep_balance_b200.launch.train_gpt_moe --steps 20

Environment knobs kept from the reference launcher (scripts/run_real_moe.sh:148-154,
scripts/pretrain_eplb_moe.py:100-176):

``EPLB_MODE=off|observe|apply``
    ``apply`` (default) balances every layer every micro-batch with replicas; ``off`` gives every rank
    zero replica slots (plain expert parallelism); ``observe`` trains like ``off`` but solves the plan
    each layer would have used and logs ``[EPLB] layer= mb= theta= imbalance= replicas= phi_token=``.
``EPLB_N_SLOT``          TOTAL expert slots per rank (default: owned experts + 2)
``GPUS_PER_NODE``        ranks per logical topology domain
``ROUTER_SKEW``          scale of the drifting router-logit bias
``ROUTER_BALANCING``     none (default) | aux_loss: auxiliary load-balancing loss on every router (``ROUTER_AUX_COEFF``)
``EPLB_TRACE_OUT/MAX/EVERY``  routing trace (format v3) written by rank 0
``EPLB_LOG=1``           print the ``[EPLB]`` line in apply mode too (one host read per layer)

``--num-micro-batches`` accumulates gradients over several micro-batches per optimizer step (expert
weight gradients in an fp32 ``main_grad``).  ``--heartbeat-file`` turns on host-side failure detection (``parallel/health.py``).
``--save/--load/--save-interval`` checkpoint the owners'
weights, optimizer state, data and skew generators; resuming reproduces the uninterrupted run.
Iteration lines use Megatron's format so ``ep_balance_b200.eval.extract_train_metrics`` parses them.
"""

from __future__ import annotations

import argparse
import os
import time

import torch
import torch.distributed as dist


def _flops_per_step(a, tokens: int) -> float:
    """Model FLOPs of one optimizer step over ``tokens`` tokens (forward + backward = 3x forward)."""
    H, S = a.hidden, a.seq_len
    attn = 4 * 2 * H * H + 2 * 2 * S * H // 2          # qkv+out projections, causal QK^T and PV
    moe = a.top_k * 3 * 2 * H * a.ffn + 2 * H * a.experts
    per_token = a.layers * (attn + moe) + 2 * H * a.vocab
    return 3.0 * per_token * tokens


def main(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--model", default=os.environ.get("MODEL", ""),
                   help="named shape from launch/recipes.py (qwen3_30b_a3b, deepseek_v2_160e, glm45_air, gpt_moe_1b); "
                        "sets layers/hidden/heads/ffn/experts/top-k, NUM_LAYERS overrides the depth")
    p.add_argument("--layers", type=int, default=16)
    p.add_argument("--hidden", type=int, default=2048)
    p.add_argument("--heads", type=int, default=16)
    p.add_argument("--ffn", type=int, default=1024)
    p.add_argument("--experts", type=int, default=64)
    p.add_argument("--top-k", type=int, default=8)
    p.add_argument("--vocab", type=int, default=32000)
    p.add_argument("--seq-len", type=int, default=2048)
    p.add_argument("--micro-batch", type=int, default=4)
    p.add_argument("--num-micro-batches", type=int, default=1)
    p.add_argument("--steps", type=int, default=10)
    p.add_argument("--lr", type=float, default=1e-4)
    p.add_argument("--log-every", type=int, default=1)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--skip-train", action="store_true",
                   help="no optimizer steps: run --eval-iters forward passes of the (loaded) model, e.g. to capture "
                        "a routing trace of a frozen checkpoint with EPLB_MODE=observe and EPLB_TRACE_OUT")
    p.add_argument("--eval-iters", type=int, default=10)
    p.add_argument("--data", default="", help="prefix of a token dataset written by launch/prepare_data.py "
                                                "(default: uniform-random token ids)")
    p.add_argument("--save", default="", help="checkpoint directory to write")
    p.add_argument("--load", default="", help="checkpoint directory to resume from (newest complete step)")
    p.add_argument("--save-interval", type=int, default=0, help="save every N steps (0: only at the end when --save is set)")
    p.add_argument("--capacity-factor", type=float, default=2.0,
                   help="receive-buffer rows per rank as a multiple of its own routed units; a rank that receives more "
                        "sets the overflow status, the step is not applied and the run stops")
    p.add_argument("--heartbeat-file", default="",
                   help="path of a shared file store: ranks publish a heartbeat per step, refuse to launch a step "
                        "when a peer is stale or reported a failure, and publish their own device status errors")
    a = p.parse_args(argv)
    if a.model:
        from .recipes import recipe

        shape = recipe(a.model, int(os.environ.get("NUM_LAYERS", "0") or 0))
        a.layers, a.hidden, a.heads, a.ffn = shape["layers"], shape["hidden"], shape["heads"], shape["ffn"]
        a.experts, a.top_k = shape["experts"], shape["top_k"]

    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    from .. import EPLBConfig, Loads, compute_metrics
    from ..core.trace import TraceWriter, build_trace_meta
    from ..models.gpt_moe import GPTMoE, GPTMoEConfig
    from ..parallel.rebalancer import EPLBRebalancer
    from ..utils.checkpoint import load_checkpoint, save_checkpoint
    from ..utils.optim import FusedAdamW
    from ..utils.workload import DriftingRouterSkew
    from .recipes import default_n_slot

    mode = os.environ.get("EPLB_MODE", "apply").strip().lower()
    if mode not in ("off", "observe", "apply"):
        raise SystemExit("EPLB_MODE must be off, observe or apply")
    home = a.experts // world
    n_slot_total = int(os.environ.get("EPLB_N_SLOT", "0") or 0) or (home + 2)
    extra = max(0, n_slot_total - home) if (mode == "apply" and world > 1) else 0
    gpn = int(os.environ.get("GPUS_PER_NODE", str(world)) or world)
    domains = world // gpn if gpn > 0 and world % gpn == 0 else 1
    M = max(1, a.num_micro_batches)
    # ROUTER_BALANCING=none (default) leaves the routing skew intact for the balancer; aux_loss adds the usual
    # auxiliary loss (coefficient ROUTER_AUX_COEFF, default 1e-2), which flattens the skew at its source
    balancing = os.environ.get("ROUTER_BALANCING", "none").strip().lower() or "none"
    if balancing not in ("none", "aux_loss"):
        raise SystemExit("ROUTER_BALANCING must be none or aux_loss")
    aux_coeff = float(os.environ.get("ROUTER_AUX_COEFF", "1e-2")) if balancing == "aux_loss" else 0.0
    cfg = GPTMoEConfig(vocab=a.vocab, layers=a.layers, hidden=a.hidden, heads=a.heads, ffn=a.ffn, experts=a.experts,
                       top_k=a.top_k, seq_len=a.seq_len, micro_batch=a.micro_batch, extra_slots=extra,
                       capacity_factor=a.capacity_factor,
                       num_domains=max(domains, 1), grad_accum_dtype=torch.float32 if M > 1 else None,
                       aux_loss_coeff=aux_coeff)
    torch.manual_seed(a.seed)
    model = GPTMoE(cfg, dev, rank=rank, world=world)
    model.sync_dense_parameters()
    # both optimizers skip their update on the device while any layer's status word is set
    dense_opt = FusedAdamW(model.dense_parameters(), lr=a.lr, guard=model.status.words)
    expert_opt = FusedAdamW(list(model.expert_parameters()), lr=a.lr, guard=model.status.words)
    skew = DriftingRouterSkew(a.layers, a.experts, rho=0.9, scale=float(os.environ.get("ROUTER_SKEW", "1.0")),
                              seed=a.seed, device=dev)
    gen = torch.Generator(device="cpu").manual_seed(1000 + rank)
    dataset = None
    if a.data:
        from ..utils.data import TokenDataset

        dataset = TokenDataset(a.data)
        if dataset.meta["vocab_size"] > a.vocab:
            raise SystemExit(f"--vocab {a.vocab} is smaller than the dataset's vocabulary {dataset.meta['vocab_size']}")
    start_step = 0
    if a.load:
        start_step, rep, shard = load_checkpoint(a.load, rank=rank, world=world)
        model.load_states(rep["model"], shard["model"])
        dense_opt.load_state_dict(rep["dense_opt"])
        expert_opt.load_state_dict(shard["expert_opt"])
        skew.g = rep["skew_g"]
        skew.gen.set_state(rep["skew_rng"])
        gen.set_state(shard["data_rng"])

    def save(step: int) -> None:
        # a step that ran with a non-zero status skipped its expert update; never write such a state down silently
        monitor.drain()
        model.check_status()
        save_checkpoint(a.save, step, rank=rank, world=world,
                        replicated={"model": model.replicated_state(), "dense_opt": dense_opt.state_dict(),
                                    "skew_g": skew.g.clone(), "skew_rng": skew.gen.get_state(), "args": vars(a)},
                        sharded={"model": model.expert_state(), "expert_opt": expert_opt.state_dict(),
                                 "data_rng": gen.get_state()})

    # ---- observer: plan that WOULD be used (observe) or WAS used (apply, EPLB_LOG=1), plus the trace
    want_log = mode == "observe" or os.environ.get("EPLB_LOG", "0") not in ("", "0")
    trace_out = os.environ.get("EPLB_TRACE_OUT", "")
    moe0 = model.blocks[0].moe
    obs_spec = moe0.spec if mode == "apply" else \
        type(moe0.spec).contiguous_main_placement(a.experts, world, 3 * a.hidden * a.ffn * 2, a.hidden * 2,
                                                  max(n_slot_total, home))
    observer = EPLBRebalancer(moe0.topo.to(dev), obs_spec.to(dev), EPLBConfig(), ring_size=0) \
        if mode == "observe" and world > 1 else None
    trace = None
    if trace_out and rank == 0:
        trace = TraceWriter(trace_out, build_trace_meta(moe0.topo, obs_spec), every=int(os.environ.get("EPLB_TRACE_EVERY", "25") or 25),
                            max_samples=int(os.environ.get("EPLB_TRACE_MAX", "0") or 0))

    def observe(step: int, mb: int) -> None:
        if not (want_log or trace is not None) or rank != 0:
            return
        for li, b in enumerate(model.blocks):
            omega = b.moe.omega().to(torch.int64)
            if trace is not None:
                trace.add(li, mb, omega.cpu())
            if not want_log:
                continue
            if observer is not None:
                plan = observer.plan_from_omega(Loads(omega))
            else:
                plan = b.moe.last_plan()
            m = compute_metrics(plan.to("cpu"), Loads(omega.cpu()), moe0.topo, obs_spec, EPLBConfig())
            print(f"[EPLB] layer={li} mb={mb} theta={m.theta} imbalance={m.imbalance:.3f} "
                  f"replicas={m.total_replicas} phi_token={m.phi_token}", flush=True)

    n_params = sum(p.numel() for p in model.dense_parameters()) + sum(p.numel() for p in model.expert_parameters()) * world
    if rank == 0:
        print(f"Total number of parameters in billions: {n_params / 1e9:.2f}", flush=True)
        print(f"[ep_balance_b200] mode={mode} world={world} domains={cfg.num_domains} extra_slots={extra} "
              f"micro_batches={M} resume_step={start_step}", flush=True)

    from ..utils.status import StatusMonitor

    monitor = StatusMonitor(model.status.words)
    guard = None
    if a.heartbeat_file:
        from ..parallel.health import Heartbeat, StepGuard

        hb = Heartbeat(dist.FileStore(a.heartbeat_file, world), rank, world, stale_after_s=120.0)
        hb.beat(start_step)
        hb.wait_for_all(300.0)
        guard = StepGuard(hb, [model.check_status], check_every=10)
    if a.skip_train:
        # frozen-checkpoint capture (reference: eval/run_expert_hotspot.sh:1-117): forward only, no skew drift
        with torch.no_grad():
            for it in range(1, a.eval_iters + 1):
                if dataset is not None:
                    ids = dataset.sample_batch(a.micro_batch, a.seq_len, gen).to(dev)
                else:
                    ids = torch.randint(0, a.vocab, (a.micro_batch, a.seq_len + 1), generator=gen).to(dev)
                loss = model(ids[:, :-1], ids[:, 1:])
                observe(it, 0)
                if rank == 0:
                    print(f" evaluation iteration {it:6d}/{a.eval_iters:6d} | lm loss: {float(loss):.6E} |", flush=True)
        if trace is not None:
            trace.flush()
        model.check_status()
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return 0
    gbs = a.micro_batch * world * M
    flops = _flops_per_step(a, a.micro_batch * a.seq_len * M)
    if world > 1:
        dist.barrier()  # start together: device-side waits on the other ranks are bounded
    for step in range(start_step + 1, a.steps + 1):
        if guard is not None:
            guard.before_step(step)
        bias = skew.step()
        t0 = time.perf_counter()
        if M > 1:
            model.zero_expert_grad_accum()
        total = torch.zeros((), device=dev)
        for mb in range(M):
            if dataset is not None:
                ids = dataset.sample_batch(a.micro_batch, a.seq_len, gen).to(dev, non_blocking=True)
            else:
                ids = torch.randint(0, a.vocab, (a.micro_batch, a.seq_len + 1), generator=gen).to(dev, non_blocking=True)
            model.set_router_bias(bias)
            loss = model(ids[:, :-1], ids[:, 1:]) / M
            loss.backward()
            total += loss.detach()
            observe(step, mb)
        model.allreduce_dense_grads()
        gn = torch.nn.utils.clip_grad_norm_(model.dense_parameters(), 1.0)
        dense_opt.step()
        expert_opt.step()      # skipped on the device while any layer's status word is set
        dense_opt.zero_grad(set_to_none=True)
        monitor.poll()         # asynchronous copy of the status words; raises for a step seen damaged (one or two steps late)
        if step % a.log_every == 0:
            torch.cuda.synchronize()
            monitor.drain()
            ms = (time.perf_counter() - t0) * 1e3
            lv = total.clone()
            if world > 1:
                dist.all_reduce(lv)
                lv /= world
            if rank == 0:
                loads = torch.stack([b.moe.rank_loads().float() for b in model.blocks])
                imb = float((loads.max(1).values / loads.mean(1).clamp_min(1)).mean())
                print(f" iteration {step:8d}/{a.steps:8d} | consumed samples: {step * gbs:12d} | "
                      f"elapsed time per iteration (ms): {ms:.1f} | throughput per GPU (TFLOP/s/GPU): {flops / ms / 1e9:.1f} | "
                      f"learning rate: {a.lr:.6E} | global batch size: {gbs:5d} | lm loss: {float(lv):.6E} | "
                      f"grad norm: {float(gn):.3f} | rank load max/mean: {imb:.3f} |", flush=True)
        if guard is not None:
            guard.after_step(step)
        if a.save and a.save_interval > 0 and step % a.save_interval == 0 and step != a.steps:
            save(step)
    if a.save:
        save(a.steps)
    if trace is not None:
        trace.flush()
    monitor.drain()
    model.check_status()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
