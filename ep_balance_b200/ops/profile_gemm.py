"""Small stand-alone workload for profiling the grouped GEMM kernel, one launch per mode.

    python -m ep_balance_b200.ops.profile_gemm [--rows 2048] [--groups 8] [--modes fwd1,dgrad2,wgrad]

Operands exceed the L2 (A 64 MB, weights 92 MB, outputs 138 MB with the defaults) but the process
holds well under 1 GB, so a full-metric capture finishes quickly.  Prints device time and TFLOP/s
per mode (CUDA events, after one warm-up launch each).
"""

from __future__ import annotations

import argparse

import torch

from .extension import load

MODE = dict(fwd1=0, fwd2=1, dgrad2=2, dgrad1=3, wgrad=4, plain=5)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=2048, help="rows per group")
    ap.add_argument("--groups", type=int, default=8)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--ffn", type=int, default=1408)
    ap.add_argument("--modes", default="fwd1,fwd2,dgrad2,dgrad1,wgrad")
    ap.add_argument("--iters", type=int, default=1)
    ap.add_argument("--ctas", type=int, default=2, choices=[1, 2])
    ap.add_argument("--fp8", action="store_true", help="also time the block-scaled fp8 GEMMs (x W1^T and act W2^T)")
    a = ap.parse_args()
    ext = load()
    dev = torch.device("cuda")
    G, H, Fd = a.groups, a.hidden, a.ffn
    rows = [a.rows] * G
    tile = 128 * a.ctas
    off = [i * ((a.rows + tile - 1) // tile * tile) for i in range(G + 1)]
    T = off[-1]
    i32 = dict(dtype=torch.int32, device=dev)
    goff, grows = torch.tensor(off, **i32), torch.tensor(rows, **i32)
    gws, totals = torch.arange(G, **i32), torch.tensor([T, G], **i32)
    status = torch.zeros(4, **i32)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    x = torch.randn(T, H, device=dev).bfloat16()
    act = torch.randn(T, Fd, device=dev).bfloat16()
    h = torch.randn(T, 2 * Fd, device=dev).bfloat16()
    w1 = (torch.randn(G, 2 * Fd, H, device=dev) * 0.02).bfloat16()
    w2 = (torch.randn(G, H, Fd, device=dev) * 0.02).bfloat16()
    out_h = torch.empty(T, H, device=dev).bfloat16()
    gw1 = torch.empty_like(w1)
    real = sum(rows)
    jobs = {
        "fwd1": (x, w1, h, act, 2 * real * H * 2 * Fd),
        "fwd2": (act, w2, out_h, None, 2 * real * Fd * H),
        "dgrad2": (x, w2, h, None, 2 * real * H * Fd),
        "dgrad1": (h, w1, out_h, None, 2 * real * 2 * Fd * H),
        "wgrad": (h, x, gw1, None, 2 * real * 2 * Fd * H),
    }
    for name in a.modes.split(","):
        A, B, o0, o1, flops = jobs[name]
        run = lambda: ext.grouped_gemm(MODE[name], A, B, o0, o1, goff, grows, gws, totals, status, sms, a.ctas)
        run()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(a.iters):
            run()
        t1.record()
        torch.cuda.synchronize()
        ms = t0.elapsed_time(t1) / a.iters
        print(f"{name:<7} {ms:8.4f} ms  {flops / ms * 1e-9:8.1f} TFLOP/s  status={status.tolist()[0]}")
    if a.fp8:
        from . import fp8

        for name, A, W, N, fctas in (("fp8_w1", x, w1, 2 * Fd, 1), ("fp8_w2", act, w2, H, 1),
                                     ("fp8_w1 pair", x, w1, 2 * Fd, 2), ("fp8_w2 pair", act, w2, H, 2)):
            if fctas == 2 and any(o % 256 for o in off):
                continue
            aq, sfa = fp8.quantize_rows(A)
            bq, sfb = fp8.quantize_weights(W)
            out = torch.empty(T, N, device=dev).bfloat16()
            run = lambda: fp8.grouped_gemm_fp8(aq, sfa, bq, sfb, out, goff, grows, gws, totals, status, sms, fctas)
            run()
            torch.cuda.synchronize()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(a.iters):
                run()
            t1.record()
            torch.cuda.synchronize()
            ms = t0.elapsed_time(t1) / a.iters
            flops = 2 * real * A.shape[1] * N
            print(f"{name:<12} {ms:8.4f} ms  {flops / ms * 1e-9:8.1f} TFLOP/s  status={status.tolist()[0]}")
            if fctas == 2:
                continue
            tq0, tq1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            tq0.record()
            for _ in range(a.iters):
                fp8.quantize_rows(A)
            tq1.record()
            torch.cuda.synchronize()
            print(f"{name:<7} quantize_rows [{A.shape[0]}, {A.shape[1]}] {tq0.elapsed_time(tq1) / a.iters:8.4f} ms")


if __name__ == "__main__":
    main()
