"""Parse a Megatron-style training log into per-iteration metrics (ms/iter, TFLOP/s/GPU, loss,
grad norm), the argument dump and the memory report.  Reference: eval/extract_train_metrics.py:29-341."""

from __future__ import annotations

import argparse
import csv
import json
import re
import statistics as st
from pathlib import Path
from typing import Any, Dict, List

ITER_RE = re.compile(
    r"iteration\s+(?P<iter>\d+)/\s*(?P<total>\d+)\s*\|\s*consumed samples:\s*(?P<samples>\d+)\s*\|"
    r"\s*elapsed time per iteration \(ms\):\s*(?P<ms>[\d.]+)\s*\|"
    r"(?:\s*throughput per GPU \(TFLOP/s/GPU\):\s*(?P<tflops>[\d.]+)\s*\|)?"
    r"\s*learning rate:\s*(?P<lr>[\dEe.+-]+)\s*\|\s*global batch size:\s*(?P<gbs>\d+)\s*\|"
    r"\s*lm loss:\s*(?P<loss>[\dEe.+-]+)\s*\|")
GRAD_NORM_RE = re.compile(r"grad norm:\s*(?P<gn>[\d.]+|nan)")
ARG_RE = re.compile(r"^\s{2}(?P<key>\w+)\s\.{2,}\s(?P<value>.*?)\s*$")
MEMORY_RE = re.compile(r"\(after (?P<iter>\d+) iterations\) memory \(MB\).*?max reserved:\s*(?P<max_reserved>[\d.]+)")
CONFIG_KEYS = set("num_layers hidden_size ffn_hidden_size num_attention_heads num_experts moe_ffn_hidden_size "
                  "moe_router_topk tensor_model_parallel_size pipeline_model_parallel_size "
                  "expert_model_parallel_size world_size seq_length micro_batch_size global_batch_size train_iters "
                  "lr bf16 seed".split())


def parse(path: Path) -> Dict[str, Any]:
    iters: List[Dict[str, Any]] = []
    config: Dict[str, str] = {}
    memory: List[Dict[str, float]] = []
    for line in Path(path).read_text(errors="replace").splitlines():
        m = ITER_RE.search(line)
        if m:
            row = {"iter": int(m["iter"]), "samples": int(m["samples"]), "ms": float(m["ms"]), "lr": float(m["lr"]),
                   "global_batch": int(m["gbs"]), "loss": float(m["loss"])}
            if m["tflops"]:
                row["tflops_per_gpu"] = float(m["tflops"])
            g = GRAD_NORM_RE.search(line)
            if g:
                row["grad_norm"] = float(g["gn"])
            iters.append(row)
            continue
        a = ARG_RE.match(line)
        if a and a["key"] in CONFIG_KEYS:
            config[a["key"]] = a["value"]
        mm = MEMORY_RE.search(line)
        if mm:
            memory.append({"iter": int(mm["iter"]), "max_reserved_mb": float(mm["max_reserved"])})
    return {"iterations": iters, "config": config, "memory": memory}


def summarize(parsed: Dict[str, Any], warmup: int = 0) -> Dict[str, Any]:
    rows = [r for r in parsed["iterations"] if r["iter"] > warmup]
    if not rows:
        return {"iterations": 0}
    out = {"iterations": len(rows), "ms_mean": st.fmean(r["ms"] for r in rows), "ms_p50": st.median(r["ms"] for r in rows),
           "loss_first": rows[0]["loss"], "loss_last": rows[-1]["loss"]}
    tf = [r["tflops_per_gpu"] for r in rows if "tflops_per_gpu" in r]
    if tf:
        out["tflops_per_gpu_mean"] = st.fmean(tf)
    if parsed["memory"]:
        out["max_reserved_mb"] = max(m["max_reserved_mb"] for m in parsed["memory"])
    return out


def main(argv=None) -> Dict[str, Any]:
    p = argparse.ArgumentParser(description=__doc__)
    p.add_argument("--log", required=True, type=Path)
    p.add_argument("--out-dir", type=Path, default=None)
    p.add_argument("--warmup", type=int, default=0)
    a = p.parse_args(argv)
    parsed = parse(a.log)
    summary = summarize(parsed, a.warmup)
    if a.out_dir:
        a.out_dir.mkdir(parents=True, exist_ok=True)
        if parsed["iterations"]:
            cols: List[str] = []
            for r in parsed["iterations"]:
                cols += [c for c in r if c not in cols]
            with open(a.out_dir / "iterations.csv", "w", newline="") as f:
                w = csv.DictWriter(f, fieldnames=cols)
                w.writeheader()
                w.writerows(parsed["iterations"])
        (a.out_dir / "summary.json").write_text(json.dumps({"summary": summary, "config": parsed["config"]}, indent=1))
    return {"summary": summary, **parsed}


if __name__ == "__main__":
    print(json.dumps(main()["summary"], indent=1))
