"""Build a token dataset for ``train_gpt_moe --data`` from local JSONL files.

    python -m ep_balance_b200.launch.prepare_data --out data/mix --token-budget 2000000 \
        --source code=raw/code.jsonl --source math=raw/math.jsonl:2 [--tokenizer /path/to/hf_tokenizer]

Mirrors the local half of the reference's data preparation (scripts/prepare_open_workload.py,
scripts/prepare_mixed_1b.sh:198-260): one ``{"text": ...}`` record per line, exact-duplicate removal,
an equal (or weighted, ``name=path:weight``) split of the token budget between the sources, and a
deterministic smooth interleave so that no long run of one source appears in the output.
Tokeniser: a local HuggingFace tokenizer directory when given, else UTF-8 bytes (vocabulary 257).

Open workloads by name (the reference's registry, scripts/prepare_open_workload.py:24-108):

    python -m ep_balance_b200.launch.prepare_data --list-workloads
    python -m ep_balance_b200.launch.prepare_data --fetch fineweb --raw-dir raw --fetch-docs 20000   # needs a network
    python -m ep_balance_b200.launch.prepare_data --out data/mix --workload fineweb --workload starcoder:2 --raw-dir raw

``--workload NAME[:weight]`` reads ``<raw-dir>/NAME.jsonl`` with the text field of that workload; ``--fetch``
streams the workload from the HuggingFace hub into that file (``datasets`` and a network are required; on a
machine without either it says what to run elsewhere and exits with an error).
"""

from __future__ import annotations

import argparse
import hashlib
import json
from typing import Dict, Iterator, List, Tuple

from ..utils.data import ByteTokenizer, write_token_dataset


# name -> where the workload lives on the HuggingFace hub and which record field holds the text
WORKLOADS: Dict[str, dict] = {
    "dapo_math":   dict(dataset="BytedTsinghua-SIA/DAPO-Math-17k", config=None, split="train", fields=("prompt", "text")),
    "fineweb":     dict(dataset="HuggingFaceFW/fineweb", config="sample-10BT", split="train", fields=("text",)),
    "dolma":       dict(dataset="allenai/dolma", config="v1_6-sample", split="train", fields=("text",)),
    "fineweb2_zh": dict(dataset="HuggingFaceFW/fineweb-2", config="cmn_Hani", split="train", fields=("text",)),
    "starcoder":   dict(dataset="bigcode/starcoderdata", config=None, split="train", fields=("content",),
                        data_dirs=("python", "cpp", "java", "rust")),
    "pes2o":       dict(dataset="allenai/peS2o", config="v2", split="train", fields=("text",)),
    "openscience": dict(dataset="nvidia/OpenScience", config="OS-Q3-235B-4", split="train", fields=("text", "input")),
    "codeforces":  dict(dataset="open-r1/codeforces", config="verifiable-prompts", split="train", fields=("prompt", "description")),
    "swe_bench":   dict(dataset="SWE-bench/SWE-bench", config="default", split="test", fields=("problem_statement", "text")),
    "gpqa":        dict(dataset="Idavidrein/gpqa", config="gpqa_main", split="train", fields=("Question", "text")),
    "wikitext":    dict(dataset="Salesforce/wikitext", config="wikitext-103-raw-v1", split="train", fields=("text",)),
    "longbench":   dict(dataset="THUDM/LongBench", config=None, split="test", fields=("context", "input")),
}


def workload_path(name: str, raw_dir: str) -> str:
    import os

    return os.path.join(raw_dir, f"{name}.jsonl")


def fetch_workload(name: str, raw_dir: str, max_docs: int) -> str:
    """Stream up to ``max_docs`` records of a catalogued workload into ``<raw_dir>/<name>.jsonl`` as
    ``{"text": ...}`` lines.  Needs the ``datasets`` package and access to the hub."""
    import os

    if name not in WORKLOADS:
        raise SystemExit(f"unknown workload {name!r}; known: {', '.join(sorted(WORKLOADS))}")
    w = WORKLOADS[name]
    out = workload_path(name, raw_dir)
    how = (f"datasets.load_dataset({w['dataset']!r}, {w['config']!r}, split={w['split']!r}, streaming=True) "
           f"-> one {{\"text\": record[{w['fields'][0]!r}]}} per line -> {out}")
    try:
        import datasets  # noqa: F401
    except ImportError:
        raise SystemExit(f"--fetch needs the `datasets` package and a network; on a connected machine run: {how}")
    os.makedirs(raw_dir, exist_ok=True)
    try:
        dirs = w.get("data_dirs") or (None,)
        streams = [iter(datasets.load_dataset(w["dataset"], w["config"], split=w["split"], streaming=True,
                                              **({"data_dir": d} if d else {}))) for d in dirs]
        n = 0
        with open(out, "w", encoding="utf-8") as f:
            while streams and n < max_docs:          # round-robin over the sub-directories
                for s in list(streams):
                    rec = next(s, None)
                    if rec is None:
                        streams.remove(s)
                        continue
                    text = next((rec[k] for k in w["fields"] if isinstance(rec.get(k), str) and rec[k].strip()), None)
                    if text:
                        f.write(json.dumps({"text": text}, ensure_ascii=False) + "\n")
                        n += 1
                        if n >= max_docs:
                            break
    except Exception as exc:  # no route to the hub, gated dataset, ...
        raise SystemExit(f"could not fetch {name}: {type(exc).__name__}: {exc}; on a connected machine run: {how}")
    return out


def read_jsonl(path: str, text_fields=("text", "content", "prompt")) -> Iterator[str]:
    with open(path, encoding="utf-8") as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            rec = json.loads(line)
            for k in text_fields:
                if isinstance(rec.get(k), str) and rec[k].strip():
                    yield rec[k]
                    break


def balanced_token_budgets(total: int, weights: List[float]) -> List[int]:
    """Split ``total`` in proportion to ``weights``; the remainder goes to the first sources."""
    s = float(sum(weights))
    out = [int(total * w / s) for w in weights]
    for i in range(total - sum(out)):
        out[i % len(out)] += 1
    return out


def smooth_interleave(counts: List[int]) -> List[int]:
    """Order in which to emit ``counts[i]`` items of source ``i`` so that every prefix holds each source in
    proportion (largest-deficit-first; ties go to the lower index).  Deterministic."""
    total = sum(counts)
    emitted = [0] * len(counts)
    order = []
    for n in range(1, total + 1):
        best, best_deficit = -1, None
        for i, c in enumerate(counts):
            if emitted[i] >= c:
                continue
            deficit = c * n / total - emitted[i]
            if best_deficit is None or deficit > best_deficit + 1e-12:
                best, best_deficit = i, deficit
        emitted[best] += 1
        order.append(best)
    return order


def collect(sources: List[Tuple[str, str, float]], tokenizer, token_budget: int):
    """Tokenise every source up to its share of the budget, dropping exact duplicates across sources."""
    budgets = balanced_token_budgets(token_budget, [w for _, _, w in sources]) if token_budget > 0 else [0] * len(sources)
    seen = set()
    per_source: List[List[List[int]]] = []
    stats: Dict[str, dict] = {}
    for (name, path, _), budget in zip(sources, budgets):
        docs, used, dup = [], 0, 0
        for text in read_jsonl(path):
            digest = hashlib.sha1(text.encode("utf-8")).digest()
            if digest in seen:
                dup += 1
                continue
            seen.add(digest)
            ids = tokenizer.encode(text)
            if not ids:
                continue
            if token_budget > 0 and used + len(ids) > budget:
                if used == 0:
                    ids = ids[:budget]      # a single oversized first document is truncated, not dropped
                else:
                    break
            docs.append(ids)
            used += len(ids)
        per_source.append(docs)
        stats[name] = {"documents": len(docs), "tokens": used, "duplicates_dropped": dup, "budget": budget}
    return per_source, stats


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--out", default="", help="output prefix (<out>.bin, .idx, .json)")
    ap.add_argument("--source", action="append", default=[], help="name=path.jsonl[:weight]")
    ap.add_argument("--workload", action="append", default=[], help="catalogued workload NAME[:weight], read from <raw-dir>/NAME.jsonl")
    ap.add_argument("--raw-dir", default="raw", help="where the workloads' JSONL files live")
    ap.add_argument("--list-workloads", action="store_true")
    ap.add_argument("--fetch", action="append", default=[], help="download a catalogued workload into <raw-dir> (needs a network)")
    ap.add_argument("--fetch-docs", type=int, default=20000, help="records to keep per fetched workload")
    ap.add_argument("--token-budget", type=int, default=0, help="total tokens to keep (0: everything)")
    ap.add_argument("--tokenizer", default="", help="local HuggingFace tokenizer directory (default: UTF-8 bytes)")
    a = ap.parse_args(argv)
    if a.list_workloads:
        for name, w in sorted(WORKLOADS.items()):
            print(f"{name:12s} {w['dataset']} config={w['config']} split={w['split']} text field={w['fields'][0]}")
        return {"workloads": sorted(WORKLOADS)}
    for name in a.fetch:
        print(f"fetched {fetch_workload(name, a.raw_dir, a.fetch_docs)}")
    if a.fetch and not (a.source or a.workload):
        return {"fetched": a.fetch}
    import os

    sources = []
    for item in a.source:
        name, rest = item.split("=", 1)
        path, _, w = rest.partition(":")
        sources.append((name, path, float(w) if w else 1.0))
    for item in a.workload:
        name, _, w = item.partition(":")
        if name not in WORKLOADS:
            raise SystemExit(f"unknown workload {name!r}; known: {', '.join(sorted(WORKLOADS))}")
        path = workload_path(name, a.raw_dir)
        if not os.path.exists(path):
            raise SystemExit(f"{path} is missing: fetch it with --fetch {name} on a machine with a network "
                             f"({WORKLOADS[name]['dataset']}), or pass --source {name}=<your.jsonl>")
        sources.append((name, path, float(w) if w else 1.0))
    if not sources or not a.out:
        raise SystemExit("nothing to do: give --out and at least one --source or --workload")
    if a.tokenizer:
        from transformers import AutoTokenizer

        hf = AutoTokenizer.from_pretrained(a.tokenizer, local_files_only=True)

        class _Tok:
            vocab_size = len(hf)
            eod = hf.eos_token_id

            @staticmethod
            def encode(text):
                return hf.encode(text, add_special_tokens=False)

        tok = _Tok()
    else:
        tok = ByteTokenizer()
    per_source, stats = collect(sources, tok, a.token_budget)
    order = smooth_interleave([len(d) for d in per_source])
    cursors = [0] * len(per_source)

    def docs():
        for s in order:
            yield per_source[s][cursors[s]]
            cursors[s] += 1

    meta = write_token_dataset(a.out, docs(), tok.vocab_size, eod=tok.eod,
                               extra_meta={"sources": stats, "tokenizer": a.tokenizer or "utf8-bytes"})
    print(json.dumps(meta))
    return meta


if __name__ == "__main__":
    main()
