"""Build a token dataset for ``train_gpt_moe --data`` from local JSONL files.

    python -m ep_balance_b200.launch.prepare_data --out data/mix --token-budget 2000000 \
        --source code=raw/code.jsonl --source math=raw/math.jsonl:2 [--tokenizer /path/to/hf_tokenizer]

Mirrors the local half of the reference's data preparation (scripts/prepare_open_workload.py,
scripts/prepare_mixed_1b.sh:198-260): one ``{"text": ...}`` record per line, exact-duplicate removal,
an equal (or weighted, ``name=path:weight``) split of the token budget between the sources, and a
deterministic smooth interleave so that no long run of one source appears in the output.  The download
half (HuggingFace datasets) needs a network and is not part of this tool: fetch the JSONL elsewhere.
Tokeniser: a local HuggingFace tokenizer directory when given, else UTF-8 bytes (vocabulary 257).
"""

from __future__ import annotations

import argparse
import hashlib
import json
from typing import Dict, Iterator, List, Tuple

from ..utils.data import ByteTokenizer, write_token_dataset


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
    ap.add_argument("--out", required=True, help="output prefix (<out>.bin, .idx, .json)")
    ap.add_argument("--source", action="append", required=True, help="name=path.jsonl[:weight]")
    ap.add_argument("--token-budget", type=int, default=0, help="total tokens to keep (0: everything)")
    ap.add_argument("--tokenizer", default="", help="local HuggingFace tokenizer directory (default: UTF-8 bytes)")
    a = ap.parse_args(argv)
    sources = []
    for item in a.source:
        name, rest = item.split("=", 1)
        path, _, w = rest.partition(":")
        sources.append((name, path, float(w) if w else 1.0))
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
