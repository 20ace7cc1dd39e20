"""Token datasets on disk: a flat ``.bin`` of token ids plus an ``.idx`` of document offsets.

    <prefix>.bin    little-endian token ids (uint16 when the vocabulary fits, else int32), documents back to back
    <prefix>.idx    int64 offsets, one per document plus the final end offset
    <prefix>.json   {"dtype", "vocab_size", "num_documents", "num_tokens", ...statistics}

The reference feeds Megatron's indexed datasets produced by its preprocessing wrapper
(scripts/prepare_open_workload.py:584-622); this is the stand-alone equivalent used by
``launch/train_gpt_moe.py --data``.  Reading is a NumPy memory map: nothing is loaded up front.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Iterable, List, Optional, Sequence

import numpy as np
import torch


class ByteTokenizer:
    """UTF-8 bytes as token ids 0..255, plus an end-of-document id 256.  Needs no vocabulary file."""

    vocab_size = 257
    eod = 256

    def encode(self, text: str) -> List[int]:
        return list(text.encode("utf-8"))


def write_token_dataset(prefix: str, documents: Iterable[Sequence[int]], vocab_size: int, eod: Optional[int] = None,
                        extra_meta: Optional[dict] = None) -> dict:
    """Write ``documents`` (iterables of token ids) under ``prefix``; returns the metadata dict."""
    dtype = np.uint16 if vocab_size <= 65536 else np.int32
    prefix_p = Path(prefix)
    prefix_p.parent.mkdir(parents=True, exist_ok=True)
    offsets = [0]
    lengths = []
    with open(f"{prefix}.bin", "wb") as f:
        for doc in documents:
            arr = np.asarray(list(doc) + ([eod] if eod is not None else []), dtype=dtype)
            arr.tofile(f)
            offsets.append(offsets[-1] + int(arr.size))
            lengths.append(int(arr.size))
    np.asarray(offsets, dtype=np.int64).tofile(f"{prefix}.idx")
    meta = {"dtype": np.dtype(dtype).name, "vocab_size": int(vocab_size), "num_documents": len(lengths),
            "num_tokens": int(offsets[-1])}
    if lengths:
        srt = sorted(lengths)
        meta.update({"doc_tokens_min": srt[0], "doc_tokens_p50": srt[len(srt) // 2],
                     "doc_tokens_p90": srt[min(len(srt) - 1, int(0.9 * len(srt)))], "doc_tokens_max": srt[-1]})
    meta.update(extra_meta or {})
    with open(f"{prefix}.json", "w") as f:
        json.dump(meta, f, indent=1)
    return meta


class TokenDataset:
    """Memory-mapped view of a dataset written by :func:`write_token_dataset`."""

    def __init__(self, prefix: str) -> None:
        with open(f"{prefix}.json") as f:
            self.meta = json.load(f)
        self.tokens = np.memmap(f"{prefix}.bin", dtype=np.dtype(self.meta["dtype"]), mode="r")
        self.offsets = np.fromfile(f"{prefix}.idx", dtype=np.int64)
        if int(self.offsets[-1]) != int(self.tokens.size):
            raise ValueError(f"{prefix}: index and token file disagree")

    def __len__(self) -> int:
        return int(self.offsets.size - 1)

    @property
    def num_tokens(self) -> int:
        return int(self.tokens.size)

    def document(self, i: int) -> np.ndarray:
        return np.asarray(self.tokens[int(self.offsets[i]):int(self.offsets[i + 1])])

    def sample_batch(self, micro_batch: int, seq_len: int, generator: torch.Generator) -> torch.Tensor:
        """``[micro_batch, seq_len + 1]`` int64 windows at random token offsets (documents are packed back to
        back, so a window may span a document boundary, as in GPT pre-training)."""
        span = seq_len + 1
        if self.num_tokens < span:
            raise ValueError("dataset is shorter than one training window")
        starts = torch.randint(0, self.num_tokens - span + 1, (micro_batch,), generator=generator).tolist()
        rows = [np.asarray(self.tokens[s:s + span]).astype(np.int64) for s in starts]
        return torch.from_numpy(np.stack(rows))
