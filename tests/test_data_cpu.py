"""Data preparation and the memory-mapped token dataset (CPU)."""

import json

import torch

from ep_balance_b200.launch.prepare_data import balanced_token_budgets, main, smooth_interleave
from ep_balance_b200.utils.data import TokenDataset


def test_smooth_interleave_keeps_every_prefix_in_proportion():
    order = smooth_interleave([6, 3, 1])
    assert sorted(order) == [0] * 6 + [1] * 3 + [2]
    assert order == smooth_interleave([6, 3, 1])          # deterministic
    for n in range(1, 11):
        seen0 = order[:n].count(0)
        assert abs(seen0 - 0.6 * n) <= 1.0
    assert max(len(run) for run in "".join(map(str, order)).split("1")) <= 3   # no long run of source 0
    assert balanced_token_budgets(10, [1, 1, 1]) == [4, 3, 3]


def test_prepare_and_read_back(tmp_path):
    a, b = tmp_path / "a.jsonl", tmp_path / "b.jsonl"
    a.write_text("\n".join(json.dumps({"text": f"alpha document number {i} " * 3}) for i in range(20)) + "\n")
    b.write_text("\n".join(json.dumps({"content": t}) for t in ["beta one", "beta two", "alpha document number 0 " * 3,
                                                                 "beta one"]) + "\n")
    meta = main(["--out", str(tmp_path / "mix"), "--source", f"a={a}", "--source", f"b={b}", "--token-budget", "600"])
    assert meta["sources"]["b"]["duplicates_dropped"] == 2     # one repeated line, one copy of a's first document
    assert meta["sources"]["a"]["tokens"] <= 300 and meta["num_tokens"] == sum(
        s["tokens"] for s in meta["sources"].values()) + meta["num_documents"]   # one end-of-document id each
    ds = TokenDataset(str(tmp_path / "mix"))
    assert len(ds) == meta["num_documents"] and ds.num_tokens == meta["num_tokens"]
    first = bytes(int(t) for t in ds.document(0)[:-1]).decode()
    assert first.startswith("alpha document number 0")
    assert int(ds.document(0)[-1]) == 256
    g = torch.Generator().manual_seed(0)
    batch = ds.sample_batch(3, 16, g)
    assert batch.shape == (3, 17) and batch.dtype == torch.int64 and int(batch.max()) <= 256
    g2 = torch.Generator().manual_seed(0)
    assert torch.equal(batch, ds.sample_batch(3, 16, g2))


def test_catalogued_workloads_resolve_to_local_files(tmp_path, capsys):
    import pytest

    from ep_balance_b200.launch.prepare_data import WORKLOADS

    assert {"fineweb", "starcoder", "dolma", "pes2o", "dapo_math"} <= set(WORKLOADS)
    assert main(["--list-workloads"])["workloads"] == sorted(WORKLOADS)
    assert "bigcode/starcoderdata" in capsys.readouterr().out
    raw = tmp_path / "raw"
    raw.mkdir()
    (raw / "fineweb.jsonl").write_text("\n".join(json.dumps({"text": f"web page {i} " * 4}) for i in range(8)) + "\n")
    (raw / "starcoder.jsonl").write_text("\n".join(json.dumps({"text": f"def f{i}(): return {i}"}) for i in range(8)) + "\n")
    meta = main(["--out", str(tmp_path / "mix"), "--workload", "fineweb", "--workload", "starcoder:3",
                 "--raw-dir", str(raw), "--token-budget", "400"])
    assert meta["sources"]["fineweb"]["budget"] == 100 and meta["sources"]["starcoder"]["budget"] == 300
    with pytest.raises(SystemExit, match="--fetch dolma"):      # a catalogued workload whose file is not there
        main(["--out", str(tmp_path / "x"), "--workload", "dolma", "--raw-dir", str(raw)])
    with pytest.raises(SystemExit, match="unknown workload"):
        main(["--out", str(tmp_path / "x"), "--workload", "nope", "--raw-dir", str(raw)])
