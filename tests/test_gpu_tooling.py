"""The sweep / comparison tooling on a GPU: a two-variant sweep of one small shape, an in-process comparison with
cuBLASLt, and the dispatch answering from the committed table."""
import csv

import pytest

from siglip_b200 import compare, sweep

pytestmark = pytest.mark.gpu


def test_small_sweep_writes_rows_and_a_table(engine, tmp_path, monkeypatch):
    monkeypatch.setitem(sweep.SHAPE_SETS, "tiny", [("fc1", 512, 256, 196), ("fc2", 256, 512, 196)])
    out = tmp_path / "tiny.csv"
    rows = sweep.run_sweep(["tiny"], m_steps=2, repeats=2, iters=3, out_path=out, variants_only={1, 6}, log=lambda *_: None)
    with open(out, newline="") as f:
        on_disk = list(csv.DictReader(f))
    assert len(on_disk) == len(rows) == 2 * 2 * 2
    assert all(r["status"] == "ok" and float(r["ms_median"]) > 0 and r["regs"] != "" for r in on_disk)
    table = sweep.best_rows(on_disk)
    assert {(t["op"], t["N"], t["K"]) for t in table} == {(1, 512, 256), (2, 256, 512)}
    assert all(t["variant"] in (1, 6) for t in table)


def test_in_process_comparison_with_cublaslt(engine):
    arms = compare.inproc_arms(["ours", "ours:v6", "cublaslt", "cublaslt_unfused"], "fc2", 2916, 1152, 4304, 729, iters=3)
    samples = {name: [fn() for _ in range(3)] for name, fn in arms.items()}
    s = compare.summarize(samples)
    assert set(s["arms"]) == {"ours", "ours:v6", "cublaslt", "cublaslt_unfused"}
    assert all(d["mean"] > 0 for d in s["arms"].values())
    assert s["anova"]["F"] is not None
    assert "ANOVA" in compare.format_table(s)


def test_dispatch_answers_from_the_committed_table(engine):
    table = sweep.best_rows(sweep.read_csv(sweep.PKG / "sweeps" / "b200.csv"))
    assert table, "the committed sweep is empty"
    for i, r in enumerate(table):
        later = [t["m_min"] for t in table[i + 1:] if (t["op"], t["N"], t["K"]) == (r["op"], r["N"], r["K"])]
        m = max(r["m_min"], 1)
        if later and later[0] <= m:
            continue
        assert engine.query_config(r["op"], m, r["N"], r["K"])["variant_id"] == r["variant"], r
    # a shape the sweep does not hold falls back to the rules
    assert engine.query_config(1, 50000, 2048, 1024)["variant_id"] == 15
    assert engine.query_config(1, 50000, 2048, 1024, out_dtype=1)["variant_id"] == 15     # e4m3 out: sixteen warps, 64-byte staging rows
