"""Sweep / comparison tooling: the parts that need no GPU (resource parsing, pruning, table building, statistics).

Counterparts in the reference: tools/grid_search.py:89-151 (pruning, ptxas parsing) and
tools/compare_all.py:338-399 (statistics, ANOVA)."""
import math

import pytest

from siglip_b200 import compare, sweep

REPORT = """\
variant_1: _ZN3sl815sl8_gemm_kernelILi2ELi256ELi128ELi5ELi4ELi2ELi0ELi3EEEv14CUtensorMap_stS1_S1_S1_NS_12KernelParamsE regs=131 stack=0 spill_stores=0 spill_loads=0
variant_1: _ZN3sl815sl8_gemm_kernelILi2ELi256ELi128ELi5ELi4ELi1ELi1ELi3EEEv14CUtensorMap_stS1_S1_S1_NS_12KernelParamsE regs=96 stack=0 spill_stores=0 spill_loads=0
variant_2: _ZN3sl815sl8_gemm_kernelILi2ELi256ELi128ELi5ELi8ELi1ELi0ELi1EEEv14CUtensorMap_stS1_S1_S1_NS_12KernelParamsE regs=94 stack=8 spill_stores=16 spill_loads=24
garbage line
"""


def test_parse_resources_reads_template_arguments_from_the_mangled_name():
    r = sweep.parse_resources(REPORT)
    assert r[(1, 2, 0)] == {"regs": 131, "stack": 0, "spill_bytes": 0}      # variant 1, FC2, bf16
    assert r[(1, 1, 1)]["regs"] == 96                                        # variant 1, FC1, e4m3
    assert r[(2, 1, 0)] == {"regs": 94, "stack": 8, "spill_bytes": 40}
    assert len(r) == 3


def test_prune_drops_single_buffer_variants_for_side_data_layers_and_spilling_kernels():
    variants = [{"variant_id": 1, "staging_buffers": 3, "smem_bytes": 218624},
                {"variant_id": 2, "staging_buffers": 1, "smem_bytes": 202240},
                {"variant_id": 9, "staging_buffers": 2, "smem_bytes": 300000}]
    res = sweep.parse_resources(REPORT)
    assert [v["variant_id"] for v in sweep.prune(variants, sweep.OPS["fc2"], res)] == [1]
    assert [v["variant_id"] for v in sweep.prune(variants, sweep.OPS["fc1"], res)] == [1]          # 2 spills, 9 too large
    assert [v["variant_id"] for v in sweep.prune(variants, sweep.OPS["fc1"], None)] == [1, 2]


def _row(op, m, n, k, variant, ms, status="ok"):
    return {"op": str(op), "M": str(m), "N": str(n), "K": str(k), "variant": str(variant), "ms_median": str(ms), "status": status}


def test_best_rows_keeps_the_previous_winner_inside_the_margin_and_merges_neighbours():
    rows = [
        _row(1, 729, 4304, 1152, 6, 0.010), _row(1, 729, 4304, 1152, 2, 0.014),
        _row(1, 1458, 4304, 1152, 6, 0.0180), _row(1, 1458, 4304, 1152, 2, 0.0179),     # 0.6 % better: keep 6
        _row(1, 2916, 4304, 1152, 6, 0.030), _row(1, 2916, 4304, 1152, 2, 0.023),       # 23 % better: switch
        _row(1, 5832, 4304, 1152, 2, 0.035), _row(1, 5832, 4304, 1152, 6, 0.050),
        _row(1, 5832, 4304, 1152, 3, 0.001, status="timeout"),                          # ignored
        _row(2, 729, 1152, 4304, 1, 0.02),
    ]
    table = sweep.best_rows(rows)
    assert table == [{"op": 1, "N": 4304, "K": 1152, "m_min": 0, "variant": 6},
                     {"op": 1, "N": 4304, "K": 1152, "m_min": 2916, "variant": 2},
                     {"op": 2, "N": 1152, "K": 4304, "m_min": 0, "variant": 1}]


def test_emit_header_writes_one_initialiser_per_row(tmp_path):
    table = [{"op": 1, "N": 4304, "K": 1152, "m_min": 0, "variant": 6}, {"op": 0, "N": 1152, "K": 588, "m_min": 2916, "variant": 5}]
    text = sweep.emit_header(table, "x.csv", tmp_path / "t.h")
    assert "{SL8_OP_FC1_GELU, 4304, 1152, 0LL, 6}," in text and "{SL8_OP_PATCH_EMBED, 1152, 588, 2916LL, 5}," in text
    assert "kSl8DispatchRows = 2;" in text
    empty = sweep.emit_header([], "x.csv", tmp_path / "e.h")
    assert "kSl8DispatchRows = 0;" in empty and "{-1, 0, 0, 0LL, 0}," in empty           # an array may not be empty


def test_the_committed_table_is_what_its_sweep_produces():
    """csrc/sl8_dispatch_table.h is generated: it must match the committed CSV it names."""
    header = sweep.TABLE_HEADER.read_text()
    csv_path = sweep.PKG.parent / header.splitlines()[0].split("--emit-table ")[1].rstrip("`.")
    if not csv_path.exists():
        assert "kSl8DispatchRows = 0;" in header
        return
    table = sweep.best_rows(sweep.read_csv(csv_path))
    for r in table:
        assert f"{{{sweep.OP_ENUM[r['op']]}, {r['N']}, {r['K']}, {r['m_min']}LL, {r['variant']}}}," in header
    assert f"kSl8DispatchRows = {len(table)};" in header


def test_anova_known_answer():
    # Textbook example: three groups, F = 9.3 exactly? computed by hand below.
    g = [[6.0, 8.0, 4.0, 5.0, 3.0, 4.0], [8.0, 12.0, 9.0, 11.0, 6.0, 8.0], [13.0, 9.0, 11.0, 8.0, 7.0, 12.0]]
    a = compare.anova_oneway(g)
    # means 5, 9, 10; grand 8; SSB = 6*(9+1+4) = 84; SSW = 16+24+28 = 68; F = (84/2)/(68/15)
    assert a["df"] == [2, 15] and a["F"] == pytest.approx(42.0 / (68.0 / 15.0))
    assert a["p"] is None or a["p"] == pytest.approx(0.0024, abs=3e-4)
    assert compare.anova_oneway([[1.0, 1.0], [1.0, 1.0]])["F"] == 0.0


def test_welch_and_summary():
    a = [10.0, 10.2, 9.8, 10.1, 9.9]
    b = [12.0, 12.3, 11.9, 12.1, 12.2]
    w = compare.welch(b, a)
    assert w["t"] > 15 and (w["p"] is None or w["p"] < 1e-6)
    s = compare.summarize({"ours": a, "other": b})
    assert s["arms"]["ours"]["n"] == 5 and s["arms"]["ours"]["mean"] == pytest.approx(10.0)
    assert s["arms"]["ours"]["ci95"][0] < 10.0 < s["arms"]["ours"]["ci95"][1]
    assert s["vs_first"]["other"]["ratio_of_means"] == pytest.approx(12.1 / 10.0)
    text = compare.format_table(s)
    assert "ours" in text and "ANOVA" in text
    assert math.isclose(compare.describe([3.0])["stdev"], 0.0)


def test_result_line_of_the_reference_harness_is_parsed():
    line = "Custom kernel: 0.531 ms\n@@RESULT ms=0.531 tflops=2062.11 checksum=1769472.000000 valid=1 c0=1728.0\n"
    assert compare.parse_result_line(line) == pytest.approx(0.531)
    assert compare.parse_result_line("no result here") is None
