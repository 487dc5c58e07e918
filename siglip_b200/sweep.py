"""Variant sweep and dispatch-table generator.

Counterpart of the reference's ``tools/grid_search.py`` (constraint pruning ``:89-116``, register / spill
parsing ``:124-151``, per-configuration timeout, CSV ``:170-251``) for the run-time variants of this library:
instead of recompiling one binary per macro combination it walks the compiled variant list
(``siglip_b200/csrc/sl8_variants.h``) through ``sl8_set_variant``, times every admissible variant on the
seeded synthetic operands of ``siglip_b200/synth.py`` over an M ladder, writes one CSV row per
(layer, shape, variant) and turns the CSV into the table ``pick_variant`` (``sl8_api.cu``) consults:
``siglip_b200/csrc/sl8_dispatch_table.h``.

    python -m siglip_b200.sweep --shapes so400m,b16 --out siglip_b200/sweeps/b200.csv     # needs a B200
    python -m siglip_b200.sweep --emit-table siglip_b200/sweeps/b200.csv                   # CPU only

A variant that trips a bounded device wait is recorded as ``timeout`` (the kernel returns, the handle is
re-created) instead of hanging the sweep; that is this library's form of grid_search's per-run timeout.
"""
from __future__ import annotations

import argparse
import csv
import re
import statistics
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
TABLE_HEADER = PKG / "csrc" / "sl8_dispatch_table.h"
OPS = {"pe": 0, "fc1": 1, "fc2": 2}
OP_NAMES = {v: k for k, v in OPS.items()}
OP_ENUM = {0: "SL8_OP_PATCH_EMBED", 1: "SL8_OP_FC1_GELU", 2: "SL8_OP_FC2_RESIDUAL"}

# (layer, N, K, rows per image): the SigLIP-So400m/14 and SigLIP-B/16 layer shapes.
SHAPE_SETS = {
    "so400m": [("pe", 1152, 588, 729), ("fc1", 4304, 1152, 729), ("fc2", 1152, 4304, 729)],
    "b16": [("pe", 768, 768, 196), ("fc1", 3072, 768, 196), ("fc2", 768, 3072, 196)],
}
CSV_FIELDS = ["op", "M", "N", "K", "variant", "cta_group", "tile_n", "tile_k", "stages", "epi_warps", "staging_buffers",
              "regs", "spill_bytes", "smem_bytes", "repeats", "iters", "ms_median", "ms_min", "ms_mean", "ms_stdev",
              "tflops", "status"]


# ----------------------------------------------------------------------------- resources (CPU)
def parse_resources(report: str) -> dict:
    """``build.resource_report()`` text -> {(variant, op, out_dtype): {"regs", "spill_bytes", "stack"}}.

    The kernel's template arguments <CG, TN, TK, STAGES, EPI_WARPS, OP, OUT, NBUF> are read back from the
    mangled name (``...ILi2ELi256ELi128ELi5ELi8ELi1ELi0ELi1EE...``)."""
    out = {}
    for line in report.splitlines():
        m = re.match(r"variant_(\d+): (\S+) regs=(\d+) stack=(\d+) spill_stores=(\d+) spill_loads=(\d+)", line)
        if not m:
            continue
        args = [int(x) for x in re.findall(r"Li(\d+)E", m.group(2))]
        if len(args) < 8:
            continue
        out[(int(m.group(1)), args[5], args[6])] = {"regs": int(m.group(3)), "stack": int(m.group(4)),
                                                    "spill_bytes": int(m.group(5)) + int(m.group(6))}
    return out


def prune(variants: list[dict], op: int, resources: dict | None = None, out_dtype: int = 0) -> list[dict]:
    """Drops the variants that cannot or should not run a layer: one staging buffer serves FC1 only (the
    residual needs a second one to land in), more than 227 KiB of shared memory, spilling kernels."""
    keep = []
    for v in variants:
        if op != OPS["fc1"] and v["staging_buffers"] < 2:
            continue
        if v.get("smem_bytes", 0) > 232448:
            continue
        r = (resources or {}).get((v["variant_id"], op, out_dtype))
        if r is not None and r["spill_bytes"] > 0:
            continue
        keep.append(v)
    return keep


# ----------------------------------------------------------------------------- table (CPU)
def best_rows(rows: list[dict], keep_margin: float = 0.02) -> list[dict]:
    """CSV rows -> dispatch rows {op, N, K, m_min, variant}.

    Per (op, N, K) the M ladder is walked upwards; the winner of the previous (smaller) M is kept unless
    another variant beats it by more than ``keep_margin`` (noise must not flip the table), and neighbouring
    M with the same winner collapse into one row whose ``m_min`` is the smallest of them (0 for the first)."""
    groups: dict[tuple, dict[int, list[dict]]] = {}
    for r in rows:
        if r["status"] != "ok":
            continue
        groups.setdefault((int(r["op"]), int(r["N"]), int(r["K"])), {}).setdefault(int(r["M"]), []).append(r)
    table = []
    for (op, n, k), by_m in sorted(groups.items()):
        prev = None
        for i, m in enumerate(sorted(by_m)):
            cands = sorted(by_m[m], key=lambda r: float(r["ms_median"]))
            best = cands[0]
            choice = int(best["variant"])
            if prev is not None and prev != choice:
                mine = [r for r in cands if int(r["variant"]) == prev]
                if mine and float(mine[0]["ms_median"]) <= float(best["ms_median"]) * (1.0 + keep_margin):
                    choice = prev
            if choice != prev:
                table.append({"op": op, "N": n, "K": k, "m_min": 0 if i == 0 else m, "variant": choice})
            prev = choice
    return table


def emit_header(table: list[dict], source: str, path: Path = TABLE_HEADER) -> str:
    lines = ["// sl8_dispatch_table.h -- GENERATED by `python -m siglip_b200.sweep --emit-table " + source + "`.",
             "// One row per (layer, N, K, smallest M) -> kernel variant, from the sweep on B200; pick_variant() takes the",
             "// row with the largest m_min <= M for an exact (layer, N, K) match and falls back to its rules otherwise.",
             "#pragma once", "",
             "struct Sl8DispatchRow { int op; int n; int k; long long m_min; int variant; };", "",
             "static const Sl8DispatchRow kSl8DispatchTable[] = {"]
    for r in table:
        lines.append(f"    {{{OP_ENUM[r['op']]}, {r['N']}, {r['K']}, {r['m_min']}LL, {r['variant']}}},")
    if not table:
        lines.append("    {-1, 0, 0, 0LL, 0},")
    lines += ["};", f"static const int kSl8DispatchRows = {max(len(table), 0)};", ""]
    text = "\n".join(lines)
    path.write_text(text)
    return text


def read_csv(path: Path) -> list[dict]:
    with open(path, newline="") as f:
        return list(csv.DictReader(f))


# ----------------------------------------------------------------------------- timing (GPU)
def time_variant(eng, go, repeats: int, iters: int) -> list[float]:
    import torch
    out = []
    go()
    torch.cuda.synchronize()
    for _ in range(repeats):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            go()
        e1.record()
        torch.cuda.synchronize()
        out.append(e0.elapsed_time(e1) / iters)
    eng.device_status()
    return out


def run_sweep(shape_sets: list[str], m_steps: int, repeats: int, iters: int, out_path: Path, variants_only=None,
              max_rows: int | None = None, log=print) -> list[dict]:
    """Times every admissible variant on every (layer, N, K) of the named shape sets for M = rows_per_image * 2^j."""
    import torch
    import siglip_b200
    from siglip_b200 import build, layers, synth
    from siglip_b200.lib import SL8Error

    dev = "cuda"
    eng = siglip_b200.Engine(0)
    resources = parse_resources(build.resource_report())
    all_variants = [dict(layers.describe_variant(v), variant_id=v) for v in range(layers.num_variants())]
    rows = []
    out_path.parent.mkdir(parents=True, exist_ok=True)
    with open(out_path, "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=CSV_FIELDS)
        w.writeheader()
        for set_name in shape_sets:
            for op_name, n, k, per_image in SHAPE_SETS[set_name]:
                op = OPS[op_name]
                for j in range(m_steps):
                    m = per_image * (1 << j)
                    if max_rows is not None and m > max_rows:
                        break
                    if op == 0:
                        p = synth.make_patch_embed(m, n, k, per_image, seed=0, device=dev, pixels=True)
                    elif op == 1:
                        p = synth.make_fc1(m, n, k, seed=0, device=dev)
                    else:
                        p = synth.make_fc2(m, n, k, seed=0, device=dev)
                    sa = torch.tensor([p.scale_a], device=dev)
                    sb = torch.tensor([p.scale_b], device=dev)
                    # Three operand sets taken in turn, so that no launch finds its A rows or its output lines in L2
                    # (the protocol of bench.py); weights, bias and table stay, as they would in a model.
                    sets = 3

                    def clone_pitched(t):
                        return torch.empty_strided(t.shape, t.stride(), dtype=t.dtype, device=t.device).copy_(t)

                    a_sets = [p.A] + [clone_pitched(p.A) for _ in range(sets - 1)]
                    d_sets = [torch.empty((m, n), dtype=torch.bfloat16, device=dev) for _ in range(sets)]
                    r_sets = [p.residual] + [p.residual.clone() for _ in range(sets - 1)] if op == 2 else None
                    tbl = eng.padded_table(p.table) if p.table is not None else None
                    turn = [0]

                    def go():
                        i = turn[0] % sets
                        turn[0] += 1
                        if op == 1:
                            eng.fc1_gelu(a_sets[i], p.B, p.bias, scale_a=sa, scale_b=sb, out=d_sets[i])
                        elif op == 2:
                            eng.fc2_residual(a_sets[i], p.B, p.bias, r_sets[i], scale_a=sa, scale_b=sb, out=d_sets[i])
                        else:
                            eng.patch_embed(a_sets[i], p.B, tbl, period=p.period, scale_a=sa, scale_b=sb, out=d_sets[i])

                    # Variants are timed in rounds (every variant once per round), not one after the other: the chip is
                    # power-bound under these kernels and whoever runs last on a warm GPU would look slower.
                    cands = [v for v in prune(all_variants, op, resources)
                             if variants_only is None or v["variant_id"] in variants_only]
                    samples = {v["variant_id"]: [] for v in cands}
                    status = {v["variant_id"]: "ok" for v in cands}
                    for rnd in range(repeats + 1):               # round 0 warms up and is not recorded
                        for v in cands:
                            vid = v["variant_id"]
                            if status[vid] != "ok":
                                continue
                            try:
                                eng.set_variant(vid)
                                ms = time_variant(eng, go, 1, iters if rnd else 3)
                                if rnd:
                                    samples[vid] += ms
                            except SL8Error as e:        # a bounded device wait ran out, or the variant refused the shape
                                status[vid] = "timeout" if "TIMEOUT" in str(e).upper() else "error"
                                eng = siglip_b200.Engine(0)
                    for v in cands:
                        vid = v["variant_id"]
                        res = resources.get((vid, op, 0), {})
                        row = {"op": op, "M": m, "N": n, "K": k, "variant": vid, "cta_group": v["cta_group"],
                               "tile_n": v["tile_n"], "tile_k": v["tile_k"], "stages": v["stages"],
                               "epi_warps": v["epi_warps"], "staging_buffers": v["staging_buffers"],
                               "regs": res.get("regs", ""), "spill_bytes": res.get("spill_bytes", ""),
                               "smem_bytes": v.get("smem_bytes", ""), "repeats": repeats, "iters": iters}
                        ms = samples[vid]
                        if status[vid] == "ok" and ms:
                            row.update(ms_median=statistics.median(ms), ms_min=min(ms), ms_mean=statistics.fmean(ms),
                                       ms_stdev=statistics.pstdev(ms), tflops=p.flops() / statistics.median(ms) / 1e9,
                                       status="ok")
                        else:
                            row.update(ms_median="", ms_min="", ms_mean="", ms_stdev="", tflops="",
                                       status=status[vid] if status[vid] != "ok" else "error")
                        w.writerow(row)
                        f.flush()
                        rows.append({k2: str(v2) for k2, v2 in row.items()})
                    ok = [r for r in rows if r["op"] == str(op) and r["M"] == str(m) and r["N"] == str(n) and r["status"] == "ok"]
                    if ok:
                        b = min(ok, key=lambda r: float(r["ms_median"]))
                        log(f"{op_name} M={m} N={n} K={k}: best v{b['variant']} {float(b['ms_median']) * 1e3:.1f} us "
                            f"{float(b['tflops']):.0f} TFLOP/s  ({len(ok)} variants)")
                    del p, a_sets, d_sets, r_sets
                    torch.cuda.empty_cache()
    eng.set_variant(-1)
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--shapes", default="so400m,b16", help="comma-separated shape sets: " + ", ".join(SHAPE_SETS))
    ap.add_argument("--m-steps", type=int, default=11, help="M = rows_per_image * 2^j for j < m-steps")
    ap.add_argument("--max-rows", type=int, default=None)
    ap.add_argument("--repeats", type=int, default=5)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--out", type=Path, default=PKG / "sweeps" / "b200.csv")
    ap.add_argument("--variants", default="", help="restrict to these variant ids")
    ap.add_argument("--emit-table", type=Path, default=None, metavar="CSV",
                    help="no GPU work: turn this CSV into csrc/sl8_dispatch_table.h")
    a = ap.parse_args(argv)
    if a.emit_table is not None:
        table = best_rows(read_csv(a.emit_table))
        try:
            shown = a.emit_table.resolve().relative_to(PKG.parent)
        except ValueError:
            shown = a.emit_table
        emit_header(table, str(shown))
        print(f"{len(table)} rows -> {TABLE_HEADER}")
        return 0
    only = {int(x) for x in a.variants.split(",")} if a.variants else None
    run_sweep(a.shapes.split(","), a.m_steps, a.repeats, a.iters, a.out, only, a.max_rows)
    print(f"wrote {a.out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
