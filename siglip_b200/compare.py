"""N-run comparison of implementations of one layer, with statistics.

Counterpart of the reference's ``tools/compare_all.py`` (N runs per binary, mean / stdev / CI, one-way ANOVA,
``:338-399``; ``@@RESULT`` parsing ``:90-100``).  An arm is either timed in-process on the seeded synthetic
operands of ``siglip_b200/synth.py``:

    ours              the library with its own dispatch
    ours:v<id>        the library with one kernel variant forced
    cublaslt          cuBLASLt FP8 GEMM (+ bias where the layer has one) through torch._scaled_mm
    cublaslt_unfused  that GEMM followed by the layer's epilogue as separate elementwise kernels

or an external command that prints the reference harness's ``@@RESULT ms=... tflops=...`` line (the
reference's own binaries, ``siglip_b200/lib/siglip_bench``), given as ``name=command``:

    python -m siglip_b200.compare --op fc2 --M 46656 --N 1152 --K 4304 --runs 10 \\
        --arms ours,ours:v13,cublaslt,cublaslt_unfused
    python -m siglip_b200.compare --runs 5 --arms "new=siglip_b200/lib/siglip_bench --layer fc1,ref=oracle/_ref/fc1-gelu"

Arms are interleaved run by run so that clock and thermal drift hit all of them alike.
"""
from __future__ import annotations

import argparse
import json
import math
import re
import shlex
import statistics
import subprocess
import sys

RESULT_RE = re.compile(r"@@RESULT\s+ms=([0-9.eE+-]+)\s+tflops=([0-9.eE+-]+)")


# ----------------------------------------------------------------------------- statistics (CPU)
def t_quantile_975(df: float) -> float:
    try:
        from scipy import stats
        return float(stats.t.ppf(0.975, df))
    except Exception:                                   # normal approximation with the usual small-sample correction
        return 1.96 + 2.4 / max(df, 1.0)


def describe(samples: list[float]) -> dict:
    n = len(samples)
    mean = statistics.fmean(samples)
    sd = statistics.stdev(samples) if n > 1 else 0.0
    half = t_quantile_975(n - 1) * sd / math.sqrt(n) if n > 1 else 0.0
    return {"n": n, "mean": mean, "median": statistics.median(samples), "stdev": sd, "min": min(samples),
            "max": max(samples), "ci95": [mean - half, mean + half]}


def anova_oneway(groups: list[list[float]]) -> dict:
    """One-way ANOVA: F = (between-group mean square) / (within-group mean square), p from the F distribution."""
    k = len(groups)
    n = sum(len(g) for g in groups)
    if k < 2 or n <= k:
        return {"F": None, "p": None, "df": [k - 1, n - k]}
    grand = sum(sum(g) for g in groups) / n
    ssb = sum(len(g) * (statistics.fmean(g) - grand) ** 2 for g in groups)
    ssw = sum(sum((x - statistics.fmean(g)) ** 2 for x in g) for g in groups)
    dfb, dfw = k - 1, n - k
    if ssw == 0.0:
        return {"F": math.inf if ssb > 0 else 0.0, "p": 0.0 if ssb > 0 else 1.0, "df": [dfb, dfw]}
    f = (ssb / dfb) / (ssw / dfw)
    try:
        from scipy import stats
        p = float(stats.f.sf(f, dfb, dfw))
    except Exception:
        p = None
    return {"F": f, "p": p, "df": [dfb, dfw]}


def welch(a: list[float], b: list[float]) -> dict:
    """Welch's unequal-variance t test of mean(a) against mean(b)."""
    na, nb = len(a), len(b)
    if na < 2 or nb < 2:
        return {"t": None, "p": None}
    va, vb = statistics.variance(a), statistics.variance(b)
    se2 = va / na + vb / nb
    if se2 == 0.0:
        same = statistics.fmean(a) == statistics.fmean(b)
        return {"t": 0.0 if same else math.inf, "p": 1.0 if same else 0.0}
    t = (statistics.fmean(a) - statistics.fmean(b)) / math.sqrt(se2)
    df = se2 ** 2 / ((va / na) ** 2 / (na - 1) + (vb / nb) ** 2 / (nb - 1))
    try:
        from scipy import stats
        p = float(2.0 * stats.t.sf(abs(t), df))
    except Exception:
        p = None
    return {"t": t, "p": p, "df": df}


def summarize(samples: dict[str, list[float]]) -> dict:
    """Per-arm statistics, the ANOVA over all arms and every arm against the first one."""
    names = list(samples)
    out = {"arms": {n: describe(samples[n]) for n in names}, "anova": anova_oneway([samples[n] for n in names]),
           "vs_first": {}}
    base = names[0]
    for n in names[1:]:
        w = welch(samples[n], samples[base])
        w["ratio_of_means"] = statistics.fmean(samples[n]) / statistics.fmean(samples[base])
        out["vs_first"][n] = w
    return out


def format_table(summary: dict, unit: str = "ms") -> str:
    lines = [f"{'arm':28s} {'n':>3s} {'mean':>10s} {'median':>10s} {'stdev':>9s} {'min':>10s} {'95% CI':>23s}   vs first"]
    first = True
    for name, d in summary["arms"].items():
        vs = ""
        if not first:
            w = summary["vs_first"][name]
            p = "n/a" if w["p"] is None else f"{w['p']:.2g}"
            vs = f"x{w['ratio_of_means']:.3f} (Welch p={p})"
        first = False
        lines.append(f"{name:28s} {d['n']:3d} {d['mean']:10.4f} {d['median']:10.4f} {d['stdev']:9.4f} {d['min']:10.4f} "
                     f"[{d['ci95'][0]:10.4f},{d['ci95'][1]:10.4f}]   {vs}")
    a = summary["anova"]
    if a["F"] is not None:
        p = "n/a" if a["p"] is None else f"{a['p']:.3g}"
        lines.append(f"one-way ANOVA over the arms: F({a['df'][0]},{a['df'][1]}) = {a['F']:.2f}, p = {p}   [{unit}]")
    return "\n".join(lines)


def parse_result_line(text: str) -> float | None:
    m = RESULT_RE.search(text)
    return float(m.group(1)) if m else None


# ----------------------------------------------------------------------------- arms
def command_arm(cmd: str, timeout: float):
    def run() -> float:
        res = subprocess.run(shlex.split(cmd), capture_output=True, text=True, timeout=timeout)
        ms = parse_result_line(res.stdout)
        if res.returncode != 0 or ms is None:
            raise RuntimeError(f"{cmd!r}: exit {res.returncode}, no @@RESULT line\n{res.stdout[-400:]}\n{res.stderr[-400:]}")
        return ms
    return run


def inproc_arms(names: list[str], op: str, M: int, N: int, K: int, period: int, iters: int):
    """Builds the operands once and returns {arm name: callable -> ms per launch}."""
    import torch
    import siglip_b200
    from siglip_b200 import synth

    dev = "cuda"
    if op == "pe":
        p = synth.make_patch_embed(M, N, K, period, seed=0, device=dev, pixels=True)
    elif op == "fc1":
        p = synth.make_fc1(M, N, K, seed=0, device=dev)
    else:
        p = synth.make_fc2(M, N, K, seed=0, device=dev)
    eng = siglip_b200.Engine(0)
    sa = torch.tensor([p.scale_a], device=dev)
    sb = torch.tensor([p.scale_b], device=dev)
    d = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    tbl = eng.padded_table(p.table) if p.table is not None else None

    def ours():
        if op == "fc1":
            eng.fc1_gelu(p.A, p.B, p.bias, scale_a=sa, scale_b=sb, out=d)
        elif op == "fc2":
            eng.fc2_residual(p.A, p.B, p.bias, p.residual, scale_a=sa, scale_b=sb, out=d)
        else:
            eng.patch_embed(p.A, p.B, tbl, period=p.period, scale_a=sa, scale_b=sb, out=d)

    kp = p.A.stride(0)                                   # cuBLASLt wants K % 16 == 0: take K at the (zero-padded) pitch
    a8 = torch.as_strided(p.A, (M, kp), (kp, 1)).view(torch.float8_e4m3fn)
    b8 = torch.as_strided(p.B, (N, kp), (kp, 1)).view(torch.float8_e4m3fn)
    s_a = torch.tensor(p.scale_a, device=dev, dtype=torch.float32)
    s_b = torch.tensor(p.scale_b, device=dev, dtype=torch.float32)
    bias = p.bias if op != "pe" else None

    def gemm():
        return torch._scaled_mm(a8, b8.t(), scale_a=s_a, scale_b=s_b, bias=bias, out_dtype=torch.bfloat16)

    def unfused():
        if op == "fc1":
            return torch.nn.functional.gelu(gemm(), approximate="tanh")
        if op == "fc2":
            return gemm().add_(p.residual)
        return gemm().view(M // p.period, p.period, N).add_(p.table)

    def timed(fn, variant=None):
        def run() -> float:
            eng.set_variant(-1 if variant is None else variant)
            for _ in range(2):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            eng.device_status()
            return e0.elapsed_time(e1) / iters
        return run

    arms = {}
    for name in names:
        if name == "ours":
            arms[name] = timed(ours)
        elif name.startswith("ours:v"):
            arms[name] = timed(ours, int(name[6:]))
        elif name == "cublaslt":
            arms[name] = timed(gemm)
        elif name == "cublaslt_unfused":
            arms[name] = timed(unfused)
        else:
            raise ValueError(f"unknown in-process arm {name!r}")
    return arms


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--op", default="fc1", choices=["pe", "fc1", "fc2"])
    ap.add_argument("--M", type=int, default=46656)
    ap.add_argument("--N", type=int, default=4304)
    ap.add_argument("--K", type=int, default=1152)
    ap.add_argument("--period", type=int, default=729)
    ap.add_argument("--runs", type=int, default=10)
    ap.add_argument("--iters", type=int, default=10, help="launches per in-process run")
    ap.add_argument("--timeout", type=float, default=600.0, help="seconds per external command")
    ap.add_argument("--arms", default="ours,cublaslt,cublaslt_unfused")
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)

    specs = [s.strip() for s in a.arms.split(",") if s.strip()]
    inproc = [s for s in specs if "=" not in s]
    arms = {}
    if inproc:
        arms.update(inproc_arms(inproc, a.op, a.M, a.N, a.K, a.period, a.iters))
    for s in specs:
        if "=" in s:
            name, cmd = s.split("=", 1)
            arms[name] = command_arm(cmd, a.timeout)
    order = [s.split("=", 1)[0] for s in specs]
    samples = {n: [] for n in order}
    for _ in range(a.runs):
        for n in order:
            samples[n].append(arms[n]())
    summary = summarize(samples)
    summary["samples_ms"] = samples
    print(json.dumps(summary) if a.json else format_table(summary))
    return 0


if __name__ == "__main__":
    sys.exit(main())
