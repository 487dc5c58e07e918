#!/usr/bin/env python
"""Benchmark of the FP8 GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config C2]

A step is one pass of the hot path over one batch of synthetic operands: one fused-GEMM launch of
libsiglip_fp8.so.  The headline workload at every N is the configuration the metric is quoted on: SigLIP-So400m
FC1 + bias + GELU(tanh), M = 46 656 rows (64 images x 729 tokens), K = 1152, N = 4304, e4m3 operands with
per-tensor scales, bf16 output.  With N GPUs every rank runs that workload on its own 64 images (rows are
independent: no collective on the data path), so the headline scales weakly and `value` is the sum over ranks.

Rank 0 prints ONE JSON line:
  value / ms_per_step   K launches between one pair of CUDA events (a burst: a few milliseconds);
  launch_stats          the same launches timed one by one (an event pair per launch): min / median / mean;
  sustained             at least a second of back-to-back launches with NVML clock and power samples taken inside
                        it: what the kernel does once the 1 kW power cap has pulled the SM clock down;
  layers                C1, C3, C4 (the other configurations): an event pair per launch, the launches back to back,
                        and the same launches replayed from a CUDA graph (a Python loop enqueues a 10 us kernel more
                        slowly than the GPU runs it); each with its roofline and the cuBLASLt FP8 GEMM on the same operands;
  chain                 C5: FC1 + GELU -> e4m3 -> FC2 + residual on this rank's share of 1024 images (strong
                        scaling: the images are divided over the ranks), device-timed and end to end from pinned host
                        memory (sl8_mlp_chain_fp8_host);
  e2e                   the headline metric through the host-operand entry point (pinned host buffers, copies in the
                        timed region); host_link = the pinned-copy bandwidth all ranks reach at the same time.
`--impl reference` times the CPU restatement of the reference's algorithm on the host cores (the reference itself
is CUDA-only, so there is no CPU build of it to run).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "fp8_tflops_fc1_gelu"          # the default workload (C2); other --config values name their own layer
METRICS = {"C1": "fp8_tflops_patch_embed", "C2": METRIC, "C3": "fp8_tflops_fc2_residual", "C4": "fp8_tflops_patch_embed"}
UNIT = "TFLOP/s"


# DRAM bytes per launch of each layer's kernel at the FULL size of its configuration (dram__bytes_read.sum +
# dram__bytes_write.sum, one-pass ncu capture of launches 11 - 19 of this bench with the caches left as the previous
# launch left them: profiles/dram_traffic_full_size.md), per GEMM row so that a changed batch scales it.
NCU_DRAM_BYTES_PER_ROW = {"C2": (53.9e6 + 401.2e6) / 46656, "C3": (310.7e6 + 108.0e6) / 46656, "C4": (119.6e6 + 428.5e6) / 186624}


# ----------------------------------------------------------------------------- peaks
def measured_peaks() -> dict:
    """Roofline denominators: the measured copy bandwidth and bf16 GEMM rate of this pool's B200s when
    the driver wrote them; otherwise the stated fallback (6.65 TB/s, 1.59 PFLOP/s bf16).  The e4m3
    tensor-core rate is twice the bf16 rate of the same tensor cores, so the FP8 peak is 2 x bf16."""
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                    bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock, board power and throttle reasons through NVML (reads only) while a timed region runs."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, device_index: int, period_s: float = 0.001):
        self.samples, self.power, self.reasons = [], [], set()
        self.sm_max = None
        self._stop = threading.Event()
        self._thread = None
        self.period = period_s
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.sm_max = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _one(self):
        try:
            self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
            self.power.append(self.nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0)
            mask = self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
            for bit, name in self.REASONS.items():
                if mask & bit:
                    self.reasons.add(name)
        except Exception:
            pass

    def _run(self):
        while not self._stop.is_set():
            self._one()
            self._stop.wait(self.period)

    def start(self):
        if self.nv is None:
            return
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def stop(self, skip_fraction: float = 0.0) -> dict:
        """Median clock / power of the samples taken (the first `skip_fraction` of them dropped: the ramp)."""
        if self.nv is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable"], "samples": 0}
        self._one()
        self._stop.set()
        self._thread.join()
        k = int(len(self.samples) * skip_fraction)
        s = sorted(self.samples[k:])
        # NVML's power figure is a running average that lags the load by about a second: the last quarter of the
        # samples is the closest this leg gets to the settled value; the maximum is reported beside it
        pw = sorted(self.power[(3 * len(self.power)) // 4:])
        out = {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.sm_max, "reasons": sorted(self.reasons),
               "samples": len(s), "power_w": pw[len(pw) // 2] if pw else None, "power_w_max": max(self.power) if self.power else None}
        if len(s) < 10:
            out["note"] = "fewer than 10 NVML samples fit into the timed region: see `sustained` for clocks under load"
        return out


# ----------------------------------------------------------------------------- CPU arm
def cpu_oracle_rate(cfg_name: str, target_seconds: float, seed: int = 0):
    """Times the CPU restatement (oracle/) on a bounded row sample of the workload, all host threads.
    Returns (TFLOP/s, cores, description, seconds)."""
    from siglip_b200 import synth
    from tests.oracle_lib import Oracle
    orc = Oracle()
    # torchrun exports OMP_NUM_THREADS=1 to its ranks; the CPU arm is meant to use every core this process may run on.
    orc.lib.sl8o_set_num_threads(len(os.sched_getaffinity(0)))
    c = synth.CONFIGS[cfg_name]
    rows_per_image = c["M"] // c["images"]

    def run(images: int) -> float:
        p = synth.make_config(cfg_name, seed=seed, images=images)
        A, B = p.A.numpy(), p.B.numpy()
        bias = p.bias.view(torch.uint16).numpy() if p.bias is not None else None
        t0 = time.perf_counter()
        if p.op == synth.OP_FC1_GELU:
            orc.fc1_gelu(A, B, p.scale_a, p.scale_b, bias)
        elif p.op == synth.OP_FC2_RESIDUAL:
            orc.fc2_residual(A, B, p.scale_a, p.scale_b, bias, p.residual.view(torch.uint16).numpy())
        else:
            orc.patch_embed(A, B, p.scale_a, p.scale_b, p.table.view(torch.uint16).numpy())
        return time.perf_counter() - t0

    t1 = run(1)                                          # one image calibrates the sample size
    images = int(max(1, min(c["images"], target_seconds / max(t1, 1e-3))))
    t = run(images)
    flops = 2.0 * images * rows_per_image * c["N"] * c["K"]
    return flops / t / 1e12, orc.num_threads(), f"{images} of {c['images']} images ({images * rows_per_image} rows) of {cfg_name}", t


def reference_arm(args, rank: int, world: int) -> None:
    if rank != 0:
        return
    from siglip_b200 import synth
    c = synth.CONFIGS[args.config]
    vals = []
    sample = ""
    cores = 0
    per_step_target = max(1.0, min(10.0, 60.0 / max(1, args.steps + args.warmup)))
    for i in range(args.warmup + args.steps):
        v, cores, sample, _t = cpu_oracle_rate(args.config, per_step_target)
        if i >= args.warmup:
            vals.append(v)
    value = sum(vals) / len(vals)
    flops = 2.0 * c["M"] * c["N"] * c["K"]
    line = {
        "impl": "reference", "metric": METRICS.get(args.config, METRIC), "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": flops / (value * 1e12) * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.config),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference project is CUDA-only; this arm times the CPU restatement of its algorithm "
                "(FP32-accumulate GEMM over dequantised e4m3 + fused epilogue) on the host cores; "
                "ms_per_step is the full workload at the measured rate",
    }
    print(json.dumps(line), flush=True)


def workload_config(name: str, images=None) -> dict:
    from siglip_b200 import synth
    c = dict(synth.CONFIGS[name])
    if images is not None:
        c["M"], c["images"] = images * (c["M"] // c["images"]), images
    op = {0: "patch-embed + periodic table add", 1: "FC1 + bias + GELU(tanh)", 2: "FC2 + bias + residual"}[c["op"]]
    return {"workload": f"SigLIP {name}: {op}, M={c['M']} ({c['images']} images) K={c['K']} N={c['N']}, "
                        "e4m3 x e4m3 -> fp32 accumulate -> bf16, per-tensor scales",
            "per_gpu_rows": c["M"], "l2": "three operand sets rotated per step (working set > 126 MB L2)"}


# ----------------------------------------------------------------------------- GPU arm
IDLE_BEFORE_BURST_S = 1.0     # host sleep before a layer's burst legs (see layer_table)


def launch_fn(eng, p, dev):
    """Returns (callable(i) launching one step on operand set i, number of sets, list of outputs)."""
    from siglip_b200 import synth
    sa = torch.tensor([p.scale_a], device=dev)
    sb = torch.tensor([p.scale_b], device=dev)
    sets = 3

    def clone_pitched(t):                       # keeps the 16-byte row pitch of a K = 588 operand
        c = torch.empty_strided(t.shape, t.stride(), dtype=t.dtype, device=t.device)
        return c.copy_(t)

    As = [p.A] + [clone_pitched(p.A) for _ in range(sets - 1)]
    Ds = [torch.empty((p.M, p.N), dtype=torch.bfloat16, device=dev) for _ in range(sets)]
    if p.op == synth.OP_FC1_GELU:
        return (lambda i: eng.fc1_gelu(As[i % sets], p.B, p.bias, scale_a=sa, scale_b=sb, out=Ds[i % sets])), sets, Ds
    if p.op == synth.OP_FC2_RESIDUAL:
        Rs = [p.residual] + [p.residual.clone() for _ in range(sets - 1)]
        return (lambda i: eng.fc2_residual(As[i % sets], p.B, p.bias, Rs[i % sets], scale_a=sa, scale_b=sb,
                                           out=Ds[i % sets])), sets, Ds
    table = eng.padded_table(p.table)            # rows past the period repeat it, as in the reference's padded table
    return (lambda i: eng.patch_embed(As[i % sets], p.B, table, period=p.period, scale_a=sa, scale_b=sb,
                                      out=Ds[i % sets])), sets, Ds


def time_steps(fn, steps: int, warmup: int, barrier) -> float:
    """ms per step: `warmup` untimed steps, then `steps` timed ones between two CUDA events on the
    stream the kernels are launched on, a barrier and a device synchronise on both sides."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    barrier()
    return e0.elapsed_time(e1) / steps


def time_graph_replay(fn, launches: int, replays: int = 4):
    """ms per launch when `launches` calls are captured once into a CUDA graph and the graph is replayed: what the
    GPU needs per launch when the host's enqueue cost (which bounds a Python loop around a kernel of a few
    microseconds) is out of the way.  None if the capture fails."""
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            # (thread-local capture mode: the NCCL watchdog and the NVML sampler threads are none of its business)
            with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
                for i in range(launches):
                    fn(i)
        torch.cuda.synchronize()
        graph.replay()                                  # warm
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(replays):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / (replays * launches)
        del graph
        return ms
    except Exception as exc:                            # a bench leg that cannot run must not take the line with it
        sys.stderr.write(f"bench: graph replay skipped ({type(exc).__name__}: {exc})\n")
        torch.cuda.synchronize()
        return None


def time_per_launch(fn, launches: int, warmup: int = 3) -> dict:
    """An event pair around every launch (on the launching stream): min / median / mean in ms."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(launches)]
    for i, (a, b) in enumerate(ev):
        a.record()
        fn(i)
        b.record()
    torch.cuda.synchronize()
    t = sorted(a.elapsed_time(b) for a, b in ev)
    return {"ms_min": t[0], "ms_median": t[len(t) // 2], "ms_mean": sum(t) / len(t), "launches": launches}


def sustained_leg(fn, flops: float, device_index: int, seconds: float, barrier) -> dict:
    """Back-to-back launches for at least `seconds`, NVML sampled inside: the rate under the power cap.
    Nothing about the GPU is set or reset; the clock is whatever the power management gives."""
    est = time_steps(fn, 20, 3, lambda: None)
    n = max(50, int(seconds * 1e3 / est))
    sampler = ClockSampler(device_index, 0.002)
    torch.cuda.synchronize()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.start()
    e0.record()
    for i in range(n):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop(skip_fraction=0.25)
    barrier()
    ms = e0.elapsed_time(e1) / n
    out = {"launches": n, "seconds": e0.elapsed_time(e1) / 1e3, "ms_per_step": ms, "tflops": flops / ms / 1e9, "clocks": clocks}
    if clocks.get("sm_mhz"):
        out["mhz_x_ms"] = clocks["sm_mhz"] * ms            # SM clock cycles per launch / 1000
        out["tflops_at_max_clock"] = out["tflops"] * clocks["sm_max_mhz"] / clocks["sm_mhz"]
    if clocks.get("power_w"):
        out["mj_per_launch"] = clocks["power_w"] * ms       # W x ms
    return out


def trace_leg(eng, fn, p, ms_untraced: float) -> dict:
    """SM clock cycles the kernel takes, from its own clock64 totals (tracing in its totals-only mode): the SM clock
    inside the kernel (cycles / event time), cycles per tile and per k-block, how often the MMA thread found the
    next stage still filling, and what the MMA thread and the epilogue waited for each other."""
    eng.trace_enable(True, coarse=True)
    for i in range(5):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n = 20
    e0.record()
    for i in range(n):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / n
    rec = eng.trace_read()
    eng.device_status()
    eng.trace_enable(False)
    cfg = eng.query_config(p.op, p.M, p.N, p.K)
    lead = rec[::cfg["cta_group"]]                  # the CTAs that issue MMAs
    tiles = sum(r["tiles"] for r in lead) / len(lead)
    cyc = [r["mma_total"] for r in lead]
    kb = (p.K + cfg["tile_k"] - 1) // cfg["tile_k"]
    mean = sum(cyc) / len(cyc)
    return {"ms_per_launch_traced": ms, "ms_per_launch_untraced": ms_untraced, "cycles_max": max(cyc), "cycles_mean": mean,
            "sm_ghz_in_kernel": max(cyc) / ms / 1e6, "tiles_per_cluster": tiles, "cycles_per_tile": mean / tiles,
            "cycles_per_k_block": mean / tiles / kb, "k_blocks_per_tile": kb,
            "k_blocks_whose_operands_were_late_pct": 100.0 * sum(r["mma_wait_operands"] for r in lead) / len(lead) / tiles / kb,
            "mma_waits_for_accumulator_cycles_per_tile": sum(r["mma_wait_accumulator"] for r in lead) / len(lead) / tiles,
            "epilogue_waits_for_accumulator_cycles_per_tile": sum(r["epi_wait_accumulator"] for r in rec) / len(rec) / tiles,
            "note": "a tcgen05.mma of a CTA pair (M 256, N 256, K 32) takes 128 cycles: 512 per full k-block of four"}


def host_link_bandwidth(dev, barrier, mib: int = 256) -> dict:
    """Pinned host <-> device copy rate of this rank with both directions (and every other rank) busy at once."""
    n = mib << 20
    h_up = torch.empty(n, dtype=torch.uint8).pin_memory()
    h_dn = torch.empty(n, dtype=torch.uint8).pin_memory()
    d_up = torch.empty(n, dtype=torch.uint8, device=dev)
    d_dn = torch.zeros(n, dtype=torch.uint8, device=dev)
    s_up, s_dn = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    for _ in range(2):
        d_up.copy_(h_up, non_blocking=True)
    torch.cuda.synchronize()
    barrier()
    reps = 4
    t0 = time.perf_counter()
    for _ in range(reps):
        with torch.cuda.stream(s_up):
            d_up.copy_(h_up, non_blocking=True)
        with torch.cuda.stream(s_dn):
            h_dn.copy_(d_dn, non_blocking=True)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    barrier()
    return {"h2d_gbs": reps * n / dt / 1e9, "d2h_gbs": reps * n / dt / 1e9, "mib_per_copy": mib, "both_directions_at_once": True}


def cublaslt_baseline(p, dev, steps: int) -> dict:
    """cuBLASLt per-tensor-scaled FP8 GEMM on the same operands (through torch._scaled_mm), as the reference's
    bench/cublas_bench.cu times it: GEMM alone (bias fused where the layer has one) and GEMM followed by the
    layer's epilogue as separate elementwise kernels.  K is taken at the operands' row pitch (the padding is
    zero), because cuBLASLt wants K % 16 == 0."""
    from siglip_b200 import synth
    try:
        kp = p.A.stride(0)
        A = torch.as_strided(p.A, (p.M, kp), (kp, 1)).view(torch.float8_e4m3fn)
        B = torch.as_strided(p.B, (p.N, kp), (kp, 1)).view(torch.float8_e4m3fn)
        sa = torch.tensor(p.scale_a, device=dev, dtype=torch.float32)
        sb = torch.tensor(p.scale_b, device=dev, dtype=torch.float32)
        bias = p.bias if p.op != synth.OP_PATCH_EMBED else None
        gemm = lambda i=0: torch._scaled_mm(A, B.t(), scale_a=sa, scale_b=sb, bias=bias, out_dtype=torch.bfloat16)
        if p.op == synth.OP_FC1_GELU:
            full = lambda i=0: torch.nn.functional.gelu(gemm(), approximate="tanh")
        elif p.op == synth.OP_FC2_RESIDUAL:
            full = lambda i=0: gemm().add_(p.residual)
        else:
            imgs = p.M // p.period
            full = lambda i=0: gemm().view(imgs, p.period, p.N).add_(p.table)
        torch.cuda.synchronize()
        time.sleep(IDLE_BEFORE_BURST_S)          # the baseline starts from an idle GPU like the legs it is compared with
        t_gemm = time_steps(gemm, steps, 3, lambda: None)
        torch.cuda.synchronize()
        time.sleep(IDLE_BEFORE_BURST_S)
        t_full = time_steps(full, steps, 3, lambda: None)
        return {"torch_scaled_mm_gemm_ms": t_gemm, "torch_scaled_mm_gemm_tflops": p.flops() / t_gemm / 1e9,
                "torch_scaled_mm_plus_epilogue_kernels_ms": t_full}
    except Exception as e:          # a torch build without _scaled_mm for this shape: report, do not fail the bench
        return {"torch_scaled_mm_error": f"{type(e).__name__}: {str(e)[:160]}"}


def host_baselines(name: str, runs: int = 20) -> dict:
    """cuBLASLt FP8 and the reference's own kernels on the configuration's shape, timed by the C++ bench host
    (siglip_b200/lib/siglip_bench) on seeded random codes: cuBLASLt through cublasLtMatmul with per-tensor scale pointers,
    the best of its heuristics, bare and with the layer's epilogue fused (GELU_BIAS; BIAS + residual as C with beta = 1;
    the table tiled to M rows as C with beta = 1); the reference kernels through oracle/_ref (baseline code, never on
    the product path; the column is left out where that build is absent)."""
    import subprocess
    exe = ROOT / "siglip_b200" / "lib" / "siglip_bench"
    out = {}
    if not exe.exists():
        return {"host_baselines_error": f"{exe} not built"}

    def run(impl):
        try:
            r = subprocess.run([str(exe), "--config", name, "--data", "random", "--impl", impl, "--runs", str(runs)],
                               capture_output=True, text=True, timeout=300)
            lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
            return json.loads(lines[-1]) if r.returncode == 0 and lines else None
        except Exception:
            return None

    lt = run("cublaslt")
    if lt:
        out.update({"cublaslt_gemm_ms": lt["gemm_ms"], "cublaslt_fused_ms": lt["fused_ms"], "cublaslt_fused": lt["fused"],
                    "cublaslt_heuristics_tried": lt["gemm_heuristics"], "cublaslt_fused_vs_this_library_max_rel_diff": lt["max_rel_diff_vs_new"]})
    else:
        out["cublaslt_error"] = "siglip_bench --impl cublaslt failed"
    so = {"C1": "pe", "C2": "fc1_so400m", "C3": "fc2_so400m", "C4": "pe_so400m"}[name]
    if (ROOT / "oracle" / "_ref" / f"libsl8_ref_{so}.so").exists() and name != "C1":      # the B/16 build is shaped for 928 256 rows
        rf = run("ref")
        if rf:
            out.update({"reference_ms": rf["ms"], "reference_build": f"oracle/_ref/libsl8_ref_{so}.so (zero-padded shape)"})
    return out


def reference_protocol_leg() -> dict:
    """The reference's own headline, on its own protocol: patch-embed at SigLIP-B/16, M = 928 256 rows, N = K = 768, the
    constant operands of its bench host, 2 warm-up + 10 timed launches under one event pair, its 32 spot checks -- run by the
    C++ host and read from the @@RESULT line its drivers parse.  The reference publishes 0.519 ms / 2108 TFLOP/s for its
    best build and 0.524 ms / 2090 TFLOP/s for its default one (CLAUDE.md:8,269); constant operands toggle few bits, so
    this figure is not comparable with the seeded random operands of every other number in this line."""
    import re
    import subprocess
    exe = ROOT / "siglip_b200" / "lib" / "siglip_bench"
    try:
        r = subprocess.run([str(exe), "--layer", "pe"], capture_output=True, text=True, timeout=300)
        m = re.search(r"@@RESULT ms=([0-9.]+) tflops=([0-9.]+) checksum=([0-9.]+) valid=([01])", r.stdout)
        if not m:
            return {"error": "no @@RESULT line"}
        ms, tf = float(m.group(1)), float(m.group(2))
        return {"workload": "SigLIP-B/16 patch-embed + table, M=928256 N=768 K=768, the reference harness's constant operands and protocol",
                "ms": ms, "tflops": tf, "valid": int(m.group(4)), "published_ms": 0.519, "published_tflops": 2108.0,
                "vs_published": tf / 2108.0, "published_source": "reference CLAUDE.md:8 (best tuned build; default build 0.524 ms)"}
    except Exception as e:
        return {"error": f"{type(e).__name__}: {str(e)[:120]}"}


def roofline_of(p, ms: float, peaks: dict, traffic=None) -> dict:
    """Roofline object of one layer: tensor-bound layers against 2 x the measured bf16 GEMM rate (the e4m3 MMA rate is
    twice bf16 on the same tensor cores), the HBM-bound one (patch-embed at K = 588) against the measured copy rate."""
    from siglip_b200 import synth
    tf = p.flops() / ms / 1e9
    gbs = p.min_bytes() / ms / 1e6
    # patch-embed at the So400m shape moves more bytes per FLOP than the machine balance: HBM-bound on paper
    hbm_bound = p.op == synth.OP_PATCH_EMBED and (p.min_bytes() / peaks["hbm_gbs"]) > (p.flops() / (2e3 * peaks["bf16_tflops"]))
    if hbm_bound:
        return {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                "traffic": traffic, "peak_source": f"{peaks['source']} copy bandwidth", "tflops": tf,
                "frac_of_nominal_4500": tf / 4500.0}
    peak = 2.0 * peaks["bf16_tflops"]
    return {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak, "traffic": traffic,
            "peak_source": f"2 x bf16 burst GEMM rate of {peaks['source']} MEASURED_PEAKS (e4m3 MMA rate is twice bf16)",
            "frac_of_nominal_4500": tf / 4500.0, "hbm_gbs_algorithmic": gbs}


def layer_table(eng, dev, launches: int, peaks: dict, names=("C1", "C3", "C4"), host: bool = True) -> dict:
    """The other configurations, timed launch by launch (an event pair per launch, three rotating operand sets,
    3 warm-up launches), each beside cuBLASLt's FP8 GEMM on the same operands."""
    from siglip_b200 import synth
    out = {}
    for name in names:
        p = synth.make_config(name, seed=0, device=dev)
        fn, _, _ = launch_fn(eng, p, dev)
        # Like the headline, which is the first thing a fresh process times, each layer's bursts start from a GPU that
        # has idled: right after seconds of dense launches the power limiter is still engaged and the same 20 launches
        # take up to 20 % longer (patch-embed C4: 166 us after an idle second, 200 us right behind 2 s of FC1).
        torch.cuda.synchronize()
        time.sleep(IDLE_BEFORE_BURST_S)
        st = time_per_launch(fn, launches)
        eng.device_status()
        b2b = time_steps(fn, launches, 3, lambda: None)          # no events between the launches
        replay = time_graph_replay(fn, launches)                 # the same launches replayed from a CUDA graph
        eng.device_status()
        # the derived figures use the shortest of the three: around a kernel of a few microseconds the two event
        # records cost as much as the kernel itself, and a Python loop enqueues more slowly than the GPU finishes
        ms = min(t for t in (st["ms_median"], b2b, replay) if t)
        row = dict(st)
        row["ms_back_to_back"] = b2b
        row["ms_graph_replay"] = replay
        row["ms_used_for_rates"] = ms
        row["idle_before_s"] = IDLE_BEFORE_BURST_S
        row.update({"tflops": p.flops() / ms / 1e9, "gbs": p.min_bytes() / ms / 1e6,
                    "images_per_s": synth.CONFIGS[name]["images"] / ms * 1e3,
                    "roofline": roofline_of(p, ms, peaks, traffic=NCU_DRAM_BYTES_PER_ROW[name] * p.M if name in NCU_DRAM_BYTES_PER_ROW else None),
                    "kernel_config": eng.query_config(p.op, p.M, p.N, p.K),
                    "workload": workload_config(name)["workload"]})
        del fn
        row.update(cublaslt_baseline(p, dev, launches))
        out[name] = row
        del p
        torch.cuda.empty_cache()
    for name in names if host else ():     # the C++ host's arms run as child processes (on GPU 0: rank 0 only)
        out[name].update(host_baselines(name))
    return out


def prep_table(eng, dev, steps: int, peaks: dict) -> dict:
    """The producer-side steps at the C4 / C2 sizes: HBM-bound byte work, reported against the measured copy bandwidth.
    Algorithmic bytes: patch unfold reads the used pixels (fp32) once and writes the operand rows at their pitch;
    abs-max reads the activation once; quantisation reads it once and writes one byte per element.  Each working
    set exceeds the 126 MB L2."""
    out = {}
    images, P = 256, 14
    g = torch.Generator(device=dev).manual_seed(0)
    pixels = torch.rand((images, 3, 384, 384), generator=g, device=dev) * 2 - 1
    scale = torch.tensor([1.0 / 448.0], device=dev)
    A = eng.patchify_quantize(pixels, P, scale)
    ms = time_steps(lambda i=0: eng.patchify_quantize(pixels, P, scale, out=A), steps, 3, lambda: None)
    nbytes = images * 3 * (27 * P) ** 2 * 4 + A.shape[0] * A.stride(0)
    out["patchify_quantize_C4"] = {"ms": ms, "gbs": nbytes / ms / 1e6, "frac_hbm_measured": nbytes / ms / 1e6 / peaks["hbm_gbs"],
                                   "bytes": nbytes, "images_per_s": images / ms * 1e3}
    del pixels, A
    x = (torch.randn((46656, 4304), generator=g, device=dev) * 0.5).to(torch.bfloat16)
    amax, sc = eng.amax_scale(x)
    ms = time_steps(lambda i=0: eng.amax_scale(x), steps, 3, lambda: None)
    nbytes = x.numel() * 2
    out["amax_scale_C2_output"] = {"ms": ms, "gbs": nbytes / ms / 1e6, "frac_hbm_measured": nbytes / ms / 1e6 / peaks["hbm_gbs"], "bytes": nbytes}
    q = eng.quantize_e4m3(x, sc)
    ms = time_steps(lambda i=0: eng.quantize_e4m3(x, sc, out=q), steps, 3, lambda: None)
    nbytes = x.numel() * 3
    out["quantize_e4m3_C2_output"] = {"ms": ms, "gbs": nbytes / ms / 1e6, "frac_hbm_measured": nbytes / ms / 1e6 / peaks["hbm_gbs"], "bytes": nbytes}
    del q
    xr = torch.randn((186624, 1152), generator=g, device=dev).to(torch.bfloat16)     # 256 images of residual stream
    gamma = torch.ones((1152,), device=dev)
    beta = torch.zeros((1152,), device=dev)
    ln = eng.layernorm_quantize(xr, gamma, beta, 1e-6, sc)
    ms = time_steps(lambda i=0: eng.layernorm_quantize(xr, gamma, beta, 1e-6, sc, out=ln), steps, 3, lambda: None)
    nbytes = xr.numel() * 3
    out["layernorm_quantize_256_images"] = {"ms": ms, "gbs": nbytes / ms / 1e6, "frac_hbm_measured": nbytes / ms / 1e6 / peaks["hbm_gbs"], "bytes": nbytes}
    eng.device_status()
    return out


def chain_leg(eng, dev, rank: int, world: int, barrier, dist, total_images: int, steps: int, warmup: int, peaks: dict,
              e2e: bool = True) -> dict:
    """C5: the MLP chain FC1 + GELU -> e4m3 -> FC2 + residual on this rank's share of `total_images` images
    (M = 746 496 rows in total at 1024; strong scaling: the images are divided over the ranks, no data crosses
    GPUs).  Device-timed (max over ranks) and, with `e2e`, end to end from pinned host memory."""
    from siglip_b200 import synth
    from siglip_b200.shard import image_range
    _, n_img = image_range(total_images, world, rank)
    M = n_img * 729
    d_model, d_ff = 1152, 4304
    p1 = synth.make_fc1(M, d_ff, d_model, seed=rank, device=dev)
    w2 = synth.make_fc2(729, d_model, d_ff, seed=rank, device=dev)          # FC2 weights and bias
    g = torch.Generator(device=dev).manual_seed(1000 + rank)
    residual = torch.randn((M, d_model), generator=g, device=dev).to(torch.bfloat16)
    sa1, sb1 = torch.tensor([p1.scale_a], device=dev), torch.tensor([p1.scale_b], device=dev)
    sb2 = torch.tensor([w2.scale_b], device=dev)
    # static activation scale of the hidden layer: amax / 448 of a one-image calibration pass
    cal = eng.fc1_gelu(p1.A[:729], p1.B, p1.bias, scale_a=sa1, scale_b=sb1)
    h_scale_f = float(cal.float().abs().max()) / 448.0
    h_scale = torch.tensor([h_scale_f], device=dev)
    H = torch.empty((M, synth.pitch128(d_ff)), dtype=torch.uint8, device=dev)[:, :d_ff]
    D = torch.empty((M, d_model), dtype=torch.bfloat16, device=dev)

    def step(i):
        eng.mlp_chain(p1.A, p1.B, p1.bias, w2.B, w2.bias, residual, scale_a=sa1, scale_w1=sb1, scale_w2=sb2,
                      hidden_scale=h_scale, hidden=H, out=D)

    torch.cuda.synchronize()
    time.sleep(IDLE_BEFORE_BURST_S)              # the same starting point as the headline and the layers: an idle GPU
    ms = time_steps(step, steps, warmup, barrier)
    eng.device_status()
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t)
    flops = 2.0 * 2.0 * total_images * 729 * d_ff * d_model
    tf = flops / ms_max / 1e9
    out = {"workload": f"SigLIP C5: MLP chain FC1+GELU (e4m3 out) -> FC2+residual, {total_images} images "
                       f"(M={total_images * 729}) split by image over {world} GPU(s), K/N 1152/4304; one step's operands "
                       "(> 0.9 GB per GPU even at 8 GPUs) exceed the 126 MB L2",
           "scaling": "strong", "images": total_images, "images_this_rank": n_img, "steps": steps, "warmup": warmup,
           "ms": ms_max, "images_per_s": total_images / ms_max * 1e3, "tflops": tf, "gpu_launches": 2 * steps,
           "kernel_config": {"fc1": eng.query_config(synth.OP_FC1_GELU, M, d_ff, d_model, 1),
                             "fc2": eng.query_config(synth.OP_FC2_RESIDUAL, M, d_model, d_ff)},
           "roofline": {"bound": "tensor", "achieved": tf / world, "peak": 2.0 * peaks["bf16_tflops"], "unit": "TFLOP/s",
                        "frac": tf / world / (2.0 * peaks["bf16_tflops"]), "traffic": None,
                        "frac_of_nominal_4500": tf / world / 4500.0}}
    if e2e:
        A_h = torch.zeros((M, p1.A.stride(0)), dtype=torch.uint8).pin_memory()[:, :d_model]
        A_h.copy_(p1.A)
        R_h = residual.cpu().pin_memory()
        D_h = torch.empty((M, d_model), dtype=torch.bfloat16).pin_memory()
        W1_h = torch.zeros((d_ff, p1.B.stride(0)), dtype=torch.uint8).pin_memory()[:, :d_model]
        W1_h.copy_(p1.B)
        W2_h = torch.zeros((d_model, w2.B.stride(0)), dtype=torch.uint8).pin_memory()[:, :d_ff]
        W2_h.copy_(w2.B)
        b1_h, b2_h = p1.bias.cpu().pin_memory(), w2.bias.cpu().pin_memory()
        run = lambda: eng.mlp_chain_host(A_h, W1_h, b1_h, W2_h, b2_h, R_h, D_h, scale_a=p1.scale_a, scale_w1=p1.scale_b,
                                         scale_w2=w2.scale_b, hidden_scale=h_scale_f)
        run()
        torch.cuda.synchronize()
        barrier()
        n = 3
        t0 = time.perf_counter()
        for _ in range(n):
            run()                                                 # blocking: returns when D is in host memory
        e_ms = (time.perf_counter() - t0) / n * 1e3
        barrier()
        t = torch.tensor([e_ms], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e_ms_max = float(t)
        same = torch.equal(D_h.to(dev).view(torch.uint16), D.view(torch.uint16))
        out["e2e"] = {"ms": e_ms_max, "images_per_s": total_images / e_ms_max * 1e3, "tflops": flops / e_ms_max / 1e9,
                      "h2d_bytes_per_step": int(M * p1.A.stride(0) + M * d_model * 2 + d_ff * p1.B.stride(0) + d_model * w2.B.stride(0)
                                                + 2 * d_ff + 2 * d_model + 16),
                      "d2h_bytes_per_step": int(M * d_model * 2), "steps": n, "matches_device_path": bool(same),
                      "note": "per rank; the hidden activations (M x 4304 e4m3) stay on the GPU"}
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="C2", choices=["C1", "C2", "C3", "C4", "C5"],
                    help="headline workload (C5: the chain leg alone, printed as its own line)")
    ap.add_argument("--no-layers", action="store_true", help="skip the per-layer table (C1, C3, C4)")
    ap.add_argument("--layers", action="store_true", help="accepted for compatibility: the table is on by default")
    ap.add_argument("--layer-names", default="C1,C3,C4", help="which configurations the per-layer table covers")
    ap.add_argument("--no-chain", action="store_true", help="skip the C5 chain leg")
    ap.add_argument("--no-sustained", action="store_true", help="skip the >= 1 s sustained leg")
    ap.add_argument("--sustained-seconds", type=float, default=1.0)
    ap.add_argument("--prep", action="store_true", help="add the producer-side steps (patch unfold, quantise, LayerNorm)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--variant", type=int, default=-1, help="force a kernel variant (sweeps)")
    ap.add_argument("--images", type=int, default=None, help="override the batch (profiling captures use a smaller case)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-operand legs (profiling captures)")
    ap.add_argument("--only-headline", action="store_true", help="headline launches only: what a profiler capture wants")
    ap.add_argument("--trace", action="store_true",
                    help="add `trace`: in-kernel clock-cycle totals of the headline kernel (sl8_trace_enable, totals only: the hot loops stay untimed)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.only_headline:
        args.no_layers = args.no_chain = args.no_sustained = args.no_e2e = args.no_cpu_baseline = True

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        reference_arm(args, rank, world)
        return

    import torch.distributed as dist
    from siglip_b200 import Engine, synth

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: there is no CPU fallback for the hot path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        barrier = lambda: dist.barrier()
    else:
        barrier = lambda: None

    peaks = measured_peaks()
    eng = Engine(local_rank)
    if args.variant >= 0:
        eng.set_variant(args.variant)
    if args.config == "C5":
        c = chain_leg(eng, dev, rank, world, barrier, dist, 1024 if args.images is None else args.images, args.steps,
                      args.warmup, peaks, e2e=not args.no_e2e)
        if rank == 0:
            print(json.dumps({"metric": "fp8_tflops_mlp_chain", "value": c["tflops"], "unit": UNIT, "n_gpus": world,
                              "steps": args.steps, "warmup": args.warmup, "ms_per_step": c["ms"], "higher_is_better": True,
                              "scaling": "strong", "vs_baseline": None, "dtype": "e4m3 x e4m3 -> f32", "data": "synthetic",
                              "config": {"workload": c["workload"]}, "images_per_s": c["images_per_s"],
                              "gpu_launches": c["gpu_launches"], "roofline": c["roofline"], "chain": c}), flush=True)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
    p = synth.make_config(args.config, seed=rank, device=dev, images=args.images)
    n_images = synth.CONFIGS[args.config]["images"] if args.images is None else args.images
    fn, _, Ds = launch_fn(eng, p, dev)
    out_bytes = p.M * p.N * 2

    # ---- headline: exactly K launches between one pair of events
    sampler = ClockSampler(local_rank)
    for i in range(args.warmup):
        fn(i)
    torch.cuda.synchronize()
    barrier()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    barrier()
    eng.device_status()
    ms = e0.elapsed_time(e1) / args.steps
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t)
    flops = p.flops()
    value = world * flops / ms_max / 1e9                      # TFLOP/s, all ranks

    trace = None
    if args.trace and rank == 0:
        trace = trace_leg(eng, fn, p, ms)
    launch_stats = time_per_launch(fn, max(20, min(args.steps, 100))) if not args.only_headline else None
    sustained = None
    if not args.no_sustained:
        sustained = sustained_leg(fn, flops, local_rank, args.sustained_seconds, barrier)
        t = torch.tensor([sustained["ms_per_step"]], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sustained["ms_per_step_max_over_ranks"] = float(t)
        sustained["tflops_all_ranks"] = world * flops / float(t) / 1e9
        # like against like: a second of launches against the cuBLAS bf16 GEMM held for seconds under the same power cap
        sustained["peak_sustained"] = 2.0 * peaks["bf16_tflops_sustained"]
        sustained["frac_of_sustained_peak"] = sustained["tflops"] / sustained["peak_sustained"]
        sustained["peak_source"] = f"2 x sustained bf16 GEMM rate of {peaks['source']} MEASURED_PEAKS"
        eng.device_status()

    e2e_value, e2e_ms_max, e2e_steps, same, side_bytes = None, None, 0, True, 0
    link = None
    if not args.no_e2e:
        link = host_link_bandwidth(dev, barrier)
        if world > 1:
            for k in ("h2d_gbs", "d2h_gbs"):
                tt = torch.tensor([link[k]], device=dev, dtype=torch.float64)
                dist.all_reduce(tt, op=dist.ReduceOp.SUM)
                link[k + "_all_ranks"] = float(tt)
        # ---- end to end: pinned host operands through the *_host entry point
        A_h = torch.zeros((p.M, p.A.stride(0)), dtype=torch.uint8).pin_memory()[:, :p.K]
        A_h.copy_(p.A)
        B_h = torch.zeros((p.N, p.B.stride(0)), dtype=torch.uint8).pin_memory()[:, :p.K]      # keeps the 16-byte row pitch of K = 588
        B_h.copy_(p.B)
        D_h = torch.empty((p.M, p.N), dtype=torch.bfloat16).pin_memory()
        side_h = None
        if p.op == synth.OP_FC1_GELU:
            bias_h = p.bias.cpu().pin_memory()
            e2e_fn = lambda: eng.fc1_gelu_host(A_h, B_h, bias_h, D_h, scale_a=p.scale_a, scale_b=p.scale_b)
            side_bytes = bias_h.numel() * 2
        elif p.op == synth.OP_FC2_RESIDUAL:
            bias_h = p.bias.cpu().pin_memory()
            side_h = p.residual.cpu().pin_memory()
            e2e_fn = lambda: eng.fc2_residual_host(A_h, B_h, bias_h, side_h, D_h, scale_a=p.scale_a, scale_b=p.scale_b)
            side_bytes = bias_h.numel() * 2 + side_h.numel() * 2
        else:
            side_h = eng.padded_table(p.table).cpu().pin_memory()
            e2e_fn = lambda: eng.patch_embed_host(A_h, B_h, side_h, D_h, period=p.period, scale_a=p.scale_a, scale_b=p.scale_b)
            side_bytes = side_h.numel() * 2
        e2e_steps = max(3, min(args.steps, 10))
        e2e_fn()
        torch.cuda.synchronize()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_fn()                                              # blocking: returns when D is in host memory
        e2e_ms = (time.perf_counter() - t0) / e2e_steps * 1e3
        barrier()
        t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms_max = float(t)
        e2e_value = world * flops / e2e_ms_max / 1e9
        same = torch.equal(D_h.to(dev).view(torch.uint16), Ds[0].view(torch.uint16)) if rank == 0 else True
        del A_h, B_h, D_h, side_h

    # ---- C5 chain on this rank's share of 1024 images (every rank takes part: max over ranks)
    chain = None
    if not args.no_chain:
        del fn
        torch.cuda.empty_cache()
        chain = chain_leg(eng, dev, rank, world, barrier, dist, 1024, max(3, min(args.steps, 10)), 3, peaks, e2e=not args.no_e2e)
        torch.cuda.empty_cache()
        fn, _, Ds = launch_fn(eng, p, dev)

    if rank == 0:
        line = {
            "metric": METRICS.get(args.config, METRIC), "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_max, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "e4m3 x e4m3 -> f32", "data": "synthetic", "config": workload_config(args.config, args.images),
            "clocks": clocks, "gpu_launches": args.steps,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(p.M * p.A.stride(0) + p.N * p.B.stride(0) + side_bytes + 12),
                    "d2h_bytes_per_step": int(out_bytes), "ms_per_step": e2e_ms_max, "steps": e2e_steps,
                    "matches_device_path": bool(same), "host_link": link},
            "images_per_s": world * n_images / ms_max * 1e3,
            "kernel_config": eng.query_config(p.op, p.M, p.N, p.K),
        }
        if trace:
            line["trace"] = trace
        if launch_stats:
            line["launch_stats"] = launch_stats
        if sustained:
            line["sustained"] = sustained
        per_row = NCU_DRAM_BYTES_PER_ROW.get(args.config)
        line["roofline"] = roofline_of(p, ms, peaks, traffic=None if per_row is None else per_row * p.M)
        line["roofline"]["traffic_note"] = ("DRAM bytes per launch from a one-pass ncu capture of this bench at full size, caches left as the "
                                            "previous launch left them (profiles/dram_traffic_full_size.md); algorithmic bytes: "
                                            f"{p.min_bytes():.0f}")
        line["roofline"]["power_note"] = ("the board sits at its 1 kW power cap under these kernels (sw_power_cap): the SM clock, not "
                                          "the tensor pipe or HBM, sets the rate; see `sustained`")
        if not args.no_cpu_baseline and world == 1:      # a reported baseline of the one-GPU run only
            v, cores, sample, secs = cpu_oracle_rate(args.config, args.cpu_seconds)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample,
                                    "seconds": secs}
        if chain:
            line["chain"] = chain
        if not args.no_layers and args.config in ("C1", "C2", "C3", "C4"):
            line["baselines"] = host_baselines(args.config)
            line["reference_protocol"] = reference_protocol_leg()
    if not args.no_layers:
        # every rank runs the table on its own GPU (the ranks stay in step); rank 0 reports its own
        tab = layer_table(eng, dev, max(20, min(args.steps, 100)), peaks, tuple(n for n in args.layer_names.split(",") if n), host=(rank == 0))
        if rank == 0:
            line["layers"] = tab
    if args.prep and rank == 0:
        line["prep"] = prep_table(eng, dev, max(20, min(args.steps, 100)), peaks)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
