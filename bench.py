#!/usr/bin/env python
"""Benchmark of the FP8 GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config C2] [--layers]

A step is one pass of the hot path over one batch of synthetic operands: one fused-GEMM
launch of libsiglip_fp8.so.  The workload at every N is the configuration the headline
metric is quoted on: SigLIP-So400m FC1 + bias + GELU(tanh), M = 46 656 rows (64 images x 729
tokens), K = 1152, N = 4304, e4m3 operands with per-tensor scales, bf16 output.  With N GPUs
every rank runs that workload on its own 64 images (rows are independent: no collective on
the data path), so the scaling is weak and `value` is the sum over ranks.

Rank 0 prints ONE JSON line.  `value` is TFLOP/s (2*M*N*K with the unpadded K and N) with the
operands resident in HBM; `e2e` is the same metric through the host-operand entry point
(pinned host buffers, host->device and device->host copies inside the timed region).
`--impl reference` times the CPU restatement of the reference's algorithm on the host cores
(the reference itself is CUDA-only, so there is no CPU build of it to run).
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


# DRAM bytes per GEMM row of the dominant kernel, from one `ncu --set full` capture per configuration on a
# smaller case (profiles/*_ncu.md: dram__bytes_read.sum + dram__bytes_write.sum divided by the rows of the
# captured launch).  Traffic grows in proportion to the rows, so a full launch is this figure times M.
NCU_DRAM_BYTES_PER_ROW = {"C2": 319.79e6 / 37908, "C3": 325.66e6 / 37908, "C4": 169.41e6 / 75816}


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
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, device_index: int, period_s: float = 0.01):
        self.samples, self.reasons = [], set()
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

    def stop(self) -> dict:
        if self.nv is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable"]}
        self._one()
        self._stop.set()
        self._thread.join()
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.sm_max, "reasons": sorted(self.reasons),
                "samples": len(s)}


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
        t_gemm = time_steps(gemm, steps, 3, lambda: None)
        t_full = time_steps(full, steps, 3, lambda: None)
        return {"cublaslt_gemm_ms": t_gemm, "cublaslt_gemm_tflops": p.flops() / t_gemm / 1e9,
                "cublaslt_unfused_ms": t_full, "cublaslt_unfused_tflops": p.flops() / t_full / 1e9}
    except Exception as e:          # a torch build without _scaled_mm for this shape: report, do not fail the bench
        return {"cublaslt_error": f"{type(e).__name__}: {str(e)[:160]}"}


def layer_table(eng, dev, steps: int, peaks: dict, names=("C1", "C2", "C3", "C4")) -> dict:
    """Per-layer numbers for every configuration with the same timing protocol, beside cuBLASLt FP8."""
    from siglip_b200 import synth
    out = {}
    for name in names:
        p = synth.make_config(name, seed=0, device=dev)
        fn, _, _ = launch_fn(eng, p, dev)
        ms = time_steps(fn, steps, 3, lambda: None)
        eng.device_status()
        tf = p.flops() / ms / 1e9
        gbs = p.min_bytes() / ms / 1e6
        out[name] = {"ms": ms, "tflops": tf, "gbs": gbs, "frac_fp8_measured": tf / (2 * peaks["bf16_tflops"]),
                     "frac_hbm_measured": gbs / peaks["hbm_gbs"], "frac_fp8_nominal_4500": tf / 4500.0,
                     "images_per_s": synth.CONFIGS[name]["images"] / ms * 1e3}
        del fn
        torch.cuda.empty_cache()
        if name == "C2":   # the opt-in GELU through the hardware tanh (SL8_FLAG_GELU_HW_TANH = 8), for information
            sa_, sb_ = torch.tensor([p.scale_a], device=dev), torch.tensor([p.scale_b], device=dev)
            d_ = torch.empty((p.M, p.N), dtype=torch.bfloat16, device=dev)
            ms_fast = time_steps(lambda i=0: eng.fc1_gelu(p.A, p.B, p.bias, scale_a=sa_, scale_b=sb_, out=d_, flags=8), steps, 3, lambda: None)
            out[name]["hw_tanh_gelu_ms"] = ms_fast
            out[name]["hw_tanh_gelu_tflops"] = p.flops() / ms_fast / 1e9
            del d_
        out[name].update(cublaslt_baseline(p, dev, steps))
        del p
        torch.cuda.empty_cache()
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


def chain_bench(args, eng, dev, rank: int, world: int, barrier, dist) -> None:
    """C5: the MLP chain FC1 + GELU -> e4m3 -> FC2 + residual on this rank's share of 1024 images (M = 746 496
    rows in total; strong scaling: the images are divided over the ranks, no data crosses GPUs)."""
    from siglip_b200 import synth
    from siglip_b200.shard import image_range
    total_images = 1024 if args.images is None else args.images
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
    h_scale = torch.tensor([float(cal.float().abs().max()) / 448.0], device=dev)
    H = torch.empty((M, synth.pitch128(d_ff)), dtype=torch.uint8, device=dev)[:, :d_ff]
    D = torch.empty((M, d_model), dtype=torch.bfloat16, device=dev)

    def step(i):
        eng.fc1_gelu(p1.A, p1.B, p1.bias, scale_a=sa1, scale_b=sb1, out=H, out_dtype=torch.uint8, out_scale=h_scale)
        eng.fc2_residual(H, w2.B, w2.bias, residual, scale_a=h_scale, scale_b=sb2, out=D)

    ms = time_steps(step, args.steps, args.warmup, barrier)
    eng.device_status()
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t)
    flops = 2.0 * 2.0 * total_images * 729 * d_ff * d_model
    if rank == 0:
        peaks = measured_peaks()
        tf = flops / ms_max / 1e9
        print(json.dumps({
            "metric": "fp8_tflops_mlp_chain", "value": tf, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_max, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "e4m3 x e4m3 -> f32", "data": "synthetic",
            "config": {"workload": f"SigLIP C5: MLP chain FC1+GELU (e4m3 out) -> FC2+residual, {total_images} images "
                                   f"(M={total_images * 729}) split by image over {world} GPU(s), K/N 1152/4304",
                       "l2": "operands of one step (> 7 GB at 1 GPU) exceed the 126 MB L2"},
            "images_per_s": total_images / ms_max * 1e3, "gpu_launches": 2 * args.steps,
            "roofline": {"bound": "tensor", "achieved": tf / world, "peak": 2.0 * peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": tf / world / (2.0 * peaks["bf16_tflops"]), "traffic": None}}), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="C2", choices=["C1", "C2", "C3", "C4", "C5"])
    ap.add_argument("--layers", action="store_true", help="also time C1, C3 and C4 and add them under 'layers'")
    ap.add_argument("--layer-names", default="C1,C2,C3,C4", help="which configurations --layers covers")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--variant", type=int, default=-1, help="force a kernel variant (sweeps)")
    ap.add_argument("--images", type=int, default=None, help="override the batch (profiling captures use a smaller case)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-operand leg (profiling captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

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
        chain_bench(args, eng, dev, rank, world, barrier, dist)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
    p = synth.make_config(args.config, seed=rank, device=dev, images=args.images)
    n_images = synth.CONFIGS[args.config]["images"] if args.images is None else args.images
    fn, _, Ds = launch_fn(eng, p, dev)
    out_bytes = p.M * p.N * 2

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

    e2e_value, e2e_ms_max, e2e_steps, same, side_bytes = None, None, 0, True, 0
    if not args.no_e2e:
        # ---- end to end: pinned host operands through the *_host entry point
        A_h = torch.zeros((p.M, p.A.stride(0)), dtype=torch.uint8).pin_memory()[:, :p.K]
        A_h.copy_(p.A)
        B_h = p.B.cpu().pin_memory()
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

    if rank == 0:
        line = {
            "metric": METRICS.get(args.config, METRIC), "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_max, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "e4m3 x e4m3 -> f32", "data": "synthetic", "config": workload_config(args.config, args.images),
            "clocks": clocks, "gpu_launches": args.steps,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(p.M * p.A.stride(0) + p.N * p.B.stride(0) + side_bytes + 12),
                    "d2h_bytes_per_step": int(out_bytes), "ms_per_step": e2e_ms_max, "steps": e2e_steps,
                    "matches_device_path": bool(same)},
            "images_per_s": world * n_images / ms_max * 1e3,
            "kernel_config": eng.query_config(p.op, p.M, p.N, p.K),
        }
        tensor_bound = p.op != synth.OP_PATCH_EMBED
        per_gpu_tf = flops / ms / 1e9
        per_gpu_gbs = p.min_bytes() / ms / 1e6
        per_row = NCU_DRAM_BYTES_PER_ROW.get(args.config)
        traffic = None if per_row is None else per_row * p.M
        if tensor_bound:
            peak = 2.0 * peaks["bf16_tflops"]
            line["roofline"] = {"bound": "tensor", "achieved": per_gpu_tf, "peak": peak, "unit": "TFLOP/s",
                                "frac": per_gpu_tf / peak, "traffic": traffic,
                                "peak_source": f"2 x bf16 burst GEMM rate of {peaks['source']} MEASURED_PEAKS (e4m3 MMA rate is twice bf16)",
                                "frac_of_nominal_4500": per_gpu_tf / 4500.0,
                                "hbm_gbs_algorithmic": per_gpu_gbs}
        else:
            line["roofline"] = {"bound": "hbm", "achieved": per_gpu_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                "frac": per_gpu_gbs / peaks["hbm_gbs"], "traffic": traffic,
                                "peak_source": f"{peaks['source']} copy bandwidth", "tflops": per_gpu_tf}
        if not args.no_cpu_baseline and world == 1:      # a reported baseline of the one-GPU run only
            v, cores, sample, secs = cpu_oracle_rate(args.config, args.cpu_seconds)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample,
                                    "seconds": secs}
        if args.layers:
            line["layers"] = layer_table(eng, dev, max(20, min(args.steps, 100)), peaks, tuple(args.layer_names.split(",")))
            line["prep"] = prep_table(eng, dev, max(20, min(args.steps, 100)), peaks)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
