"""Two measurements that say what bounds a layer, on a B200.

    python -m siglip_b200.diagnose kfit                 # time per tile = a * k-blocks + b, fitted over K
    SL8_DIAG=1 python -m siglip_b200.build --force      # measurement build: the switches below exist only there
    python -m siglip_b200.diagnose parts                # the layer with parts of its epilogue switched off

``kfit`` times FC1 at the So400m M and N for K = 576, 1152, 2304 and 4608 (4, 9, 18, 36 k-blocks of 128 bytes) and fits
the time of one 256x256 tile to ``a * k_blocks + b``: ``a`` is the cost of streaming one k-block of operands through
the ring and the tensor pipe, ``b`` what every tile pays on top (its epilogue and output store, as far as they do not
hide behind the next tile's MMAs).  ``parts`` repeats the launch with the epilogue's tensor-memory loads, its
arithmetic, its output stores, its side-data loads or all of it switched off, which shows which of them ``b`` is made of.
The counterpart in the reference is its clock64 instrumentation (``kernel_body.cuh`` under ``-DTIMING``,
``docs/clock64_timing_analysis.md``).
"""
from __future__ import annotations

import argparse
import sys

# Measurement switches of a library built with -DSL8_DIAG (sl8_kernel.cuh).
SKIP_SIDE, SKIP_STORE, SKIP_EPILOGUE, SKIP_TMEM_LD, SKIP_MATH = 0x100, 0x800, 0x2000, 0x20000, 0x40000
PARTS = [("all on", 0), ("no tcgen05.ld", SKIP_TMEM_LD), ("no arithmetic", SKIP_MATH), ("no stores", SKIP_STORE),
         ("no arithmetic, no stores", SKIP_MATH | SKIP_STORE), ("no epilogue", SKIP_EPILOGUE)]


def _time_us(eng, fn, iters: int) -> float:
    import torch
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    eng.device_status()
    return e0.elapsed_time(e1) / iters * 1e3


def fit_tile_cost(t_short: float, kb_short: int, t_long: float, kb_long: int) -> tuple:
    """(a, b) of t = a * k_blocks + b through two (k_blocks, time per tile) points."""
    a = (t_long - t_short) / (kb_long - kb_short)
    return a, t_short - kb_short * a


def kfit(iters: int) -> int:
    import torch
    import siglip_b200
    import siglip_b200.lib as L
    from siglip_b200 import synth
    eng = siglip_b200.Engine(0)
    M, N = 46656, 4304
    rounds = -(-((M + 255) // 256 * ((N + 255) // 256)) // 74)          # tiles per CTA pair, rounded up
    cases = ((2, L.SL8_FLAG_NO_ACTIVATION, "eight warps, no activation"), (15, 0, "sixteen warps, exact GELU"))
    per_tile = {}
    for K in (576, 1152, 2304, 4608):
        p = synth.make_fc1(M, N, K, seed=0, device="cuda")
        sa, sb = torch.tensor([p.scale_a], device="cuda"), torch.tensor([p.scale_b], device="cuda")
        D = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
        for vid, flags, name in cases:
            eng.set_variant(vid)
            us = _time_us(eng, lambda: eng.fc1_gelu(p.A, p.B, p.bias, scale_a=sa, scale_b=sb, out=D, flags=flags), iters)
            per_tile[(name, K)] = us / rounds * 1e3
            print(f"K={K:5d} ({K // 128:2d} k-blocks)  {name}: {us:7.1f} us  {p.flops() / us / 1e6:5.0f} TFLOP/s  "
                  f"{per_tile[(name, K)]:6.0f} ns per tile", flush=True)
        del p, D
    for _, _, name in cases:
        a, b = fit_tile_cost(per_tile[(name, 1152)], 9, per_tile[(name, 4608)], 36)
        print(f"{name}: a = {a:.0f} ns per k-block, b = {b:.0f} ns per tile; K = 2304 predicted "
              f"{18 * a + b:.0f} ns per tile, measured {per_tile[(name, 2304)]:.0f}")
    return 0


def parts(iters: int) -> int:
    import torch
    import siglip_b200
    import siglip_b200.lib as L
    from siglip_b200 import synth
    eng = siglip_b200.Engine(0)

    def row(name, call, cases):
        try:
            print(name + ": " + " | ".join(f"{n} {_time_us(eng, lambda f=f: call(f), iters):.1f}" for n, f in cases) + "  (us)", flush=True)
        except L.SL8Error as e:
            print(f"{name}: {e} -- the measurement switches need a library built with SL8_DIAG=1", file=sys.stderr)
            raise SystemExit(2)

    p = synth.make_config("C2", seed=0, device="cuda")
    sa, sb = torch.tensor([p.scale_a], device="cuda"), torch.tensor([p.scale_b], device="cuda")
    D = torch.empty((p.M, p.N), dtype=torch.bfloat16, device="cuda")
    for vid, base, name in ((2, L.SL8_FLAG_NO_ACTIVATION, "FC1 C2, eight warps, no activation"), (15, 0, "FC1 C2, sixteen warps, exact GELU")):
        eng.set_variant(vid)
        row(name, lambda f: eng.fc1_gelu(p.A, p.B, p.bias, scale_a=sa, scale_b=sb, out=D, flags=base | f), PARTS)
    del p, D
    p = synth.make_config("C3", seed=0, device="cuda")
    sa, sb = torch.tensor([p.scale_a], device="cuda"), torch.tensor([p.scale_b], device="cuda")
    D = torch.empty((p.M, p.N), dtype=torch.bfloat16, device="cuda")
    eng.set_variant(-1)
    row("FC2 C3", lambda f: eng.fc2_residual(p.A, p.B, p.bias, p.residual, scale_a=sa, scale_b=sb, out=D, flags=f),
        PARTS + [("no residual loads", SKIP_SIDE)])
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=["kfit", "parts"])
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args(argv)
    return kfit(a.iters) if a.what == "kfit" else parts(a.iters)


if __name__ == "__main__":
    sys.exit(main())
