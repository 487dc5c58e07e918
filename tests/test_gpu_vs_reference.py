"""Side by side with the reference's OWN kernels on identical seeded operands.

`make -C oracle ref` compiles the reference's three layer sources (from where they lie) into
oracle/_ref/libsl8_ref_{pe,fc1,fc2}.so behind a small launch shim (oracle/ref_shim.cu).  The
reference is shaped at compile time: M = 928 256 rows and its SigLIP-B/16 N, K, operands consumed as
raw e4m3 codes (scale 1), fp32 bias, a 32x32-blocked bf16 bias+pos table.  `make -C oracle ref_so400m` compiles
the same sources for the zero-padded SigLIP-So400m shapes (libsl8_ref_*_so400m.so).  Each test feeds both
implementations the same random codes at exactly that shape (this library on the unpadded views), compares the outputs, arbitrates on a
row sample with the CPU oracle, prints both kernels' times (CUDA events) and appends them to
ref_compare.txt in the directory SL8_REPORT_DIR names, when it is set.

The reference's own validation uses constant rows (every output row equal), so it cannot see a
permutation of rows; these tests can.
"""
import ctypes as C
import os
from pathlib import Path

import numpy as np
import pytest
import torch

from tests.tolerance import check_bf16, bf16_bits_to_f32

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
REF_DIR = ROOT / "oracle" / "_ref"
DEV = "cuda"


def load_ref(name):
    so = REF_DIR / f"libsl8_ref_{name}.so"
    if not so.exists():
        pytest.skip(f"{so} not built (make -C oracle ref needs the reference checkout)")
    lib = C.CDLL(str(so))
    lib.sl8_ref_shape.argtypes = [C.POINTER(C.c_longlong), C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int),
                                  C.POINTER(C.c_int)]
    lib.sl8_ref_launch.argtypes = [C.c_void_p] * 6
    lib.sl8_ref_launch.restype = C.c_int
    m, n, k, s, t = C.c_longlong(), C.c_int(), C.c_int(), C.c_int(), C.c_int()
    lib.sl8_ref_shape(C.byref(m), C.byref(n), C.byref(k), C.byref(s), C.byref(t))
    return lib, m.value, n.value, k.value, s.value, t.value


def raw_codes(rows, cols, std, seed):
    """N(0, std) rounded straight to e4m3 (scale 1), generated on the device in row slabs."""
    g = torch.Generator(device=DEV)
    g.manual_seed(seed)
    out = torch.empty((rows, cols), dtype=torch.uint8, device=DEV)
    step = 1 << 16
    for r0 in range(0, rows, step):
        r1 = min(rows, r0 + step)
        x = torch.randn((r1 - r0, cols), generator=g, device=DEV) * std
        out[r0:r1] = x.clamp_(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
    return out


def time_ms(fn, iters=10):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def record(line):
    print(line)
    out = os.environ.get("SL8_REPORT_DIR")
    if out and Path(out).is_dir():
        with open(Path(out) / "ref_compare.txt", "a") as f:
            f.write(line + "\n")


def compare(name, D_ref, D_new, oracle_rows_fn, M, N, K, t_ref, t_new):
    """oracle_rows_fn(rows, a_rows) -> oracle output for output rows `rows` computed from operand rows `a_rows`.

    This library must match the oracle.  The reference is then classified: it either matches the oracle too,
    or matches the oracle evaluated with the ACCUMULATOR rows r ^ 64 -- its epilogue warps 2..5 address TMEM
    lane group (warp - 2) % 4 (kernel_body.cuh:640-641,66) while the hardware gives warp w the lanes of
    group w % 4, which swaps the 32-row groups of every 128-row block in pairs; its constant-row self-test
    cannot see that."""
    D_ref = D_ref.contiguous()
    same = (D_ref.view(torch.uint16) == D_new.view(torch.uint16))
    exact = float(same.float().mean())
    flops = 2.0 * M * N * K
    record(f"{name}: M={M} N={N} K={K}  reference {t_ref:.3f} ms ({flops / t_ref / 1e9:.0f} TFLOP/s)  "
           f"this library {t_new:.3f} ms ({flops / t_new / 1e9:.0f} TFLOP/s)  outputs bit-identical {exact:.6f}")
    rows = np.unique(np.r_[0:64, M // 2:M // 2 + 64, M - 64:M, np.random.default_rng(0).integers(0, M, 128)])
    want = oracle_rows_fn(rows, rows)
    st_new = check_bf16(D_new[rows].view(torch.uint16).cpu().numpy(), want, f"{name}: this library vs oracle")
    ref_bits = D_ref[rows].view(torch.uint16).cpu().numpy()
    try:
        st_ref = check_bf16(ref_bits, want, f"{name}: reference vs oracle")
        record(f"{name}: vs CPU oracle on {len(rows)} rows: this library exact {st_new['exact']:.5f}, reference exact {st_ref['exact']:.5f}")
        return "matches"
    except AssertionError:
        pass
    swapped = oracle_rows_fn(rows, rows ^ 64)
    st_sw = check_bf16(ref_bits, swapped, f"{name}: reference vs oracle with accumulator rows r ^ 64")
    record(f"{name}: vs CPU oracle on {len(rows)} rows: this library exact {st_new['exact']:.5f}; the reference does NOT match the "
           f"oracle, it matches the oracle with accumulator rows r ^ 64 (exact {st_sw['exact']:.5f}): rows of its output are permuted")
    return "row-permuted"


# Shapes the reference is compiled for -> the shape the two libraries are compared on.  The So400m builds
# (`make -C oracle ref_so400m`) are compiled for zero-padded shapes (N to a multiple of 256, K to a multiple of 128, M to
# a multiple of 256): the reference runs on the padded operands, this library on the unpadded views of the SAME buffers.
# (compare() looks operand rows r ^ 64 up as well: near the end of M those lie in the zero padding, so the oracle is
# fed from the padded buffers.)
TRUE_SHAPE = {"pe_so400m": (186624, 1152, 588), "fc1_so400m": (46656, 4304, 1152), "fc2_so400m": (46656, 1152, 4304)}


def padded_codes(rows_p, cols_p, rows, cols, std, seed):
    """[rows_p, cols_p] e4m3 codes, N(0, std) in the leading [rows, cols] block and zero elsewhere."""
    out = torch.zeros((rows_p, cols_p), dtype=torch.uint8, device=DEV)
    out[:rows, :cols] = raw_codes(rows, cols, std, seed)
    return out


@pytest.mark.parametrize("build", ["pe", "pe_so400m"])
def test_patch_embed_vs_reference(engine, oracle, build):
    lib, Mp, Np, Kp, period, table_rows = load_ref(build)
    M, N, K = TRUE_SHAPE.get(build, (Mp, Np, Kp))
    lib.sl8_ref_make_table.argtypes = [C.c_void_p] * 4
    lib.sl8_ref_make_table.restype = C.c_int
    Ap, Bp = padded_codes(Mp, Kp, M, K, 1.0, 1), padded_codes(Np, Kp, N, K, 0.02, 2)
    A, B = Ap[:M, :K], Bp[:N, :K]
    g = torch.Generator(device=DEV).manual_seed(3)
    bias_p = torch.zeros((Np,), device=DEV)
    bias_p[:N] = torch.randn((N,), generator=g, device=DEV) * 0.01
    pos_p = torch.zeros((period, Np), device=DEV)
    pos_p[:, :N] = torch.randn((period, N), generator=g, device=DEV) * 0.02
    blocked = torch.zeros((table_rows * Np,), dtype=torch.bfloat16, device=DEV)
    assert lib.sl8_ref_make_table(bias_p.data_ptr(), pos_p.data_ptr(), blocked.data_ptr(), None) == 0
    bias, pos = bias_p[:N].contiguous(), pos_p[:, :N].contiguous()
    table = engine.make_table(bias, pos)                                   # same arithmetic, row-major, padded
    assert torch.equal(table[:period], (bias[None, :] + pos).to(torch.bfloat16))
    D_ref = torch.zeros((Mp, Np), dtype=torch.bfloat16, device=DEV)
    D_new = torch.zeros((M, N), dtype=torch.bfloat16, device=DEV)
    run_ref = lambda: lib.sl8_ref_launch(Ap.data_ptr(), Bp.data_ptr(), blocked.data_ptr(), D_ref.data_ptr(), None, None)
    run_new = lambda: engine.patch_embed(A, B, table, period=period, out=D_new)
    assert run_ref() == 0
    run_new()
    engine.device_status()
    t_ref, t_new = time_ms(run_ref), time_ms(run_new)
    Bn, tn = B.contiguous().cpu().numpy(), table[:period].contiguous().view(torch.uint16).cpu().numpy()

    def orc(rows, a_rows):
        out = np.empty((len(rows), N), dtype=np.uint16)
        for i, (r, a) in enumerate(zip(rows, a_rows)):          # one row at a time keeps each row's table phase right
            out[i] = oracle.patch_embed(Ap[a:a + 1, :K].contiguous().cpu().numpy(), Bn, 1.0, 1.0, tn, row_phase=int(r % period))[0]
        return out

    assert compare(f"patch-embed [{build}]", D_ref[:M, :N], D_new, orc, M, N, K, t_ref, t_new) in ("matches", "row-permuted")


@pytest.mark.parametrize("build", ["fc1", "fc1_so400m"])
def test_fc1_vs_reference(engine, oracle, build):
    lib, Mp, Np, Kp, _, _ = load_ref(build)
    M, N, K = TRUE_SHAPE.get(build, (Mp, Np, Kp))
    Ap, Bp = padded_codes(Mp, Kp, M, K, 1.0, 4), padded_codes(Np, Kp, N, K, 0.02, 5)
    A, B = Ap[:M, :K], Bp[:N, :K]
    g = torch.Generator(device=DEV).manual_seed(6)
    bias_p = torch.zeros((Np,), device=DEV)
    bias_p[:N] = torch.randn((N,), generator=g, device=DEV) * 0.01
    bias = bias_p[:N]
    D_ref = torch.zeros((Mp, Np), dtype=torch.bfloat16, device=DEV)
    D_new = torch.zeros((M, N), dtype=torch.bfloat16, device=DEV)
    run_ref = lambda: lib.sl8_ref_launch(Ap.data_ptr(), Bp.data_ptr(), bias_p.data_ptr(), D_ref.data_ptr(), None, None)
    run_new = lambda: engine.fc1_gelu(A, B, bias, out=D_new)
    assert run_ref() == 0
    run_new()
    engine.device_status()
    t_ref, t_new = time_ms(run_ref, 5), time_ms(run_new, 5)
    Bn, bn = B.contiguous().cpu().numpy(), bias.cpu().numpy()
    orc = lambda rows, a_rows: oracle.fc1_gelu(Ap[torch.as_tensor(a_rows, device=DEV)][:, :K].contiguous().cpu().numpy(), Bn, 1.0, 1.0, bn, flags=1)
    assert compare(f"FC1+GELU [{build}]", D_ref[:M, :N], D_new, orc, M, N, K, t_ref, t_new) in ("matches", "row-permuted")


@pytest.mark.parametrize("build", ["fc2", "fc2_so400m"])
def test_fc2_vs_reference(engine, oracle, build):
    lib, Mp, Np, Kp, _, _ = load_ref(build)
    M, N, K = TRUE_SHAPE.get(build, (Mp, Np, Kp))
    Ap, Bp = padded_codes(Mp, Kp, M, K, 0.5, 7), padded_codes(Np, Kp, N, K, 0.02, 8)
    A, B = Ap[:M, :K], Bp[:N, :K]
    g = torch.Generator(device=DEV).manual_seed(9)
    bias_p = torch.zeros((Np,), device=DEV)
    bias_p[:N] = torch.randn((N,), generator=g, device=DEV) * 0.01
    bias = bias_p[:N]
    res_p = torch.zeros((Mp, Np), dtype=torch.bfloat16, device=DEV)
    res_p[:M, :N] = torch.randn((M, N), generator=g, device=DEV).to(torch.bfloat16)
    residual = res_p[:M, :N]
    D_ref = torch.zeros((Mp, Np), dtype=torch.bfloat16, device=DEV)
    D_new = torch.zeros((M, N), dtype=torch.bfloat16, device=DEV)
    run_ref = lambda: lib.sl8_ref_launch(Ap.data_ptr(), Bp.data_ptr(), bias_p.data_ptr(), D_ref.data_ptr(), res_p.data_ptr(), None)
    run_new = lambda: engine.fc2_residual(A, B, bias, residual, out=D_new)
    assert run_ref() == 0
    run_new()
    engine.device_status()
    t_ref, t_new = time_ms(run_ref, 5), time_ms(run_new, 5)
    Bn, bn = B.contiguous().cpu().numpy(), bias.cpu().numpy()

    def orc(rows, a_rows):
        idx, aidx = torch.as_tensor(rows, device=DEV), torch.as_tensor(a_rows, device=DEV)
        return oracle.fc2_residual(Ap[aidx][:, :K].contiguous().cpu().numpy(), Bn, 1.0, 1.0, bn,
                                   residual[idx].contiguous().view(torch.uint16).cpu().numpy(), flags=1)

    assert compare(f"FC2+residual [{build}]", D_ref[:M, :N], D_new, orc, M, N, K, t_ref, t_new) in ("matches", "row-permuted")
