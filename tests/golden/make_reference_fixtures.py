"""Generates tests/golden/ref_{pe,fc1,fc2}.npz: outputs of the REFERENCE's own kernels on seeded operands.

Needs a B200 and `make -C oracle ref` (the reference's three layer sources compiled in place into
oracle/_ref/libsl8_ref_*.so).  The reference is shaped at compile time (M = 928 256 rows, SigLIP-B/16 N and K), so
whole outputs cannot be committed; each fixture keeps a sample: R output rows x C output columns of the reference's
result and of this library's, with exactly the operand slices a CPU evaluation of those entries needs -- the A rows
(and the rows r ^ 64, see tests/test_gpu_vs_reference.py), the B rows of the sampled columns, bias, table or residual
entries.  tests/test_golden_fixtures.py replays them through the CPU oracle without a GPU.

    python tests/golden/make_reference_fixtures.py --out tests/golden
"""
import argparse
import ctypes as C
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
DEV = "cuda"


def load_ref(name):
    lib = C.CDLL(str(ROOT / "oracle" / "_ref" / f"libsl8_ref_{name}.so"))
    lib.sl8_ref_shape.argtypes = [C.POINTER(C.c_longlong)] + [C.POINTER(C.c_int)] * 4
    lib.sl8_ref_launch.argtypes = [C.c_void_p] * 6
    lib.sl8_ref_launch.restype = C.c_int
    m, n, k, s, t = C.c_longlong(), C.c_int(), C.c_int(), C.c_int(), C.c_int()
    lib.sl8_ref_shape(C.byref(m), C.byref(n), C.byref(k), C.byref(s), C.byref(t))
    return lib, m.value, n.value, k.value, s.value, t.value


def raw_codes(rows, cols, std, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    out = torch.empty((rows, cols), dtype=torch.uint8, device=DEV)
    for r0 in range(0, rows, 1 << 16):
        r1 = min(rows, r0 + (1 << 16))
        x = torch.randn((r1 - r0, cols), generator=g, device=DEV) * std
        out[r0:r1] = x.clamp_(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
    return out


def sample(M, N, seed):
    rng = np.random.default_rng(seed)
    rows = np.unique(np.r_[0:4, 64:68, 188:200, M // 2:M // 2 + 4, M - 4:M, rng.integers(0, M, 8)])
    cols = np.unique(np.r_[0:8, N - 8:N, rng.integers(0, N, 48)])
    return rows.astype(np.int64), cols.astype(np.int64)


def gather(t, rows, cols=None):
    idx = torch.as_tensor(rows, device=DEV)
    x = t[idx]
    if cols is not None:
        x = x[:, torch.as_tensor(cols, device=DEV)]
    return x


def bits(t):
    return t.contiguous().view(torch.uint16).cpu().numpy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", type=Path, default=Path(__file__).resolve().parent)
    a = ap.parse_args()
    a.out.mkdir(parents=True, exist_ok=True)
    import siglip_b200
    eng = siglip_b200.Engine(0)

    # ---- patch-embed
    lib, M, N, K, period, table_rows = load_ref("pe")
    lib.sl8_ref_make_table.argtypes = [C.c_void_p] * 4
    lib.sl8_ref_make_table.restype = C.c_int
    A, B = raw_codes(M, K, 1.0, 1), raw_codes(N, K, 0.02, 2)
    g = torch.Generator(device=DEV).manual_seed(3)
    bias = torch.randn((N,), generator=g, device=DEV) * 0.01
    pos = torch.randn((period, N), generator=g, device=DEV) * 0.02
    blocked = torch.zeros((table_rows * N,), dtype=torch.bfloat16, device=DEV)
    assert lib.sl8_ref_make_table(bias.data_ptr(), pos.data_ptr(), blocked.data_ptr(), None) == 0
    table = eng.make_table(bias, pos)
    D_ref = torch.zeros((M, N), dtype=torch.bfloat16, device=DEV)
    D_new = torch.zeros((M, N), dtype=torch.bfloat16, device=DEV)
    assert lib.sl8_ref_launch(A.data_ptr(), B.data_ptr(), blocked.data_ptr(), D_ref.data_ptr(), None, None) == 0
    eng.patch_embed(A, B, table, period=period, out=D_new)
    eng.device_status()
    rows, cols = sample(M, N, 11)
    np.savez_compressed(a.out / "ref_pe.npz", M=M, N=N, K=K, period=period, rows=rows, cols=cols,
                        A_rows=gather(A, rows).cpu().numpy(), A_partner=gather(A, rows ^ 64).cpu().numpy(),
                        B_cols=gather(B, cols).cpu().numpy(),
                        table_rc=bits(gather(table, rows % period, cols)),
                        ref_out=bits(gather(D_ref, rows, cols)), new_out=bits(gather(D_new, rows, cols)))
    del A, B, D_ref, D_new

    # ---- FC1 + GELU
    lib, M, N, K, _, _ = load_ref("fc1")
    A, B = raw_codes(M, K, 1.0, 4), raw_codes(N, K, 0.02, 5)
    g = torch.Generator(device=DEV).manual_seed(6)
    bias = torch.randn((N,), generator=g, device=DEV) * 0.01
    D_ref = torch.zeros((M, N), dtype=torch.bfloat16, device=DEV)
    D_new = torch.zeros((M, N), dtype=torch.bfloat16, device=DEV)
    assert lib.sl8_ref_launch(A.data_ptr(), B.data_ptr(), bias.data_ptr(), D_ref.data_ptr(), None, None) == 0
    eng.fc1_gelu(A, B, bias, out=D_new)
    eng.device_status()
    rows, cols = sample(M, N, 12)
    np.savez_compressed(a.out / "ref_fc1.npz", M=M, N=N, K=K, rows=rows, cols=cols,
                        A_rows=gather(A, rows).cpu().numpy(), A_partner=gather(A, rows ^ 64).cpu().numpy(),
                        B_cols=gather(B, cols).cpu().numpy(), bias_cols=bias[torch.as_tensor(cols, device=DEV)].cpu().numpy(),
                        ref_out=bits(gather(D_ref, rows, cols)), new_out=bits(gather(D_new, rows, cols)))
    del A, B, D_ref, D_new

    # ---- FC2 + residual
    lib, M, N, K, _, _ = load_ref("fc2")
    A, B = raw_codes(M, K, 0.5, 7), raw_codes(N, K, 0.02, 8)
    g = torch.Generator(device=DEV).manual_seed(9)
    bias = torch.randn((N,), generator=g, device=DEV) * 0.01
    residual = torch.randn((M, N), generator=g, device=DEV).to(torch.bfloat16)
    D_ref = torch.zeros((M, N), dtype=torch.bfloat16, device=DEV)
    D_new = torch.zeros((M, N), dtype=torch.bfloat16, device=DEV)
    assert lib.sl8_ref_launch(A.data_ptr(), B.data_ptr(), bias.data_ptr(), D_ref.data_ptr(), residual.data_ptr(), None) == 0
    eng.fc2_residual(A, B, bias, residual, out=D_new)
    eng.device_status()
    rows, cols = sample(M, N, 13)
    np.savez_compressed(a.out / "ref_fc2.npz", M=M, N=N, K=K, rows=rows, cols=cols,
                        A_rows=gather(A, rows).cpu().numpy(), A_partner=gather(A, rows ^ 64).cpu().numpy(),
                        B_cols=gather(B, cols).cpu().numpy(), bias_cols=bias[torch.as_tensor(cols, device=DEV)].cpu().numpy(),
                        residual_rc=bits(gather(residual, rows, cols)),
                        ref_out=bits(gather(D_ref, rows, cols)), new_out=bits(gather(D_new, rows, cols)))
    for f in sorted(a.out.glob("ref_*.npz")):
        print(f, f.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
