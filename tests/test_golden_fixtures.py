"""Replays the committed outputs of the REFERENCE's own kernels (tests/golden/ref_*.npz, made on a B200 by
tests/golden/make_reference_fixtures.py) through the CPU oracle: no GPU needed.

Each fixture holds a sample of output entries of the reference kernel and of this library on the same seeded
operands, plus the operand slices those entries depend on.  This library's entries must be the oracle's.  The
reference's entries must be the oracle's too, either on the same A rows or -- its epilogue warps read the TMEM lane
group (warp - 2) % 4 where the hardware gives warp w the group w % 4 (kernel_body.cuh:640-641,66) -- on the rows
r ^ 64; which of the two is recorded in the assertion message, never anything else."""
from pathlib import Path

import numpy as np
import pytest

from tests.tolerance import check_bf16

GOLDEN = Path(__file__).resolve().parent / "golden"


def load(name):
    f = GOLDEN / f"ref_{name}.npz"
    if not f.exists():
        pytest.skip(f"{f} not generated yet")
    return np.load(f)


def classify(name, fx, oracle_fn):
    want = oracle_fn(fx["A_rows"])
    check_bf16(fx["new_out"], want, f"{name}: this library vs oracle (golden sample)")
    try:
        check_bf16(fx["ref_out"], want, f"{name}: reference vs oracle")
        return "matches"
    except AssertionError:
        swapped = oracle_fn(fx["A_partner"])
        check_bf16(fx["ref_out"], swapped, f"{name}: reference vs oracle on accumulator rows r ^ 64")
        return "row-permuted"


def test_reference_patch_embed_outputs(oracle):
    fx = load("pe")
    one = np.float32(1.0)

    def fn(a_rows):
        out = np.empty(fx["ref_out"].shape, dtype=np.uint16)
        for i in range(a_rows.shape[0]):              # a one-row "table" per output row: its own table entries
            out[i] = oracle.patch_embed(np.ascontiguousarray(a_rows[i:i + 1]), np.ascontiguousarray(fx["B_cols"]), float(one),
                                        float(one), np.ascontiguousarray(fx["table_rc"][i:i + 1]), 0)[0]
        return out

    assert classify("patch-embed", fx, fn) in ("matches", "row-permuted")


def test_reference_fc1_outputs(oracle):
    fx = load("fc1")
    fn = lambda a_rows: oracle.fc1_gelu(np.ascontiguousarray(a_rows), np.ascontiguousarray(fx["B_cols"]), 1.0, 1.0,
                                        np.ascontiguousarray(fx["bias_cols"]), flags=1)
    assert classify("FC1+GELU", fx, fn) in ("matches", "row-permuted")


def test_reference_fc2_outputs(oracle):
    fx = load("fc2")
    fn = lambda a_rows: oracle.fc2_residual(np.ascontiguousarray(a_rows), np.ascontiguousarray(fx["B_cols"]), 1.0, 1.0,
                                            np.ascontiguousarray(fx["bias_cols"]), np.ascontiguousarray(fx["residual_rc"]), flags=1)
    assert classify("FC2+residual", fx, fn) in ("matches", "row-permuted")
