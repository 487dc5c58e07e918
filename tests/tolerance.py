"""The parity bar between the CUDA path and the CPU oracle, in one place.

Floating-point outputs (FP32 accumulation order differs between the tensor core and the
CPU, and the GELU uses hardware exp2 / reciprocal):

    |got - ref| <= RTOL * |ref| + ATOL_RMS * rms(ref)        RTOL = 1e-2, ATOL_RMS = 2.5e-3

i.e. 1 % relative error on every element, with an absolute floor of 0.25 % of the output's
root-mean-square for elements that are small through cancellation (where one bf16 ulp of an
intermediate -- the reference rounds the patch-embed accumulator to bf16 before adding the
table -- is large compared with the result).  On top of that at least EXACT_MIN of the
elements must be bit-identical to the oracle: an indexing or swizzle mistake cannot hide
inside a tolerance.

e4m3 outputs: every code within one e4m3 ulp (adjacent code) of the oracle's code, and at
least EXACT_MIN bit-identical.
"""
import numpy as np

RTOL = 1e-2
ATOL_RMS = 2.5e-3
EXACT_MIN = 0.99


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def check_bf16(got_bits: np.ndarray, ref_bits: np.ndarray, what: str = "") -> dict:
    assert got_bits.shape == ref_bits.shape, (got_bits.shape, ref_bits.shape)
    g = bf16_bits_to_f32(got_bits).astype(np.float64)
    r = bf16_bits_to_f32(ref_bits).astype(np.float64)
    assert np.isfinite(r).all(), "oracle produced non-finite values"
    rms = float(np.sqrt(np.mean(r * r)))
    err = np.abs(g - r)
    tol = RTOL * np.abs(r) + ATOL_RMS * rms
    bad = ~(err <= tol)
    exact = float(np.mean(got_bits == ref_bits))
    stats = dict(bad=int(bad.sum()), size=int(r.size), exact=exact, max_err=float(np.nanmax(err)), rms=rms)
    if bad.any():
        idx = np.argwhere(bad)
        i = tuple(idx[0])
        raise AssertionError(
            f"{what}: {bad.sum()} of {r.size} elements outside |err| <= {RTOL}*|ref| + {ATOL_RMS}*rms ({rms:.4g}); "
            f"first at {i}: got {g[i]!r} ref {r[i]!r}; bad rows {np.unique(idx[:, 0])[:16].tolist()} "
            f"bad cols {np.unique(idx[:, -1])[:16].tolist()}")
    assert exact >= EXACT_MIN, f"{what}: only {exact:.4f} of the elements are bit-identical to the oracle"
    return stats


def e4m3_order_key(codes: np.ndarray) -> np.ndarray:
    """Maps e4m3 codes to integers ordered like their values, so adjacent values differ by one."""
    c = codes.astype(np.int32)
    mag = c & 0x7F
    return np.where(c & 0x80, -mag, mag)


def check_e4m3(got: np.ndarray, ref: np.ndarray, what: str = "") -> dict:
    assert got.shape == ref.shape
    d = np.abs(e4m3_order_key(got) - e4m3_order_key(ref))
    exact = float(np.mean(got == ref))
    assert d.max() <= 1, f"{what}: e4m3 codes differ by {d.max()} ulp at {np.argwhere(d > 1)[:4].tolist()}"
    assert exact >= EXACT_MIN, f"{what}: only {exact:.4f} of the codes are bit-identical to the oracle"
    return dict(exact=exact, max_ulp=int(d.max()))
