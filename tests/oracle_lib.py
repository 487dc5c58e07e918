"""numpy-facing wrapper of the CPU oracle (oracle/libsl8_oracle.so).  Test infrastructure."""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

ORACLE_DIR = Path(__file__).resolve().parent.parent / "oracle"
ORACLE_SO = ORACLE_DIR / "libsl8_oracle.so"

_P, _I, _I64, _U, _F = C.c_void_p, C.c_int, C.c_int64, C.c_uint, C.c_float


def build_oracle() -> Path:
    src = ORACLE_DIR / "sl8_oracle.c"
    if not ORACLE_SO.exists() or ORACLE_SO.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(ORACLE_DIR), "libsl8_oracle.so"], check=True, capture_output=True)
    return ORACLE_SO


def _np_ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _pitch(a: np.ndarray) -> int:
    assert a.ndim == 2 and a.strides[1] == a.itemsize
    return a.strides[0] // a.itemsize


class Oracle:
    def __init__(self):
        self.lib = C.CDLL(str(build_oracle()))
        L = self.lib
        L.sl8o_e4m3_to_f32.restype = _F
        L.sl8o_e4m3_to_f32.argtypes = [C.c_uint8]
        L.sl8o_f32_to_e4m3.restype = C.c_uint8
        L.sl8o_f32_to_e4m3.argtypes = [_F]
        L.sl8o_bf16_to_f32.restype = _F
        L.sl8o_bf16_to_f32.argtypes = [C.c_uint16]
        L.sl8o_f32_to_bf16.restype = C.c_uint16
        L.sl8o_f32_to_bf16.argtypes = [_F]
        L.sl8o_bf16_add.restype = C.c_uint16
        L.sl8o_bf16_add.argtypes = [C.c_uint16, C.c_uint16]
        L.sl8o_gelu_tanh.restype = _F
        L.sl8o_gelu_tanh.argtypes = [_F]
        L.sl8o_num_threads.restype = _I
        L.sl8o_set_num_threads.argtypes = [_I]
        L.sl8o_gemm_fp8_f32.restype = _I
        L.sl8o_gemm_fp8_f32.argtypes = [_P, _I64, _P, _I64, _I64, _I, _I, _P, _I64]
        L.sl8o_patch_embed.restype = _I
        L.sl8o_patch_embed.argtypes = [_P, _I64, _P, _I64, _F, _F, _P, _I64, _I, _I, _P, _I64, _I64, _I, _I, _U]
        L.sl8o_fc1_gelu.restype = _I
        L.sl8o_fc1_gelu.argtypes = [_P, _I64, _P, _I64, _F, _F, _P, _P, _I64, _I, _F, _I64, _I, _I, _U]
        L.sl8o_fc2_residual.restype = _I
        L.sl8o_fc2_residual.argtypes = [_P, _I64, _P, _I64, _F, _F, _P, _P, _I64, _P, _I64, _I64, _I, _I, _U]
        L.sl8o_combine_bias_pos.argtypes = [_P, _P, _I, _I, _P]
        L.sl8o_quantize_e4m3.argtypes = [_P, _I64, _F, _P]
        L.sl8o_dequantize_e4m3.argtypes = [_P, _I64, _P]
        L.sl8o_patchify_quantize.restype = _I
        L.sl8o_patchify_quantize.argtypes = [_P, _I, _I, _I, _I, _I, _F, _P, _I64, _I]
        L.sl8o_amax.restype = _F
        L.sl8o_amax.argtypes = [_P, _I64, _I, _I64]
        L.sl8o_quantize_rows_e4m3.restype = _I
        L.sl8o_quantize_rows_e4m3.argtypes = [_P, _I64, _I, _I64, _F, _P, _I64]
        L.sl8o_layernorm_quantize.restype = _I
        L.sl8o_layernorm_quantize.argtypes = [_P, _I64, _I, _I64, _P, _P, _F, _F, _P, _I64]

    # ---- scalars
    def e4m3_lut(self) -> np.ndarray:
        return np.array([self.lib.sl8o_e4m3_to_f32(i) for i in range(256)], dtype=np.float32)

    def num_threads(self) -> int:
        return self.lib.sl8o_num_threads()

    # ---- producer-side steps; pixels / x are fp32 arrays
    def patchify_quantize(self, pixels, patch, scale, lda, row_bytes):
        images, Cc, H, W = pixels.shape
        rows = images * (H // patch) * (W // patch)
        A = np.full((rows, lda), 0xAA, dtype=np.uint8)          # what is not written stays recognisable
        px = np.ascontiguousarray(pixels, dtype=np.float32)
        rc = self.lib.sl8o_patchify_quantize(_np_ptr(px), images, Cc, H, W, patch, scale, _np_ptr(A), lda, row_bytes)
        assert rc == 0
        return A

    def amax(self, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        return float(self.lib.sl8o_amax(_np_ptr(x), x.shape[0], x.shape[1], x.shape[1]))

    def quantize_rows(self, x, scale):
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.empty(x.shape, dtype=np.uint8)
        rc = self.lib.sl8o_quantize_rows_e4m3(_np_ptr(x), x.shape[0], x.shape[1], x.shape[1], scale, _np_ptr(out), x.shape[1])
        assert rc == 0
        return out

    def layernorm_quantize(self, x, gamma, beta, eps, scale):
        x = np.ascontiguousarray(x, dtype=np.float32)
        g = np.ascontiguousarray(gamma, dtype=np.float32)
        b = np.ascontiguousarray(beta, dtype=np.float32)
        out = np.empty(x.shape, dtype=np.uint8)
        rc = self.lib.sl8o_layernorm_quantize(_np_ptr(x), x.shape[0], x.shape[1], x.shape[1], _np_ptr(g), _np_ptr(b), eps, scale,
                                              _np_ptr(out), x.shape[1])
        assert rc == 0
        return out

    # ---- layers; A, B uint8 2-D (K contiguous); outputs uint16 (bf16 bits) or uint8 (e4m3 codes)
    def gemm(self, A, B):
        M, K = A.shape
        N = B.shape[0]
        acc = np.empty((M, N), dtype=np.float32)
        rc = self.lib.sl8o_gemm_fp8_f32(_np_ptr(A), _pitch(A), _np_ptr(B), _pitch(B), M, N, K, _np_ptr(acc), N)
        assert rc == 0
        return acc

    def patch_embed(self, A, B, sa, sb, table, row_phase=0, flags=0):
        M, K = A.shape
        N = B.shape[0]
        D = np.empty((M, N), dtype=np.uint16)
        rc = self.lib.sl8o_patch_embed(_np_ptr(A), _pitch(A), _np_ptr(B), _pitch(B), sa, sb, _np_ptr(table),
                                       _pitch(table), table.shape[0], row_phase, _np_ptr(D), N, M, N, K, flags)
        assert rc == 0
        return D

    def fc1_gelu(self, A, B, sa, sb, bias, out_e4m3=False, out_scale=1.0, flags=0):
        M, K = A.shape
        N = B.shape[0]
        D = np.empty((M, N), dtype=np.uint8 if out_e4m3 else np.uint16)
        rc = self.lib.sl8o_fc1_gelu(_np_ptr(A), _pitch(A), _np_ptr(B), _pitch(B), sa, sb, _np_ptr(bias), _np_ptr(D), N,
                                    1 if out_e4m3 else 0, out_scale, M, N, K, flags)
        assert rc == 0
        return D

    def fc2_residual(self, A, B, sa, sb, bias, residual, flags=0):
        M, K = A.shape
        N = B.shape[0]
        D = np.empty((M, N), dtype=np.uint16)
        rc = self.lib.sl8o_fc2_residual(_np_ptr(A), _pitch(A), _np_ptr(B), _pitch(B), sa, sb, _np_ptr(bias),
                                        _np_ptr(residual), _pitch(residual), _np_ptr(D), N, M, N, K, flags)
        assert rc == 0
        return D

    def combine_bias_pos(self, bias_f32, pos_f32):
        period, N = pos_f32.shape
        t = np.empty((period, N), dtype=np.uint16)
        self.lib.sl8o_combine_bias_pos(_np_ptr(np.ascontiguousarray(bias_f32)), _np_ptr(np.ascontiguousarray(pos_f32)),
                                       period, N, _np_ptr(t))
        return t


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
