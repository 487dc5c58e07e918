"""ctypes binding of libsiglip_fp8.so: one Python function per symbol of include/siglip_fp8.h.

The library is looked up in-tree (``siglip_b200/lib/libsiglip_fp8.so``, produced by
``python -m siglip_b200.build``).  A missing library is an error, never a fallback.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "lib" / "libsiglip_fp8.so"
_lib = None

SL8_OK = 0
SL8_ERR_INVALID_VALUE = -1
SL8_ERR_ALIGNMENT = -2
SL8_ERR_UNSUPPORTED = -3
SL8_ERR_CUDA = -4
SL8_ERR_DEVICE_TIMEOUT = -5
SL8_ERR_ARCH = -6
SL8_ERR_NO_DEVICE = -7

SL8_OUT_BF16, SL8_OUT_E4M3 = 0, 1
SL8_OP_PATCH_EMBED, SL8_OP_FC1_GELU, SL8_OP_FC2_RESIDUAL = 0, 1, 2
SL8_FLAG_NONE, SL8_FLAG_BIAS_F32, SL8_FLAG_PE_F32_ADD, SL8_FLAG_NO_ACTIVATION, SL8_FLAG_GELU_HW_TANH = 0, 1, 2, 4, 8
SL8_DT_F32, SL8_DT_BF16 = 0, 1

_ERR_NAMES = {
    -1: "SL8_ERR_INVALID_VALUE", -2: "SL8_ERR_ALIGNMENT", -3: "SL8_ERR_UNSUPPORTED", -4: "SL8_ERR_CUDA",
    -5: "SL8_ERR_DEVICE_TIMEOUT", -6: "SL8_ERR_ARCH", -7: "SL8_ERR_NO_DEVICE",
}


class SL8Error(RuntimeError):
    """A call into libsiglip_fp8.so returned a negative status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"{_ERR_NAMES.get(code, code)}: {message}")
        self.code = code


class Config(C.Structure):
    """Mirror of ``sl8_config``."""
    _fields_ = [(n, C.c_int) for n in ("cta_group", "tile_m", "tile_n", "tile_k", "stages", "epi_warps",
                                       "staging_buffers", "grid", "smem_bytes", "variant_id")]

    def as_dict(self) -> dict:
        return {n: getattr(self, n) for n, _ in self._fields_}


# name -> (restype, argtypes); the exported symbols of include/siglip_fp8.h, all of them.
_P, _I, _I64, _U, _F = C.c_void_p, C.c_int, C.c_int64, C.c_uint, C.c_float
SIGNATURES = {
    "sl8_create": (_I, [C.POINTER(_P), _I]),
    "sl8_destroy": (_I, [_P]),
    "sl8_last_error_string": (C.c_char_p, [_P]),
    "sl8_version": (C.c_char_p, []),
    "sl8_patch_embed_fp8": (_I, [_P, _P, _I64, _P, _I64, _P, _P, _P, _I64, _I, _I, _I, _P, _I64, _I64, _I, _I, _U, _P]),
    "sl8_make_periodic_table": (_I, [_P, _P, _P, _I, _I, _P, _I64, _I, _P]),
    "sl8_extend_periodic_table": (_I, [_P, _P, _I64, _I, _I, _P, _I64, _I, _P]),
    "sl8_padded_table_rows": (_I, [_I]),
    "sl8_fc1_gelu_fp8": (_I, [_P, _P, _I64, _P, _I64, _P, _P, _P, _P, _I64, _I, _P, _I64, _I, _I, _U, _P]),
    "sl8_linear_bias_fp8": (_I, [_P, _P, _I64, _P, _I64, _P, _P, _P, _P, _I64, _I, _P, _I64, _I, _I, _U, _P]),
    "sl8_fc2_residual_fp8": (_I, [_P, _P, _I64, _P, _I64, _P, _P, _P, _P, _I64, _P, _I64, _I64, _I, _I, _U, _P]),
    "sl8_patchify_quantize_e4m3": (_I, [_P, _P, _I, _I, _I, _I, _I, _I, _P, _P, _I64, _P]),
    "sl8_amax_scale": (_I, [_P, _P, _I, _I64, _I, _I64, _P, _P, _P]),
    "sl8_quantize_e4m3": (_I, [_P, _P, _I, _I64, _I, _I64, _P, _P, _I64, _P]),
    "sl8_layernorm_quantize_e4m3": (_I, [_P, _P, _I, _I64, _I, _I64, _P, _P, _F, _P, _P, _I64, _P]),
    "sl8_patch_embed_fp8_host": (_I, [_P, _P, _I64, _P, _I64, _F, _F, _P, _I64, _I, _I, _I, _P, _I64, _I64, _I, _I, _U]),
    "sl8_fc1_gelu_fp8_host": (_I, [_P, _P, _I64, _P, _I64, _F, _F, _P, _P, _I64, _I, _F, _I64, _I, _I, _U]),
    "sl8_fc2_residual_fp8_host": (_I, [_P, _P, _I64, _P, _I64, _F, _F, _P, _P, _I64, _P, _I64, _I64, _I, _I, _U]),
    "sl8_mlp_chain_fp8": (_I, [_P, _P, _I64, _P, _I64, _P, _P, _P, _P, _I64, _P, _P, _I64, _P, _P, _P, _I64, _P, _I64, _I64, _I, _I, _U, _P]),
    "sl8_mlp_chain_fp8_host": (_I, [_P, _P, _I64, _P, _I64, _F, _F, _P, _F, _P, _I64, _F, _P, _P, _I64, _P, _I64, _I64, _I, _I, _U]),
    "sl8_query_config": (_I, [_P, _I, _I, _I64, _I, _I, C.POINTER(Config)]),
    "sl8_num_variants": (_I, []),
    "sl8_describe_variant": (_I, [_I, C.POINTER(Config)]),
    "sl8_set_variant": (_I, [_P, _I]),
    "sl8_device_status": (_I, [_P, _P, C.POINTER(C.c_uint * 4)]),
    "sl8_set_wait_budget_ms": (_I, [_P, _I]),
    "sl8_set_wait_budget_us": (_I, [_P, _I64]),
    "sl8_trace_enable": (_I, [_P, _I]),
    "sl8_trace_read": (_I, [_P, C.POINTER(C.c_longlong), _I]),
    "sl8_fc1_gelu_fp8_static": (_I, [_P, _I64, _P, _I64, _P, _P, _P, _P, _I64, _I, _P, _I64, _I, _I, _U, _P, _P, _P]),
}


def library_path() -> Path:
    return _LIB_PATH


def load_library() -> C.CDLL:
    """Loads libsiglip_fp8.so and types its entry points.  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        raise SL8Error(SL8_ERR_CUDA, f"{_LIB_PATH} is missing: run `python -m siglip_b200.build` "
                                     "(nvcc, sm_100a); there is no fallback path")
    lib = C.CDLL(str(_LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError here = header and library disagree
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
