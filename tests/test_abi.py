"""CPU-side checks of the drop-in boundary: the library builds, loads, exports every symbol
the header declares, and the entry points that need no GPU behave."""
import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    from siglip_b200 import build
    build.build()
    import siglip_b200.lib as L
    return L.load_library()


def header_symbols():
    text = (ROOT / "include" / "siglip_fp8.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sl8_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree(lib):
    import siglip_b200.lib as L
    syms = header_symbols()
    assert len(syms) >= 16
    assert sorted(L.SIGNATURES) == syms
    for s in syms:
        assert hasattr(lib, s), f"libsiglip_fp8.so does not export {s}"


def test_version_and_variants(lib):
    from siglip_b200.layers import num_variants, describe_variant
    assert b"sm_100a" in lib.sl8_version()
    n = num_variants()
    assert n >= 4
    seen = set()
    for v in range(n):
        c = describe_variant(v)
        assert c["variant_id"] == v and c["cta_group"] in (1, 2) and c["tile_m"] == 128 * c["cta_group"]
        assert c["tile_n"] in (128, 256) and c["tile_k"] in (128, 256) and c["smem_bytes"] <= 232448
        seen.add((c["cta_group"], c["tile_n"], c["stages"], c["epi_warps"], c["staging_buffers"]))
    assert len(seen) == n
    with pytest.raises(Exception):
        describe_variant(n)


def test_query_config_without_handle(lib):
    import siglip_b200.lib as L
    cfg = L.Config()
    assert lib.sl8_query_config(None, L.SL8_OP_FC1_GELU, L.SL8_OUT_BF16, 46656, 4304, 1152, C.byref(cfg)) == 0
    assert cfg.tile_n == 256 and cfg.grid in (148, 296 // 2)
    assert lib.sl8_query_config(None, L.SL8_OP_FC2_RESIDUAL, L.SL8_OUT_BF16, 46656, 1152, 4304, C.byref(cfg)) == 0
    assert cfg.tile_n == 256
    assert lib.sl8_query_config(None, L.SL8_OP_FC2_RESIDUAL, L.SL8_OUT_BF16, 729, 1152, 4304, C.byref(cfg)) == 0
    assert cfg.tile_n == 128 and cfg.cta_group == 1       # too few 256-wide tiles for 148 SMs
    assert lib.sl8_query_config(None, 7, 0, 10, 16, 16, C.byref(cfg)) == L.SL8_ERR_INVALID_VALUE


def test_null_handle_is_rejected(lib):
    import siglip_b200.lib as L
    assert lib.sl8_destroy(None) == L.SL8_ERR_INVALID_VALUE
    assert lib.sl8_set_variant(None, 0) == L.SL8_ERR_INVALID_VALUE
    assert lib.sl8_fc1_gelu_fp8(None, None, 0, None, 0, None, None, None, None, 0, 0, None, 1, 16, 16, 0, None) \
        == L.SL8_ERR_INVALID_VALUE


def test_create_without_gpu_reports_no_device(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import siglip_b200
    with pytest.raises(siglip_b200.SL8Error) as e:
        siglip_b200.Engine(0)
    assert e.value.code == siglip_b200.lib.SL8_ERR_NO_DEVICE
    assert "no CUDA device" in str(e.value)
