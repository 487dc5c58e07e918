"""The C++ bench host (siglip_b200/lib/siglip_bench) speaks the reference harness's protocol: its result lines
must parse with the regular expressions of the reference's drivers (tools/grid_search.py:155,
tools/compare_all.py:93, tools/stat_test.py:27) and its closed-form spot checks -- the reference's own
(patch_embed.cu:273-306, fc1_gelu.cu:200-225, fc2.cu:231-259) -- must pass."""
import re
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

BENCH = Path(__file__).resolve().parent.parent / "siglip_b200" / "lib" / "siglip_bench"
GRID_SEARCH_RE = r'@@RESULT ms=([\d.]+) tflops=([\d.]+) checksum=([\d.]+) valid=([01]) c0=([\d.]+)'
COMPARE_ALL_RE = r'@@RESULT ms=([\d.]+) tflops=([\d.]+) checksum=[\d.]+ valid=([01])'
STAT_TEST_RE = r"Custom kernel:\s+([\d.]+)\s+ms"


@pytest.mark.parametrize("layer,extra", [("pe", []), ("fc1", []), ("fc2", []), ("pe", ["--N", "1152", "--K", "588", "--period", "729"])])
def test_bench_host_protocol(layer, extra):
    if not BENCH.exists():
        pytest.fail(f"{BENCH} missing: python -m siglip_b200.build")
    # 37 x 196 + 5 rows: a partial last tile, spots that land in every image phase
    out = subprocess.run([str(BENCH), "--layer", layer, "--M", "72581", *extra], capture_output=True, text=True, timeout=300)
    text = out.stdout + out.stderr
    assert out.returncode == 0, text[-2000:]
    line = [l for l in text.splitlines() if l.startswith("@@RESULT")]
    assert len(line) == 1, text[-2000:]
    m = re.match(GRID_SEARCH_RE, line[0])
    assert m and re.match(COMPARE_ALL_RE, line[0]) and re.search(STAT_TEST_RE, text)
    ms, tflops, checksum, valid, c0 = float(m.group(1)), float(m.group(2)), float(m.group(3)), int(m.group(4)), float(m.group(5))
    assert valid == 1 and ms > 0 and tflops > 0 and checksum > 0
    if layer == "pe" and not extra:
        assert c0 == 1728.0        # 768 * 2.25 + bf16(1 + 3), rounded to even: the reference prints the same c0


@pytest.mark.parametrize("config,layer,N", [("C1", "pe", 768), ("C3", "fc2", 1152)])
def test_bench_host_named_configs_and_json_line(config, layer, N):
    import json
    out = subprocess.run([str(BENCH), "--config", config, "--runs", "3"], capture_output=True, text=True, timeout=300)
    text = out.stdout + out.stderr
    assert out.returncode == 0, text[-2000:]
    js = [json.loads(l) for l in text.splitlines() if l.startswith("{")]
    assert len(js) == 1 and js[0]["layer"] == layer and js[0]["N"] == N and js[0]["valid"] == 1 and js[0]["tflops"] > 0
    assert re.search(GRID_SEARCH_RE, text)
