"""Builds libsiglip_fp8.so (the CUDA kernels and the C ABI) in-tree for sm_100a.

    python -m siglip_b200.build [--force] [--verbose]

Every kernel configuration of ``csrc/sl8_variants.h`` is one translation unit
(``sl8_variant.cu`` compiled with ``-DSL8_VARIANT_ID=<id>``), so they compile in
parallel; ``sl8_api.cu`` holds the C ABI.  The result is ``siglip_b200/lib/libsiglip_fp8.so``.
nvcc cross-compiles without a GPU.  This is the build-system counterpart of the
reference's Makefile (Makefile:1-28: one nvcc line per layer binary).
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import re
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "lib" / "obj"
LIB = PKG / "lib" / "libsiglip_fp8.so"
BENCH = PKG / "lib" / "siglip_bench"      # per-layer bench host speaking the reference harness's @@RESULT protocol

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ARCH_FLAGS + ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden",
                           "-Xptxas", "-v"]
if os.environ.get("SL8_DIAG"):          # measurement aids in the kernels (see SL8_DBG in sl8_kernel.cuh)
    NVCC_FLAGS.append("-DSL8_DIAG")
NVCC_FLAGS += os.environ.get("SL8_NVCC_DEFINES", "").split()   # tuning macros, e.g. -DSL8_MMA_UNROLL=2


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found: the CUDA toolkit is needed to build libsiglip_fp8.so")
    return exe


def variant_ids() -> list[int]:
    text = (CSRC / "sl8_variants.h").read_text()
    body = text.split("#define SL8_VARIANT_LIST(X)")[1].split("#define SL8_NUM_VARIANTS")[0]
    ids = [int(m) for m in re.findall(r"X\((\d+),", body)]
    declared = int(re.search(r"#define SL8_NUM_VARIANTS (\d+)", text).group(1))
    if ids != list(range(declared)):
        raise RuntimeError(f"SL8_VARIANT_LIST ids {ids} do not match SL8_NUM_VARIANTS {declared}")
    return ids


def sources_mtime() -> float:
    files = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
    files.append(PKG.parent / "include" / "siglip_fp8.h")
    return max(f.stat().st_mtime for f in files)


def compile_one(args: tuple[list[str], Path, bool]) -> str:
    cmd, log, verbose = args
    res = subprocess.run(cmd, capture_output=True, text=True)
    log.write_text(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed: {' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)
    return res.stderr


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compiles what is out of date and returns the path of the shared library."""
    if LIB.exists() and BENCH.exists() and not force and min(LIB.stat().st_mtime, BENCH.stat().st_mtime) >= sources_mtime():
        return LIB
    OBJ.mkdir(parents=True, exist_ok=True)
    for stale in list(OBJ.glob("variant_*.o")) + list(OBJ.glob("variant_*.log")):
        stale.unlink()
    exe = nvcc()
    jobs = []
    objs = []
    for vid in variant_ids():
        o = OBJ / f"variant_{vid}.o"
        objs.append(o)
        jobs.append(([exe, *NVCC_FLAGS, f"-DSL8_VARIANT_ID={vid}", "-c", str(CSRC / "sl8_variant.cu"), "-o", str(o)],
                     OBJ / f"variant_{vid}.log", verbose))
    for name in ("api", "static", "prep"):
        o = OBJ / f"{name}.o"
        objs.append(o)
        jobs.append(([exe, *NVCC_FLAGS, "-c", str(CSRC / f"sl8_{name}.cu"), "-o", str(o)], OBJ / f"{name}.log", verbose))
    with cf.ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as pool:
        list(pool.map(compile_one, jobs))
    link = [exe, *ARCH_FLAGS, "-shared", "-o", str(LIB), *map(str, objs), "-cudart", "static"]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed: {' '.join(link)}\n{res.stdout}\n{res.stderr}")
    bench = [exe, *ARCH_FLAGS, "-O3", "-std=c++17", "-lineinfo", str(CSRC / "sl8_bench.cu"), "-o", str(BENCH),
             f"-L{LIB.parent}", "-lsiglip_fp8", "-lcublasLt", "-ldl", "-Xlinker", "-rpath=$ORIGIN", "-cudart", "static"]
    res = subprocess.run(bench, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"bench host build failed: {' '.join(bench)}\n{res.stdout}\n{res.stderr}")
    return LIB


def resource_report() -> str:
    """Registers / spills / shared memory per kernel, from the ptxas logs of the last build."""
    out = []
    for log in sorted(OBJ.glob("variant_*.log"), key=lambda p: int(p.stem.split("_")[1])):
        text = log.read_text()
        pat = (r"Compiling entry function '(\S+)' for 'sm_100a'\n.*?\n\s*(\d+) bytes stack frame, (\d+) bytes spill stores,"
               r" (\d+) bytes spill loads\n.*?Used (\d+) registers")
        for name, stack, st, ld, regs in re.findall(pat, text):
            out.append(f"{log.stem}: {name} regs={regs} stack={stack} spill_stores={st} spill_loads={ld}")
    return "\n".join(out)


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--report", action="store_true", help="print registers/spills per kernel after building")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
    if a.report:
        print(resource_report())
