"""siglip_b200 -- B200 (sm_100a) FP8 GEMM engine for the three dense contractions of a
SigLIP ViT encoder block: patch-embed + periodic table add, FC1 + bias + GELU(tanh),
FC2 + bias + residual.

The product is the C-ABI shared library ``libsiglip_fp8.so`` (declared in
``include/siglip_fp8.h``).  This package holds its CUDA sources (``csrc/``), its build
step (``build.py``), a ctypes binding (``lib.py``), the host-side layer interface over
torch tensors (``layers.py``) and the seeded synthetic operands of the benchmark
configurations (``synth.py``).  There is no CPU fallback: without the built library, or
without an sm_100 device, the calls raise.
"""
from .lib import SL8Error, load_library, library_path  # noqa: F401
from .layers import Engine  # noqa: F401

__all__ = ["Engine", "SL8Error", "load_library", "library_path"]
