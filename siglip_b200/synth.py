"""Seeded synthetic operands with the shapes and value distributions of the benchmark
configurations (SigLIP-B/16 patch-embed; SigLIP-So400m FC1, FC2, patch-embed).

The reference's bench hosts fill constant operands (A = 1.5 everywhere, B rows alternating
1.5 / 1.0: patch_embed.cu:121-145) which cannot reveal a permuted row or K index; these
generators draw activations from N(0, 1) (pixels from U[-1, 1]), weights from N(0, 0.02),
bias from N(0, 0.01), the positional table from N(0, 0.02) and the residual from N(0, 1),
and quantise e4m3 operands per tensor with scale = amax / 448.

Everything is produced by torch on the requested device from an explicit seed, so a CPU
oracle and the GPU path can be fed bit-identical bytes.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

E4M3_MAX = 448.0

OP_PATCH_EMBED, OP_FC1_GELU, OP_FC2_RESIDUAL = 0, 1, 2

# name -> (op, M, N, K, period); M = images x tokens per image
CONFIGS = {
    "C1": dict(op=OP_PATCH_EMBED, M=32 * 196, N=768, K=768, period=196, images=32),
    "C2": dict(op=OP_FC1_GELU, M=64 * 729, N=4304, K=1152, period=0, images=64),
    "C3": dict(op=OP_FC2_RESIDUAL, M=64 * 729, N=1152, K=4304, period=0, images=64),
    "C4": dict(op=OP_PATCH_EMBED, M=256 * 729, N=1152, K=588, period=729, images=256),
}


def pitch16(k: int) -> int:
    """Smallest legal row pitch in bytes for K one-byte elements: TMA wants global strides in multiples of 16."""
    return (k + 15) // 16 * 16


def pitch128(k: int) -> int:
    """Row pitch that starts every row on a 128-byte line.  A TMA box row is 128 bytes; with a pitch that is
    not a multiple of 128 each box row straddles two lines and the operand stream is measurably slower."""
    return (k + 127) // 128 * 128


# Row pitch rule used by the generators below for e4m3 operands (K contiguous).
DEFAULT_PITCH = pitch128


def quantize_e4m3(x: torch.Tensor, scale: Optional[float] = None, pitch: Optional[int] = None):
    """Per-tensor quantisation: returns (uint8 codes [rows, K] viewed out of a [rows, pitch] buffer, scale)."""
    if scale is None:
        amax = float(x.abs().max())
        scale = amax / E4M3_MAX if amax > 0 else 1.0
    q = (x.float() / scale).clamp_(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(torch.uint8)
    rows, k = q.shape
    pitch = DEFAULT_PITCH(k) if pitch is None else pitch
    if pitch == k:
        return q.contiguous(), scale
    buf = torch.zeros((rows, pitch), dtype=torch.uint8, device=x.device)
    buf[:, :k] = q
    return buf[:, :k], scale


@dataclass
class Problem:
    op: int
    M: int
    N: int
    K: int
    A: torch.Tensor                      # uint8 codes [M, K], row pitch a multiple of 16
    B: torch.Tensor                      # uint8 codes [N, K]
    scale_a: float
    scale_b: float
    bias: Optional[torch.Tensor] = None      # bf16 [N]
    table: Optional[torch.Tensor] = None     # bf16 [period, N]   (patch-embed)
    residual: Optional[torch.Tensor] = None  # bf16 [M, N]        (FC2)
    period: int = 0
    extra: dict = field(default_factory=dict)

    def flops(self) -> float:
        return 2.0 * self.M * self.N * self.K

    def min_bytes(self, out_bytes: int = 2) -> float:
        """Algorithmic HBM bytes: operands once, output once, side inputs once."""
        b = self.M * self.K + self.N * self.K + out_bytes * self.M * self.N
        if self.bias is not None:
            b += 2 * self.N
        if self.table is not None:
            b += 2 * self.period * self.N
        if self.residual is not None:
            b += 2 * self.M * self.N
        return float(b)


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def _randn_chunked(rows: int, cols: int, g: torch.Generator, device, std: float = 1.0, uniform: bool = False):
    """Row-chunked generation so the fp32 staging of a large operand stays small on the device."""
    return (torch.rand((rows, cols), generator=g, device=device) * 2 - 1) if uniform \
        else torch.randn((rows, cols), generator=g, device=device) * std


def make_patch_embed(M: int, N: int, K: int, period: int, seed: int = 0, device="cpu", pixels: bool = False) -> Problem:
    g = _gen(seed, device)
    x = _randn_chunked(M, K, g, device, uniform=pixels)
    w = torch.randn((N, K), generator=g, device=device) * 0.02
    table = (torch.randn((period, N), generator=g, device=device) * 0.02).to(torch.bfloat16)
    A, sa = quantize_e4m3(x)
    B, sb = quantize_e4m3(w)
    return Problem(OP_PATCH_EMBED, M, N, K, A, B, sa, sb, table=table, period=period)


def make_fc1(M: int, N: int, K: int, seed: int = 0, device="cpu") -> Problem:
    g = _gen(seed, device)
    x = _randn_chunked(M, K, g, device)
    w = torch.randn((N, K), generator=g, device=device) * 0.02
    bias = (torch.randn((N,), generator=g, device=device) * 0.01).to(torch.bfloat16)
    A, sa = quantize_e4m3(x)
    B, sb = quantize_e4m3(w)
    return Problem(OP_FC1_GELU, M, N, K, A, B, sa, sb, bias=bias)


def make_fc2(M: int, N: int, K: int, seed: int = 0, device="cpu", act: Optional[torch.Tensor] = None,
             act_scale: Optional[float] = None) -> Problem:
    """FC2 operands.  ``act`` (uint8 e4m3 codes [M, K]) is the quantised GELU output of an FC1 when the
    caller has one; otherwise activations are drawn with the distribution a GELU of N(0, 0.68) has."""
    g = _gen(seed + 1, device)
    if act is None:
        pre = torch.randn((M, K), generator=g, device=device) * 0.68
        h = torch.nn.functional.gelu(pre, approximate="tanh")
        A, sa = quantize_e4m3(h)
    else:
        A, sa = act, float(act_scale)
    w = torch.randn((N, K), generator=g, device=device) * 0.02
    bias = (torch.randn((N,), generator=g, device=device) * 0.01).to(torch.bfloat16)
    residual = torch.randn((M, N), generator=g, device=device).to(torch.bfloat16)
    B, sb = quantize_e4m3(w)
    return Problem(OP_FC2_RESIDUAL, M, N, K, A, B, sa, sb, bias=bias, residual=residual)


def make_config(name: str, seed: int = 0, device="cpu", images: Optional[int] = None) -> Problem:
    """Operands of benchmark configuration ``name`` (C1..C4); ``images`` overrides the batch."""
    c = CONFIGS[name]
    rows_per_image = c["M"] // c["images"]
    M = c["M"] if images is None else images * rows_per_image
    if c["op"] == OP_PATCH_EMBED:
        return make_patch_embed(M, c["N"], c["K"], c["period"], seed, device, pixels=(name == "C4"))
    if c["op"] == OP_FC1_GELU:
        return make_fc1(M, c["N"], c["K"], seed, device)
    return make_fc2(M, c["N"], c["K"], seed, device)
