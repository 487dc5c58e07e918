"""Host-side layer interface over torch tensors: the three launches of the reference's
per-layer bench hosts (patch_embed.cu:216, fc1_gelu.cu:147, fc2.cu:178) as methods of one
``Engine`` bound to a GPU.  torch supplies device memory and streams; all arithmetic happens
inside libsiglip_fp8.so.

Operand conventions (those of the reference): ``A`` is [M, K] e4m3 with K contiguous,
``B`` is [N, K] e4m3 (weights stored out x in), outputs are [M, N] row-major.  e4m3
tensors may be ``torch.float8_e4m3fn`` or raw ``torch.uint8`` codes.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import lib as _l


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _is_fp8(t: torch.Tensor) -> bool:
    return t.dtype in (torch.uint8, torch.float8_e4m3fn)


class Engine:
    """One handle of libsiglip_fp8.so (``sl8_create``) on CUDA device ``device``."""

    def __init__(self, device: int = 0):
        self._lib = _l.load_library()
        self._h = C.c_void_p()
        self.device = int(device)
        rc = self._lib.sl8_create(C.byref(self._h), self.device)
        if rc != _l.SL8_OK:
            raise _l.SL8Error(rc, self._lib.sl8_last_error_string(None).decode())

    # ------------------------------------------------------------------ plumbing
    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h.value:
            self._lib.sl8_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def _check(self, rc: int) -> None:
        if rc != _l.SL8_OK:
            raise _l.SL8Error(rc, self._lib.sl8_last_error_string(self._h).decode())

    def _stream(self, stream) -> int:
        if stream is None:
            stream = torch.cuda.current_stream(self.device)
        return stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream)

    def _operands(self, A: torch.Tensor, B: torch.Tensor):
        if not (_is_fp8(A) and _is_fp8(B)):
            raise TypeError("A and B must be float8_e4m3fn or uint8 (raw e4m3 codes)")
        if A.dim() != 2 or B.dim() != 2 or A.stride(1) != 1 or B.stride(1) != 1:
            raise ValueError("A [M, K] and B [N, K] must be 2-D with K contiguous")
        if not (A.is_cuda and B.is_cuda):
            raise ValueError("A and B must be CUDA tensors (use the *_host methods for host operands)")
        self._on_device("A", A)
        self._on_device("B", B)
        M, K = A.shape
        N, Kb = B.shape
        if K != Kb:
            raise ValueError(f"K mismatch: A has {K}, B has {Kb}")
        return M, N, K

    @staticmethod
    def _new_out(M: int, N: int, dtype: torch.dtype, device) -> torch.Tensor:
        return torch.empty((M, N), dtype=dtype, device=device)

    def _on_device(self, name: str, t: Optional[torch.Tensor]) -> None:
        """Every device operand must live on the GPU this handle is bound to: the library dereferences
        the pointer on that GPU whatever device the tensor says it is on."""
        if t is None:
            return
        if not t.is_cuda:
            raise ValueError(f"{name} must be a CUDA tensor")
        if t.device.index != self.device:
            raise ValueError(f"{name} is on cuda:{t.device.index}, this engine is bound to cuda:{self.device}")

    def _check_out(self, out: torch.Tensor, M: int, N: int, allowed: tuple) -> torch.Tensor:
        """A caller-supplied output: [M, N], N contiguous, on this engine's GPU, of an element type the
        layer can write.  The kernel's output type is then taken from the tensor, never from a keyword."""
        if out.dtype not in allowed:
            raise TypeError(f"out has dtype {out.dtype}; this layer writes {' / '.join(str(a) for a in allowed)}")
        if out.dim() != 2 or tuple(out.shape) != (M, N):
            raise ValueError(f"out has shape {tuple(out.shape)}, expected ({M}, {N})")
        if out.stride(1) != 1:
            raise ValueError("out must have its N dimension contiguous")
        self._on_device("out", out)
        return out

    _E4M3_TYPES = (torch.float8_e4m3fn, torch.uint8)

    def _resolve_out(self, out, out_dtype, M: int, N: int, device):
        """(output tensor, SL8_OUT_*) of the layers that can write bf16 or e4m3.  With `out` given its dtype
        decides; an explicit out_dtype that contradicts it is an error."""
        if out is None:
            out_dtype = torch.bfloat16 if out_dtype is None else out_dtype
            if out_dtype != torch.bfloat16 and out_dtype not in self._E4M3_TYPES:
                raise TypeError("out_dtype must be bfloat16, float8_e4m3fn or uint8 (raw e4m3 codes)")
            out = self._new_out(M, N, out_dtype, device)
        else:
            self._check_out(out, M, N, (torch.bfloat16,) + self._E4M3_TYPES)
            if out_dtype is not None:
                same = (out_dtype == out.dtype) or (out_dtype in self._E4M3_TYPES and out.dtype in self._E4M3_TYPES)
                if not same:
                    raise TypeError(f"out_dtype {out_dtype} contradicts out.dtype {out.dtype}")
        return out, (_l.SL8_OUT_E4M3 if out.dtype in self._E4M3_TYPES else _l.SL8_OUT_BF16)

    # ------------------------------------------------------------------ layers
    def patch_embed(self, A, B, table, *, period: Optional[int] = None, scale_a=None, scale_b=None, row_phase: int = 0,
                    out=None, flags: int = 0, stream=None) -> torch.Tensor:
        """D = bf16(bf16(sa*sb*A.B^T) + table[(m + row_phase) % period]).

        ``table`` is bf16 [rows, N]; ``period`` defaults to its row count.  A table made by
        :meth:`padded_table` (rows past the period repeat it) takes the fast path."""
        M, N, K = self._operands(A, B)
        if table.dtype != torch.bfloat16 or table.dim() != 2 or table.shape[1] != N or table.stride(1) != 1:
            raise ValueError("table must be bf16 [rows, N] with N contiguous")
        period = table.shape[0] if period is None else int(period)
        for name, t in (("table", table), ("scale_a", scale_a), ("scale_b", scale_b)):
            self._on_device(name, t)
        D = self._new_out(M, N, torch.bfloat16, A.device) if out is None else self._check_out(out, M, N, (torch.bfloat16,))
        self._check(self._lib.sl8_patch_embed_fp8(
            self._h, A.data_ptr(), A.stride(0), B.data_ptr(), B.stride(0), _ptr(scale_a), _ptr(scale_b),
            table.data_ptr(), table.stride(0), period, table.shape[0], int(row_phase), D.data_ptr(), D.stride(0),
            M, N, K, int(flags), self._stream(stream)))
        return D

    def padded_table(self, table: torch.Tensor, stream=None) -> torch.Tensor:
        """bf16 [period, N] -> bf16 [sl8_padded_table_rows(period), N] whose extra rows repeat the period."""
        period, N = table.shape
        rows = self._lib.sl8_padded_table_rows(period)
        out = torch.empty((rows, N), dtype=torch.bfloat16, device=table.device)
        self._check(self._lib.sl8_extend_periodic_table(self._h, table.data_ptr(), table.stride(0), period, N,
                                                        out.data_ptr(), out.stride(0), rows, self._stream(stream)))
        return out

    def make_table(self, bias: Optional[torch.Tensor], pos: torch.Tensor, stream=None) -> torch.Tensor:
        """fp32 bias [N] (or None) and fp32 pos [period, N] -> padded bf16 table of bf16(bias + pos)."""
        period, N = pos.shape
        rows = self._lib.sl8_padded_table_rows(period)
        out = torch.empty((rows, N), dtype=torch.bfloat16, device=pos.device)
        pos = pos.contiguous().float()
        b = None if bias is None else bias.contiguous().float()
        self._check(self._lib.sl8_make_periodic_table(self._h, _ptr(b), pos.data_ptr(), period, N, out.data_ptr(),
                                                      out.stride(0), rows, self._stream(stream)))
        return out

    def fc1_gelu(self, A, B, bias, *, scale_a=None, scale_b=None, out_dtype=None, out_scale=None,
                 out=None, flags: int = 0, stream=None) -> torch.Tensor:
        """D = cast(gelu_tanh(sa*sb*A.B^T + bias) / out_scale); bias bf16 [N] (fp32 with SL8_FLAG_BIAS_F32).
        The output type is that of ``out`` when it is given, else ``out_dtype`` (default bf16)."""
        M, N, K = self._operands(A, B)
        if bias is not None and bias.dtype == torch.float32:
            flags |= _l.SL8_FLAG_BIAS_F32
        elif bias is not None and bias.dtype != torch.bfloat16:
            raise TypeError("bias must be bf16 or fp32")
        for name, t in (("bias", bias), ("scale_a", scale_a), ("scale_b", scale_b), ("out_scale", out_scale)):
            self._on_device(name, t)
        D, out_code = self._resolve_out(out, out_dtype, M, N, A.device)
        self._check(self._lib.sl8_fc1_gelu_fp8(
            self._h, A.data_ptr(), A.stride(0), B.data_ptr(), B.stride(0), _ptr(scale_a), _ptr(scale_b), _ptr(bias),
            D.data_ptr(), D.stride(0), out_code, _ptr(out_scale), M, N, K,
            int(flags), self._stream(stream)))
        return D

    def linear_bias(self, A, B, bias, *, scale_a=None, scale_b=None, out_dtype=None, out_scale=None,
                    out=None, flags: int = 0, stream=None) -> torch.Tensor:
        """D = cast((sa*sb*A.B^T + bias) / out_scale): the Q / K / V projections (no activation)."""
        M, N, K = self._operands(A, B)
        if bias is not None and bias.dtype == torch.float32:
            flags |= _l.SL8_FLAG_BIAS_F32
        elif bias is not None and bias.dtype != torch.bfloat16:
            raise TypeError("bias must be bf16 or fp32")
        for name, t in (("bias", bias), ("scale_a", scale_a), ("scale_b", scale_b), ("out_scale", out_scale)):
            self._on_device(name, t)
        D, out_code = self._resolve_out(out, out_dtype, M, N, A.device)
        self._check(self._lib.sl8_linear_bias_fp8(
            self._h, A.data_ptr(), A.stride(0), B.data_ptr(), B.stride(0), _ptr(scale_a), _ptr(scale_b), _ptr(bias),
            D.data_ptr(), D.stride(0), out_code, _ptr(out_scale), M, N, K,
            int(flags), self._stream(stream)))
        return D

    def fc2_residual(self, A, B, bias, residual, *, scale_a=None, scale_b=None, out=None, flags: int = 0,
                     stream=None) -> torch.Tensor:
        """D = bf16((sa*sb*A.B^T + bias) + residual); residual bf16 [M, N]."""
        M, N, K = self._operands(A, B)
        if bias is not None and bias.dtype == torch.float32:
            flags |= _l.SL8_FLAG_BIAS_F32
        if residual.dtype != torch.bfloat16 or residual.shape != (M, N) or residual.stride(1) != 1:
            raise ValueError("residual must be bf16 [M, N] with N contiguous")
        for name, t in (("bias", bias), ("residual", residual), ("scale_a", scale_a), ("scale_b", scale_b)):
            self._on_device(name, t)
        D = self._new_out(M, N, torch.bfloat16, A.device) if out is None else self._check_out(out, M, N, (torch.bfloat16,))
        self._check(self._lib.sl8_fc2_residual_fp8(
            self._h, A.data_ptr(), A.stride(0), B.data_ptr(), B.stride(0), _ptr(scale_a), _ptr(scale_b), _ptr(bias),
            residual.data_ptr(), residual.stride(0), D.data_ptr(), D.stride(0), M, N, K, int(flags),
            self._stream(stream)))
        return D

    def mlp_chain(self, A, W1, bias1, W2, bias2, residual, *, scale_a, scale_w1, scale_w2, hidden_scale, hidden=None,
                  out=None, flags: int = 0, stream=None) -> torch.Tensor:
        """D = FC2(e4m3(GELU(FC1(A)) / hidden_scale)) + residual: the block's MLP as one call (sl8_mlp_chain_fp8).
        ``hidden`` is the e4m3 scratch [M, d_ff] (uint8, row pitch a multiple of 16 bytes); allocated when None."""
        M, d_ff, d_model = self._operands(A, W1)
        n2, k2 = W2.shape
        if (n2, k2) != (d_model, d_ff) or not _is_fp8(W2) or W2.stride(1) != 1:
            raise ValueError(f"W2 must be e4m3 [{d_model}, {d_ff}] with K contiguous")
        if residual.dtype != torch.bfloat16 or tuple(residual.shape) != (M, d_model) or residual.stride(1) != 1:
            raise ValueError("residual must be bf16 [M, d_model] with d_model contiguous")
        if hidden_scale is None:
            raise ValueError("hidden_scale (device float) is required: the scale of the e4m3 hidden activations")
        if bias1 is not None and bias1.dtype == torch.float32:
            flags |= _l.SL8_FLAG_BIAS_F32
        if hidden is None:
            hidden = torch.empty((M, (d_ff + 127) // 128 * 128), dtype=torch.uint8, device=A.device)[:, :d_ff]
        self._check_out(hidden, M, d_ff, self._E4M3_TYPES)
        for name, t in (("W2", W2), ("bias1", bias1), ("bias2", bias2), ("residual", residual), ("scale_a", scale_a),
                        ("scale_w1", scale_w1), ("scale_w2", scale_w2), ("hidden_scale", hidden_scale)):
            self._on_device(name, t)
        D = self._new_out(M, d_model, torch.bfloat16, A.device) if out is None else self._check_out(out, M, d_model, (torch.bfloat16,))
        self._check(self._lib.sl8_mlp_chain_fp8(
            self._h, A.data_ptr(), A.stride(0), W1.data_ptr(), W1.stride(0), _ptr(scale_a), _ptr(scale_w1), _ptr(bias1),
            hidden.data_ptr(), hidden.stride(0), _ptr(hidden_scale), W2.data_ptr(), W2.stride(0), _ptr(scale_w2), _ptr(bias2),
            residual.data_ptr(), residual.stride(0), D.data_ptr(), D.stride(0), M, d_model, d_ff, int(flags),
            self._stream(stream)))
        return D

    def mlp_chain_host(self, A, W1, bias1, W2, bias2, residual, out, *, scale_a, scale_w1, scale_w2, hidden_scale, flags=0):
        """The MLP on HOST tensors (pinned memory gives full bus speed): A and the residual go up, D comes down, the
        hidden activations stay on the GPU (sl8_mlp_chain_fp8_host).  Blocking."""
        M, d_model = A.shape
        d_ff = W1.shape[0]
        if bias1 is not None and bias1.dtype == torch.float32:
            flags |= _l.SL8_FLAG_BIAS_F32
        self._check(self._lib.sl8_mlp_chain_fp8_host(
            self._h, A.data_ptr(), A.stride(0), W1.data_ptr(), W1.stride(0), float(scale_a), float(scale_w1), _ptr(bias1),
            float(hidden_scale), W2.data_ptr(), W2.stride(0), float(scale_w2), _ptr(bias2), residual.data_ptr(),
            residual.stride(0), out.data_ptr(), out.stride(0), M, d_model, d_ff, int(flags)))
        return out

    # ------------------------------------------------------------------ producer-side steps
    @staticmethod
    def _dt(x) -> int:
        if x.dtype == torch.float32:
            return _l.SL8_DT_F32
        if x.dtype == torch.bfloat16:
            return _l.SL8_DT_BF16
        raise TypeError("expected an fp32 or bf16 tensor")

    def patchify_quantize(self, pixels, patch: int, scale=None, *, out=None, pitch=None, stream=None) -> torch.Tensor:
        """pixels [images, C, H, W] (fp32 / bf16) -> A [images * (H // patch) * (W // patch), C * patch * patch] e4m3
        codes (uint8) at a row pitch that is a multiple of 128 bytes: the patch-embed GEMM's operand."""
        if pixels.dim() != 4 or not pixels.is_contiguous():
            raise ValueError("pixels must be a contiguous [images, C, H, W] tensor")
        images, Cc, H, W = pixels.shape
        K = Cc * patch * patch
        rows = images * (H // patch) * (W // patch)
        if out is None:
            pitch = (K + 127) // 128 * 128 if pitch is None else int(pitch)
            out = torch.empty((rows, pitch), dtype=torch.uint8, device=pixels.device)[:, :K]
        self._check(self._lib.sl8_patchify_quantize_e4m3(
            self._h, pixels.data_ptr(), self._dt(pixels), images, Cc, H, W, int(patch), _ptr(scale), out.data_ptr(),
            out.stride(0), self._stream(stream)))
        return out

    def amax_scale(self, x, stream=None):
        """(amax, scale) as one-element device tensors: max |x| and amax / 448."""
        amax = torch.empty((1,), dtype=torch.float32, device=x.device)
        scale = torch.empty((1,), dtype=torch.float32, device=x.device)
        self._check(self._lib.sl8_amax_scale(self._h, x.data_ptr(), self._dt(x), x.shape[0], x.shape[1], x.stride(0),
                                             amax.data_ptr(), scale.data_ptr(), self._stream(stream)))
        return amax, scale

    def quantize_e4m3(self, x, scale=None, *, out=None, stream=None) -> torch.Tensor:
        """e4m3 codes (uint8) of x / scale, row pitch a multiple of 128 bytes unless `out` is given."""
        rows, cols = x.shape
        if out is None:
            out = torch.empty((rows, (cols + 127) // 128 * 128), dtype=torch.uint8, device=x.device)[:, :cols]
        self._check(self._lib.sl8_quantize_e4m3(self._h, x.data_ptr(), self._dt(x), rows, cols, x.stride(0), _ptr(scale),
                                                out.data_ptr(), out.stride(0), self._stream(stream)))
        return out

    def layernorm_quantize(self, x, gamma=None, beta=None, eps: float = 1e-6, scale=None, *, out=None, stream=None) -> torch.Tensor:
        """e4m3 codes (uint8) of LayerNorm(x) / scale: FC1's A operand, row pitch a multiple of 128 bytes."""
        rows, cols = x.shape
        if out is None:
            out = torch.empty((rows, (cols + 127) // 128 * 128), dtype=torch.uint8, device=x.device)[:, :cols]
        self._check(self._lib.sl8_layernorm_quantize_e4m3(
            self._h, x.data_ptr(), self._dt(x), rows, cols, x.stride(0), _ptr(gamma), _ptr(beta), float(eps), _ptr(scale),
            out.data_ptr(), out.stride(0), self._stream(stream)))
        return out

    # ------------------------------------------------------------------ host operands
    def patch_embed_host(self, A, B, table, out, *, period=None, scale_a=1.0, scale_b=1.0, row_phase=0, flags=0):
        M, K = A.shape
        N = B.shape[0]
        period = table.shape[0] if period is None else int(period)
        self._check(self._lib.sl8_patch_embed_fp8_host(
            self._h, A.data_ptr(), A.stride(0), B.data_ptr(), B.stride(0), float(scale_a), float(scale_b),
            table.data_ptr(), table.stride(0), period, table.shape[0], int(row_phase), out.data_ptr(), out.stride(0),
            M, N, K, int(flags)))
        return out

    def fc1_gelu_host(self, A, B, bias, out, *, scale_a=1.0, scale_b=1.0, out_scale=1.0, flags=0):
        M, K = A.shape
        N = B.shape[0]
        if bias is not None and bias.dtype == torch.float32:
            flags |= _l.SL8_FLAG_BIAS_F32
        e4 = out.dtype in (torch.float8_e4m3fn, torch.uint8)
        self._check(self._lib.sl8_fc1_gelu_fp8_host(
            self._h, A.data_ptr(), A.stride(0), B.data_ptr(), B.stride(0), float(scale_a), float(scale_b),
            _ptr(bias), out.data_ptr(), out.stride(0), _l.SL8_OUT_E4M3 if e4 else _l.SL8_OUT_BF16,
            float(out_scale), M, N, K, int(flags)))
        return out

    def fc2_residual_host(self, A, B, bias, residual, out, *, scale_a=1.0, scale_b=1.0, flags=0):
        M, K = A.shape
        N = B.shape[0]
        if bias is not None and bias.dtype == torch.float32:
            flags |= _l.SL8_FLAG_BIAS_F32
        self._check(self._lib.sl8_fc2_residual_fp8_host(
            self._h, A.data_ptr(), A.stride(0), B.data_ptr(), B.stride(0), float(scale_a), float(scale_b),
            _ptr(bias), residual.data_ptr(), residual.stride(0), out.data_ptr(), out.stride(0), M, N, K,
            int(flags)))
        return out

    # ------------------------------------------------------------------ dispatch and watchdog
    def query_config(self, op: int, M: int, N: int, K: int, out_dtype: int = _l.SL8_OUT_BF16) -> dict:
        cfg = _l.Config()
        self._check(self._lib.sl8_query_config(self._h, op, out_dtype, M, N, K, C.byref(cfg)))
        return cfg.as_dict()

    def set_variant(self, variant_id: int) -> None:
        self._check(self._lib.sl8_set_variant(self._h, int(variant_id)))

    def set_wait_budget_ms(self, ms: int) -> None:
        self._check(self._lib.sl8_set_wait_budget_ms(self._h, int(ms)))

    def set_wait_budget_us(self, us: int) -> None:
        self._check(self._lib.sl8_set_wait_budget_us(self._h, int(us)))

    def device_status(self, stream=None) -> None:
        """Synchronises the stream and raises SL8Error(SL8_ERR_DEVICE_TIMEOUT) if a device wait expired."""
        detail = (C.c_uint * 4)()
        rc = self._lib.sl8_device_status(self._h, self._stream(stream), C.byref(detail))
        self.last_status_detail = tuple(int(x) for x in detail)      # (code, barrier / stage index, tile, block)
        self._check(rc)


    # ------------------------------------------------------------------ tracing
    TRACE_FIELDS = ("producer_wait", "producer_total", "mma_wait_operands", "mma_wait_accumulator", "mma_total",
                    "epi_wait_accumulator", "epi_total", "epi_wait_store", "tiles", "epi_wait_tmem_load",
                    "epi_math", "epi_store_issue", "epi_refill", "epi_prefetch_issue", "mma_issue", "mma_commit")

    def trace_enable(self, on=True, coarse: bool = False) -> None:
        """Tracing on / off; ``coarse`` records the per-role totals only and leaves the hot loops untimed."""
        self._check(self._lib.sl8_trace_enable(self._h, (2 if coarse else 1) if on else 0))

    def trace_read(self, max_blocks: int = 512) -> list:
        """Per-CTA cycle totals of the last launch (see sl8_trace_read)."""
        buf = (C.c_longlong * (max_blocks * 16))()
        n = self._lib.sl8_trace_read(self._h, buf, max_blocks)
        if n < 0:
            self._check(n)
        return [{k: buf[b * 16 + i] for i, k in enumerate(self.TRACE_FIELDS)} for b in range(n)]


def num_variants() -> int:
    return _l.load_library().sl8_num_variants()


def describe_variant(variant_id: int) -> dict:
    cfg = _l.Config()
    rc = _l.load_library().sl8_describe_variant(int(variant_id), C.byref(cfg))
    if rc != _l.SL8_OK:
        raise _l.SL8Error(rc, "no such variant")
    return cfg.as_dict()
