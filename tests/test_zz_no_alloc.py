"""sl8_fc1_gelu_fp8_static: FC1 for callers that may not allocate device memory (an enqueue callback of an
inference plug-in, a serving loop with a frozen memory pool).  Its status block and trace records live in a
__device__ array inside the library instead of cudaMalloc'ed memory, so it needs no handle.

Called twice in a row through the C ABI (the array is shared by every call and keeps what the previous one left:
the second call, with tracing on, runs on an array the first one has used), each result compared with the
handle-based sl8_fc1_gelu_fp8 on the same operands: same arithmetic, so the outputs must be bit-identical, and the
status words copied back must be zero although the host buffer was poisoned beforehand.  This file sorts last on
purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes as C

import pytest
import torch

from siglip_b200 import synth
import siglip_b200.lib as L

pytestmark = pytest.mark.gpu

DEV = "cuda"


def static_call(lib, p, sa, sb, out, status, trace=None, out_scale=None):
    e4 = out.dtype == torch.uint8
    return lib.sl8_fc1_gelu_fp8_static(
        p.A.data_ptr(), p.A.stride(0), p.B.data_ptr(), p.B.stride(0), sa.data_ptr(), sb.data_ptr(), p.bias.data_ptr(),
        out.data_ptr(), out.stride(0), L.SL8_OUT_E4M3 if e4 else L.SL8_OUT_BF16, None if out_scale is None else out_scale.data_ptr(),
        p.M, p.N, p.K, 0, status.data_ptr(), None if trace is None else trace.data_ptr(), torch.cuda.current_stream().cuda_stream)


def test_static_entry_point_matches_handle_based_call_twice(engine):
    lib = L.load_library()
    for call, (M, N, K, seed) in enumerate([(4864, 1024, 1152, 1), (5000, 1072, 588, 2)]):
        p = synth.make_fc1(M, N, K, seed=seed, device=DEV)
        sa = torch.tensor([p.scale_a], device=DEV)
        sb = torch.tensor([p.scale_b], device=DEV)
        want = engine.fc1_gelu(p.A, p.B, p.bias, scale_a=sa, scale_b=sb)
        engine.device_status()
        got = torch.full((M, N), -3.0, dtype=torch.bfloat16, device=DEV)
        status = torch.full((4,), 0xFFFFFFFF, dtype=torch.int64).to(torch.int32).pin_memory()   # poisoned
        trace = torch.zeros((512 * 16,), dtype=torch.int64).pin_memory()        # SL8_STATIC_MAX_CTAS records
        ctas = static_call(lib, p, sa, sb, got, status, trace if call == 1 else None)
        torch.cuda.synchronize()
        assert ctas > 0, f"call {call}: status code {ctas}"
        assert status.tolist() == [0, 0, 0, 0], f"call {call}: device status {status.tolist()}"
        assert torch.equal(got.view(torch.uint16), want.view(torch.uint16)), f"call {call}: outputs differ"
        if call == 1:       # tracing on: one record per CTA, the leaders report their tiles
            rec = trace[: ctas * 16].view(ctas, 16)
            tiles = ((M + 255) // 256) * ((N + 255) // 256)
            assert int(rec[::2, 8].sum()) == tiles


def test_static_entry_point_e4m3_and_errors(engine):
    lib = L.load_library()
    p = synth.make_fc1(2560, 2048, 1152, seed=3, device=DEV)
    sa, sb = torch.tensor([p.scale_a], device=DEV), torch.tensor([p.scale_b], device=DEV)
    osc = torch.tensor([0.01], device=DEV)
    want = engine.fc1_gelu(p.A, p.B, p.bias, scale_a=sa, scale_b=sb, out_dtype=torch.uint8, out_scale=osc)
    got = torch.zeros((p.M, p.N), dtype=torch.uint8, device=DEV)
    status = torch.zeros((4,), dtype=torch.int32).pin_memory()
    assert static_call(lib, p, sa, sb, got, status, out_scale=osc) > 0
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    # refusals: bad alignment, N not a multiple of 16, a flag this entry point does not take
    bad = lib.sl8_fc1_gelu_fp8_static(p.A.data_ptr() + 8, p.A.stride(0), p.B.data_ptr(), p.B.stride(0), None, None, None,
                                      got.data_ptr(), got.stride(0), L.SL8_OUT_E4M3, None, p.M, p.N, p.K, 0, None, None, None)
    assert bad == L.SL8_ERR_ALIGNMENT
    bad = lib.sl8_fc1_gelu_fp8_static(p.A.data_ptr(), p.A.stride(0), p.B.data_ptr(), p.B.stride(0), None, None, None,
                                      got.data_ptr(), got.stride(0), L.SL8_OUT_E4M3, None, p.M, 40, p.K, 0, None, None, None)
    assert bad == L.SL8_ERR_UNSUPPORTED
    bad = lib.sl8_fc1_gelu_fp8_static(p.A.data_ptr(), p.A.stride(0), p.B.data_ptr(), p.B.stride(0), None, None, None,
                                      got.data_ptr(), got.stride(0), L.SL8_OUT_E4M3, None, p.M, p.N, p.K, L.SL8_FLAG_PE_F32_ADD, None, None, None)
    assert bad == L.SL8_ERR_INVALID_VALUE
    # a scale pointer that is not 4-byte aligned is refused on the host (the kernel would fault on it)
    bad = lib.sl8_fc1_gelu_fp8_static(p.A.data_ptr(), p.A.stride(0), p.B.data_ptr(), p.B.stride(0), sa.data_ptr() + 2, None, None,
                                      got.data_ptr(), got.stride(0), L.SL8_OUT_E4M3, None, p.M, p.N, p.K, 0, None, None, None)
    assert bad == L.SL8_ERR_ALIGNMENT
