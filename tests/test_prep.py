"""Producer-side steps: patch unfold + quantisation, abs-max scale, row quantisation.

CPU: the oracle's restatement against an independent numpy formulation (unfold by reshape/transpose, e4m3 through
the 256-entry decode table).  GPU: the CUDA kernels against the oracle, bit for bit (byte work)."""
import numpy as np
import pytest
import torch

DEV = "cuda"


def nearest_e4m3(oracle, v):
    """Independent of the oracle's encoder: nearest representable value by search in the decode table, ties to the
    even code, saturating at +-448."""
    lut = oracle.e4m3_lut().astype(np.float64)
    finite = np.array([c for c in range(256) if np.isfinite(lut[c])])
    vals = lut[finite]
    order = np.argsort(vals, kind="stable")
    vals, codes = vals[order], finite[order]
    v = np.clip(np.asarray(v, dtype=np.float64), -448.0, 448.0)
    idx = np.clip(np.searchsorted(vals, v), 1, len(vals) - 1)
    lo, hi = vals[idx - 1], vals[idx]
    pick_hi = (v - lo) > (hi - v)
    tie = (v - lo) == (hi - v)
    even_hi = (codes[idx] & 1) == 0
    pick_hi = np.where(tie, even_hi, pick_hi)
    out = np.where(pick_hi, codes[idx], codes[idx - 1]).astype(np.uint8)
    out = np.where(v == 0.0, np.where(np.signbit(v), 0x80, 0x00), out).astype(np.uint8)
    return out


def unfold_numpy(pixels, P):
    images, C, H, W = pixels.shape
    gh, gw = H // P, W // P
    x = pixels[:, :, :gh * P, :gw * P].reshape(images, C, gh, P, gw, P)
    return x.transpose(0, 2, 4, 1, 3, 5).reshape(images * gh * gw, C * P * P)      # (img, gy, gx) x (c, py, px)


def test_oracle_patchify_matches_an_unfold_by_reshape(oracle):
    rng = np.random.default_rng(0)
    pixels = rng.uniform(-1, 1, size=(2, 3, 30, 45)).astype(np.float32)           # 30 = 2*14 + 2, 45 = 3*14 + 3
    scale = np.float32(1.0 / 448.0)
    A = oracle.patchify_quantize(pixels, 14, float(scale), lda=640, row_bytes=640)
    want = unfold_numpy(pixels, 14) * (np.float32(1.0) / scale)
    assert A.shape == (2 * 2 * 3, 640)
    codes = nearest_e4m3(oracle, want.astype(np.float32))
    assert np.array_equal(A[:, :588], codes)
    assert not A[:, 588:].any()
    short = oracle.patchify_quantize(pixels, 14, float(scale), lda=1024, row_bytes=592)
    assert np.array_equal(short[:, :588], codes) and not short[:, 588:592].any() and (short[:, 592:] == 0xAA).all()


def test_oracle_amax_and_row_quantisation(oracle):
    rng = np.random.default_rng(1)
    x = (rng.standard_normal((37, 50)) * 3).astype(np.float32)
    x[5, 7] = -123.5
    assert oracle.amax(x) == 123.5
    scale = np.float32(123.5 / 448.0)
    q = oracle.quantize_rows(x, float(scale))
    assert np.array_equal(q, nearest_e4m3(oracle, x * (np.float32(1.0) / scale)))
    assert q[5, 7] == 0xFE                                                          # -448: the largest magnitude
    big = oracle.quantize_rows(np.array([[1e9, -1e9, 0.0]], dtype=np.float32), 1.0)
    assert big.tolist() == [[0x7E, 0xFE, 0x00]]                                      # saturation, not NaN


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("images,C,H,W,P", [(3, 3, 384, 384, 14), (2, 3, 224, 224, 16), (1, 1, 30, 45, 7)])
def test_patchify_quantize_on_gpu(engine, oracle, dtype, images, C, H, W, P):
    g = torch.Generator(device=DEV).manual_seed(images * 100 + P)
    pixels = (torch.rand((images, C, H, W), generator=g, device=DEV) * 2 - 1).to(dtype)
    scale = torch.tensor([1.0 / 448.0], device=DEV)
    A = engine.patchify_quantize(pixels, P, scale)
    engine.device_status()
    K = C * P * P
    pitch = A.stride(0)
    full = torch.as_strided(A, (A.shape[0], pitch), (pitch, 1)).cpu().numpy()
    row_bytes = pitch if pitch - K < 128 else (K + 15) // 16 * 16
    ref = oracle.patchify_quantize(pixels.float().cpu().numpy(), P, float(scale.item()), lda=pitch, row_bytes=row_bytes)
    assert np.array_equal(full[:, :row_bytes], ref[:, :row_bytes])
    assert full.shape[0] == images * (H // P) * (W // P)


@pytest.mark.gpu
def test_patchify_feeds_the_patch_embed_gemm(engine, oracle):
    """Pixels -> operand rows -> patch-embed GEMM, against the oracle run on the oracle's own operand rows."""
    from siglip_b200 import synth
    from tests.tolerance import check_bf16
    images, P = 2, 14
    g = torch.Generator(device=DEV).manual_seed(5)
    pixels = torch.rand((images, 3, 384, 384), generator=g, device=DEV) * 2 - 1
    scale_a = 1.0 / 448.0
    A = engine.patchify_quantize(pixels, P, torch.tensor([scale_a], device=DEV))
    p = synth.make_patch_embed(images * 729, 1152, 588, 729, seed=6, device=DEV, pixels=True)
    D = engine.patch_embed(A, p.B, engine.padded_table(p.table), period=729, scale_a=torch.tensor([scale_a], device=DEV),
                           scale_b=torch.tensor([p.scale_b], device=DEV))
    engine.device_status()
    A_ref = oracle.patchify_quantize(pixels.cpu().numpy(), P, scale_a, lda=640, row_bytes=640)[:, :588]
    ref = oracle.patch_embed(np.ascontiguousarray(A_ref), p.B.cpu().numpy(), scale_a, p.scale_b,
                             p.table.view(torch.uint16).cpu().numpy(), 0)
    check_bf16(D.view(torch.uint16).cpu().numpy(), ref, "patchify -> patch-embed")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,cols", [(1000, 4304), (37, 50), (729, 1152)])
def test_amax_and_quantize_on_gpu(engine, oracle, dtype, rows, cols):
    g = torch.Generator(device=DEV).manual_seed(rows + cols)
    x = (torch.randn((rows, cols), generator=g, device=DEV) * 2.5).to(dtype)
    x[rows // 2, cols // 3] = -77.0
    amax, scale = engine.amax_scale(x)
    engine.device_status()
    xf = x.float().cpu().numpy()
    assert amax.item() == oracle.amax(xf) == 77.0
    assert scale.item() == np.float32(77.0) / np.float32(448.0)
    q = engine.quantize_e4m3(x, scale)
    engine.device_status()
    assert np.array_equal(q.cpu().numpy(), oracle.quantize_rows(xf, scale.item()))
    zero_amax, zero_scale = engine.amax_scale(torch.zeros((4, 8), dtype=dtype, device=DEV))
    assert zero_amax.item() == 0.0 and zero_scale.item() == 1.0


@pytest.mark.gpu
def test_dynamic_quantisation_between_fc1_and_fc2(engine, oracle):
    """FC1 (bf16 out) -> abs-max scale -> e4m3 codes -> FC2, against the oracle on the same codes."""
    from siglip_b200 import synth
    from tests.tolerance import check_bf16
    M = 600
    p1 = synth.make_fc1(M, 4304, 1152, seed=41, device=DEV)
    p2 = synth.make_fc2(M, 1152, 4304, seed=42, device=DEV)
    sa1, sb1 = torch.tensor([p1.scale_a], device=DEV), torch.tensor([p1.scale_b], device=DEV)
    H = engine.fc1_gelu(p1.A, p1.B, p1.bias, scale_a=sa1, scale_b=sb1)
    amax, hs = engine.amax_scale(H)
    Hq = engine.quantize_e4m3(H, hs)
    D = engine.fc2_residual(Hq, p2.B, p2.bias, p2.residual, scale_a=hs, scale_b=torch.tensor([p2.scale_b], device=DEV))
    engine.device_status()
    assert Hq.stride(0) % 128 == 0
    codes = Hq.cpu().numpy()
    assert np.array_equal(codes, oracle.quantize_rows(H.float().cpu().numpy(), hs.item()))
    ref = oracle.fc2_residual(np.ascontiguousarray(codes), p2.B.cpu().numpy(), hs.item(), p2.scale_b,
                              p2.bias.view(torch.uint16).cpu().numpy(), p2.residual.view(torch.uint16).cpu().numpy())
    check_bf16(D.view(torch.uint16).cpu().numpy(), ref, "fc1 -> dynamic quantisation -> fc2")


@pytest.mark.gpu
def test_prep_argument_checks(engine):
    from siglip_b200.lib import SL8Error
    px = torch.zeros((1, 3, 28, 28), device=DEV)
    narrow = torch.empty((4, 512), dtype=torch.uint8, device=DEV)
    with pytest.raises(SL8Error):
        engine.patchify_quantize(px, 14, out=narrow)                                 # row pitch 512 < K = 588
    with pytest.raises(TypeError):
        engine.amax_scale(torch.zeros((2, 2), dtype=torch.float16, device=DEV))


def test_oracle_layernorm_quantize_against_numpy(oracle):
    rng = np.random.default_rng(2)
    x = (rng.standard_normal((33, 1152)) * 1.7 + 0.3).astype(np.float32)
    gamma = (1.0 + 0.1 * rng.standard_normal(1152)).astype(np.float32)
    beta = (0.05 * rng.standard_normal(1152)).astype(np.float32)
    scale, eps = 0.01, 1e-6
    q = oracle.layernorm_quantize(x, gamma, beta, eps, scale)
    xd = x.astype(np.float64)
    mean = xd.mean(axis=1, keepdims=True)
    var = ((xd - mean) ** 2).mean(axis=1, keepdims=True)
    y = (xd - mean) / np.sqrt(var + eps) * gamma + beta
    want = nearest_e4m3(oracle, (y / scale).astype(np.float32))
    lut = oracle.e4m3_lut()
    same = q == want
    assert same.mean() > 0.999                               # float vs double intermediates: a rounding tie now and then
    assert np.all(np.abs(lut[q] - lut[want]) <= np.maximum(np.abs(lut[want]) * 0.13, 2.0 ** -9))   # never more than one code


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,cols", [(1000, 1152), (77, 768), (5, 4304 - 4304 % 8)])
def test_layernorm_quantize_on_gpu(engine, oracle, dtype, rows, cols):
    from tests.tolerance import check_e4m3
    g = torch.Generator(device=DEV).manual_seed(rows * 7 + cols)
    x = (torch.randn((rows, cols), generator=g, device=DEV) * 1.5 + 0.25).to(dtype)
    gamma = 1.0 + 0.1 * torch.randn((cols,), generator=g, device=DEV)
    beta = 0.05 * torch.randn((cols,), generator=g, device=DEV)
    scale = torch.tensor([0.0125], device=DEV)
    q = engine.layernorm_quantize(x, gamma, beta, 1e-6, scale)
    engine.device_status()
    ref = oracle.layernorm_quantize(x.float().cpu().numpy(), gamma.cpu().numpy(), beta.cpu().numpy(), 1e-6, float(scale.item()))
    check_e4m3(q.cpu().numpy(), ref, f"layernorm-quantize {rows}x{cols}")
    assert q.stride(0) % 128 == 0
    plain = engine.layernorm_quantize(x, None, None, 1e-6, scale)                  # gamma = 1, beta = 0
    ref_plain = oracle.layernorm_quantize(x.float().cpu().numpy(), np.ones(cols, np.float32), np.zeros(cols, np.float32), 1e-6,
                                          float(scale.item()))
    check_e4m3(plain.cpu().numpy(), ref_plain, "layernorm-quantize without affine")


@pytest.mark.gpu
def test_layernorm_quantize_feeds_fc1(engine, oracle):
    """Residual stream -> LayerNorm -> e4m3 -> FC1, against the oracle's FC1 on the codes the kernel produced."""
    from siglip_b200 import synth
    from tests.tolerance import check_bf16
    M = 500
    g = torch.Generator(device=DEV).manual_seed(9)
    x = torch.randn((M, 1152), generator=g, device=DEV).to(torch.bfloat16)
    scale = torch.tensor([4.0 / 448.0], device=DEV)
    A = engine.layernorm_quantize(x, None, None, 1e-6, scale)
    p = synth.make_fc1(M, 4304, 1152, seed=10, device=DEV)
    D = engine.fc1_gelu(A, p.B, p.bias, scale_a=scale, scale_b=torch.tensor([p.scale_b], device=DEV))
    engine.device_status()
    ref = oracle.fc1_gelu(np.ascontiguousarray(A.cpu().numpy()), p.B.cpu().numpy(), float(scale.item()), p.scale_b,
                          p.bias.view(torch.uint16).cpu().numpy())
    check_bf16(D.view(torch.uint16).cpu().numpy(), ref, "layernorm -> fc1")
