"""Pins the CPU oracle to the reference's own known answers.

The reference validates each layer binary against closed forms of constant operands
(patch_embed.cu:121-145,273-306; fc1_gelu.cu:67-85,200-225; fc2.cu:59-66,88-116,231-259;
periodic rows of cutlass_bench.cu:757).  The same operands are rebuilt here, at a smaller M
(the closed forms do not depend on M), and the oracle must reproduce every expected value
bit for bit.
"""
import numpy as np
import pytest

from tests.oracle_lib import bf16_bits_to_f32, f32_to_bf16_bits

SEQ_LEN = 196  # kernel_common.cuh:79


def ref_operands(M, N, K):
    A = np.full((M, K), 0x3C, dtype=np.uint8)                         # 1.5  (patch_embed.cu:121)
    B = np.empty((N, K), dtype=np.uint8)
    B[0::2] = 0x3C                                                    # even rows 1.5
    B[1::2] = 0x38                                                    # odd rows 1.0 (patch_embed.cu:124-127)
    bias = np.arange(1, N + 1, dtype=np.float32)                      # bias[c] = c + 1
    return A, B, bias


def acc_closed_form(N, K):
    bval = np.where(np.arange(N) % 2 == 1, 1.0, 1.5).astype(np.float32)
    return (np.float32(K) * np.float32(1.5) * bval).astype(np.float32)   # K * 1.5 * b, exact in fp32


def spot_positions(M, N):
    """The reference's 32 spots plus its period-wrap rows."""
    pos = [(s * M // 32, (s * 47) % N) for s in range(32)]
    for r in (0, 1, 195, 196, 197, M // 2, M - 1):
        for c in (0, 1, 47, N - 1):
            pos.append((r, c))
    return pos


def test_codec_known_values(oracle):
    lut = oracle.e4m3_lut()
    assert lut[0x3C] == 1.5 and lut[0x38] == 1.0          # the two codes the reference fills with
    assert lut[0x7E] == 448.0 and lut[0x01] == 2.0 ** -9
    assert np.isnan(lut[0x7F]) and np.isnan(lut[0xFF])
    assert oracle.lib.sl8o_f32_to_e4m3(1.5) == 0x3C and oracle.lib.sl8o_f32_to_e4m3(1e9) == 0x7E
    assert oracle.lib.sl8o_f32_to_bf16(1728.0) == 0x44D8   # 1728 is exact in bf16


def test_patch_embed_reference_known_answers(oracle):
    M, N, K = 2 * 196 + 120, 768, 768
    A, B, bias = ref_operands(M, N, K)
    pos = (3.0 * (np.arange(SEQ_LEN, dtype=np.float32)[:, None] + 1.0)) * np.ones((1, N), dtype=np.float32)
    table = oracle.combine_bias_pos(bias, pos)                         # bf16(bias + pos), patch_embed.cu:96
    assert np.array_equal(table, f32_to_bf16_bits(bias[None, :] + pos))
    D = oracle.patch_embed(A, B, 1.0, 1.0, table)
    acc = acc_closed_form(N, K)
    # patch_embed.cu:281-292: bf16( float(bf16(gemm)) + float(combined) )
    gemm_bf16 = bf16_bits_to_f32(f32_to_bf16_bits(acc))
    rows = np.arange(M) % SEQ_LEN
    expect = f32_to_bf16_bits(gemm_bf16[None, :] + bf16_bits_to_f32(table)[rows])
    for r, c in spot_positions(M, N):
        assert D[r, c] == expect[r, c], (r, c)
    assert np.array_equal(D, expect)
    assert bf16_bits_to_f32(D[0, :2]).tolist() == [1728.0, 1160.0]     # 1728 + 4 ties to even; 1152 + 5 -> 1160


def test_fc1_reference_known_answers(oracle):
    M, N, K = 320, 3072, 768
    A, B, bias = ref_operands(M, N, K)
    D = oracle.fc1_gelu(A, B, 1.0, 1.0, bias, flags=1)                 # fp32 bias as the reference
    x = acc_closed_form(N, K) + bias                                    # fc1_gelu.cu:207-211
    k = np.float32(0.7978845608)
    g = np.float32(0.5) * x * (np.float32(1.0) + np.tanh(k * (x + np.float32(0.044715) * x * x * x), dtype=np.float32))
    expect = np.broadcast_to(f32_to_bf16_bits(g.astype(np.float32)), (M, N))
    for r, c in spot_positions(M, N):
        assert D[r, c] == expect[r, c], (r, c)
    assert np.array_equal(D, expect)


def test_fc2_reference_known_answers(oracle):
    M, N, K = 384, 768, 3072
    A, B, bias = ref_operands(M, N, K)
    r_idx = np.arange(M, dtype=np.float32)[:, None] % 128
    c_idx = np.arange(N, dtype=np.float32)[None, :]
    residual = f32_to_bf16_bits(r_idx * np.float32(0.25) + c_idx * np.float32(0.125))   # fc2.cu:59-66
    D = oracle.fc2_residual(A, B, 1.0, 1.0, bias, residual, flags=1)
    expect = f32_to_bf16_bits((acc_closed_form(N, K) + bias)[None, :] + bf16_bits_to_f32(residual))  # fc2.cu:239-245
    for r, c in spot_positions(M, N):
        assert D[r, c] == expect[r, c], (r, c)
    assert np.array_equal(D, expect)


def test_historical_checksum(oracle):
    """data/clock64_timing.txt:10-11 records checksum 1769472.0 = 1024 x 1728 for the older
    all-1.5 operands with a zero table: 1024 strided samples of 768 * 1.5 * 1.5."""
    M, N, K = 256, 768, 768
    A = np.full((M, K), 0x3C, dtype=np.uint8)
    B = np.full((N, K), 0x3C, dtype=np.uint8)
    table = np.zeros((SEQ_LEN, N), dtype=np.uint16)
    D = bf16_bits_to_f32(oracle.patch_embed(A, B, 1.0, 1.0, table)).ravel()
    stride = D.size // 1024
    assert float(np.sum(D[::stride][:1024], dtype=np.float64)) == 1769472.0


def test_gemm_against_float64(oracle):
    """The FP32-accumulate GEMM against an independent float64 product of the decoded operands."""
    rng = np.random.default_rng(7)
    for (M, N, K) in [(37, 48, 588), (130, 80, 76), (5, 16, 4304)]:
        A = rng.integers(0, 256, size=(M, K), dtype=np.uint8)
        B = rng.integers(0, 256, size=(N, K), dtype=np.uint8)
        A[(A & 0x7F) == 0x7F] = 0x3C
        B[(B & 0x7F) == 0x7F] = 0x38
        lut = oracle.e4m3_lut().astype(np.float64)
        ref = lut[A] @ lut[B].T
        mag = np.abs(lut[A]) @ np.abs(lut[B]).T
        got = oracle.gemm(A, B)
        assert np.all(np.abs(got - ref) <= 1e-6 * mag + 1e-30)


def test_bf16_add_single_rounding(oracle):
    """add.rn.bf16x2 rounds the exact sum once; spot values incl. ties."""
    f = oracle.lib
    one = 0x3F80
    assert f.sl8o_bf16_add(one, 0x3B80) == 0x3F80          # 1 + 2^-8: tie, rounds to even (1.0)
    assert f.sl8o_bf16_add(0x3F81, 0x3B80) == 0x3F82       # 1.0078125 + 2^-8: tie, rounds to even
    assert f.sl8o_bf16_add(one, 0x3B81) == 0x3F81          # just above the tie
    assert f.sl8o_bf16_add(0x44D8, 0x4080) == 0x44D8       # 1728 + 4 = 1732 -> tie between 1728 and 1736: even
    assert bf16_bits_to_f32(np.array([f.sl8o_bf16_add(0x44D8, 0x4100)], dtype=np.uint16))[0] == 1736.0


def test_linear_bias_is_fc1_without_the_activation(oracle):
    """Flag 4 of the FC1 oracle: acc * scale + bias, rounded once; closed form on the reference's constant operands
    (acc = 2.25 K on even columns, 1.5 K on odd ones: patch_embed.cu:121-145)."""
    M, N, K = 64, 128, 256
    A, B, bias = ref_operands(M, N, K)
    D = oracle.fc1_gelu(A, B, 1.0, 1.0, bias, flags=1 | 4)
    want = acc_closed_form(N, K) + bias
    assert np.array_equal(D, np.broadcast_to(f32_to_bf16_bits(want.astype(np.float32)), (M, N)))
