"""Parity at the sizes the benchmark configurations are quoted on (C1 .. C4, C5's chain on one 64-image shard).

C1 is small enough for the CPU oracle to compute whole.  At the So400m sizes (46 656 and 186 624 rows) the
oracle computes runs of rows chosen at every kind of tile boundary plus seeded random ones -- a GEMM row
depends on its own row of A only -- and the rest of the matrix is covered by properties that need no oracle:

  * two launches give bit-identical outputs;
  * rows computed as a shard of their own (the way images are divided over GPUs: another M, another tile
    grid, for patch-embed another row phase) are bit-identical to the same rows of the full launch, both for a
    shard that starts on an image boundary and for one that starts in the middle of an image and of a tile;
  * every output is finite.

The reference checks 32 spot elements per run (patch_embed.cu:281-292, fc1_gelu.cu:207-211, fc2.cu:239-245).
"""
import numpy as np
import pytest
import torch

from siglip_b200 import synth
from tests.tolerance import check_bf16, check_e4m3

pytestmark = pytest.mark.gpu

DEV = "cuda"
RUN = 8                     # rows per sampled run


def dscalar(x):
    return torch.tensor([x], dtype=torch.float32, device=DEV)


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.uint16).cpu().numpy()


def sample_runs(M: int, seed: int, random_runs: int = 24) -> list:
    """First rows of RUN-row runs: around the 128- and 256-row tile edges at both ends of the matrix, around an
    image boundary (729 rows), the last rows, and seeded random places."""
    starts = {0, 124, 252, 725, 729 - 4, M - RUN, M - 128 - 4, M - 256 - 4, (M // 2 // 256) * 256 - 4}
    rng = np.random.default_rng(seed)
    starts.update(int(x) for x in rng.integers(0, M - RUN, size=random_runs))
    return sorted(s for s in starts if 0 <= s <= M - RUN)


def launch(engine, p, A=None, residual=None, row_phase=0, table=None):
    """One call of the layer `p` describes, on `A` / `residual` (default: the whole problem)."""
    A = p.A if A is None else A
    kw = dict(scale_a=dscalar(p.scale_a), scale_b=dscalar(p.scale_b))
    if p.op == synth.OP_FC1_GELU:
        D = engine.fc1_gelu(A, p.B, p.bias, **kw)
    elif p.op == synth.OP_FC2_RESIDUAL:
        D = engine.fc2_residual(A, p.B, p.bias, p.residual if residual is None else residual, **kw)
    else:
        D = engine.patch_embed(A, p.B, table, period=p.period, row_phase=row_phase, **kw)
    engine.device_status()
    return D


def oracle_rows(oracle, p, s: int) -> np.ndarray:
    """The oracle's output for rows s .. s + RUN - 1."""
    A = np.ascontiguousarray(p.A[s:s + RUN].cpu().numpy())
    B = p.B.cpu().numpy()
    if p.op == synth.OP_FC1_GELU:
        return oracle.fc1_gelu(A, B, p.scale_a, p.scale_b, bits(p.bias))
    if p.op == synth.OP_FC2_RESIDUAL:
        return oracle.fc2_residual(A, B, p.scale_a, p.scale_b, bits(p.bias), bits(p.residual[s:s + RUN]))
    return oracle.patch_embed(A, B, p.scale_a, p.scale_b, bits(p.table), row_phase=s % p.period)


def check_full_size(engine, oracle, p, what: str, seed: int):
    table = engine.padded_table(p.table) if p.table is not None else None
    D = launch(engine, p, table=table)
    assert bool(torch.isfinite(D.view(-1)[::97].float()).all()) and bool(torch.isfinite(D[-300:].float()).all())

    # sampled runs against the oracle, judged together (one rms, one share of bit-identical elements)
    runs = sample_runs(p.M, seed)
    got = np.concatenate([bits(D[s:s + RUN]) for s in runs])
    ref = np.concatenate([oracle_rows(oracle, p, s) for s in runs])
    stats = check_bf16(got, ref, f"{what}: {len(runs)} runs of {RUN} rows")

    # determinism
    D2 = launch(engine, p, table=table)
    assert torch.equal(D.view(torch.uint16), D2.view(torch.uint16)), f"{what}: two launches differ"
    del D2

    # shards: images 5 .. 20 on their own, and a range that starts inside an image and inside a tile
    rows_per_image = p.period if p.period else 729
    for r0, r1 in ((5 * rows_per_image, 21 * rows_per_image), (3 * rows_per_image + 77, 9 * rows_per_image + 301)):
        if r1 > p.M:
            continue
        res = p.residual[r0:r1] if p.residual is not None else None
        Ds = launch(engine, p, A=p.A[r0:r1], residual=res, row_phase=r0 % rows_per_image, table=table)
        assert torch.equal(Ds.view(torch.uint16), D[r0:r1].view(torch.uint16)), f"{what}: shard rows {r0}..{r1} differ from the full launch"
    return stats


def test_c1_whole_matrix_against_the_oracle(engine, oracle):
    p = synth.make_config("C1", seed=0, device=DEV)
    D = launch(engine, p, table=engine.padded_table(p.table))
    ref = oracle.patch_embed(p.A.cpu().numpy(), p.B.cpu().numpy(), p.scale_a, p.scale_b, bits(p.table))
    check_bf16(bits(D), ref, "C1 patch-embed 6272x768x768")


@pytest.mark.parametrize("name", ["C2", "C4"])
def test_full_size_fc1_and_patch_embed(engine, oracle, name):
    p = synth.make_config(name, seed=0, device=DEV)
    c = synth.CONFIGS[name]
    assert (p.M, p.N, p.K) == (c["M"], c["N"], c["K"])
    check_full_size(engine, oracle, p, name, seed=11)


def test_full_size_chain_fc1_e4m3_into_fc2(engine, oracle):
    """C3 as the configuration defines it: FC2's operand is the e4m3 output of a seeded FC1 at the C2 size (one
    64-image shard of the C5 chain).  FC1's codes are checked on sampled runs, FC2 in full-size fashion on the very
    codes FC1 wrote."""
    c2, c3 = synth.CONFIGS["C2"], synth.CONFIGS["C3"]
    p1 = synth.make_config("C2", seed=0, device=DEV)
    h_scale = 0.0125
    H = torch.zeros((c2["M"], synth.pitch128(c2["N"])), dtype=torch.uint8, device=DEV)[:, :c2["N"]]
    engine.fc1_gelu(p1.A, p1.B, p1.bias, scale_a=dscalar(p1.scale_a), scale_b=dscalar(p1.scale_b), out=H,
                    out_dtype=torch.uint8, out_scale=dscalar(h_scale))
    engine.device_status()
    runs = sample_runs(c2["M"], seed=12)
    got = np.concatenate([H[s:s + RUN].cpu().numpy() for s in runs])
    B1 = p1.B.cpu().numpy()
    ref = np.concatenate([oracle.fc1_gelu(np.ascontiguousarray(p1.A[s:s + RUN].cpu().numpy()), B1, p1.scale_a, p1.scale_b,
                                          bits(p1.bias), out_e4m3=True, out_scale=h_scale) for s in runs])
    check_e4m3(got, ref, "C2 -> e4m3 codes")
    del p1
    p3 = synth.make_fc2(c3["M"], c3["N"], c3["K"], seed=0, device=DEV, act=H, act_scale=h_scale)
    check_full_size(engine, oracle, p3, "C3 on FC1's codes", seed=13)


def committed_dispatch_rows():
    """(op, N, K) -> sorted [(m_min, variant)] of the committed, generated dispatch table."""
    import re
    from pathlib import Path
    text = (Path(__file__).resolve().parent.parent / "siglip_b200" / "csrc" / "sl8_dispatch_table.h").read_text()
    ops = {"SL8_OP_PATCH_EMBED": 0, "SL8_OP_FC1_GELU": 1, "SL8_OP_FC2_RESIDUAL": 2}
    table = {}
    for op, n, k, m, v in re.findall(r"\{(SL8_OP_\w+), (\d+), (\d+), (\d+)LL, (\d+)\}", text):
        table.setdefault((ops[op], int(n), int(k)), []).append((int(m), int(v)))
    return {key: sorted(rows) for key, rows in table.items()}


def table_variant(table, op, M, N, K):
    rows = [v for m, v in table[(op, N, K)] if m <= M]
    return rows[-1]


def test_c5_chain_at_its_real_size(engine, oracle):
    """C5 whole: 1024 images, M = 746 496 rows, through sl8_mlp_chain_fp8.  The hidden codes (FC1 -> e4m3) and the
    output (FC2 on those very codes + residual) are checked on sampled row runs at tile edges, image edges, both ends
    and seeded random places; the launches must pick the variants the committed sweep names for this M."""
    d_model, d_ff, M = 1152, 4304, 1024 * 729
    table = committed_dispatch_rows()
    assert engine.query_config(synth.OP_FC1_GELU, M, d_ff, d_model, 1)["variant_id"] == table_variant(table, 1, M, d_ff, d_model)
    assert engine.query_config(synth.OP_FC2_RESIDUAL, M, d_model, d_ff)["variant_id"] == table_variant(table, 2, M, d_model, d_ff)
    p1 = synth.make_fc1(M, d_ff, d_model, seed=0, device=DEV)
    w2 = synth.make_fc2(729, d_model, d_ff, seed=0, device=DEV)
    g = torch.Generator(device=DEV).manual_seed(77)
    residual = torch.empty((M, d_model), dtype=torch.bfloat16, device=DEV)
    for r0 in range(0, M, 1 << 17):                                   # fp32 staging of the residual in slabs
        r1 = min(M, r0 + (1 << 17))
        residual[r0:r1] = torch.randn((r1 - r0, d_model), generator=g, device=DEV).to(torch.bfloat16)
    h_scale = 0.0125
    H = torch.empty((M, synth.pitch128(d_ff)), dtype=torch.uint8, device=DEV)[:, :d_ff]
    D = engine.mlp_chain(p1.A, p1.B, p1.bias, w2.B, w2.bias, residual, scale_a=dscalar(p1.scale_a), scale_w1=dscalar(p1.scale_b),
                         scale_w2=dscalar(w2.scale_b), hidden_scale=dscalar(h_scale), hidden=H)
    engine.device_status()
    assert bool(torch.isfinite(D.view(-1)[::9973].float()).all())
    runs = sample_runs(M, seed=21, random_runs=16)
    B1, B2 = p1.B.cpu().numpy(), w2.B.cpu().numpy()
    got_h = np.concatenate([H[s:s + RUN].cpu().numpy() for s in runs])
    ref_h = np.concatenate([oracle.fc1_gelu(np.ascontiguousarray(p1.A[s:s + RUN].cpu().numpy()), B1, p1.scale_a, p1.scale_b,
                                            bits(p1.bias), out_e4m3=True, out_scale=h_scale) for s in runs])
    check_e4m3(got_h, ref_h, "C5: hidden codes")
    got_d = np.concatenate([bits(D[s:s + RUN]) for s in runs])
    ref_d = np.concatenate([oracle.fc2_residual(np.ascontiguousarray(H[s:s + RUN].cpu().numpy()), B2, h_scale, w2.scale_b,
                                                bits(w2.bias), bits(residual[s:s + RUN])) for s in runs])
    check_bf16(got_d, ref_d, "C5: FC2 + residual on the hidden codes")


@pytest.mark.parametrize("layer", ["fc1", "fc2", "pe"])
def test_m_ladder_points_pick_the_committed_variant_and_match_the_oracle(engine, oracle, layer):
    """The M ladder of the sweep (729 * 2^j rows, the sizes the dispatch table has break points for): at every point
    the library picks the variant the committed table names, and sampled row runs match the oracle."""
    table = committed_dispatch_rows()
    op, N, K = {"fc1": (1, 4304, 1152), "fc2": (2, 1152, 4304), "pe": (0, 1152, 588)}[layer]
    make = {"fc1": lambda M: synth.make_fc1(M, N, K, seed=3, device=DEV),
            "fc2": lambda M: synth.make_fc2(M, N, K, seed=3, device=DEV),
            "pe": lambda M: synth.make_patch_embed(M, N, K, 729, seed=3, device=DEV, pixels=True)}[layer]
    for j in (0, 2, 4, 7, 8, 9):                      # 729 ... 373 248 rows (46 656 and 186 624 have tests of their own)
        M = 729 * 2 ** j
        assert engine.query_config(op, M, N, K)["variant_id"] == table_variant(table, op, M, N, K), f"{layer} M={M}"
        p = make(M)
        D = launch(engine, p, table=engine.padded_table(p.table) if p.table is not None else None)
        runs = sample_runs(M, seed=30 + j, random_runs=6) if M > 2 * 729 else [0, M - RUN]
        got = np.concatenate([bits(D[s:s + RUN]) for s in runs])
        ref = np.concatenate([oracle_rows(oracle, p, s) for s in runs])
        check_bf16(got, ref, f"{layer} M={M}: {len(runs)} runs of {RUN} rows")
        del p, D
        torch.cuda.empty_cache()
