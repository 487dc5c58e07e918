"""Host-side logic that needs no GPU: synthetic operands, quantisation, sharding (incl. a
world_size-2 gloo run of the shard arithmetic the bench uses)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from siglip_b200 import synth
from siglip_b200.shard import image_range, row_range


def test_quantize_matches_oracle(oracle):
    g = torch.Generator().manual_seed(0)
    x = torch.randn((64, 588), generator=g)
    q, s = synth.quantize_e4m3(x)
    assert q.stride(0) == 640 and q.shape == (64, 588)      # rows start on 128-byte lines
    q16, _ = synth.quantize_e4m3(x, pitch=synth.pitch16(588))
    assert q16.stride(0) == 592 and torch.equal(q16, q)
    assert abs(s - float(x.abs().max()) / 448.0) < 1e-12
    want = np.array([[oracle.lib.sl8o_f32_to_e4m3(float(v)) for v in row] for row in (x / s).numpy()[:8]], dtype=np.uint8)
    assert np.array_equal(q.numpy()[:8], want)
    assert int(q.max()) >= 0x7E or int((q & 0x7F).max()) == 0x7E      # amax maps to +-448


def test_config_shapes():
    assert synth.CONFIGS["C1"]["M"] == 6272 and synth.CONFIGS["C2"]["M"] == 46656
    assert synth.CONFIGS["C4"]["M"] == 186624 and synth.CONFIGS["C4"]["K"] == 588
    p = synth.make_config("C4", images=2)
    assert p.A.shape == (1458, 588) and p.A.stride(0) == 640 and p.table.shape == (729, 1152)
    assert p.flops() == 2.0 * 1458 * 1152 * 588
    p = synth.make_config("C3", images=1)
    assert p.residual.shape == (729, 1152) and p.bias.dtype == torch.bfloat16
    q = synth.make_config("C3", images=1)
    assert torch.equal(p.A, q.A) and torch.equal(p.residual, q.residual)      # seeded


@pytest.mark.parametrize("total,world", [(1024, 1), (1024, 2), (1024, 8), (10, 4), (3, 8)])
def test_image_ranges_partition(total, world):
    covered = []
    for r in range(world):
        first, n = image_range(total, world, r)
        covered.extend(range(first, first + n))
    assert covered == list(range(total))
    sizes = [image_range(total, world, r)[1] for r in range(world)]
    assert max(sizes) - min(sizes) <= 1
    assert row_range(total, 729, world, 0)[0] == 0 and row_range(total, 729, world, 0)[2] == 0


def _worker(rank, world, port, total_images):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    first, n = image_range(total_images, world, rank)
    # every rank "processes" its images; the only communication is the bench's reduction of counts and times
    done = torch.tensor([float(n), float(first)])
    t = torch.tensor([0.5 + rank])
    dist.all_reduce(done[:1], op=dist.ReduceOp.SUM)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    assert int(done[0]) == total_images and float(t) == 0.5 + world - 1
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharding_gloo():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, 129), nprocs=2, join=True)


# ---- Engine argument validation: refused on the host, before any launch ---------------------------------------------
class _FakeCuda:
    """Stands in for a CUDA tensor where only its placement matters (no GPU is needed to test the refusal)."""

    def __init__(self, index):
        self.is_cuda = True
        self.device = torch.device("cuda", index)


def _bare_engine(device=0):
    from siglip_b200.layers import Engine
    eng = Engine.__new__(Engine)          # no handle: the checks under test run before the library is called
    eng.device = device
    eng._h = None
    return eng


def test_out_tensor_is_validated_before_launch():
    eng = _bare_engine()
    M, N = 8, 32
    with pytest.raises(TypeError):        # a one-byte buffer where the layer writes bf16
        eng._check_out(torch.empty((M, N), dtype=torch.uint8), M, N, (torch.bfloat16,))
    with pytest.raises(ValueError):       # wrong shape
        eng._check_out(torch.empty((M, N + 16), dtype=torch.bfloat16), M, N, (torch.bfloat16,))
    with pytest.raises(ValueError):       # N not contiguous
        eng._check_out(torch.empty((N, M), dtype=torch.bfloat16).t(), M, N, (torch.bfloat16,))
    with pytest.raises(ValueError):       # host memory
        eng._check_out(torch.empty((M, N), dtype=torch.bfloat16), M, N, (torch.bfloat16,))


def test_output_type_comes_from_out():
    from siglip_b200 import lib as l
    eng = _bare_engine()
    eng._on_device = lambda name, t: None                 # placement is covered by its own test
    M, N = 8, 32
    out8 = torch.empty((M, N), dtype=torch.uint8)
    assert eng._resolve_out(out8, None, M, N, "cpu")[1] == l.SL8_OUT_E4M3            # no keyword needed
    assert eng._resolve_out(out8, torch.float8_e4m3fn, M, N, "cpu")[1] == l.SL8_OUT_E4M3
    out16 = torch.empty((M, N), dtype=torch.bfloat16)
    assert eng._resolve_out(out16, None, M, N, "cpu")[1] == l.SL8_OUT_BF16
    with pytest.raises(TypeError):        # the bf16 kernel must never be pointed at a one-byte buffer
        eng._resolve_out(out8, torch.bfloat16, M, N, "cpu")
    with pytest.raises(TypeError):
        eng._resolve_out(out16, torch.uint8, M, N, "cpu")
    with pytest.raises(TypeError):
        eng._resolve_out(None, torch.float16, M, N, "cpu")
    fresh, code = eng._resolve_out(None, None, M, N, "cpu")
    assert fresh.dtype == torch.bfloat16 and code == l.SL8_OUT_BF16


def test_operands_must_live_on_the_engines_gpu():
    eng = _bare_engine(device=0)
    eng._on_device("A", _FakeCuda(0))
    eng._on_device("bias", None)
    with pytest.raises(ValueError, match="cuda:1"):
        eng._on_device("residual", _FakeCuda(1))
    with pytest.raises(ValueError):
        eng._on_device("table", torch.empty(4))
    with pytest.raises(ValueError):       # fc1_gelu refuses host operands before touching the library
        eng.fc1_gelu(torch.empty((4, 16), dtype=torch.uint8), torch.empty((16, 16), dtype=torch.uint8), None)
