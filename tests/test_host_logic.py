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
