"""A bounded device-side wait that really runs out, in the only form that leaves the GPU healthy: a short budget, a
copy that is never issued (so the barrier it would complete is never completed), and a kernel that gives up, records
where, lets its in-flight work land, frees its tensor memory and returns.  The host then reads
SL8_ERR_DEVICE_TIMEOUT with the role, the stage, the tile and the block, and the next launch in the same process
(a handle created without the switch) is correct.  Nothing here traps, faults or spins without a limit.

The switch that drops the copy (environment variable SL8_TEST_DROP_B=1, read when a handle is created) is a test
aid of the library: the B operand of k-block 1 of every cluster's first tile is not loaded, so the MMA-issuing
thread (and the producers behind it) wait for that stage until a budget is spent.  The reference's counterpart spins for ever
(kernel_common.cuh:166-178).
"""
import os

import numpy as np
import pytest
import torch

import siglip_b200
import siglip_b200.lib as L
from siglip_b200 import synth
from tests.tolerance import check_bf16

pytestmark = pytest.mark.gpu

DEV = "cuda"
ST_PRODUCER_EMPTY_WAIT, ST_MMA_FULL_WAIT = 1, 2          # sl8_kernel.cuh: which role gave up


def dscalar(x):
    return torch.tensor([x], dtype=torch.float32, device=DEV)


@pytest.mark.parametrize("variant,cta_group", [(6, 1), (1, 2)])
def test_a_wait_that_runs_out_returns_a_status_and_leaves_the_handle_usable(oracle, variant, cta_group):
    M, N, K = 256, 256, 1024                      # one 256 x 256 tile (or four 128 x 128 ones), eight k-blocks
    p = synth.make_fc2(M, N, K, seed=5, device=DEV)
    kw = dict(scale_a=dscalar(p.scale_a), scale_b=dscalar(p.scale_b))
    os.environ["SL8_TEST_DROP_B"] = "1"
    try:
        eng = siglip_b200.Engine(0)
    finally:
        del os.environ["SL8_TEST_DROP_B"]
    try:
        assert siglip_b200.layers.describe_variant(variant)["cta_group"] == cta_group
        eng.set_variant(variant)
        eng.set_wait_budget_us(3000)
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        eng.fc2_residual(p.A, p.B, p.bias, p.residual, **kw)
        t1.record()
        with pytest.raises(L.SL8Error) as err:
            eng.device_status()
        assert err.value.code == L.SL8_ERR_DEVICE_TIMEOUT
        # Two waits hang on the stage whose copy never came: the MMA thread's (for the operands) and, once the ring
        # is full, the producers' (for that stage to be handed back).  Whichever budget is spent first reports.
        assert "MMA thread waiting for operands" in str(err.value) or "producer waiting for a free stage" in str(err.value)
        code, stage, tile, block = eng.last_status_detail
        assert code in (ST_PRODUCER_EMPTY_WAIT, ST_MMA_FULL_WAIT) and stage == 1      # k-block 1 lives in stage 1 of the ring
        assert tile < 4 and block < 4 * cta_group
        ms = t0.elapsed_time(t1)
        # budget 3 ms, + at most a third of a millisecond per parked poll of the other roles, + the 0.2 ms drain:
        # a pair whose second CTA had to sit out a budget of its own would take twice as long
        assert 3.0 <= ms < 5.5, f"kernel took {ms:.2f} ms to give up"
        eng.device_status()                                        # the status block was cleared by the read
    finally:
        eng.close()

    # the same process, a fresh handle without the switch: the GPU context is healthy and the layer is right
    with siglip_b200.Engine(0) as good:
        good.set_variant(variant)
        D = good.fc2_residual(p.A, p.B, p.bias, p.residual, **kw)
        good.device_status()
        ref = oracle.fc2_residual(p.A.cpu().numpy(), p.B.cpu().numpy(), p.scale_a, p.scale_b,
                                  p.bias.view(torch.uint16).cpu().numpy(), p.residual.view(torch.uint16).cpu().numpy())
        check_bf16(D.view(torch.uint16).cpu().numpy(), ref, "fc2 after a timed-out launch")


def test_wait_budget_arguments(engine):
    with pytest.raises(L.SL8Error):
        engine.set_wait_budget_us(0)
    engine.set_wait_budget_us(2_000_000)
    engine.set_wait_budget_ms(2000)
