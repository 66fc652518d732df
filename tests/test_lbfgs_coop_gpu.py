"""The L-BFGS step as one cooperative launch ("lbfgs_coop": 1 keeps the direction vector on
chip, 2 leaves it in L2 and only replaces the kernel boundaries between passes by grid
barriers): the parity cases of test_lbfgs_gpu.py run again through both.  It must give
the bits of the oracle, like the multi-launch step, in every mode, for ragged and
unaligned tensors, and at the 10^7-variable size it was built for; a problem too large
for the on-chip storage silently takes the multi-launch step.
"""
import numpy as np
import pytest

import test_lbfgs_gpu as TL

pytestmark = pytest.mark.gpu


@pytest.fixture(params=[1, 2], ids=["direction_on_chip", "direction_in_l2"])
def coop(request, gm, dev):
    L = gm.lib
    before = L.gm_device_get_tuning(dev.h, b"lbfgs_coop")
    gm.check(L.gm_device_set_tuning(dev.h, b"lbfgs_coop", request.param), "single-launch step on")
    launches = L.gm_device_launch_count(dev.h)
    yield lambda: L.gm_device_launch_count(dev.h) - launches
    gm.check(L.gm_device_set_tuning(dev.h, b"lbfgs_coop", before), "restore")


@pytest.mark.parametrize("mode", [0, 1, 3])
def test_well_conditioned_50_iterations(gm, dev, oracle, coop, mode):
    TL.test_lbfgs_well_conditioned_50_iterations(gm, dev, oracle, mode)
    assert coop() == 50, "one launch per step"


@pytest.mark.parametrize("mode", [0, 3])
def test_ill_conditioned_as_configured(gm, dev, oracle, coop, mode):
    TL.test_lbfgs_ill_conditioned_as_configured(gm, dev, oracle, mode)


def test_multi_tensor_short_history(gm, dev, oracle, coop):
    TL.test_lbfgs_multi_tensor_short_history(gm, dev, oracle)


@pytest.mark.parametrize("shifts", [[1], [0, 0, 0, 2, 0, 1, 0]], ids=["all_off_by_one", "columns_disagree"])
def test_unaligned_buffers(gm, dev, oracle, coop, shifts):
    TL.test_lbfgs_unaligned_buffers(gm, dev, oracle, shifts)


def test_single_slot_history(gm, dev, oracle, coop):
    TL.test_lbfgs_single_slot_history(gm, dev, oracle)


def test_10m_variables_history_10(gm, dev, oracle, coop):
    """n = 10,000,000: 2,442 chunks, 16 or 17 per SM -- shared memory and the register chunks
    are both full.  14 iterations (history full and wrapping), everything compared on the last."""
    oracle.set_threads(oracle.all_cores())
    try:
        gm.check(gm.lib.gm_lbfgs_set_mode(dev.h, 3), "mode")
        P = TL.LbfgsProblem(gm, dev, oracle, [10_000_000], 10, -0.3, 0.3, seed=77)
        try:
            with np.errstate(all="ignore"):
                for it in range(14):
                    P.step(3)
                    P.compare(it, full=(it == 13))
        finally:
            P.free()
        assert coop() == 14
    finally:
        oracle.set_threads(1)


def test_too_large_for_the_chip_takes_the_multi_launch_step(gm, dev, oracle, coop, request):
    if "direction_in_l2" in request.node.name:
        pytest.skip("the L2 form has no size limit")
    n = 17 * gm.lib.gm_device_sm_count(dev.h) * 4096 + 4096
    oracle.set_threads(oracle.all_cores())
    try:
        P = TL.LbfgsProblem(gm, dev, oracle, [n], 2, -0.2, 0.2, seed=5)
        try:
            for it in range(3):
                P.step(3)
                P.compare(it, full=False)
        finally:
            P.free()
        assert coop() > 3
    finally:
        oracle.set_threads(1)


# ---- launch-strategy switches of the multi-launch step: every setting gives the oracle's bits ----
@pytest.fixture(params=[("lbfgs_defer", 0), ("lbfgs_prewait", 0), ("lbfgs_prewait", 2)],
                ids=["own_final_sum", "no_early_loads", "early_loads_and_l2_prefetch"])
def multi_launch_switch(request, gm, dev):
    L = gm.lib
    name, value = request.param
    before = L.gm_device_get_tuning(dev.h, name.encode())
    assert before >= 0, f"unknown switch {name}"
    gm.check(L.gm_device_set_tuning(dev.h, name.encode(), value), "switch")
    yield
    gm.check(L.gm_device_set_tuning(dev.h, name.encode(), before), "restore")


@pytest.mark.parametrize("mode", [0, 3])
def test_switches_well_conditioned(gm, dev, oracle, multi_launch_switch, mode):
    TL.test_lbfgs_well_conditioned_50_iterations(gm, dev, oracle, mode)


def test_switches_ill_conditioned_pairs_rejected(gm, dev, oracle, multi_launch_switch):
    TL.test_lbfgs_ill_conditioned_as_configured(gm, dev, oracle, 0)


def test_switches_ragged_and_unaligned(gm, dev, oracle, multi_launch_switch):
    TL.test_lbfgs_multi_tensor_short_history(gm, dev, oracle)
    TL.test_lbfgs_unaligned_buffers(gm, dev, oracle, [0, 0, 0, 2, 0, 1, 0])
