"""The mixed-precision step through its other launch strategies: the update fed by
an asynchronous shared-memory ring (after the overflow-check kernel), and the whole
step as one cooperative launch with a grid-wide barrier.  Every strategy must
produce the bits of the oracle, so the parity cases of test_mixed_gpu.py are run
again under each of them.  Also: the bounded barrier wait gives up when nothing
releases it, and the device stays usable.
"""
import ctypes as C

import numpy as np
import pytest

import test_mixed_gpu as TM
import workloads as W

pytestmark = pytest.mark.gpu


@pytest.fixture(params=[0, 1, 2], ids=["two_launches", "check_then_ring", "one_cooperative_launch"])
def strategy(request, gm, dev):
    L = gm.lib
    before = L.gm_device_get_tuning(dev.h, b"mixed_ring")
    gm.check(L.gm_device_set_tuning(dev.h, b"mixed_ring", request.param), "set strategy")
    yield request.param
    gm.check(L.gm_device_set_tuning(dev.h, b"mixed_ring", before), "restore strategy")


def test_ragged_list_with_overflows_and_growth(gm, dev, oracle, strategy):
    sizes = W.ragged_sizes(48, 393_217, 1024, 65536)
    skips, scales, st = TM.run_mixed(gm, dev, oracle, sizes, 150, 25, 0.03, 25, seed=40 + strategy)
    assert skips >= 1 and len(scales) >= 2 and st.adam_t == 150 - skips


@pytest.mark.parametrize("seed", range(4))
def test_random_alignments(gm, dev, oracle, strategy, seed):
    TM.test_random_alignments_mixed(gm, dev, oracle, seed)


def test_16_byte_but_not_32_byte_aligned_fp32_streams(gm, dev, oracle, strategy):
    TM.test_fp32_streams_on_16_but_not_32_byte_boundaries(gm, dev, oracle)


@pytest.mark.parametrize("case", ["inf_first", "nan_last", "neg_inf_middle"])
def test_overflow_skips_everything(gm, dev, oracle, strategy, case):
    TM.test_overflow_anywhere_skips_everything(gm, dev, oracle, case)


def test_late_resume(gm, dev, oracle, strategy):
    TM.test_resume_at_a_late_step_with_slow_betas(gm, dev, oracle)


def test_list_smaller_than_the_grid(gm, dev, oracle, strategy):
    """Fewer tiles than resident CTAs: most CTAs have nothing to do but must still meet at the barrier."""
    skips, scales, st = TM.run_mixed(gm, dev, oracle, [5, 2049, 300], 12, 4, 0.2, 3, seed=9)
    assert st.adam_t == 12 - skips


def test_fast_division_switch_changes_no_bit(gm, dev, oracle, strategy):
    L = gm.lib
    before = L.gm_device_get_tuning(dev.h, b"mixed_fastdiv")
    try:
        for on in (0, 1):
            gm.check(L.gm_device_set_tuning(dev.h, b"mixed_fastdiv", on), "fastdiv")
            TM.run_mixed(gm, dev, oracle, [70_001, 9, 8192], 10, 100, 0.0, 5, seed=3)
    finally:
        L.gm_device_set_tuning(dev.h, b"mixed_fastdiv", before)


def test_bounded_barrier_wait_gives_up(gm, dev):
    """A wait on a word that nothing sets, with a budget of about a millisecond: the kernel
    returns, says that it gave up, and the next launches on the device work."""
    L = gm.lib
    gave_up = C.c_int(-1)
    gm.check(L.gm_selftest_barrier_timeout(dev.h, 2_000_000, C.byref(gave_up)), "selftest")
    assert gave_up.value == 1
    assert L.gm_selftest_barrier_timeout(dev.h, 0, C.byref(gave_up)) == -10
    p = dev.to_device(np.arange(8, dtype=np.float32))
    assert np.array_equal(dev.to_host(p, 8), np.arange(8, dtype=np.float32))
    dev.free(p)
    assert L.gm_device_set_tuning(dev.h, b"no_such_switch", 1) == -10
    assert L.gm_device_get_tuning(dev.h, b"no_such_switch") == -1
