"""The CUDA kernels against the committed fixtures of tests/golden/ (inputs and
expected outputs stored as bits; made by tests/golden/make_golden.py)."""
import ctypes as C
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "optimizer_steps.npz")


def bits(a):
    return np.asarray(a, dtype=np.float32).view(np.uint32)


def same_bits(a, b):
    """Bitwise equality; NaNs match NaNs whatever their payload (x86 and the GPU differ there)."""
    a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
    na, nb = np.isnan(a), np.isnan(b)
    return np.array_equal(na, nb) and np.array_equal(bits(a)[~na], bits(b)[~nb])


@pytest.fixture(scope="module")
def G():
    return np.load(GOLDEN)


def run3(gm, dev, G, nstate, call):
    w0 = G["w0"]
    n = w0.size
    dw = dev.to_device(w0)
    dg = dev.alloc(4 * n)
    ds = [dev.to_device(np.zeros(n, np.float32)) for _ in range(nstate)]
    one = lambda p: gm.uarray([p])
    for s in (1, 2, 3):
        dev.upload(dg, G[f"g{s}"])
        rc = call(one(dw), one(dg), [one(p) for p in ds], gm.iarray([4 * n]), s)
        assert rc == 0, gm.last_error()
    out = [dev.to_host(dw, n)] + [dev.to_host(p, n) for p in ds]
    for p in [dw, dg] + ds:
        dev.free(p)
    return out


def test_golden_elementwise_rules(gm, dev, G):
    L, h = gm.lib, dev.h
    cases = [
        (("adam_w", "adam_m", "adam_v"), 2, lambda w, g, s, z, t: L.execute_adam_step_cuda(h, w, g, s[0], s[1], 1, z, 1e-3, 0.9, 0.999, 1e-8, 0.0, t)),
        (("adam_wd_w", "adam_wd_m", "adam_wd_v"), 2, lambda w, g, s, z, t: L.execute_adam_step_cuda(h, w, g, s[0], s[1], 1, z, 1e-3, 0.9, 0.999, 1e-8, 0.01, t)),
        (("nadam_w", "nadam_m", "nadam_v"), 2, lambda w, g, s, z, t: L.execute_nadam_step_cuda(h, w, g, s[0], s[1], 1, z, 0.002, 0.9, 0.999, 1e-8, 0.0, t)),
        (("sgd_plain_w",), 0, lambda w, g, s, z, t: L.execute_sgd_step_cuda(h, w, g, None, 1, z, 0.01, 0.0, 0.0, 0, t)),
        (("sgd_mom_w", "sgd_mom_mom"), 1, lambda w, g, s, z, t: L.execute_sgd_step_cuda(h, w, g, s[0], 1, z, 0.01, 0.9, 0.0, 0, t)),
        (("sgd_nesterov_w", "sgd_nesterov_mom"), 1, lambda w, g, s, z, t: L.execute_sgd_step_cuda(h, w, g, s[0], 1, z, 0.01, 0.9, 1e-4, 1, t)),
        (("rmsprop_w", "rmsprop_sq"), 1, lambda w, g, s, z, t: L.execute_rmsprop_step_cuda(h, w, g, s[0], None, None, 1, z, 0.01, 0.99, 1e-8, 0.0, 0.0, False, t)),
        (("rmsprop_cm_w", "rmsprop_cm_sq", "rmsprop_cm_mom", "rmsprop_cm_gavg"), 3, lambda w, g, s, z, t: L.execute_rmsprop_step_cuda(h, w, g, s[0], s[1], s[2], 1, z, 0.01, 0.99, 1e-8, 1e-3, 0.9, True, t)),
        (("adagrad_w", "adagrad_sq"), 1, lambda w, g, s, z, t: L.execute_adagrad_step_cuda(h, w, g, s[0], 1, z, 0.01, 1e-10, 0.0)),
        (("adadelta_w", "adadelta_sq", "adadelta_upd"), 2, lambda w, g, s, z, t: L.execute_adadelta_step_cuda(h, w, g, s[0], s[1], 1, z, 0.9, 1e-6, 0.0)),
    ]
    for names, nstate, call in cases:
        got = run3(gm, dev, G, nstate, call)
        for name, a in zip(names, got):
            assert np.array_equal(bits(a), bits(G[name])), name


def test_golden_mixed_precision(gm, dev, G):
    L = gm.lib
    sizes = [257, 64]
    init = gm.LossScale(scale=65536.0, growth=2.0, backoff=0.5, max_scale=16777216.0, interval=2,
                        good_steps=0, adam_t=0, skipped=0, last_overflow=0)
    mx = L.gm_mixed_create(dev.h, C.byref(init), 0.9, 0.999, 0)
    dw = [dev.to_device(G[f"mixed_master0_{k}"]) for k in range(2)]
    dm = [dev.to_device(np.zeros(n, np.float32)) for n in sizes]
    dv = [dev.to_device(np.zeros(n, np.float32)) for n in sizes]
    dg = [dev.alloc(2 * n) for n in sizes]
    dp = [dev.to_device(np.zeros(n, np.uint16)) for n in sizes]
    lst = dev.tensor_list([dg, dw, dm, dv, dp], sizes, [2, 4, 4, 4, 2])
    try:
        for s in range(1, 7):
            for k in range(2):
                dev.upload(dg[k], G[f"mixed_g16_{s}_{k}"])
            gm.check(L.gm_mixed_step_async(dev.h, mx, lst, 1e-3, 1e-8, 0.0), "mixed")
            st = gm.LossScale()
            gm.check(L.gm_mixed_get_state(dev.h, mx, C.byref(st)), "state")
            want = G["mixed_traj"][s - 1]
            assert [st.scale, st.good_steps, st.adam_t, st.skipped, st.last_overflow] == list(want), f"step {s}"
        for k, n in enumerate(sizes):
            assert np.array_equal(bits(dev.to_host(dw[k], n)), bits(G[f"mixed_master_{k}"]))
            assert np.array_equal(bits(dev.to_host(dm[k], n)), bits(G[f"mixed_m_{k}"]))
            assert np.array_equal(bits(dev.to_host(dv[k], n)), bits(G[f"mixed_v_{k}"]))
            assert np.array_equal(dev.to_host(dp[k], n, np.uint16), G[f"mixed_p16_{k}"])
    finally:
        L.gm_tensor_list_destroy(lst)
        L.gm_mixed_destroy(mx)
        for p in dw + dm + dv + dg + dp:
            dev.free(p)


@pytest.mark.parametrize("mode", [0, 1, 3])
def test_golden_lbfgs(gm, dev, G, mode):
    L = gm.lib
    n, hs = 300, 3
    D, b = G["lbfgs_D"], G["lbfgs_b"]
    z = lambda k=n: dev.to_device(np.zeros(k, np.float32))
    dx, dg, dold, ddir, dalpha = z(), z(), z(), z(), z(hs)
    ds, dy, drho = [z() for _ in range(hs)], [z() for _ in range(hs)], [z(1) for _ in range(hs)]
    gm.check(L.gm_lbfgs_set_mode(dev.h, mode), "mode")
    try:
        hc = hi = 0
        for it in range(8):
            x = dev.to_host(dx, n)
            dev.upload(dg, (D * x - b).astype(np.float32))
            step = C.c_float()
            rc = L.execute_lbfgs_step_cuda(dev.h, gm.uarray([dx]), gm.uarray([dg]), gm.uarray([dold]), gm.uarray([ddir]),
                                           gm.uarray(ds), gm.uarray(dy), gm.uarray(drho), dalpha, 1, gm.iarray([4 * n]),
                                           hs, hc, hi, 1.0, 1e-4, 0.9, 20, 0.0, 0.0, C.byref(step))
            assert rc == 0, gm.last_error()
            hi, hc = (hi + 1) % hs, min(hc + 1, hs)
            rho = np.array([dev.to_host(p, 1)[0] for p in drho], np.float32)
            assert same_bits(rho, G[f"lbfgs_rho_mode{mode}"][it]), f"iteration {it}"
        # mode 1 ascends (reference signs) and has overflowed to NaN by iteration 8
        assert same_bits(dev.to_host(dx, n), G[f"lbfgs_x_mode{mode}"])
    finally:
        gm.check(L.gm_lbfgs_set_mode(dev.h, 3), "mode")
        for p in [dx, dg, dold, ddir, dalpha] + ds + dy + drho:
            dev.free(p)


def test_golden_dot(gm, dev, G):
    pa, pb = dev.to_device(G["dot_a"]), dev.to_device(G["dot_b"])
    out = C.c_float()
    gm.check(gm.lib.gm_dot_canonical(dev.h, pa, pb, 5000, C.byref(out)), "dot")
    assert bits(np.float32(out.value)) == bits(G["dot_value"][0])
    dev.free(pa)
    dev.free(pb)
