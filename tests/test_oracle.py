"""CPU checks of the oracle itself (no GPU).

The reference has no golden vector for an optimizer step (its rules run inside
Apple's MPSGraph and its tests never read a result back), so the oracle is
checked three ways: against hand-computed one-element cases, against a second
restatement in numpy float32 (tests/np_rules.py), and against the committed
fixtures of tests/golden/ (a regression pin).  fp16 conversion is checked
against numpy's IEEE binary16 for every half and for rounding boundaries.
"""
import os

import numpy as np
import pytest

import np_rules as R
import workloads as W

f32 = np.float32
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "optimizer_steps.npz")


def bits(a):
    return np.asarray(a, dtype=np.float32).view(np.uint32)


def same(a, b):
    return np.array_equal(bits(a), bits(b))


# ---------------------------------------------------------------- hand-computed

def test_adam_first_step_by_hand(oracle):
    """w=1, g=0.5, m=v=0, t=1: m'=0.05, v'=0.00025, m^=0.5, v^=0.25, update=0.5/(0.5+1e-8)."""
    O = oracle
    w, g, m, v = (np.array([x], f32) for x in (1.0, 0.5, 0.0, 0.0))
    O.adam_step(w, g, m, v, 0.1, 0.9, 0.999, 1e-8, 0.0, 1)
    omb1, omb2 = f32(1) - f32(0.9), f32(1) - f32(0.999)
    m1 = f32(0.5) * omb1
    v1 = f32(0.25) * omb2
    bc1, bc2 = f32(1) - f32(0.9), f32(1) - f32(0.999)       # powf(b, 1) == b
    upd = (m1 / bc1) / (np.sqrt(v1 / bc2) + f32(1e-8))
    assert same(m, [m1]) and same(v, [v1]) and same(w, [f32(1.0) - upd * f32(0.1)])
    assert abs(float(w[0]) - 0.9) < 1e-6


def test_sgd_momentum_and_nesterov_by_hand(oracle):
    O = oracle
    w, g, mom = np.array([2.0], f32), np.array([1.0], f32), np.array([0.5], f32)
    O.sgd_step(w, g, mom, 0.1, 0.9, 0.0, 0)                 # m' = 0.45+1 = 1.45 ; w' = 2 - 0.145
    assert same(mom, [f32(0.5) * f32(0.9) + f32(1.0)])
    assert same(w, [f32(2.0) - f32(0.1) * (f32(0.5) * f32(0.9) + f32(1.0))])
    w, mom = np.array([2.0], f32), np.array([0.5], f32)
    O.sgd_step(w, g, mom, 0.1, 0.9, 0.0, 1)                 # step = lr*(mu*m' + g)
    m2 = f32(0.5) * f32(0.9) + f32(1.0)
    assert same(w, [f32(2.0) - f32(0.1) * (f32(0.9) * m2 + f32(1.0))])
    w = np.array([2.0], f32)
    O.sgd_step(w, g, None, 0.1, 0.9, 0.5, 0)                # no buffer: plain rule with decay
    assert same(w, [f32(2.0) - f32(0.1) * (f32(1.0) + f32(2.0) * f32(0.5))])


def test_adagrad_adadelta_rmsprop_by_hand(oracle):
    O = oracle
    w, g, sq = np.array([1.0], f32), np.array([2.0], f32), np.array([5.0], f32)
    O.adagrad_step(w, g, sq, 0.3, 1e-10, 0.0)               # G'=9, sqrt=3, w' = 1 - (0.3/3)*2
    assert same(sq, [9.0]) and same(w, [f32(1.0) - (f32(0.3) / (f32(3.0) + f32(1e-10))) * f32(2.0)])
    w, sq, up = np.array([1.0], f32), np.array([0.0], f32), np.array([0.0], f32)
    O.adadelta_step(w, g, sq, up, 0.9, 1e-6, 0.0)
    e = f32(4.0) * (f32(1) - f32(0.9))
    neg = -((np.sqrt(f32(0.0) + f32(1e-6)) / np.sqrt(e + f32(1e-6))) * f32(2.0))
    assert same(sq, [e]) and same(w, [f32(1.0) + neg]) and same(up, [(neg * neg) * (f32(1) - f32(0.9))])
    w, sq = np.array([1.0], f32), np.array([0.0], f32)
    O.rmsprop_step(w, g, sq, None, None, 0.01, 0.99, 1e-8, 0.0, 0.0, False)
    s2 = f32(4.0) * (f32(1) - f32(0.99))
    assert same(sq, [s2]) and same(w, [f32(1.0) - (f32(2.0) / np.sqrt(s2 + f32(1e-8))) * f32(0.01)])


def test_rmsprop_reference_writeback_quirk(oracle):
    """With persist_aux=0 the momentum / gradient-average buffers stay untouched,
    as in cgo_bridge/bridge_optimizer.m:915-937."""
    O = oracle
    w, g, sq = np.array([1.0], f32), np.array([2.0], f32), np.array([0.0], f32)
    mom, ga = np.array([0.25], f32), np.array([0.125], f32)
    O.rmsprop_step(w, g, sq, mom, ga, 0.01, 0.99, 1e-8, 0.0, 0.9, True, False)
    assert same(mom, [0.25]) and same(ga, [0.125])
    O.rmsprop_step(w, g, sq, mom, ga, 0.01, 0.99, 1e-8, 0.0, 0.9, True, True)
    assert not same(mom, [0.25]) and not same(ga, [0.125])


def test_host_scalars(oracle):
    O = oracle
    bc1, bc2, omb1, omb2 = O.adam_scalars(0.9, 0.999, 1)
    assert same([bc1, bc2, omb1, omb2], [f32(1) - f32(0.9), f32(1) - f32(0.999), f32(1) - f32(0.9), f32(1) - f32(0.999)])
    bc1, bc2, _, _ = O.adam_scalars(0.9, 0.999, 100000)
    assert bc1 == 1.0 and bc2 == 1.0                        # both powers underflow below half an ulp of 1
    mu = O.nadam_mu_next(0.9, 1)
    assert abs(float(mu) - 0.9 * (1 - 0.5 * 0.96 ** (2 * 0.004))) < 1e-6


# ---------------------------------------------------------------- numpy cross-check

@pytest.mark.filterwarnings("ignore::RuntimeWarning")
@pytest.mark.parametrize("special", [False, True], ids=["dense", "zeros_and_denormals"])
@pytest.mark.parametrize("wd", [0.0, 0.01])
def test_rules_match_numpy_restatement(oracle, wd, special):
    """special: a third of the gradient entries are +0 or -0 (their state stays zero: the
    untouched-parameter case the kernels shortcut), and weights and gradients carry
    denormals, 1e-30 and 1e30, so the two restatements are compared where rounding and
    the sign of zero matter most."""
    O = oracle
    n = 10_007
    w0 = O.fill_uniform(n, -0.5, 0.5, 3, 1)
    if special:
        w0[::11] = 0.0
        w0[5::97] = np.float32(1e-42)
        w0[7::101] = np.float32(-1e30)
    z = lambda: np.zeros(n, f32)
    state = {
        "adam": [w0.copy(), z(), z()], "nadam": [w0.copy(), z(), z()], "sgd": [w0.copy(), z()],
        "nest": [w0.copy(), z()], "rms": [w0.copy(), z()], "rmscm": [w0.copy(), z(), z(), z()],
        "adagrad": [w0.copy(), z()], "adadelta": [w0.copy(), z(), z()],
    }
    ref = {k: [a.copy() for a in v] for k, v in state.items()}
    for t in range(1, 8):
        g = O.scale_subset(O.fill_normal(n, 0, 0.01, 3, 10 + t), 10, 100.0, 3, 40 + t)
        if special:
            g[::3] = 0.0
            g[::6] = -0.0
            g[1::91] = np.float32(1e-42)
            g[2::89] = np.float32(1e-30)
            g[4::83] = np.float32(1e18)
        bc1, bc2, _, _ = O.adam_scalars(0.9, 0.999, t)
        s = state
        O.adam_step(s["adam"][0], g, s["adam"][1], s["adam"][2], 1e-3, 0.9, 0.999, 1e-8, wd, t)
        ref["adam"] = list(R.adam(*ref["adam"][:1], g, *ref["adam"][1:], 1e-3, 0.9, 0.999, 1e-8, wd, bc1, bc2))
        O.nadam_step(s["nadam"][0], g, s["nadam"][1], s["nadam"][2], 2e-3, 0.9, 0.999, 1e-8, wd, t)
        ref["nadam"] = list(R.nadam(ref["nadam"][0], g, ref["nadam"][1], ref["nadam"][2], 2e-3, 0.9, 0.999, 1e-8, wd,
                                    bc1, bc2, O.nadam_mu_next(0.9, t)))
        O.sgd_step(s["sgd"][0], g, s["sgd"][1], 0.01, 0.9, wd, 0)
        ref["sgd"] = list(R.sgd(ref["sgd"][0], g, ref["sgd"][1], 0.01, 0.9, wd, False))
        O.sgd_step(s["nest"][0], g, s["nest"][1], 0.01, 0.9, wd, 1)
        ref["nest"] = list(R.sgd(ref["nest"][0], g, ref["nest"][1], 0.01, 0.9, wd, True))
        O.rmsprop_step(s["rms"][0], g, s["rms"][1], None, None, 0.01, 0.99, 1e-8, wd, 0.0, False)
        r = R.rmsprop(ref["rms"][0], g, ref["rms"][1], None, None, 0.01, 0.99, 1e-8, wd, 0.0, False)
        ref["rms"] = [r[0], r[1]]
        O.rmsprop_step(s["rmscm"][0], g, s["rmscm"][1], s["rmscm"][2], s["rmscm"][3], 0.01, 0.99, 1e-8, wd, 0.9, True, True)
        ref["rmscm"] = list(R.rmsprop(ref["rmscm"][0], g, ref["rmscm"][1], ref["rmscm"][2], ref["rmscm"][3],
                                      0.01, 0.99, 1e-8, wd, 0.9, True))
        O.adagrad_step(s["adagrad"][0], g, s["adagrad"][1], 0.01, 1e-10, wd)
        ref["adagrad"] = list(R.adagrad(ref["adagrad"][0], g, ref["adagrad"][1], 0.01, 1e-10, wd))
        O.adadelta_step(s["adadelta"][0], g, s["adadelta"][1], s["adadelta"][2], 0.9, 1e-6, wd)
        ref["adadelta"] = list(R.adadelta(ref["adadelta"][0], g, ref["adadelta"][1], ref["adadelta"][2], 0.9, 1e-6, wd))
    for k in state:
        for a, b in zip(state[k], ref[k]):
            assert same(a, b), f"{k}: the C oracle and the numpy restatement disagree"


# ---------------------------------------------------------------- fp16

def test_f16_to_f32_all_halves(oracle):
    h = np.arange(65536, dtype=np.uint16)
    got = oracle.f16_to_f32(h)
    want = h.view(np.float16).astype(np.float32)
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(bits(got)[~nan], bits(want)[~nan])


def test_f32_to_f16_rounding(oracle):
    O = oracle
    h = np.arange(0x7c00, dtype=np.uint16)                   # all non-negative finite halves
    f = O.f16_to_f32(h)
    mids = ((f[:-1].astype(np.float64) + f[1:].astype(np.float64)) / 2).astype(np.float32)   # exact ties
    around = np.concatenate([f, mids, np.nextafter(mids, f32(np.inf)), np.nextafter(mids, f32(-np.inf)),
                             np.array([65504, 65519.996, 65520, 65536, 1e30, 2.0 ** -25, 2.0 ** -24,
                                       np.nextafter(f32(2.0 ** -25), f32(1)), 0.0], f32)])
    x = np.concatenate([around, -around, O.fill_normal(200_000, 0, 1, 9, 9) * f32(300.0)])
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(O.f32_to_f16(x), want)
    special = O.f32_to_f16(np.array([np.inf, -np.inf, np.nan], f32))
    assert special[0] == 0x7c00 and special[1] == 0xfc00 and (special[2] & 0x7c00) == 0x7c00 and (special[2] & 0x3ff)


# ---------------------------------------------------------------- loss scale

def test_loss_scale_state_machine(oracle):
    """docs/tutorials/mixed-precision.md:617-629 and training/model_trainer.go:258-270."""
    O = oracle
    st = O.new_loss_scale()
    assert (st.scale, st.growth, st.backoff, st.interval) == (65536.0, 2.0, 0.5, 2000)
    st = O.new_loss_scale(interval=3, max_scale=262144.0)
    n = 8
    master, m, v = ([np.zeros(n, f32)] for _ in range(3))
    p16 = [np.zeros(n, np.uint16)]
    clean = [O.f32_to_f16(np.full(n, 0.5, f32))]
    bad = [clean[0].copy()]
    bad[0][n - 1] = 0x7e00
    seq = [clean, clean, clean, clean, bad, clean, clean, clean, clean, clean, clean]
    scales, ts = [], []
    for g in seq:
        O.mixed_adam_step(g, master, m, v, p16, 1e-3, 0.9, 0.999, 1e-8, 0.0, st)
        scales.append(st.scale)
        ts.append(st.adam_t)
    assert scales == [65536, 65536, 131072, 131072, 65536, 65536, 65536, 131072, 131072, 131072, 262144]
    assert ts == [1, 2, 3, 4, 4, 5, 6, 7, 8, 9, 10]          # the counter does not advance on the skipped step
    assert st.skipped == 1
    for _ in range(6):
        O.mixed_adam_step(clean, master, m, v, p16, 1e-3, 0.9, 0.999, 1e-8, 0.0, st)
    assert st.scale == 262144.0                                # clamped at max_scale


def test_mixed_step_equals_fp32_adam_on_unscaled_grads(oracle):
    O = oracle
    n = 1000
    w0 = O.fill_uniform(n, -1, 1, 4, 1)
    g16 = O.f32_to_f16(O.fill_normal(n, 0, 1e-3, 4, 2) * f32(65536.0))
    master, m, v, p16 = [w0.copy()], [np.zeros(n, f32)], [np.zeros(n, f32)], [np.zeros(n, np.uint16)]
    st = O.new_loss_scale()
    assert O.mixed_adam_step([g16], master, m, v, p16, 1e-3, 0.9, 0.999, 1e-8, 0.0, st) == 0
    g = (O.f16_to_f32(g16) * (f32(1.0) / f32(65536.0))).astype(f32)
    w, m2, v2 = w0.copy(), np.zeros(n, f32), np.zeros(n, f32)
    O.adam_step(w, g, m2, v2, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1)
    assert same(master[0], w) and same(m[0], m2) and same(v[0], v2)
    assert np.array_equal(p16[0], O.f32_to_f16(w))


# ---------------------------------------------------------------- reductions and L-BFGS

@pytest.mark.parametrize("n", [1, 3, 255, 4096, 4097, 70_001])
def test_canonical_dot_matches_numpy_restatement(oracle, n):
    a = oracle.fill_normal(n, 0, 1, 5, n)
    b = oracle.fill_normal(n, 0, 1, 6, n)
    assert bits(oracle.dot_canonical(a, b)) == bits(R.dot_canonical(a, b))
    exact = float(np.dot(a.astype(np.float64), b.astype(np.float64)))
    assert abs(float(oracle.dot_canonical(a, b)) - exact) <= 1e-5 * max(1.0, float(np.abs(a * b).sum()))


def lbfgs_run(O, n, hs, iters, mode, order=0, lo=-0.2, hi=0.2, seed=7):
    D = O.fill_loguniform(n, lo, hi, seed, 1)
    b = O.fill_normal(n, 0, 1, seed, 2)
    x, old, d = (np.zeros(n, f32) for _ in range(3))
    s = [[np.zeros(n, f32)] for _ in range(hs)]
    y = [[np.zeros(n, f32)] for _ in range(hs)]
    rho, alpha = np.zeros(hs, f32), np.zeros(hs, f32)
    hc = hi_ = 0
    hist = []
    for _ in range(iters):
        g = (D * x - b).astype(f32)
        rc, step = O.lbfgs_step([x], [g], [old], [d], s, y, rho, alpha, hs, hc, hi_, 1.0, mode, order)
        assert rc == 0 and step == 1.0
        hi_, hc = (hi_ + 1) % hs, min(hc + 1, hs)
        hist.append((x.copy(), rho.copy(), g))
    return D, b, hist


def test_lbfgs_reference_order_rejects_every_pair(oracle):
    """Statement order of bridge_optimizer.m:1232-1312: old_g is overwritten before
    y is formed, so y == 0, rho == 0, and each step is x += g (the double negation
    of :1026-1038 and :1204-1213 makes the step ascend)."""
    D, b, hist = lbfgs_run(oracle, 500, 4, 5, mode=0)
    x_prev = np.zeros(500, f32)
    for x, rho, g in hist:
        assert (rho == 0).all()
        assert same(x, x_prev + f32(1.0) * g)
        x_prev = x


def test_lbfgs_working_mode_converges(oracle):
    D, b, hist = lbfgs_run(oracle, 2000, 10, 25, mode=3)
    gmax = [float(np.abs(g).max()) for _, _, g in hist]
    assert min(gmax) < 1e-5
    assert (hist[12][1] != 0).all()                            # every stored pair accepted
    first = hist[0][0]
    assert same(first, b)                                      # x1 = x0 - g0 = b when x0 = 0


def test_lbfgs_orders_agree_within_rounding(oracle):
    _, _, a = lbfgs_run(oracle, 3000, 5, 8, mode=3, order=0)
    _, _, s = lbfgs_run(oracle, 3000, 5, 8, mode=3, order=1)
    for (xa, _, _), (xs, _, _) in zip(a, s):
        assert np.allclose(xa, xs, rtol=1e-3, atol=1e-4)


def test_sequential_order_carries_one_accumulator_across_tensors_for_sy(oracle):
    """bridge_optimizer.m:1272-1297 adds every s*y product of every tensor into one
    fp32 accumulator, unlike the loop dots (:1073-1109) that sum per tensor first."""
    O = oracle
    sizes = [301, 77, 1025]
    rng = np.random.default_rng(4)
    mk = lambda: [rng.standard_normal(n).astype(f32) for n in sizes]
    z = lambda: [np.zeros(n, f32) for n in sizes]
    x, old, d = z(), mk(), z()
    g = mk()
    s, y = [mk(), mk()], [z(), z()]
    rho, alpha = np.zeros(2, f32), np.zeros(2, f32)
    s_prev = [a.copy() for a in s[0]]
    old_before = [a.copy() for a in old]
    rc, _ = O.lbfgs_step(x, g, old, d, s, y, rho, alpha, 2, 1, 1, 1.0, 1, 1)
    assert rc == 0
    acc = f32(0.0)
    for t in range(len(sizes)):
        yt = (g[t] - old_before[t]).astype(f32)
        for k in range(sizes[t]):
            acc = f32(acc + f32(s_prev[t][k] * yt[k]))
    assert bits(rho[0]) == bits(f32(1.0) / acc)


def test_threads_change_no_bit(oracle):
    """The pthread split of the independent loops must give the results of one thread."""
    O = oracle
    n = 300_007
    def run():
        a = O.fill_normal(n, 0, 1, 9, 1)
        u = O.fill_uniform(n, -1, 1, 9, 2)
        d = O.fill_loguniform(n, -1, 1, 9, 3)
        h = O.f32_to_f16(a)
        back = O.f16_to_f32(h)
        sc = O.scale_to_f16(a, 3.0)
        dot = O.dot_canonical(a, u)
        st = O.new_loss_scale()
        w, m, v = u.copy(), np.zeros(n, f32), np.zeros(n, f32)
        p = O.f32_to_f16(w)
        O.mixed_adam_step([h], [w], [m], [v], [p], 1e-3, 0.9, 0.999, 1e-8, 0.01, st)
        _, _, hist = lbfgs_run(O, 200_000, 3, 4, mode=3)
        ss = O.sumsq_f16_layout([h], [3], 8192, 0.5)
        return [a, u, d, h, back, sc, np.array([dot, ss]), w, m, v, p, hist[-1][0]]
    one = run()
    O.set_threads(5)
    try:
        many = run()
    finally:
        O.set_threads(1)
    for x, y in zip(one, many):
        assert np.array_equal(x.view(np.uint8), y.view(np.uint8))
    assert np.array_equal(one[5], O.f32_to_f16((one[0] * f32(3.0)).astype(f32)))


@pytest.mark.parametrize("sizes,heads", [([5], [0]), ([70_001, 9, 8192 * 2 + 3], [3, 7, 0]), ([4099, 33], [-1, 1]),
                                         ([2], [7])])
def test_layout_sumsq_matches_numpy_restatement(oracle, sizes, heads):
    O = oracle
    g16 = [O.f32_to_f16(O.fill_normal(n, 0, 30.0, 12, k)) for k, n in enumerate(sizes)]
    inv = 1.0 / 64.0
    got = O.sumsq_f16_layout(g16, heads, 8192, inv)
    assert bits(got) == bits(R.sumsq_f16_layout(g16, heads, 8192, inv))
    exact = sum(O.sumsq_f16(g, inv) for g in g16)
    assert abs(float(got) - exact) <= 1e-5 * exact
    # a smaller chunk is another (equally valid) order: same value within rounding
    assert abs(float(O.sumsq_f16_layout(g16, heads, 2048, inv)) - exact) <= 1e-5 * exact


def test_canonical_sumsq_is_the_list_dot_of_g_with_itself(oracle):
    O = oracle
    g = [O.fill_normal(n, 0, 1, 13, k) for k, n in enumerate([4097, 3, 70_001])]
    got = O.sumsq_canonical(g)
    parts = np.concatenate([np.array([R.dot_canonical(a[c * 4096:(c + 1) * 4096], a[c * 4096:(c + 1) * 4096])
                                      for c in range((a.size + 4095) // 4096)], f32) for a in g])
    assert bits(got) == bits(R._reduce_lanes(R._reduce_partials_to_lanes(parts)))


def test_clip_coefficient(oracle):
    O = oracle
    assert O.clip_coef(4.0, 1.0) == f32(1.0) / f32(f32(2.0) + f32(1e-6))
    assert O.clip_coef(0.25, 1.0) == 1.0                       # norm below the limit: untouched
    assert O.clip_coef(0.0, 1.0) == 1.0
    assert O.clip_coef(np.inf, 1.0) == 0.0
    assert O.clip_coef(np.nan, 1.0) == 1.0
    for ss, mx in ((3.7, 0.5), (1e-12, 1e-7), (1e30, 2.0)):
        assert bits(O.clip_coef(ss, mx)) == bits(R.clip_coef(ss, mx))


def test_clipped_mixed_step_is_the_plain_step_on_clipped_gradients(oracle):
    O = oracle
    sizes, heads = [1000, 4099], [1, 5]
    rng = np.random.default_rng(8)
    g16 = [O.f32_to_f16(rng.standard_normal(n).astype(f32) * f32(65536 * 1e-2)) for n in sizes]
    mk = lambda: ([O.fill_uniform(n, -1, 1, 3, k) for k, n in enumerate(sizes)], [np.zeros(n, f32) for n in sizes],
                  [np.zeros(n, f32) for n in sizes], [np.zeros(n, np.uint16) for n in sizes])
    w, m, v, p = mk()
    st = O.new_loss_scale()
    skipped, ss, coef = O.mixed_adam_step_clipped(g16, w, m, v, p, 1e-3, 0.9, 0.999, 1e-8, 0.0, 0.25, heads, 8192, st)
    assert skipped == 0 and 0 < coef < 1 and bits(coef) == bits(O.clip_coef(ss, 0.25))
    assert bits(ss) == bits(O.sumsq_f16_layout(g16, heads, 8192, 1.0 / 65536.0))
    # the same update by hand: unscale, clip, fp32 Adam
    w2, m2, v2, _ = mk()
    for t in range(2):
        g = (O.f16_to_f32(g16[t]) * f32(1.0 / 65536.0)).astype(f32)
        g = (g * coef).astype(f32)
        O.adam_step(w2[t], g, m2[t], v2[t], 1e-3, 0.9, 0.999, 1e-8, 0.0, 1)
        assert same(w[t], w2[t]) and same(m[t], m2[t]) and same(v[t], v2[t])
        assert np.array_equal(p[t], O.f32_to_f16(w[t]))
    # an overflow step: not finite sum, skipped
    g16[1][7] = 0x7c00
    skipped, ss, coef = O.mixed_adam_step_clipped(g16, w, m, v, p, 1e-3, 0.9, 0.999, 1e-8, 0.0, 0.25, heads, 8192, st)
    assert skipped == 1 and not np.isfinite(ss) and st.scale == 32768.0


# ---------------------------------------------------------------- generators, fixtures

def test_generators_are_deterministic_and_shaped(oracle):
    O = oracle
    a, b = O.fill_normal(100_000, 0, 0.01, 1, 2), O.fill_normal(100_000, 0, 0.01, 1, 2)
    assert same(a, b) and not same(a, O.fill_normal(100_000, 0, 0.01, 1, 3))
    assert abs(float(a.std()) - 0.01) < 2e-4 and abs(float(a.mean())) < 2e-4
    u = O.fill_uniform(100_000, -2, 3, 1, 4)
    assert u.min() >= -2 and u.max() <= 3 and abs(float(u.mean()) - 0.5) < 0.02
    d = O.fill_loguniform(100_000, -2, 2, 1, 5)
    assert d.min() >= 1e-2 * 0.999 and d.max() <= 1e2 * 1.001
    h = O.scale_subset(np.ones(100_000, f32), 10, 100.0, 1, 6)
    assert 700 < int((h == 100).sum()) < 1300                  # about 1 %
    sizes = W.ragged_sizes(48, 25_165_824, 4096, 4_194_304)
    assert sum(sizes) == 25_165_824 and all(s % 8 for s in sizes) and len(sizes) == 48


def test_oracle_reproduces_golden_fixtures(oracle):
    O = oracle
    G = np.load(GOLDEN)
    w0 = G["w0"]
    n = w0.size
    z = lambda: np.zeros(n, f32)
    w, m, v = w0.copy(), z(), z()
    for s in (1, 2, 3):
        O.adam_step(w, G[f"g{s}"], m, v, 1e-3, 0.9, 0.999, 1e-8, 0.0, s)
    assert same(w, G["adam_w"]) and same(m, G["adam_m"]) and same(v, G["adam_v"])
    w, sq, up = w0.copy(), z(), z()
    for s in (1, 2, 3):
        O.adadelta_step(w, G[f"g{s}"], sq, up, 0.9, 1e-6, 0.0)
    assert same(w, G["adadelta_w"]) and same(up, G["adadelta_upd"])
    assert bits(O.dot_canonical(G["dot_a"], G["dot_b"])) == bits(G["dot_value"][0])
    assert same(np.array([O.adam_scalars(0.9, 0.999, t) for t in range(1, 21)], f32), G["adam_scalars"])
    # the numpy restatement reproduces the same fixtures
    w, m, v = w0.copy(), z(), z()
    for s in (1, 2, 3):
        bc1, bc2 = G["adam_scalars"][s - 1][:2]
        w, m, v = R.adam(w, G[f"g{s}"], m, v, 1e-3, 0.9, 0.999, 1e-8, 0.0, bc1, bc2)
    assert same(w, G["adam_w"])
