"""Parity at the sizes AND lengths the benchmark configurations state.

The other GPU files cover the rules on small lists for many steps and the large
lists for a few steps; the cases here run each large configuration for its
whole stated length:

  * mixed-precision Adam: 25,165,824 parameters in 48 ragged tensors, 500 steps,
    a seeded 0.1 % chance per step of one inf/NaN in one tensor; the loss-scale
    state is compared after every step, every buffer every 50 steps and after
    every skipped step;
  * fp32 Adam on 2^30 parameters in 256 tensors: 20 steps, a strided sample of
    every tensor compared after every step;
  * L-BFGS, n = 10,000,000, history 10, 50 iterations: the configured
    ill-conditioned quadratic in the reference's statement order and in the
    working mode, and a well-conditioned quadratic in the working mode.

The oracle's independent loops are split over the host cores here (same bits as
one thread; tests/test_oracle.py checks that) so that these cases take minutes,
not an hour.  They are marked `slow` as well as `gpu`.
"""
import ctypes as C

import numpy as np
import pytest

import workloads as W

pytestmark = [pytest.mark.gpu, pytest.mark.slow]


@pytest.fixture()
def fast_oracle(oracle):
    oracle.set_threads(oracle.all_cores())
    yield oracle
    oracle.set_threads(1)


def test_mixed_adam_25m_params_500_steps_seeded_injection(gm, dev, fast_oracle):
    from test_mixed_gpu import PackedArenas, same_state, LR, B1, B2, EPS, WD
    O, L = fast_oracle, gm.lib
    sizes = W.ragged_sizes(48, 25_165_824, 4096, 4_194_304)
    total = sum(sizes)
    assert total == 25_165_824 and all(s % 8 for s in sizes)
    bounds = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    split = lambda flat: [flat[bounds[t]:bounds[t + 1]] for t in range(len(sizes))]

    # flat host copies; the per-tensor views alias them, so the oracle updates them in place
    w_flat = O.fill_uniform(total, -0.05, 0.05, 31, 1)
    m_flat, v_flat = np.zeros(total, np.float32), np.zeros(total, np.float32)
    p_flat = O.f32_to_f16(w_flat)
    master, m, v, p16 = split(w_flat), split(m_flat), split(v_flat), split(p_flat)
    st = O.new_loss_scale()                                   # 65536, x2 after 2000 clean steps, x0.5 on overflow
    A = PackedArenas(gm, dev, sizes)
    lead = int(A.offs[0])

    def put_flat(key, flat):
        dev.upload(A.base[key] + A.eb[key] * lead, flat)

    def get_flat(key):
        return dev.to_host(A.base[key] + A.eb[key] * lead, total, np.uint16 if A.eb[key] == 2 else np.float32)

    mx = L.gm_mixed_create(dev.h, None, B1, B2, 0)
    assert mx, gm.last_error()
    inject = np.random.default_rng(20261)                     # seeded: which steps overflow, where and with what
    steps, skips, compared = 500, 0, 0
    try:
        for key in "gwmvp":                                     # the words around the tensors start at zero too
            gm.check(L.gm_buffer_zero(dev.h, A.base[key], A.total * A.eb[key]), "zero")
        for key, flat in (("w", w_flat), ("m", m_flat), ("v", v_flat), ("p", p_flat)):
            put_flat(key, flat)
        for step in range(1, steps + 1):
            z = O.fill_normal(total, 0.0, 1e-3, 777, step)    # fresh N(0, 1e-3^2) gradients every step
            g_flat = O.scale_to_f16(z, st.scale)              # ... times the current loss scale, as fp16
            if inject.random() < 0.001 or step == 137:        # 0.1 % per step; one fixed step so that a skip is certain
                t = int(inject.integers(len(sizes)))
                e = int(inject.integers(sizes[t]))
                g_flat[bounds[t] + e] = [0x7c00, 0xfc00, 0x7e00][int(inject.integers(3))]
            put_flat("g", g_flat)
            gm.check(L.gm_mixed_step_async(dev.h, mx, A.list, LR, EPS, WD), "mixed step")
            skipped = O.mixed_adam_step(split(g_flat), master, m, v, p16, LR, B1, B2, EPS, WD, st)
            skips += skipped
            got = gm.LossScale()
            gm.check(L.gm_mixed_get_state(dev.h, mx, C.byref(got)), "state")
            assert same_state(got, st), (f"step {step}: device scale={got.scale} good={got.good_steps} t={got.adam_t} "
                                         f"skipped={got.skipped} vs oracle scale={st.scale} good={st.good_steps} "
                                         f"t={st.adam_t} skipped={st.skipped}")
            if step % 50 == 0 or skipped or step == steps:
                compared += 1
                for key, want in (("w", w_flat), ("m", m_flat), ("v", v_flat)):
                    assert np.array_equal(get_flat(key).view(np.uint32), want.view(np.uint32)), f"step {step}: {key} differs"
                got_p = get_flat("p")
                assert np.array_equal(got_p, p_flat), f"step {step}: fp16 parameters differ from the oracle"
                assert np.array_equal(got_p, O.f32_to_f16(w_flat)), f"step {step}: fp16 parameters != half_rn(master)"
        assert skips >= 1 and st.skipped == skips and st.adam_t == steps - skips
        assert compared >= 11
        # nothing outside the tensors was written (the element in front and the slack behind)
        for key in "wmv":
            assert dev.to_host(A.base[key], 1)[0] == 0.0
            assert not dev.to_host(A.base[key] + 4 * (lead + total), 16).any()
    finally:
        L.gm_mixed_destroy(mx)
        A.close()


def test_adam_2p30_params_256_tensors_20_steps_sampled(gm, dev, oracle):
    """fp32 Adam, lr 1e-3, betas 0.9/0.999, eps 1e-8, on 1,073,741,824 parameters in 256 flat
    tensors of 4,194,304; 20 steps with fresh N(0, 0.01^2) gradients each step.  The rule is
    elementwise, so a strided sample of every tensor (plus both ends) carried through all 20
    steps on the oracle pins the whole trajectory of those elements; guard words behind each
    arena and a no-element-skipped count cover the rest."""
    torch = pytest.importorskip("torch")
    from test_full_size_gpu import sample_indices
    O, L = oracle, gm.lib
    T, E = 256, 4_194_304
    n = T * E
    free_b, _ = torch.cuda.mem_get_info()
    if free_b < 18 * 2 ** 30:
        pytest.skip("needs 18 GiB of free device memory")
    gen = torch.Generator(device="cuda")
    gen.manual_seed(20264)
    guard = 1024
    lim = (6.0 / 4096.0) ** 0.5                               # He-uniform, fan-in 4096
    w = torch.empty(n + guard, dtype=torch.float32, device="cuda").uniform_(-lim, lim, generator=gen)
    g = torch.empty(n + guard, dtype=torch.float32, device="cuda")
    m = torch.zeros(n + guard, dtype=torch.float32, device="cuda")
    v = torch.zeros(n + guard, dtype=torch.float32, device="cuda")
    for a in (w, m, v):
        a[n:] = 7.0
    torch.cuda.synchronize()
    ptrs = lambda a: [a.data_ptr() + 4 * t * E for t in range(T)]
    lst = dev.tensor_list([ptrs(w), ptrs(g), ptrs(m), ptrs(v)], [E] * T)
    idx = sample_indices(E)
    flat = torch.from_numpy(np.concatenate([idx + t * E for t in range(T)])).cuda()
    ws, ms, vs = (a[flat].cpu().numpy() for a in (w, m, v))    # the oracle's copy of the sampled elements
    try:
        for step in range(1, 21):
            g.normal_(0.0, 0.01, generator=gen)
            torch.cuda.synchronize()
            gs = g[flat].cpu().numpy()
            hy = gm.Hyper(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=step)
            gm.check(L.gm_step_async(dev.h, gm.RULE_ADAM, lst, C.byref(hy)), "adam")
            dev.sync()
            O.adam_step(ws, gs, ms, vs, 1e-3, 0.9, 0.999, 1e-8, 0.0, step)
            for k, a, want in (("w", w, ws), ("m", m, ms), ("v", v, vs)):
                got = a[flat].cpu().numpy()
                assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"step {step}: {k} sample differs"
        assert bool((w[n:] == 7.0).all()) and bool((m[n:] == 7.0).all()) and bool((v[n:] == 7.0).all())
        assert int((v[:n] == 0).sum()) <= int((g[:n] == 0).sum()), "an element was skipped"
    finally:
        L.gm_tensor_list_destroy(lst)
        del w, g, m, v
        torch.cuda.empty_cache()


@pytest.mark.parametrize("name,mode,lo,hi", [
    ("configured_problem_reference_order_identical_through_the_overflow", 0, -2.0, 2.0),
    ("configured_problem_working_mode_identical_through_the_overflow", 3, -2.0, 2.0),
    ("well_conditioned_problem_working_mode", 3, -0.3, 0.3),
])
def test_lbfgs_10m_variables_history_10_50_iterations(gm, dev, fast_oracle, name, mode, lo, hi):
    """n = 10,000,000, m = 10, unit step, no line search, 50 iterations.  On the configured
    problem (D log-uniform in [1e-2, 1e2]) the unit step overflows within ~15 iterations
    in every mode: iterates, alpha and rho are identical bit for bit up to and including
    the overflow, and afterwards the NaN positions are equal (NaN payloads are not
    compared).  The well-conditioned problem (D in [0.5, 2]) converges, so its accept/skip
    decisions are real ones."""
    from test_lbfgs_gpu import LbfgsProblem
    gm.check(gm.lib.gm_lbfgs_set_mode(dev.h, mode), "mode")
    P = LbfgsProblem(gm, dev, fast_oracle, [10_000_000], 10, lo, hi, seed=77)
    try:
        finite_iterations, best = 0, np.inf
        with np.errstate(all="ignore"):
            for it in range(50):
                P.step(mode)
                P.compare(it, full=(it in (0, 12, 49)))
                if np.isfinite(P.x[0]).all():
                    finite_iterations += 1
                    best = min(best, float(np.abs(P.gradient(P.x)[0]).max()))
                if it == 20 and name.startswith("well"):
                    assert (P.rho != 0).all(), "every stored pair is accepted while the iteration converges"
        if name.startswith("well"):
            # The reference has no termination test (lbfgs.go:245-301): once the gradient is at rounding
            # level the curvature pairs are noise and later iterations wander, so convergence is judged on
            # the best iterate; parity above covers all 50 iterations whatever they do.
            assert best < 1e-4 and finite_iterations >= 25, (best, finite_iterations)
        else:
            assert 3 <= finite_iterations < 50, "the configured problem overflows under a unit step"
        if mode == 0:
            assert (P.rho == 0).all() or not np.isfinite(P.rho).all()
    finally:
        P.free()
        gm.lib.gm_lbfgs_set_mode(dev.h, 3)
