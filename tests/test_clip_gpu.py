"""Deterministic gradient norm, global-norm clipping and the constant-divisor
division, on the GPU against the CPU oracle, bit for bit.

The reference has no clipping code (docs/guides/optimizers.md:568-569 names the
concept); the formula is coef = min(1, max_norm / (sqrt(sum g^2) + 1e-6)) in
binary32, every gradient multiplied by coef (one rounding) before the rule.
"""
import ctypes as C

import numpy as np
import pytest

import workloads as W

pytestmark = pytest.mark.gpu

f32 = np.float32


def bits(x):
    return np.asarray(x, dtype=f32).view(np.uint32)


def test_clipped_adam_mlp_100_steps(gm, dev, oracle):
    """Config-1 shape (MLP, 101,770 parameters in 4 tensors), 100 Adam steps with the
    gradients clipped to a global norm that the N(0, 0.01^2) gradients exceed on every
    step: sum of squares, coefficient, parameters and both moments bit for bit."""
    O, L = oracle, gm.lib
    shapes = W.MLP_SHAPES
    sizes = [W.numel(s) for s in shapes]
    w = W.he_uniform_weights(O, shapes, W.MLP_FAN_IN)
    m = [np.zeros(n, f32) for n in sizes]
    v = [np.zeros(n, f32) for n in sizes]
    d = {k: [dev.to_device(a) for a in arrs] for k, arrs in (("w", w), ("m", m), ("v", v))}
    d["g"] = [dev.alloc(4 * n) for n in sizes]
    lst = dev.tensor_list([d["w"], d["g"], d["m"], d["v"]], sizes)
    max_norm = 1.0                                            # ||g|| is about 0.01*sqrt(101770) = 3.2
    try:
        for step in range(1, 101):
            g = W.normal_grads(O, shapes, step)
            for p, a in zip(d["g"], g):
                dev.upload(p, a)
            hy = gm.Hyper(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=step)
            gm.check(L.gm_step_with_clip_async(dev.h, gm.RULE_ADAM, lst, C.byref(hy), max_norm), "clipped step")
            out = (C.c_float * 3)()
            gm.check(L.gm_last_clip(dev.h, out), "last clip")
            ss = O.sumsq_canonical(g)
            coef = O.clip_coef(ss, max_norm)
            assert bits(out[0]) == bits(ss), f"step {step}: sum of squares {out[0]} vs {ss}"
            assert bits(out[1]) == bits(coef) and 0 < coef < 1, f"step {step}: coefficient {out[1]} vs {coef}"
            for t in range(len(sizes)):
                gc = (g[t] * coef).astype(f32)
                O.adam_step(w[t], gc, m[t], v[t], 1e-3, 0.9, 0.999, 1e-8, 0.0, step)
            if step % 10 == 0 or step == 1:
                for key, want in (("w", w), ("m", m), ("v", v)):
                    for t, n in enumerate(sizes):
                        got = dev.to_host(d[key][t], n)
                        assert np.array_equal(bits(got), bits(want[t])), f"step {step}: {key}[{t}] differs"
    finally:
        L.gm_tensor_list_destroy(lst)
        for arrs in d.values():
            for p in arrs:
                dev.free(p)


def test_clip_leaves_small_gradients_alone_and_works_for_every_rule(gm, dev, oracle):
    """A norm below the limit gives coef == 1 and the unclipped bits; the coefficient
    reaches the other rules too (SGD with momentum checked); unaligned gradient tensors
    take the element-wise loads in the same order."""
    O, L = oracle, gm.lib
    sizes = [4097, 3, 70_001]
    base = {k: dev.alloc(4 * (sum(sizes) + 16)) for k in "wgm"}
    offs = np.concatenate([[1], 1 + np.cumsum(sizes)[:-1]])           # every tensor off the 16-byte boundary
    ptrs = {k: [base[k] + 4 * int(o) for o in offs] for k in "wgm"}
    lst = dev.tensor_list([ptrs["w"], ptrs["g"], ptrs["m"]], sizes)
    w = [O.fill_uniform(n, -0.1, 0.1, 61, k) for k, n in enumerate(sizes)]
    mom = [np.zeros(n, f32) for n in sizes]
    try:
        for step, (std, max_norm) in enumerate([(0.01, 100.0), (0.5, 2.0), (0.5, 1e-3)], start=1):
            g = [O.fill_normal(n, 0.0, std, 61, 100 * step + k) for k, n in enumerate(sizes)]
            for key, arrs in (("w", w), ("g", g), ("m", mom)):
                for p, a in zip(ptrs[key], arrs):
                    dev.upload(p, a)
            hy = gm.Hyper(lr=0.01, beta1=0.9, weight_decay=0.0, step=step)
            gm.check(L.gm_step_with_clip_async(dev.h, gm.RULE_SGD, lst, C.byref(hy), max_norm), "clipped sgd")
            out = (C.c_float * 3)()
            gm.check(L.gm_last_clip(dev.h, out), "last clip")
            ss = O.sumsq_canonical(g)
            coef = O.clip_coef(ss, max_norm)
            assert bits(out[0]) == bits(ss) and bits(out[1]) == bits(coef)
            assert (coef == 1.0) == (step == 1)
            for t, n in enumerate(sizes):
                O.sgd_step(w[t], (g[t] * coef).astype(f32), mom[t], 0.01, 0.9, 0.0, False)
                assert np.array_equal(bits(dev.to_host(ptrs["w"][t], n)), bits(w[t])), f"step {step}: w[{t}]"
                assert np.array_equal(bits(dev.to_host(ptrs["m"][t], n)), bits(mom[t])), f"step {step}: momentum[{t}]"
        bad = gm.Hyper(lr=0.01, beta1=0.9, step=1)
        assert L.gm_step_with_clip_async(dev.h, gm.RULE_SGD, lst, C.byref(bad), 0.0) == -10
        assert L.gm_grad_clip_coef_async(dev.h, lst, 1.0, 0) == -4
    finally:
        L.gm_tensor_list_destroy(lst)
        for p in base.values():
            dev.free(p)


def test_clipped_mixed_adam(gm, dev, oracle):
    """Mixed-precision Adam with clipping: the overflow-check pass also forms the norm of
    the unscaled gradients and the coefficient; the sum (in the order of the list's
    layout), the coefficient, master/m/v and the fp16 parameters match the oracle bit
    for bit over 40 steps that include an overflow and a growth of the scale."""
    from test_mixed_gpu import PackedArenas, same_state, LR, B1, B2, EPS, WD
    O, L = oracle, gm.lib
    sizes = W.ragged_sizes(12, 98_311, 1024, 40_000) + [3, 8191]
    A = PackedArenas(gm, dev, sizes)
    heads = [L.gm_tensor_list_head(A.list, t) for t in range(len(sizes))]
    chunk = L.gm_tensor_list_chunk_elems(A.list)
    assert chunk == 8192 and all(-1 <= h < 8 for h in heads) and any(h > 0 for h in heads)
    rng = np.random.default_rng(77)
    master = [O.fill_uniform(n, -0.05, 0.05, 71, k) for k, n in enumerate(sizes)]
    m = [np.zeros(n, f32) for n in sizes]
    v = [np.zeros(n, f32) for n in sizes]
    p16 = [O.f32_to_f16(a) for a in master]
    st = O.new_loss_scale(interval=15)
    init = gm.LossScale(scale=st.scale, growth=st.growth, backoff=st.backoff, max_scale=st.max_scale, interval=15,
                        good_steps=0, adam_t=0, skipped=0, last_overflow=0)
    mx = L.gm_mixed_create(dev.h, C.byref(init), B1, B2, 0)
    assert mx, gm.last_error()
    max_norm = 0.2                                            # ||g|| is about 1e-3*sqrt(106505) = 0.33
    gm.check(L.gm_mixed_set_clip(mx, max_norm), "set clip")
    try:
        for key, arrs in (("w", master), ("m", m), ("v", v), ("p", p16)):
            A.put(key, arrs)
        clipped_steps = 0
        for step in range(1, 41):
            std = 1e-3 if step % 4 else 2e-4                  # every fourth step stays below the limit
            g16 = [O.scale_to_f16((rng.standard_normal(n) * std).astype(f32), st.scale) for n in sizes]
            if step == 9:
                g16[5][11] = 0x7e00
            A.put("g", g16)
            gm.check(L.gm_mixed_step_async(dev.h, mx, A.list, LR, EPS, WD), "mixed step")
            skipped, ss, coef = O.mixed_adam_step_clipped(g16, master, m, v, p16, LR, B1, B2, EPS, WD, max_norm, heads, chunk, st)
            got_ss, got_coef = C.c_float(), C.c_float()
            gm.check(L.gm_mixed_last_clip(dev.h, mx, C.byref(got_ss), C.byref(got_coef)), "last clip")
            if skipped:
                assert not np.isfinite(got_ss.value) and step == 9
            else:
                assert bits(got_ss.value) == bits(ss), f"step {step}: sum of squares {got_ss.value} vs {ss}"
                assert bits(got_coef.value) == bits(coef), f"step {step}: coefficient {got_coef.value} vs {coef}"
                clipped_steps += int(coef < 1.0)
            got = gm.LossScale()
            gm.check(L.gm_mixed_get_state(dev.h, mx, C.byref(got)), "state")
            assert same_state(got, st), f"step {step}: loss-scale state differs"
            if step % 8 == 0 or skipped or step == 40:
                for key, want in (("w", master), ("m", m), ("v", v)):
                    got_list, _ = A.get(key)
                    for t, (a, b) in enumerate(zip(got_list, want)):
                        assert np.array_equal(bits(a), bits(b)), f"step {step}: {key}[{t}] differs"
                got_p, _ = A.get("p")
                for t, (a, b) in enumerate(zip(got_p, p16)):
                    assert np.array_equal(a, b), f"step {step}: p16[{t}] differs"
        assert 20 <= clipped_steps <= 32 and st.skipped == 1 and len({st.scale, 65536.0}) == 2
        # clipping off again: the plain step, coefficient 1
        gm.check(L.gm_mixed_set_clip(mx, 0.0), "clip off")
        g16 = [O.scale_to_f16((rng.standard_normal(n) * 1e-3).astype(f32), st.scale) for n in sizes]
        A.put("g", g16)
        gm.check(L.gm_mixed_step_async(dev.h, mx, A.list, LR, EPS, WD), "mixed step")
        O.mixed_adam_step(g16, master, m, v, p16, LR, B1, B2, EPS, WD, st)
        got_list, _ = A.get("w")
        for t, (a, b) in enumerate(zip(got_list, master)):
            assert np.array_equal(bits(a), bits(b)), f"unclipped step: w[{t}] differs"
        assert L.gm_mixed_set_clip(mx, -1.0) == -10 and L.gm_mixed_set_clip(mx, float("nan")) == -10
    finally:
        L.gm_mixed_destroy(mx)
        A.close()


def test_mixed_grad_norm_is_deterministic_and_matches_the_layout_order(gm, dev, oracle):
    """The norm taken by the overflow check alone (no clipping): same bits as the oracle's
    layout-ordered sum, and the same bits on a second run over the same data."""
    from test_mixed_gpu import PackedArenas, LR, B1, B2, EPS, WD
    O, L = oracle, gm.lib
    sizes = [9, 70_001, 8192 * 3 + 5, 4096]
    for lead in (1, 4, 8):
        A = PackedArenas(gm, dev, sizes, lead=lead)
        heads = [L.gm_tensor_list_head(A.list, t) for t in range(len(sizes))]
        mx = L.gm_mixed_create(dev.h, None, B1, B2, 0)
        gm.check(L.gm_mixed_enable_grad_norm(mx, 1), "norm on")
        try:
            zeros = [np.zeros(n, f32) for n in sizes]
            for key in "wmv":
                A.put(key, zeros)
            A.put("p", [np.zeros(n, np.uint16) for n in sizes])
            g16 = [O.f32_to_f16(O.fill_normal(n, 0, 40.0, 81, k)) for k, n in enumerate(sizes)]
            A.put("g", g16)
            seen = []
            for _ in range(2):
                gm.check(L.gm_mixed_step_async(dev.h, mx, A.list, LR, EPS, WD), "step")
                out = C.c_float()
                gm.check(L.gm_mixed_last_grad_sumsq(dev.h, mx, C.byref(out)), "sumsq")
                seen.append(f32(out.value))
            want = O.sumsq_f16_layout(g16, heads, 8192, 1.0 / 65536.0)
            assert bits(seen[0]) == bits(want) and bits(seen[1]) == bits(want), (lead, heads, seen, want)
        finally:
            L.gm_mixed_destroy(mx)
            A.close()


def test_constant_divisor_division_is_exact_for_every_dividend(gm, dev, oracle):
    """All 2^32 dividends against the IEEE division, for the bias corrections 1 - beta^t of the
    default betas (every step until beta1's correction reaches 1, and beta2's at a spread of
    steps) and for divisors at the edges of the enabled range."""
    O, L = oracle, gm.lib
    divisors = {}
    for t in list(range(1, 181)) + [250, 500, 1000, 2000, 4000, 8000, 12000, 16000]:
        bc1, bc2, _, _ = O.adam_scalars(0.9, 0.999, t)
        divisors[float(bc1)] = f"1-0.9^{t}"
        divisors[float(bc2)] = f"1-0.999^{t}"
    for t in (1, 2, 3, 50, 5000):
        divisors[float(O.adam_scalars(0.99, 0.9999, t)[1])] = f"1-0.9999^{t}"
    divisors[1.0] = "one"
    divisors[float(f32(2.0 ** -24))] = "lower edge"
    divisors[0.75] = "0.75"
    enabled = 0
    for c, name in divisors.items():
        count, first, allowed = C.c_uint64(), C.c_uint32(), C.c_int()
        gm.check(L.gm_selftest_const_div(dev.h, c, C.byref(count), C.byref(first), C.byref(allowed)), "selftest")
        assert count.value == 0, f"c = {c!r} ({name}): {count.value} dividends differ, first 0x{first.value:08x}"
        enabled += allowed.value
    assert enabled >= 180
    # outside the enabled range the library keeps the IEEE division
    allowed = C.c_int(7)
    count = C.c_uint64(9)
    for c in (1.5, 1e-9, float(np.uint32(0x3effffff).view(f32)), float("nan")):
        gm.check(L.gm_selftest_const_div(dev.h, c, C.byref(count), None, C.byref(allowed)), "selftest")
        assert allowed.value == 0 and count.value == 0
