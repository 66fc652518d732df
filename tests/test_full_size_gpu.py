"""Parity at the full sizes of the benchmark configurations.

The oracle is scalar, so full-size checks use what the domain offers: the
rules are elementwise, hence any subset of elements is independently
verifiable -- inputs are filled on the device, a strided sample plus the head
and tail of every tensor is copied back before and after the step, and the
oracle is run on exactly those bits.  The mixed-precision and L-BFGS
configurations are small enough (25 M / 10 M elements) to run whole for a few
steps.
"""
import ctypes as C

import numpy as np
import pytest

import workloads as W

pytestmark = pytest.mark.gpu


def sample_indices(n, stride=4099, edge=64):
    idx = np.unique(np.concatenate([np.arange(0, min(edge, n)), np.arange(max(0, n - edge), n), np.arange(0, n, stride)]))
    return idx.astype(np.int64)


def test_adam_2p30_params_256_tensors_sampled(gm, dev, oracle):
    """fp32 Adam on 1,073,741,824 parameters in 256 flat tensors of 4,194,304 (16 GiB of
    arenas), 3 steps; every tensor is checked on ~1,150 sampled elements per step,
    and untouched guard words after each arena stay intact."""
    torch = pytest.importorskip("torch")
    O, L = oracle, gm.lib
    T, E = 256, 4_194_304
    n = T * E
    free_b, _ = torch.cuda.mem_get_info()
    if free_b < 18 * 2 ** 30:
        pytest.skip("needs 18 GiB of free device memory")
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1234)
    guard = 1024
    w = torch.empty(n + guard, dtype=torch.float32, device="cuda").uniform_(-0.04, 0.04, generator=gen)
    g = torch.empty(n + guard, dtype=torch.float32, device="cuda")
    m = torch.zeros(n + guard, dtype=torch.float32, device="cuda")
    v = torch.zeros(n + guard, dtype=torch.float32, device="cuda")
    for a in (w, m, v):
        a[n:] = 7.0
    torch.cuda.synchronize()
    ptrs = lambda a: [a.data_ptr() + 4 * t * E for t in range(T)]
    lst = dev.tensor_list([ptrs(w), ptrs(g), ptrs(m), ptrs(v)], [E] * T)
    assert L.gm_tensor_list_total(lst) == n
    idx = sample_indices(E)
    flat = torch.from_numpy(np.concatenate([idx + t * E for t in range(T)])).cuda()
    try:
        for step in (1, 2, 3):
            g.normal_(0.0, 0.01, generator=gen)
            torch.cuda.synchronize()
            before = {k: a[flat].cpu().numpy() for k, a in (("w", w), ("g", g), ("m", m), ("v", v))}
            hy = gm.Hyper(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=step)
            gm.check(L.gm_step_async(dev.h, gm.RULE_ADAM, lst, C.byref(hy)), "adam")
            dev.sync()
            ws, ms, vs = before["w"].copy(), before["m"].copy(), before["v"].copy()
            O.adam_step(ws, before["g"], ms, vs, 1e-3, 0.9, 0.999, 1e-8, 0.0, step)
            for k, a, want in (("w", w, ws), ("m", m, ms), ("v", v, vs)):
                got = a[flat].cpu().numpy()
                assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"step {step}: {k} sample differs"
            assert bool((w[n:] == 7.0).all()) and bool((m[n:] == 7.0).all()) and bool((v[n:] == 7.0).all())
            # size-independent property: no element was skipped (v > 0 wherever g != 0)
            assert int((v[:n] == 0).sum()) <= int((g[:n] == 0).sum())
    finally:
        L.gm_tensor_list_destroy(lst)
        del w, g, m, v
        torch.cuda.empty_cache()


def test_adam_one_tensor_past_2p31_elements(gm, dev, oracle):
    """Maximum sizes: one tensor of 2^31 + 5,001 elements (8 GiB per stream, more than an
    `int` can count in elements or bytes), every stream starting one element past a
    16-byte boundary, so element offsets, chunk counts and the ragged tail all run in
    64-bit arithmetic.  Two Adam steps; a strided sample, both ends and the elements on
    either side of index 2^31 are compared with the oracle."""
    torch = pytest.importorskip("torch")
    O, L = oracle, gm.lib
    n = 2 ** 31 + 5001
    free_b, _ = torch.cuda.mem_get_info()
    if free_b < 40 * 2 ** 30:
        pytest.skip("needs 40 GiB of free device memory")
    gen = torch.Generator(device="cuda")
    gen.manual_seed(4321)
    pad = 8
    w = torch.empty(n + pad, dtype=torch.float32, device="cuda").uniform_(-0.04, 0.04, generator=gen)
    g = torch.empty(n + pad, dtype=torch.float32, device="cuda")
    m = torch.zeros(n + pad, dtype=torch.float32, device="cuda")
    v = torch.zeros(n + pad, dtype=torch.float32, device="cuda")
    for a in (w, m, v):
        a[0] = 7.0
        a[n + 1:] = 7.0
    lst = dev.tensor_list([[a.data_ptr() + 4] for a in (w, g, m, v)], [n])
    assert L.gm_tensor_list_total(lst) == n
    assert L.gm_tensor_list_num_chunks(lst) == (n - 3 + 4095) // 4096      # 3 elements peeled up to the boundary
    mid = np.arange(2 ** 31 - 64, 2 ** 31 + 64)
    idx = np.unique(np.concatenate([sample_indices(n, stride=1_000_003), mid])).astype(np.int64)
    flat = torch.from_numpy(idx + 1).cuda()                 # +1: the tensors start at element 1 of the allocations
    try:
        for step in (1, 2):
            g.normal_(0.0, 0.01, generator=gen)
            torch.cuda.synchronize()
            before = {k: a[flat].cpu().numpy() for k, a in (("w", w), ("g", g), ("m", m), ("v", v))}
            hy = gm.Hyper(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=step)
            gm.check(L.gm_step_async(dev.h, gm.RULE_ADAM, lst, C.byref(hy)), "adam")
            dev.sync()
            ws, ms, vs = before["w"].copy(), before["m"].copy(), before["v"].copy()
            O.adam_step(ws, before["g"], ms, vs, 1e-3, 0.9, 0.999, 1e-8, 0.0, step)
            for k, a, want in (("w", w, ws), ("m", m, ms), ("v", v, vs)):
                got = a[flat].cpu().numpy()
                assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"step {step}: {k} sample differs"
            for a in (w, m, v):
                assert float(a[0]) == 7.0 and bool((a[n + 1:] == 7.0).all()), "wrote outside the tensor"
            # no element skipped: v stays 0 only where g is 0
            assert int((v[1:n + 1] == 0).sum()) <= int((g[1:n + 1] == 0).sum())
    finally:
        L.gm_tensor_list_destroy(lst)
        del w, g, m, v
        torch.cuda.empty_cache()


def test_mixed_adam_25m_params_48_ragged_tensors(gm, dev, oracle):
    """The mixed-precision configuration at its full size: 25,165,824 parameters in 48
    log-uniform tensors (4 Ki - 4 Mi, none a multiple of 8) packed back to back, fp16
    gradients N(0, 1e-3^2) x scale; 6 steps, an injected NaN on step 3; everything is
    compared whole against the oracle."""
    from test_mixed_gpu import PackedArenas, same_state, LR, B1, B2, EPS, WD
    O, L = oracle, gm.lib
    sizes = W.ragged_sizes(48, 25_165_824, 4096, 4_194_304)
    assert sum(sizes) == 25_165_824
    rng = np.random.default_rng(3)
    master = [O.fill_uniform(n, -0.05, 0.05, 3, 500 + k) for k, n in enumerate(sizes)]
    m = [np.zeros(n, np.float32) for n in sizes]
    v = [np.zeros(n, np.float32) for n in sizes]
    p16 = [O.f32_to_f16(a) for a in master]
    st = O.new_loss_scale()
    A = PackedArenas(gm, dev, sizes)
    mx = L.gm_mixed_create(dev.h, None, B1, B2, 0)
    try:
        for key, arrs in (("w", master), ("m", m), ("v", v), ("p", p16)):
            A.put(key, arrs)
        for step in range(1, 7):
            scale = np.float32(st.scale)
            g16 = [O.f32_to_f16(rng.standard_normal(n, dtype=np.float32) * np.float32(1e-3) * scale) for n in sizes]
            if step == 3:
                g16[17][sizes[17] - 1] = 0x7e00
            A.put("g", g16)
            gm.check(L.gm_mixed_step_async(dev.h, mx, A.list, LR, EPS, WD), "mixed")
            O.mixed_adam_step(g16, master, m, v, p16, LR, B1, B2, EPS, WD, st)
            got = gm.LossScale()
            gm.check(L.gm_mixed_get_state(dev.h, mx, C.byref(got)), "state")
            assert same_state(got, st), f"step {step}: loss-scale state differs"
        assert st.skipped == 1 and st.adam_t == 5 and st.scale == 32768.0
        for key, want in (("w", master), ("m", m), ("v", v)):
            got_list, _ = A.get(key)
            for t, (a, b) in enumerate(zip(got_list, want)):
                assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), f"{key}[{t}] differs"
        got_p, _ = A.get("p")
        for t, (a, b) in enumerate(zip(got_p, p16)):
            assert np.array_equal(a, b) and np.array_equal(a, O.f32_to_f16(master[t])), f"p16[{t}]"
    finally:
        L.gm_mixed_destroy(mx)
        A.close()


def test_lbfgs_10m_variables_history_10(gm, dev, oracle):
    """L-BFGS at n = 10,000,000, m = 10, on the well-conditioned quadratic for 14
    iterations (history full and wrapping): iterates and rho bit for bit, plus the
    configured ill-conditioned problem for 6 iterations."""
    from test_lbfgs_gpu import LbfgsProblem
    gm.check(gm.lib.gm_lbfgs_set_mode(dev.h, 3), "mode")
    for lo, hi, iters in ((-0.3, 0.3, 14), (-2.0, 2.0, 6)):
        P = LbfgsProblem(gm, dev, oracle, [10_000_000], 10, lo, hi, seed=77)
        try:
            with np.errstate(all="ignore"):
                for it in range(iters):
                    P.step(3)
                    P.compare(it, full=(it == iters - 1))
        finally:
            P.free()
