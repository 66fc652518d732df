"""The host mirror of the optimizer package driving the real CUDA library:
Optimizer.Step through the drop-in entries against the oracle, a checkpoint
round trip (GetState -> LoadState into a fresh optimizer -> identical
continuation), the LR hook, and L-BFGS with its own Step signature."""
import ctypes as C

import numpy as np
import pytest

import hostlib as HL
import workloads as W

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def H(gm):
    lib = HL.load_host()
    assert lib.gmh_init(HL.CUDA.encode()) == 0, HL.err(lib)
    return lib


def put(gm, arrays):
    ptrs = []
    for a in arrays:
        p = gm.lib.allocate_cuda_buffer(gm_dev, a.size * 4, 1)
        gm.check(gm.lib.copy_float32_array_to_cuda_buffer(p, a.ctypes.data, a.size), "upload")
        ptrs.append(p)
    return ptrs


def get(gm, ptrs, sizes):
    out = []
    for p, n in zip(ptrs, sizes):
        a = np.empty(n, np.float32)
        gm.check(gm.lib.copy_cuda_buffer_to_float32_array(p, a.ctypes.data, n), "download")
        out.append(a)
    return out


gm_dev = 0


def test_adam_through_host_mirror_with_checkpoint_resume(gm, H, oracle):
    global gm_dev
    O = oracle
    dev = H.gmh_device_create()
    gm_dev = dev
    assert dev, HL.err(H)
    mm = H.gmh_mm_create(dev)
    shapes = [list(s) for s in W.MLP_SHAPES]
    sizes = [W.numel(s) for s in shapes]
    w_cpu = W.he_uniform_weights(O, W.MLP_SHAPES, W.MLP_FAN_IN)
    m_cpu = [np.zeros(n, np.float32) for n in sizes]
    v_cpu = [np.zeros(n, np.float32) for n in sizes]
    wp = put(gm, w_cpu)
    gp = put(gm, [np.zeros(n, np.float32) for n in sizes])
    opt = HL.make_optimizer(H, "Adam", [], shapes, mm, dev)
    assert opt, HL.err(H)
    assert H.gmh_optimizer_set_weight_buffers(opt, HL.uarr(wp), 4) == 0

    def step(o, k, lr):
        grads = W.normal_grads(O, W.MLP_SHAPES, k)
        for p, g in zip(gp, grads):
            gm.check(gm.lib.copy_float32_array_to_cuda_buffer(p, g.ctypes.data, g.size), "upload")
        assert H.gmh_optimizer_step(o, HL.uarr(gp), 4, 0.0) == 0, HL.err(H)
        for t in range(4):
            O.adam_step(w_cpu[t], grads[t], m_cpu[t], v_cpu[t], lr, 0.9, 0.999, 1e-8, 0.0, k)

    for k in range(1, 6):
        step(opt, k, 1e-3)
    # LR hook: a StepLR scheduler changes the rate the next step uses
    sched = H.gmh_sched_create(0, 1, 0.5, 0.0, b"")
    assert H.gmh_apply_scheduler(sched, opt, 1, 0, 1e-3) == 0
    lr2 = float(np.float32(1e-3 * 0.5))
    step(opt, 6, lr2)
    for a, b in zip(get(gm, wp, sizes), w_cpu):
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))

    # checkpoint: state out, into a fresh optimizer, continue
    st = H.gmh_optimizer_get_state(opt)
    assert st and H.gmh_state_num_tensors(st) == 8
    saved = H.gmh_state_new(b"Adam")
    for i in range(8):
        n = H.gmh_state_tensor_numel(st, i)
        buf = np.empty(n, np.float32)
        H.gmh_state_tensor_data(st, i, buf.ctypes.data)
        H.gmh_state_add_tensor(saved, H.gmh_state_tensor_name(st, i), H.gmh_state_tensor_type(st, i), buf.ctypes.data, n)
        if i == 1:
            assert np.array_equal(buf.view(np.uint32), m_cpu[1].view(np.uint32))      # momentum_1
        if i == 4:
            assert np.array_equal(buf.view(np.uint32), v_cpu[0].view(np.uint32))      # variance_0
    H.gmh_state_set_float64(saved, b"step_count", 6.0)                  # as a JSON checkpoint delivers it
    H.gmh_state_set_float64(saved, b"learning_rate", lr2)
    H.gmh_optimizer_destroy(opt)
    opt2 = HL.make_optimizer(H, "Adam", [], shapes, mm, dev)
    assert H.gmh_optimizer_set_weight_buffers(opt2, HL.uarr(wp), 4) == 0
    assert H.gmh_optimizer_load_state(opt2, saved) == 0, HL.err(H)
    assert H.gmh_optimizer_step_count(opt2) == 6
    step(opt2, 7, lr2)
    for a, b in zip(get(gm, wp, sizes), w_cpu):
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), "resumed run diverged from the uninterrupted one"
    H.gmh_state_destroy(st)
    H.gmh_state_destroy(saved)
    H.gmh_sched_destroy(sched)
    H.gmh_optimizer_destroy(opt2)
    for p in wp + gp:
        gm.lib.deallocate_cuda_buffer(p)
    H.gmh_mm_destroy(mm)
    H.gmh_device_destroy(dev)


@pytest.mark.parametrize("kind,cfg", [("SGD", [0.01, 0.9, 0.0, 1]), ("RMSProp", [0.01, 0.99, 1e-8, 0.0, 0.9, 1]),
                                      ("AdaGrad", []), ("AdaDelta", [0.9, 1e-6, 0.0]), ("Nadam", [])])
def test_other_rules_through_host_mirror(gm, H, oracle, kind, cfg):
    global gm_dev
    O = oracle
    dev = H.gmh_device_create()
    gm_dev = dev
    mm = H.gmh_mm_create(dev)
    shapes = [[1000], [33, 7]]
    sizes = [1000, 231]
    w_cpu = [O.fill_uniform(n, -0.5, 0.5, 8, k) for k, n in enumerate(sizes)]
    z = lambda: [np.zeros(n, np.float32) for n in sizes]
    s1, s2, s3 = z(), z(), z()
    wp, gp = put(gm, w_cpu), put(gm, z())
    opt = HL.make_optimizer(H, kind, cfg, shapes, mm, dev)
    assert opt, HL.err(H)
    H.gmh_optimizer_set_weight_buffers(opt, HL.uarr(wp), 2)
    for k in range(1, 5):
        grads = [O.fill_normal(n, 0, 0.01, 8, 10 * k + t) for t, n in enumerate(sizes)]
        for p, g in zip(gp, grads):
            gm.check(gm.lib.copy_float32_array_to_cuda_buffer(p, g.ctypes.data, g.size), "upload")
        assert H.gmh_optimizer_step(opt, HL.uarr(gp), 2, 0.0) == 0, HL.err(H)
        for t in range(2):
            if kind == "SGD":
                O.sgd_step(w_cpu[t], grads[t], s1[t], 0.01, 0.9, 0.0, 1)
            elif kind == "RMSProp":
                O.rmsprop_step(w_cpu[t], grads[t], s1[t], s2[t], s3[t], 0.01, 0.99, 1e-8, 0.0, 0.9, True, True)
            elif kind == "AdaGrad":
                O.adagrad_step(w_cpu[t], grads[t], s1[t], 0.01, 1e-10, 0.0)
            elif kind == "AdaDelta":
                O.adadelta_step(w_cpu[t], grads[t], s1[t], s2[t], 0.9, 1e-6, 0.0)
            else:
                O.nadam_step(w_cpu[t], grads[t], s1[t], s2[t], 0.002, 0.9, 0.999, 1e-8, 0.0, k)
    for a, b in zip(get(gm, wp, sizes), w_cpu):
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), kind
    H.gmh_optimizer_destroy(opt)
    for p in wp + gp:
        gm.lib.deallocate_cuda_buffer(p)
    H.gmh_mm_destroy(mm)
    H.gmh_device_destroy(dev)


def test_lbfgs_through_host_mirror(gm, H, oracle):
    global gm_dev
    O = oracle
    dev = H.gmh_device_create()
    gm_dev = dev
    mm = H.gmh_mm_create(dev)
    n, m = 20_000, 4
    D = O.fill_loguniform(n, -0.2, 0.2, 12, 1)
    b = O.fill_normal(n, 0, 1, 12, 2)
    x, old, d = (np.zeros(n, np.float32) for _ in range(3))
    s = [[np.zeros(n, np.float32)] for _ in range(m)]
    y = [[np.zeros(n, np.float32)] for _ in range(m)]
    rho, alpha = np.zeros(m, np.float32), np.zeros(m, np.float32)
    wp, gp = put(gm, [x]), put(gm, [x])
    opt = HL.make_optimizer(H, "LBFGS", [m], [[n]], mm, dev)
    assert opt, HL.err(H)
    H.gmh_optimizer_set_weight_buffers(opt, HL.uarr(wp), 1)
    hc = hi = 0
    for it in range(12):
        g = (D * x - b).astype(np.float32)
        gm.check(gm.lib.copy_float32_array_to_cuda_buffer(gp[0], g.ctypes.data, n), "upload")
        assert H.gmh_optimizer_step(opt, HL.uarr(gp), 1, float(it)) == 0, HL.err(H)
        O.lbfgs_step([x], [g], [old], [d], s, y, rho, alpha, m, hc, hi, 1.0, 3, 0)
        hi, hc = (hi + 1) % m, min(hc + 1, m)
        got = get(gm, wp, [n])[0]
        assert np.array_equal(got.view(np.uint32), x.view(np.uint32)), f"iteration {it}"
        r = np.zeros(m, np.float32)
        assert H.gmh_lbfgs_read_rho(opt, r.ctypes.data, m) == m
        assert np.array_equal(r.view(np.uint32), rho.view(np.uint32)), f"iteration {it}: rho"
    cnt, idx = C.c_int(), C.c_int()
    H.gmh_lbfgs_history(opt, C.byref(cnt), C.byref(idx))
    assert (cnt.value, idx.value) == (hc, hi)
    H.gmh_optimizer_destroy(opt)
    for p in wp + gp:
        gm.lib.deallocate_cuda_buffer(p)
    H.gmh_mm_destroy(mm)
    H.gmh_device_destroy(dev)


def test_mixed_adam_through_host_mirror_with_checkpoint_resume(gm, H, oracle):
    """The mixed-precision optimizer type on the real library: fp16 gradients in, fp32
    master weights and fp16 parameters out, the loss scale growing (interval 4) and
    backing off (one injected inf) on the device; then GetState -> the checkpoint's JSON
    text -> decoded payload (float64 numbers) -> LoadState into a fresh optimizer -> the
    continuation equals the oracle's uninterrupted run bit for bit."""
    O, L = oracle, gm.lib
    dev = H.gmh_device_create()
    assert dev, HL.err(H)
    mm = H.gmh_mm_create(dev)
    shapes = [[33], [4097], [7, 9]]
    sizes = [33, 4097, 63]
    lr, b1, b2, eps, wd = 1e-3, 0.9, 0.999, 1e-8, 0.01
    cfg = [lr, b1, b2, eps, wd, 65536.0, 2.0, 0.5, 4]
    master = [O.fill_uniform(n, -0.05, 0.05, 21, 50 + k) for k, n in enumerate(sizes)]
    m = [np.zeros(n, np.float32) for n in sizes]
    v = [np.zeros(n, np.float32) for n in sizes]
    p16 = [O.f32_to_f16(w) for w in master]
    st = O.new_loss_scale(interval=4)

    def alloc16(arr):
        p = L.allocate_cuda_buffer(dev, arr.size * 2, 1)
        assert p, gm.last_error()
        gm.check(L.copy_data_to_cuda_buffer(p, arr.ctypes.data, arr.size * 2), "upload")
        return p

    wp = [alloc16(a) for a in p16]
    gp = [alloc16(np.zeros(n, np.uint16)) for n in sizes]

    def make():
        o = HL.make_optimizer(H, "MixedAdam", cfg, shapes, mm, dev)
        assert o, HL.err(H)
        assert H.gmh_optimizer_set_weight_buffers(o, HL.uarr(wp), 3) == 0
        return o

    rng = np.random.default_rng(5)

    def step(o, k, inject):
        scale = np.float32(st.scale)
        g16 = [O.f32_to_f16(rng.standard_normal(n, dtype=np.float32) * np.float32(1e-3) * scale) for n in sizes]
        if inject:
            g16[1][4000] = 0x7c00
        for p, g in zip(gp, g16):
            gm.check(L.copy_data_to_cuda_buffer(p, g.ctypes.data, g.size * 2), "upload")
        assert H.gmh_optimizer_step(o, HL.uarr(gp), 3, 0.0) == 0, HL.err(H)
        skipped = O.mixed_adam_step(g16, master, m, v, p16, lr, b1, b2, eps, wd, st)
        assert skipped == (1 if inject else 0)
        ls = HL.LossScaleC()
        assert H.gmh_mixed_loss_scale(o, C.byref(ls)) == 0, HL.err(H)
        assert (ls.scale, ls.good_steps, ls.adam_t, ls.skipped) == (st.scale, st.good_steps, st.adam_t, st.skipped), f"step {k}"

    def compare(o, what):
        for t, n in enumerate(sizes):
            got = np.empty(n, np.float32)
            assert H.gmh_mixed_read_master(o, t, got.ctypes.data, n) == 0, HL.err(H)
            assert np.array_equal(got.view(np.uint32), master[t].view(np.uint32)), f"{what}: master_{t}"
            h = np.empty(n, np.uint16)
            gm.check(L.gm_buffer_download(dev, wp[t], h.ctypes.data, n * 2), "download")
            assert np.array_equal(h, p16[t]), f"{what}: fp16 parameters {t}"

    opt = make()
    for t, w in enumerate(master):
        assert H.gmh_mixed_init_master(opt, t, w.ctypes.data, w.size) == 0, HL.err(H)
    for k in range(1, 7):
        step(opt, k, inject=(k == 3))
    compare(opt, "before the checkpoint")
    assert st.scale == 32768.0 and st.skipped == 1 and st.good_steps == 3    # halved at step 3; the 4th clean step comes after the resume

    got = H.gmh_optimizer_get_state(opt)
    assert got and H.gmh_state_num_tensors(got) == 9
    # through the checkpoint's JSON text and back: parameters return as float64, tensors keep their bits
    text = H.gmh_state_to_json(got)
    assert text, HL.err(H)
    saved = H.gmh_state_from_json(text)
    assert saved and H.gmh_state_num_tensors(saved) == 9, HL.err(H)
    val = C.c_double()
    assert H.gmh_state_get_param(saved, b"adam_step", C.byref(val)) == 0 and val.value == 5.0
    assert H.gmh_state_get_param(saved, b"loss_scale", C.byref(val)) == 0 and val.value == 32768.0
    H.gmh_state_destroy(got)
    H.gmh_optimizer_destroy(opt)

    opt2 = make()
    assert H.gmh_optimizer_load_state(opt2, saved) == 0, HL.err(H)
    assert H.gmh_optimizer_step_count(opt2) == 6
    for k in range(7, 12):
        step(opt2, k, inject=(k == 9))
    compare(opt2, "after the resume")
    H.gmh_state_destroy(saved)
    H.gmh_optimizer_destroy(opt2)
    for p in wp + gp:
        L.deallocate_cuda_buffer(p)
    H.gmh_mm_destroy(mm)
    H.gmh_device_destroy(dev)


def test_adam_with_state_in_a_flat_arena(gm, H, oracle):
    """The memory manager on one flat arena of the real library: the optimizer's moment
    buffers are carved from it (256-byte aligned, back to back), more of them than the
    reference's tier cap allows, and the steps still equal the oracle's."""
    global gm_dev
    O = oracle
    dev = H.gmh_device_create()
    gm_dev = dev
    mm = H.gmh_mm_create(dev)
    assert H.gmh_mm_use_arena(mm, 8 << 20) == 0, HL.err(H)
    nt = 130                                                   # 260 state buffers of the 1 KB tier: over its cap of 100
    shapes = [[200]] * nt
    sizes = [200] * nt
    w_cpu = [O.fill_uniform(200, -0.3, 0.3, 9, t) for t in range(nt)]
    m_cpu = [np.zeros(200, np.float32) for _ in range(nt)]
    v_cpu = [np.zeros(200, np.float32) for _ in range(nt)]
    wp = put(gm, w_cpu)
    gp = put(gm, [np.zeros(200, np.float32) for _ in range(nt)])
    opt = HL.make_optimizer(H, "Adam", [], shapes, mm, dev)
    assert opt, HL.err(H)
    assert H.gmh_optimizer_set_weight_buffers(opt, HL.uarr(wp), nt) == 0
    for k in range(1, 4):
        grads = [O.fill_normal(200, 0.0, 0.01, 9, 1000 * k + t) for t in range(nt)]
        for p, g in zip(gp, grads):
            gm.check(gm.lib.copy_float32_array_to_cuda_buffer(p, g.ctypes.data, g.size), "upload")
        assert H.gmh_optimizer_step(opt, HL.uarr(gp), nt, 0.0) == 0, HL.err(H)
        for t in range(nt):
            O.adam_step(w_cpu[t], grads[t], m_cpu[t], v_cpu[t], 1e-3, 0.9, 0.999, 1e-8, 0.0, k)
    for a, b in zip(get(gm, wp, sizes), w_cpu):
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    st = H.gmh_optimizer_get_state(opt)
    assert st and H.gmh_state_num_tensors(st) == 2 * nt
    buf = np.empty(200, np.float32)
    H.gmh_state_tensor_data(st, nt + 3, buf.ctypes.data)            # variance_3
    assert np.array_equal(buf.view(np.uint32), v_cpu[3].view(np.uint32))
    H.gmh_state_destroy(st)
    H.gmh_optimizer_destroy(opt)
    for p in wp + gp:
        gm.lib.deallocate_cuda_buffer(p)
    H.gmh_mm_destroy(mm)
    H.gmh_device_destroy(dev)


def test_synchronize_with_a_deadline(gm, dev):
    """gm_device_synchronize_timeout returns GM_ERR_TIMEOUT (-12) while the stream still has
    work and GM_OK once it has drained; nothing is cancelled by the timeout."""
    import ctypes as C
    L = gm.lib
    n = 1 << 26
    bufs = [dev.alloc(4 * n) for _ in range(4)]
    for p in bufs:
        gm.check(L.gm_buffer_zero(dev.h, p, 4 * n), "zero")
    lst = dev.tensor_list([[p] for p in bufs], [n])
    try:
        assert L.gm_device_synchronize_timeout(dev.h, 1000) == 0
        hy = gm.Hyper(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=1)
        for step in range(1, 201):                          # about 60 ms of queued work
            hy.step = step
            gm.check(L.gm_step_async(dev.h, gm.RULE_ADAM, lst, C.byref(hy)), "adam")
        assert L.gm_device_synchronize_timeout(dev.h, 0) == -12
        assert "did not drain" in gm.last_error()
        assert L.gm_device_synchronize_timeout(dev.h, 20000) == 0
        assert L.gm_device_synchronize_timeout(dev.h, -1) == -10
        assert L.gm_device_synchronize_timeout(0, 5) == -1
    finally:
        L.gm_tensor_list_destroy(lst)
        for p in bufs:
            dev.free(p)


def test_mixed_adam_gradient_clipping_through_host_mirror(gm, H, oracle):
    """SetGradClip on the MixedAdam optimizer type: the norm, the coefficient and the clipped
    update match the oracle bit for bit (the mirror's buffers are all 256-byte aligned, so
    every tensor's offset from a 16-byte boundary is 0)."""
    O, L = oracle, gm.lib
    dev = H.gmh_device_create()
    assert dev, HL.err(H)
    mm = H.gmh_mm_create(dev)
    shapes, sizes = [[9000], [130], [64, 33]], [9000, 130, 2112]
    lr, b1, b2, eps, wd = 1e-3, 0.9, 0.999, 1e-8, 0.0
    master = [O.fill_uniform(n, -0.05, 0.05, 23, 50 + k) for k, n in enumerate(sizes)]
    m = [np.zeros(n, np.float32) for n in sizes]
    v = [np.zeros(n, np.float32) for n in sizes]
    p16 = [O.f32_to_f16(w) for w in master]
    st = O.new_loss_scale(interval=2000)

    def alloc16(arr):
        p = L.allocate_cuda_buffer(dev, arr.size * 2, 1)
        assert p, gm.last_error()
        gm.check(L.copy_data_to_cuda_buffer(p, arr.ctypes.data, arr.size * 2), "upload")
        return p

    wp = [alloc16(a) for a in p16]
    gp = [alloc16(np.zeros(n, np.uint16)) for n in sizes]
    opt = HL.make_optimizer(H, "MixedAdam", [lr, b1, b2, eps, wd, 65536.0, 2.0, 0.5, 2000], shapes, mm, dev)
    assert opt, HL.err(H)
    try:
        assert H.gmh_optimizer_set_weight_buffers(opt, HL.uarr(wp), 3) == 0
        for t, w in enumerate(master):
            assert H.gmh_mixed_init_master(opt, t, w.ctypes.data, w.size) == 0, HL.err(H)
        assert H.gmh_mixed_set_clip(opt, 0.05) == 0, HL.err(H)
        assert H.gmh_mixed_set_clip(opt, -1.0) != 0
        rng = np.random.default_rng(6)
        for step in range(1, 6):
            g16 = [O.scale_to_f16((rng.standard_normal(n) * 1e-3).astype(np.float32), st.scale) for n in sizes]
            for p, g in zip(gp, g16):
                gm.check(L.copy_data_to_cuda_buffer(p, g.ctypes.data, g.size * 2), "upload")
            assert H.gmh_optimizer_step(opt, HL.uarr(gp), 3, 0.0) == 0, HL.err(H)
            skipped, ss, coef = O.mixed_adam_step_clipped(g16, master, m, v, p16, lr, b1, b2, eps, wd, 0.05, [0, 0, 0], 8192, st)
            got_ss, got_coef = C.c_float(), C.c_float()
            assert H.gmh_mixed_last_clip(opt, C.byref(got_ss), C.byref(got_coef)) == 0, HL.err(H)
            assert not skipped and 0 < coef < 1
            assert np.float32(got_ss.value).view(np.uint32) == ss.view(np.uint32), f"step {step}: {got_ss.value} vs {ss}"
            assert np.float32(got_coef.value).view(np.uint32) == coef.view(np.uint32), f"step {step}"
        for t, n in enumerate(sizes):
            got = np.empty(n, np.float32)
            assert H.gmh_mixed_read_master(opt, t, got.ctypes.data, n) == 0, HL.err(H)
            assert np.array_equal(got.view(np.uint32), master[t].view(np.uint32)), f"master_{t}"
    finally:
        H.gmh_optimizer_destroy(opt)
        for p in wp + gp:
            L.deallocate_cuda_buffer(p)
        H.gmh_mm_destroy(mm)
        H.gmh_device_destroy(dev)
