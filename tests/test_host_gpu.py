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
