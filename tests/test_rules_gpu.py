"""GPU parity of the six elementwise rules against the CPU oracle, called
through the drop-in C entries (execute_*_step_cuda).

Tolerance: the required bound is 2 ulp per step and 1e-5 relative after 100
steps.  The kernels use the same IEEE operations in the same order as the
oracle, so the tests first demand bit equality and report the ulp distance if
that ever fails.
"""
import ctypes as C

import numpy as np
import pytest

import workloads as W

pytestmark = pytest.mark.gpu

MAX_ULP = 2
REL_TOL = 1e-5


class DeviceSet:
    """One device buffer per tensor, allocated through allocate_cuda_buffer."""

    def __init__(self, gm, dev, arrays):
        self.gm, self.dev = gm, dev
        self.n = [a.size for a in arrays]
        self.ptrs = []
        for a in arrays:
            p = gm.lib.allocate_cuda_buffer(dev.h, a.size * 4, 1)
            assert p, gm.last_error()
            gm.check(gm.lib.copy_float32_array_to_cuda_buffer(p, a.ctypes.data, a.size), "upload")
            self.ptrs.append(p)

    def upload(self, arrays):
        for p, a in zip(self.ptrs, arrays):
            self.gm.check(self.gm.lib.copy_float32_array_to_cuda_buffer(p, a.ctypes.data, a.size), "upload")

    def download(self):
        out = []
        for p, n in zip(self.ptrs, self.n):
            a = np.empty(n, dtype=np.float32)
            self.gm.check(self.gm.lib.copy_cuda_buffer_to_float32_array(p, a.ctypes.data, n), "download")
            out.append(a)
        return out

    def array(self):
        return self.gm.uarray(self.ptrs)

    def free(self):
        for p in self.ptrs:
            self.gm.lib.deallocate_cuda_buffer(p)


def zeros_like(ws):
    return [np.zeros_like(w) for w in ws]


def assert_close(name, step, got, want):
    for t, (a, b) in enumerate(zip(got, want)):
        if np.array_equal(a.view(np.uint32), b.view(np.uint32)):
            continue
        finite = np.isfinite(a) & np.isfinite(b)
        assert np.array_equal(np.isfinite(a), np.isfinite(b)), f"{name} step {step} tensor {t}: finiteness differs"
        ulp = W.ulp_distance(a[finite], b[finite])
        assert ulp.max() <= MAX_ULP, f"{name} step {step} tensor {t}: {ulp.max()} ulp apart (limit {MAX_ULP})"


def assert_rel(name, got, want):
    for t, (a, b) in enumerate(zip(got, want)):
        denom = np.maximum(np.abs(b), np.float32(1e-30))
        rel = np.abs(a.astype(np.float64) - b.astype(np.float64)) / denom
        # entries at zero are compared absolutely
        rel = np.where(np.abs(b) < 1e-30, np.abs(a), rel)
        assert rel.max() <= REL_TOL, f"{name} tensor {t}: relative error {rel.max():.3e} > {REL_TOL}"


def run_rule(gm, dev, O, name, shapes, fan_in, steps, heavy_tail, state_count, gpu_step, cpu_step):
    w_cpu = W.he_uniform_weights(O, shapes, fan_in)
    states_cpu = [zeros_like(w_cpu) for _ in range(state_count)]
    w_gpu = DeviceSet(gm, dev, w_cpu)
    g_gpu = DeviceSet(gm, dev, zeros_like(w_cpu))
    states_gpu = [DeviceSet(gm, dev, s) for s in states_cpu]
    sizes = gm.iarray([a.size * 4 for a in w_cpu])
    exact = True
    try:
        for step in range(1, steps + 1):
            grads = W.normal_grads(O, shapes, step, 0.01, heavy_tail)
            g_gpu.upload(grads)
            rc = gpu_step(w_gpu.array(), g_gpu.array(), [s.array() for s in states_gpu], len(shapes), sizes, step)
            assert rc == 0, f"{name} step {step}: code {rc}: {gm.last_error()}"
            for t in range(len(shapes)):
                cpu_step(w_cpu[t], grads[t], [s[t] for s in states_cpu], step)
            if step <= 3 or step % 10 == 0 or step == steps:
                got_w = w_gpu.download()
                assert_close(name + ".w", step, got_w, w_cpu)
                for k, s in enumerate(states_gpu):
                    assert_close(f"{name}.state{k}", step, s.download(), states_cpu[k])
                exact = exact and all(np.array_equal(a.view(np.uint32), b.view(np.uint32)) for a, b in zip(got_w, w_cpu))
        assert_rel(name + ".w", w_gpu.download(), w_cpu)
        for k, s in enumerate(states_gpu):
            assert_rel(f"{name}.state{k}", s.download(), states_cpu[k])
    finally:
        for s in [w_gpu, g_gpu] + states_gpu:
            s.free()
    return exact


def test_adam_mlp_100_steps(gm, dev, oracle):
    """fp32 Adam, lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, no decay, MLP 784-128-10, 100 steps."""
    O = oracle
    lr, b1, b2, eps, wd = 1e-3, 0.9, 0.999, 1e-8, 0.0

    def gpu(w, g, st, n, sizes, step):
        return gm.lib.execute_adam_step_cuda(dev.h, w, g, st[0], st[1], n, sizes, lr, b1, b2, eps, wd, step)

    def cpu(w, g, st, step):
        O.adam_step(w, g, st[0], st[1], lr, b1, b2, eps, wd, step)

    exact = run_rule(gm, dev, O, "adam", W.MLP_SHAPES, W.MLP_FAN_IN, 100, False, 2, gpu, cpu)
    assert exact, "Adam is expected to be bit-identical to the oracle"


CNN_CASES = {
    "sgd_momentum": 1, "sgd_nesterov": 1, "rmsprop": 1, "adagrad": 1, "adadelta": 2, "nadam": 2,
    "adam_decay": 2,
}


@pytest.mark.parametrize("case", list(CNN_CASES))
def test_cnn_rules_100_steps(gm, dev, oracle, case):
    """SGD-momentum, RMSProp, AdaGrad, AdaDelta, NAdam on the 8 CNN tensors with
    heavy-tailed gradients (1 % of entries x100), 100 steps.  Learning rates the
    configuration leaves open use the reference defaults (sgd.go:48-55 0.01,
    rmsprop.go:54-63 0.01, adagrad.go:42-48 0.01, nadam.go:47-55 0.002)."""
    O = oracle
    L = gm.lib

    if case in ("sgd_momentum", "sgd_nesterov"):
        nest = 1 if case == "sgd_nesterov" else 0
        wd = 1e-4 if nest else 0.0
        gpu = lambda w, g, st, n, sz, step: L.execute_sgd_step_cuda(dev.h, w, g, st[0], n, sz, 0.01, 0.9, wd, nest, step)
        cpu = lambda w, g, st, step: O.sgd_step(w, g, st[0], 0.01, 0.9, wd, nest)
    elif case == "rmsprop":
        gpu = lambda w, g, st, n, sz, step: L.execute_rmsprop_step_cuda(dev.h, w, g, st[0], None, None, n, sz, 0.01, 0.99, 1e-8, 0.0, 0.0, False, step)
        cpu = lambda w, g, st, step: O.rmsprop_step(w, g, st[0], None, None, 0.01, 0.99, 1e-8, 0.0, 0.0, False)
    elif case == "adagrad":
        gpu = lambda w, g, st, n, sz, step: L.execute_adagrad_step_cuda(dev.h, w, g, st[0], n, sz, 0.01, 1e-10, 0.0)
        cpu = lambda w, g, st, step: O.adagrad_step(w, g, st[0], 0.01, 1e-10, 0.0)
    elif case == "adadelta":
        gpu = lambda w, g, st, n, sz, step: L.execute_adadelta_step_cuda(dev.h, w, g, st[0], st[1], n, sz, 0.9, 1e-6, 0.0)
        cpu = lambda w, g, st, step: O.adadelta_step(w, g, st[0], st[1], 0.9, 1e-6, 0.0)
    elif case == "nadam":
        gpu = lambda w, g, st, n, sz, step: L.execute_nadam_step_cuda(dev.h, w, g, st[0], st[1], n, sz, 0.002, 0.9, 0.999, 1e-8, 0.0, step)
        cpu = lambda w, g, st, step: O.nadam_step(w, g, st[0], st[1], 0.002, 0.9, 0.999, 1e-8, 0.0, step)
    else:   # Adam with weight decay: exercises the decay branch
        gpu = lambda w, g, st, n, sz, step: L.execute_adam_step_cuda_pooled(dev.h, w, g, st[0], st[1], n, sz, 1e-3, 0.9, 0.999, 1e-8, 0.01, step, 0)
        cpu = lambda w, g, st, step: O.adam_step(w, g, st[0], st[1], 1e-3, 0.9, 0.999, 1e-8, 0.01, step)

    exact = run_rule(gm, dev, O, case, W.CNN_SHAPES, W.CNN_FAN_IN, 100, True, CNN_CASES[case], gpu, cpu)
    assert exact, f"{case} is expected to be bit-identical to the oracle"


@pytest.mark.parametrize("mode", ["plain", "momentum", "centered", "both"])
def test_rmsprop_modes(gm, dev, oracle, mode):
    """RMSProp with momentum and/or centering keeps its extra state between steps."""
    O = oracle
    mom = 0.9 if mode in ("momentum", "both") else 0.0
    cen = mode in ("centered", "both")
    shapes, fan = [(1000,), (37,), (4099,)], [10, 10, 10]
    nstate = 1 + (1 if mom > 0 else 0) + (1 if cen else 0)

    def gpu(w, g, st, n, sz, step):
        k = 1
        mb = gb = None
        if mom > 0:
            mb = st[k]; k += 1
        if cen:
            gb = st[k]
        return gm.lib.execute_rmsprop_step_cuda(dev.h, w, g, st[0], mb, gb, n, sz, 0.01, 0.99, 1e-8, 1e-3, mom, cen, step)

    def cpu(w, g, st, step):
        k = 1
        mb = gb = None
        if mom > 0:
            mb = st[k]; k += 1
        if cen:
            gb = st[k]
        O.rmsprop_step(w, g, st[0], mb, gb, 0.01, 0.99, 1e-8, 1e-3, mom, cen, True)

    assert run_rule(gm, dev, O, "rmsprop-" + mode, shapes, fan, 20, True, nstate, gpu, cpu)


def test_plain_sgd_and_small_sizes(gm, dev, oracle):
    """Vanilla SGD (no momentum buffers) on every size from 1 to 130 elements."""
    O = oracle
    shapes = [(n,) for n in range(1, 131)]
    fan = [4] * len(shapes)

    def gpu(w, g, st, n, sz, step):
        return gm.lib.execute_sgd_step_cuda(dev.h, w, g, None, n, sz, 0.05, 0.0, 0.0, 0, step)

    def cpu(w, g, st, step):
        O.sgd_step(w, g, None, 0.05, 0.0, 0.0, 0)

    assert run_rule(gm, dev, O, "sgd-plain", shapes, fan, 5, False, 0, gpu, cpu)


def test_misaligned_views_inside_an_arena(gm, dev, oracle):
    """Tensors packed back to back in flat arenas, so most start off a 16-byte
    boundary; one tensor's streams disagree on alignment and takes the scalar path."""
    O = oracle
    L = gm.lib
    sizes = [5, 1, 3, 4097, 8191, 2, 70001, 33, 16385]
    total = sum(sizes) + 16
    rng_w = O.fill_uniform(total, -1.0, 1.0, 7, 1)
    host = {k: np.zeros(total, dtype=np.float32) for k in "wgmv"}
    host["w"][:] = rng_w
    arena = L.gm_arena_create(dev.h, 4 * total * 4 + 4096)
    assert arena
    base = {k: L.gm_arena_alloc(arena, total * 4) for k in "wgmv"}
    assert all(base.values())
    offs = np.concatenate([[0], np.cumsum(sizes)[:-1]]).astype(np.int64) + 1      # +1: nothing starts aligned
    # the last tensor's v stream is shifted by one more element: inconsistent alignment
    shift = {k: [0] * len(sizes) for k in "wgmv"}
    shift["v"][-1] = 1
    ptrs = {k: [base[k] + 4 * (int(o) + shift[k][i]) for i, o in enumerate(offs)] for k in "wgmv"}
    lr, b1, b2, eps, wd = 1e-3, 0.9, 0.999, 1e-8, 0.0
    try:
        for step in range(1, 4):
            host["g"][:] = O.fill_normal(total, 0.0, 0.01, 7, 10 + step)
            for k in "wgmv":
                dev.upload(base[k], host[k])
            rc = L.execute_adam_step_cuda(dev.h, gm.uarray(ptrs["w"]), gm.uarray(ptrs["g"]), gm.uarray(ptrs["m"]),
                                          gm.uarray(ptrs["v"]), len(sizes), gm.iarray([4 * s for s in sizes]),
                                          lr, b1, b2, eps, wd, step)
            assert rc == 0, gm.last_error()
            want = {k: host[k].copy() for k in "wmv"}
            for i, (o, n) in enumerate(zip(offs, sizes)):
                sl = {k: slice(int(o) + shift[k][i], int(o) + shift[k][i] + n) for k in "wgmv"}
                w, m, v = (np.ascontiguousarray(want[k][sl[k]]) for k in "wmv")
                O.adam_step(w, np.ascontiguousarray(host["g"][sl["g"]]), m, v, lr, b1, b2, eps, wd, step)
                want["w"][sl["w"]], want["m"][sl["m"]], want["v"][sl["v"]] = w, m, v
            for k in "wmv":
                got = dev.to_host(base[k], total)
                # bytes between and around the tensors must be untouched
                assert np.array_equal(got.view(np.uint32), want[k].view(np.uint32)), f"stream {k} step {step}"
                host[k] = got
    finally:
        L.gm_arena_destroy(arena)


def test_equal_tensors_inside_an_arena(gm, dev, oracle):
    """Seven tensors of one size (12291 elements: three chunks and a ragged tail),
    each starting 3 elements before a 16-byte boundary, through the drop-in Adam
    entry with weight decay."""
    O, L = oracle, gm.lib
    nt, each = 7, 12291
    stride = each + 1                                   # keeps every start at 16k + 4 bytes
    assert (stride * 4) % 16 == 0
    total = nt * stride + 8
    offs = [1 + i * stride for i in range(nt)]
    host = {k: np.zeros(total, dtype=np.float32) for k in "wgmv"}
    host["w"][:] = O.fill_uniform(total, -1.0, 1.0, 9, 1)
    base = {k: dev.to_device(host[k]) for k in "wgmv"}
    ptrs = {k: [base[k] + 4 * o for o in offs] for k in "wgmv"}
    lr, b1, b2, eps, wd = 1e-3, 0.9, 0.999, 1e-8, 0.01

    def expect(step):
        want = {k: host[k].copy() for k in "wmv"}
        for o in offs:
            sl = slice(o, o + each)
            w, m, v = (np.ascontiguousarray(want[k][sl]) for k in "wmv")
            O.adam_step(w, np.ascontiguousarray(host["g"][sl]), m, v, lr, b1, b2, eps, wd, step)
            want["w"][sl], want["m"][sl], want["v"][sl] = w, m, v
        return want

    try:
        for step in range(1, 4):
            host["g"][:] = O.fill_normal(total, 0.0, 0.01, 9, 10 + step)
            dev.upload(base["g"], host["g"])
            rc = L.execute_adam_step_cuda(dev.h, gm.uarray(ptrs["w"]), gm.uarray(ptrs["g"]), gm.uarray(ptrs["m"]),
                                          gm.uarray(ptrs["v"]), nt, gm.iarray([4 * each] * nt), lr, b1, b2, eps, wd, step)
            assert rc == 0, gm.last_error()
            want = expect(step)
            for k in "wmv":
                got = dev.to_host(base[k], total)
                assert np.array_equal(got.view(np.uint32), want[k].view(np.uint32)), f"stream {k} step {step}"
                host[k] = got
    finally:
        for k in "wgmv":
            dev.free(base[k])


def test_error_codes(gm, dev):
    L = gm.lib
    p = L.allocate_cuda_buffer(dev.h, 64, 1)
    one = gm.uarray([p])
    sizes = gm.iarray([64])
    assert L.execute_adam_step_cuda(0, one, one, one, one, 1, sizes, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1) == -1
    nil = gm.uarray([0])
    assert L.execute_adam_step_cuda(dev.h, one, nil, one, one, 1, sizes, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1) == -4
    assert L.execute_adam_step_cuda(dev.h, one, one, one, one, 1, gm.iarray([128]), 1e-3, 0.9, 0.999, 1e-8, 0.0, 1) == -9
    assert L.execute_adam_step_cuda(dev.h, one, one, one, one, 1, gm.iarray([6]), 1e-3, 0.9, 0.999, 1e-8, 0.0, 1) == -9
    assert L.execute_rmsprop_step_cuda(dev.h, one, one, one, None, None, 1, sizes, 0.01, 0.99, 1e-8, 0.0, 0.9, False, 1) == -5
    assert L.execute_rmsprop_step_cuda(dev.h, one, one, one, None, None, 1, sizes, 0.01, 0.99, 1e-8, 0.0, 0.0, True, 1) == -6
    assert L.allocate_cuda_buffer(dev.h, 0, 1) == 0
    assert L.allocate_cuda_buffer(0, 64, 1) == 0
    # empty inputs: no tensors, a zero-byte tensor, an empty tensor list
    assert L.execute_adam_step_cuda(dev.h, one, one, one, one, 0, sizes, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1) == -10
    assert L.execute_adam_step_cuda(dev.h, one, one, one, one, 1, gm.iarray([0]), 1e-3, 0.9, 0.999, 1e-8, 0.0, 1) == -9
    assert L.execute_sgd_step_cuda(dev.h, one, one, None, 0, sizes, 0.01, 0.0, 0.0, 0, 1) == -10
    with pytest.raises(gm.GmError):
        dev.tensor_list([[], []], [])
    # Adam's step count starts at 1 (bias correction 1 - beta^0 would divide by zero)
    lst = dev.tensor_list([[p], [p], [p], [p]], [16])
    hy = gm.Hyper(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, step=0)
    assert L.gm_step_async(dev.h, gm.RULE_ADAM, lst, C.byref(hy)) == -10
    assert L.gm_step_async(dev.h, 17, lst, C.byref(hy)) == -10
    L.gm_tensor_list_destroy(lst)
    L.deallocate_cuda_buffer(p)


def test_convert_roundtrip(gm, dev, oracle):
    """fp32 -> fp16 is round-to-nearest-even, fp16 -> fp32 is exact (bridge_memory.m:362-376)."""
    O = oracle
    n = 100003
    exps = (np.arange(n) % 12 - 6).astype(np.float32)
    x = (O.fill_normal(n, 0.0, 1.0, 3, 3) * np.float32(10.0) ** exps).astype(np.float32)
    x[:8] = [0.0, -0.0, 65504.0, 65520.0, 1e-8, 6e-8, np.inf, -np.inf]
    src = dev.to_device(x)
    dst = dev.alloc(n * 2)
    back = dev.alloc(n * 4)
    shape = gm.iarray([n])
    gm.check(gm.lib.convert_tensor_type_cuda(src, dst, shape, 1, 0, 2, dev.h), "f32->f16")
    h = dev.to_host(dst, n, np.uint16)
    assert np.array_equal(h, O.f32_to_f16(x))
    gm.check(gm.lib.convert_tensor_type_cuda(dst, back, shape, 1, 2, 0, dev.h), "f16->f32")
    assert np.array_equal(dev.to_host(back, n).view(np.uint32), O.f16_to_f32(h).view(np.uint32))
    assert gm.lib.convert_tensor_type_cuda(src, dst, shape, 1, 0, 1, dev.h) == -11
    # buffers off the 16-byte boundary take the element-wise kernels; same results
    src1 = dev.to_device(np.concatenate([[np.float32(0)], x]))
    dst1 = dev.alloc((n + 8) * 2)
    back1 = dev.alloc((n + 8) * 4)
    gm.check(gm.lib.convert_tensor_type_cuda(src1 + 4, dst1 + 2, shape, 1, 0, 2, dev.h), "f32->f16 unaligned")
    assert np.array_equal(dev.to_host(dst1, n + 1, np.uint16)[1:], O.f32_to_f16(x))
    gm.check(gm.lib.convert_tensor_type_cuda(dst1 + 2, back1 + 4, shape, 1, 2, 0, dev.h), "f16->f32 unaligned")
    assert np.array_equal(dev.to_host(back1, n + 1)[1:].view(np.uint32), O.f16_to_f32(h).view(np.uint32))
    for n_small in (1, 7, 8, 9, 4096):                          # vector passes and the ragged tail
        gm.check(gm.lib.convert_tensor_type_cuda(src, dst, gm.iarray([n_small]), 1, 0, 2, dev.h), "small")
        assert np.array_equal(dev.to_host(dst, n_small, np.uint16), O.f32_to_f16(x[:n_small]))
    for p in (src1, dst1, back1):
        dev.free(p)
    tiny = dev.alloc(64)                                      # a destination that cannot hold the result is refused
    assert gm.lib.convert_tensor_type_cuda(src, tiny, shape, 1, 0, 2, dev.h) == -9
    assert gm.lib.convert_tensor_type_cuda(tiny, back, shape, 1, 2, 0, dev.h) == -9
    dev.free(tiny)
    for p in (src, dst, back):
        dev.free(p)


@pytest.mark.parametrize("sizes", [[5000, 12, 70001, 4096, 333], [12288] * 6], ids=["ragged", "equal"])
def test_host_buffer_step_matches_oracle(gm, dev, oracle, sizes):
    """gm_step_host: gradients come from (pinned) host memory and the new parameters
    return to host memory, pipelined over slices; the result equals the oracle's and
    the device copies agree with what was downloaded.  With equal tensors the slice
    boundaries fall on tensor boundaries (1, 3 slices) or inside tensors (5, 64)."""
    import ctypes as C
    O, L = oracle, gm.lib
    n = sum(sizes)
    offs = np.concatenate([[0], np.cumsum(sizes)[:-1]])
    w = O.fill_uniform(n, -0.2, 0.2, 61, 1)
    m, v = np.zeros(n, np.float32), np.zeros(n, np.float32)
    dw, dg, dm, dv = dev.to_device(w), dev.alloc(4 * n), dev.to_device(m), dev.to_device(v)
    ptrs = lambda base: [base + 4 * int(o) for o in offs]
    lst = dev.tensor_list([ptrs(dw), ptrs(dg), ptrs(dm), ptrs(dv)], sizes)
    hg = L.gm_host_alloc_pinned(4 * n)
    hw = L.gm_host_alloc_pinned(4 * n)
    assert hg and hw
    hg_arr = np.ctypeslib.as_array(C.cast(hg, C.POINTER(C.c_float)), shape=(n,))
    hw_arr = np.ctypeslib.as_array(C.cast(hw, C.POINTER(C.c_float)), shape=(n,))
    try:
        for step, slices in [(1, 1), (2, 3), (3, 5), (4, 64)]:
            g = O.fill_normal(n, 0.0, 0.01, 61, 10 + step)
            hg_arr[:] = g
            hy = gm.Hyper(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=step)
            gm.check(L.gm_step_host(dev.h, gm.RULE_ADAM, lst, C.byref(hy), hg, hw, slices), "gm_step_host")
            for o, k in zip(offs, sizes):
                sl = slice(int(o), int(o) + k)
                ws, ms, vs = (np.ascontiguousarray(x[sl]) for x in (w, m, v))
                O.adam_step(ws, np.ascontiguousarray(g[sl]), ms, vs, 1e-3, 0.9, 0.999, 1e-8, 0.0, step)
                w[sl], m[sl], v[sl] = ws, ms, vs
            assert np.array_equal(hw_arr.view(np.uint32), w.view(np.uint32)), f"step {step}: downloaded parameters"
            assert np.array_equal(dev.to_host(dw, n).view(np.uint32), w.view(np.uint32)), f"step {step}: device parameters"
        assert np.array_equal(dev.to_host(dv, n).view(np.uint32), v.view(np.uint32))
        # tensors that do not lie back to back on the device (here: a gap after the first) move one by one
        gap = dev.tensor_list([[dw, dw + 4 * 6000], [dg, dg + 4 * 6000], [dm, dm + 4 * 6000], [dv, dv + 4 * 6000]], [5000, 100])
        before = {k: dev.to_host(p, n) for k, p in (("w", dw), ("m", dm), ("v", dv))}
        g2 = O.fill_normal(5100, 0.0, 0.01, 61, 99)
        hg_arr[:5100] = g2
        hy = gm.Hyper(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, step=5)
        gm.check(L.gm_step_host(dev.h, gm.RULE_ADAM, gap, C.byref(hy), hg, hw, 2), "gm_step_host on separate tensors")
        for lo, cnt, src in ((0, 5000, 0), (6000, 100, 5000)):
            ws, ms, vs = (np.ascontiguousarray(before[k][lo:lo + cnt]) for k in "wmv")
            O.adam_step(ws, np.ascontiguousarray(g2[src:src + cnt]), ms, vs, 1e-3, 0.9, 0.999, 1e-8, 0.0, 5)
            assert np.array_equal(hw_arr[src:src + cnt].view(np.uint32), ws.view(np.uint32)), "downloaded parameters (separate tensors)"
            assert np.array_equal(dev.to_host(dw, n)[lo:lo + cnt].view(np.uint32), ws.view(np.uint32))
        assert np.array_equal(dev.to_host(dw, n)[5000:6000].view(np.uint32), before["w"][5000:6000].view(np.uint32)), "the gap was written"
        L.gm_tensor_list_destroy(gap)
    finally:
        L.gm_tensor_list_destroy(lst)
        L.gm_host_free_pinned(hg)
        L.gm_host_free_pinned(hw)
        for p in (dw, dg, dm, dv):
            dev.free(p)


FUZZ_RULES = ["sgd_plain", "sgd_momentum", "adam", "nadam", "rmsprop", "rmsprop_both", "adagrad", "adadelta"]


@pytest.mark.parametrize("seed", range(6))
def test_random_ragged_lists_every_rule(gm, dev, oracle, seed):
    """Seeded fuzz through the tensor-list entry: 1-12 tensors of 1-20,000 elements
    (sizes biased towards the chunk and vector boundaries), each stream of each tensor at
    its own random element offset inside one arena, so aligned, peelable and
    inconsistently aligned tensors all occur; every rule, three steps, bit-exact, and no
    byte outside the tensors may change."""
    O, L = oracle, gm.lib
    rng = np.random.default_rng(1000 + seed)
    special = [1, 2, 3, 4, 5, 7, 8, 255, 256, 257, 1023, 1024, 1025, 4095, 4096, 4097, 4099, 8191, 8192, 8193, 12289]
    for rule in FUZZ_RULES:
        nt = int(rng.integers(1, 13))
        sizes = [int(rng.choice(special)) if rng.random() < 0.5 else int(rng.integers(1, 20001)) for _ in range(nt)]
        ns = {"sgd_plain": 2, "sgd_momentum": 3, "adam": 4, "nadam": 4, "rmsprop": 3, "rmsprop_both": 5, "adagrad": 3,
              "adadelta": 4}[rule]
        same_alignment = rng.random() < 0.6                    # else every stream draws its own offset
        span = sum(sizes) + 8 * nt + 16
        host = [np.zeros(span, np.float32) for _ in range(ns)]
        offs = [[0] * nt for _ in range(ns)]
        at = 4
        for t, n in enumerate(sizes):
            base_shift = int(rng.integers(0, 4))
            for s in range(ns):
                offs[s][t] = at + (base_shift if same_alignment else int(rng.integers(0, 4)))
            at += n + 8
        host[0][:] = O.fill_uniform(span, -0.5, 0.5, 77 + seed, 1)
        canary = [h.copy() for h in host]
        bufs = [dev.to_device(h) for h in host]
        lst = dev.tensor_list([[bufs[s] + 4 * offs[s][t] for t in range(nt)] for s in range(ns)], sizes)
        wd = float(rng.choice([0.0, 0.01]))
        hy = {"sgd_plain": gm.Hyper(lr=0.05, beta1=0.0, weight_decay=wd),
              "sgd_momentum": gm.Hyper(lr=0.05, beta1=0.9, weight_decay=wd, nesterov=int(rng.integers(0, 2))),
              "adam": gm.Hyper(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=wd),
              "nadam": gm.Hyper(lr=2e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=wd),
              "rmsprop": gm.Hyper(lr=0.01, beta1=0.99, eps=1e-8, weight_decay=wd),
              "rmsprop_both": gm.Hyper(lr=0.01, beta1=0.99, eps=1e-8, weight_decay=wd, momentum=0.9, centered=1),
              "adagrad": gm.Hyper(lr=0.01, eps=1e-10, weight_decay=wd),
              "adadelta": gm.Hyper(beta1=0.9, eps=1e-6, weight_decay=wd)}[rule]
        rid = {"sgd_plain": gm.RULE_SGD, "sgd_momentum": gm.RULE_SGD, "adam": gm.RULE_ADAM, "nadam": gm.RULE_NADAM,
               "rmsprop": gm.RULE_RMSPROP, "rmsprop_both": gm.RULE_RMSPROP, "adagrad": gm.RULE_ADAGRAD,
               "adadelta": gm.RULE_ADADELTA}[rule]
        try:
            for step in (1, 2, 3):
                g_full = O.fill_normal(span, 0.0, 0.01, 77 + seed, 10 + step)
                for t, n in enumerate(sizes):
                    host[1][offs[1][t]:offs[1][t] + n] = g_full[offs[1][t]:offs[1][t] + n]
                dev.upload(bufs[1], host[1])
                hy.step = step
                gm.check(L.gm_step_async(dev.h, rid, lst, C.byref(hy)), rule)
                dev.sync()
                for t, n in enumerate(sizes):
                    x = [np.ascontiguousarray(host[s][offs[s][t]:offs[s][t] + n]) for s in range(ns)]
                    if rule == "sgd_plain":
                        O.sgd_step(x[0], x[1], None, hy.lr, 0.0, wd, 0)
                    elif rule == "sgd_momentum":
                        O.sgd_step(x[0], x[1], x[2], hy.lr, 0.9, wd, hy.nesterov)
                    elif rule == "adam":
                        O.adam_step(x[0], x[1], x[2], x[3], hy.lr, 0.9, 0.999, 1e-8, wd, step)
                    elif rule == "nadam":
                        O.nadam_step(x[0], x[1], x[2], x[3], hy.lr, 0.9, 0.999, 1e-8, wd, step)
                    elif rule == "rmsprop":
                        O.rmsprop_step(x[0], x[1], x[2], None, None, hy.lr, 0.99, 1e-8, wd, 0.0, False)
                    elif rule == "rmsprop_both":
                        O.rmsprop_step(x[0], x[1], x[2], x[3], x[4], hy.lr, 0.99, 1e-8, wd, 0.9, True, True)
                    elif rule == "adagrad":
                        O.adagrad_step(x[0], x[1], x[2], hy.lr, 1e-10, wd)
                    else:
                        O.adadelta_step(x[0], x[1], x[2], x[3], 0.9, 1e-6, wd)
                    for s in range(ns):
                        if s != 1:
                            host[s][offs[s][t]:offs[s][t] + n] = x[s]
                for s in range(ns):
                    got = dev.to_host(bufs[s], span)
                    assert np.array_equal(got.view(np.uint32), host[s].view(np.uint32)), (
                        f"seed {seed} {rule} step {step} stream {s}: sizes {sizes} offsets {offs[s]}")
            # bytes between the tensors still hold what they held at the start
            for s in range(ns):
                mask = np.ones(span, bool)
                for t, n in enumerate(sizes):
                    mask[offs[s][t]:offs[s][t] + n] = False
                assert np.array_equal(host[s][mask].view(np.uint32), canary[s][mask].view(np.uint32))
        finally:
            L.gm_tensor_list_destroy(lst)
            for b in bufs:
                dev.free(b)


@pytest.mark.parametrize("rule", FUZZ_RULES)
def test_untouched_parameters_stay_exact(gm, dev, oracle, rule):
    """Parameters a model never touches: gradient exactly zero (+0 and -0) and all state
    zero for 60 % of the elements, scattered and in whole 4,096-element runs.  The
    kernels take exact shortcuts for 0/b and sqrt(0) there; results, including the sign
    of every zero, must still equal the oracle's for three steps.  A few denormal, tiny
    and huge values ride along so the division's and square root's own slow paths run too."""
    O, L = oracle, gm.lib
    n = 3 * 4096 + 77
    rng = np.random.default_rng(42)
    ns = {"sgd_plain": 2, "sgd_momentum": 3, "adam": 4, "nadam": 4, "rmsprop": 3, "rmsprop_both": 5, "adagrad": 3,
          "adadelta": 4}[rule]
    dead = rng.random(n) < 0.4
    dead[4096:8192] = True
    host = [np.zeros(n, np.float32) for _ in range(ns)]
    host[0][:] = O.fill_uniform(n, -0.5, 0.5, 5, 1)
    host[0][::97] = 0.0                                      # some parameters are zero themselves
    host[0][7::101] = np.float32(-1e30)
    bufs = [dev.to_device(h) for h in host]
    lst = dev.tensor_list([[b] for b in bufs], [n])
    hy = {"sgd_plain": gm.Hyper(lr=0.05, beta1=0.0), "sgd_momentum": gm.Hyper(lr=0.05, beta1=0.9, nesterov=1),
          "adam": gm.Hyper(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8), "nadam": gm.Hyper(lr=2e-3, beta1=0.9, beta2=0.999, eps=1e-8),
          "rmsprop": gm.Hyper(lr=0.01, beta1=0.99, eps=1e-8),
          "rmsprop_both": gm.Hyper(lr=0.01, beta1=0.99, eps=1e-8, momentum=0.9, centered=1),
          "adagrad": gm.Hyper(lr=0.01, eps=1e-10), "adadelta": gm.Hyper(beta1=0.9, eps=1e-6)}[rule]
    rid = {"sgd_plain": gm.RULE_SGD, "sgd_momentum": gm.RULE_SGD, "adam": gm.RULE_ADAM, "nadam": gm.RULE_NADAM,
           "rmsprop": gm.RULE_RMSPROP, "rmsprop_both": gm.RULE_RMSPROP, "adagrad": gm.RULE_ADAGRAD,
           "adadelta": gm.RULE_ADADELTA}[rule]
    try:
        for step in (1, 2, 3):
            g = O.fill_normal(n, 0.0, 0.01, 5, 10 + step)
            g[dead] = 0.0
            g[dead & (np.arange(n) % 3 == 0)] = -0.0
            g[1::91] = np.float32(1e-42)                     # denormal, tiny and huge gradients: the
            g[2::89] = np.float32(1e-30)                     # intrinsics' own special-case paths
            g[4::83] = np.float32(1e18)
            host[1][:] = g
            dev.upload(bufs[1], host[1])
            hy.step = step
            gm.check(L.gm_step_async(dev.h, rid, lst, C.byref(hy)), rule)
            dev.sync()
            x = host
            if rule == "sgd_plain":
                O.sgd_step(x[0], x[1], None, hy.lr, 0.0, 0.0, 0)
            elif rule == "sgd_momentum":
                O.sgd_step(x[0], x[1], x[2], hy.lr, 0.9, 0.0, 1)
            elif rule == "adam":
                O.adam_step(x[0], x[1], x[2], x[3], hy.lr, 0.9, 0.999, 1e-8, 0.0, step)
            elif rule == "nadam":
                O.nadam_step(x[0], x[1], x[2], x[3], hy.lr, 0.9, 0.999, 1e-8, 0.0, step)
            elif rule == "rmsprop":
                O.rmsprop_step(x[0], x[1], x[2], None, None, hy.lr, 0.99, 1e-8, 0.0, 0.0, False)
            elif rule == "rmsprop_both":
                O.rmsprop_step(x[0], x[1], x[2], x[3], x[4], hy.lr, 0.99, 1e-8, 0.0, 0.9, True, True)
            elif rule == "adagrad":
                O.adagrad_step(x[0], x[1], x[2], hy.lr, 1e-10, 0.0)
            else:
                O.adadelta_step(x[0], x[1], x[2], x[3], 0.9, 1e-6, 0.0)
            for s in range(ns):
                got = dev.to_host(bufs[s], n)
                assert np.array_equal(got.view(np.uint32), host[s].view(np.uint32)), f"{rule} step {step} stream {s}"
    finally:
        L.gm_tensor_list_destroy(lst)
        for b in bufs:
            dev.free(b)
