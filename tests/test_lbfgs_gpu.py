"""GPU parity of the L-BFGS step (execute_lbfgs_step_cuda) against the CPU
oracle: iterates, history vectors, rho/alpha and therefore every curvature-pair
accept/skip decision must match bit for bit, in every mode.

The objective is f(x) = 1/2 x'Dx - b'x with diagonal D; the harness forms the
gradient g = D*x - b on the host from the device's own iterate (numpy float32,
one rounding per operation), so both sides see identical gradient bits.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def same_bits(a, b):
    """Bitwise equality, except that any NaN matches any NaN (payloads differ
    between x86 and the GPU)."""
    na, nb = np.isnan(a), np.isnan(b)
    if not np.array_equal(na, nb):
        return False
    return np.array_equal(a.view(np.uint32)[~na], b.view(np.uint32)[~nb])


class LbfgsProblem:
    def __init__(self, gm, dev, O, sizes, m, lo_exp, hi_exp, seed, shifts=None):
        self.gm, self.dev, self.O, self.sizes, self.m = gm, dev, O, sizes, m
        self.D = [O.fill_loguniform(n, lo_exp, hi_exp, seed, 1 + k) for k, n in enumerate(sizes)]
        self.b = [O.fill_normal(n, 0.0, 1.0, seed, 100 + k) for k, n in enumerate(sizes)]
        z = lambda: [np.zeros(n, dtype=np.float32) for n in sizes]
        # oracle side
        self.x, self.old_g, self.dir = z(), z(), z()
        self.s = [z() for _ in range(m)]
        self.y = [z() for _ in range(m)]
        self.rho = np.zeros(m, dtype=np.float32)
        self.alpha = np.zeros(m, dtype=np.float32)
        # device side
        # shifts: element offsets (cycled over the buffers as they are allocated) that move
        # buffers off their 16-byte boundary, so some tensors take the element-wise path
        self._bases = []
        self._count = 0

        def alloc(n):
            base = dev.to_device(np.zeros(n + 8, dtype=np.float32))
            self._bases.append(base)
            shift = shifts[self._count % len(shifts)] if shifts else 0
            self._count += 1
            return base + 4 * shift
        self.dx = [alloc(n) for n in sizes]
        self.dg = [alloc(n) for n in sizes]
        self.dold = [alloc(n) for n in sizes]
        self.ddir = [alloc(n) for n in sizes]
        self.ds = [[alloc(n) for n in sizes] for _ in range(m)]
        self.dy = [[alloc(n) for n in sizes] for _ in range(m)]
        self.drho = [alloc(1) for _ in range(m)]
        self.dalpha = alloc(m)
        self.hc = self.hi = 0

    def free(self):
        for p in self._bases:
            self.dev.free(p)

    def gradient(self, x):
        return [(D * xi - b).astype(np.float32) for D, xi, b in zip(self.D, x, self.b)]

    def step(self, mode, pooled=False):
        gm, L, O = self.gm, self.gm.lib, self.O
        nt, m = len(self.sizes), self.m
        g = self.gradient(self.x)
        for p, a in zip(self.dg, g):
            self.dev.upload(p, a)
        s_flat = [self.ds[k][t] for k in range(m) for t in range(nt)]       # [slot*nt + tensor]
        y_flat = [self.dy[k][t] for k in range(m) for t in range(nt)]
        step_out = C.c_float(-1.0)
        args = [self.dev.h, gm.uarray(self.dx), gm.uarray(self.dg), gm.uarray(self.dold), gm.uarray(self.ddir),
                gm.uarray(s_flat), gm.uarray(y_flat), gm.uarray(self.drho), self.dalpha, nt,
                gm.iarray([4 * n for n in self.sizes]), m, self.hc, self.hi, 1.0, 1e-4, 0.9, 20, 0.0, 0.0]
        if pooled:
            rc = L.execute_lbfgs_step_cuda_pooled(*args, 0, C.byref(step_out))
        else:
            rc = L.execute_lbfgs_step_cuda(*args, C.byref(step_out))
        assert rc == 0, gm.last_error()
        assert step_out.value == 1.0
        rc, step_cpu = O.lbfgs_step(self.x, g, self.old_g, self.dir, self.s, self.y, self.rho, self.alpha,
                                    m, self.hc, self.hi, 1.0, mode, 0)
        assert rc == 0 and step_cpu == 1.0
        # history bookkeeping of optimizer/lbfgs.go:287-290
        self.hi = (self.hi + 1) % m
        self.hc = min(self.hc + 1, m)

    def compare(self, it, full):
        dev = self.dev
        got_rho = np.array([dev.to_host(p, 1)[0] for p in self.drho], dtype=np.float32)
        assert same_bits(got_rho, self.rho), f"iteration {it}: rho {got_rho} vs {self.rho}"
        # accept/skip decisions are the zero pattern of rho
        assert np.array_equal(got_rho == 0, self.rho == 0), f"iteration {it}: skip decisions differ"
        got_alpha = dev.to_host(self.dalpha, self.m)
        assert same_bits(got_alpha, self.alpha), f"iteration {it}: alpha {got_alpha} vs {self.alpha}"
        for t, n in enumerate(self.sizes):
            assert same_bits(dev.to_host(self.dx[t], n), self.x[t]), f"iteration {it}: x[{t}] differs"
            assert same_bits(dev.to_host(self.ddir[t], n), self.dir[t]), f"iteration {it}: direction[{t}] differs"
            if full:
                assert same_bits(dev.to_host(self.dold[t], n), self.old_g[t]), f"iteration {it}: old_g[{t}]"
                for k in range(self.m):
                    assert same_bits(dev.to_host(self.ds[k][t], n), self.s[k][t]), f"iteration {it}: s[{k}][{t}]"
                    assert same_bits(dev.to_host(self.dy[k][t], n), self.y[k][t]), f"iteration {it}: y[{k}][{t}]"


@pytest.mark.parametrize("mode", [0, 1, 3])
def test_lbfgs_well_conditioned_50_iterations(gm, dev, oracle, mode):
    """D in [0.5, 2]: the corrected modes converge, so all 50 iterations carry
    finite iterates and real accept decisions; m=10."""
    gm.check(gm.lib.gm_lbfgs_set_mode(dev.h, mode), "mode")
    P = LbfgsProblem(gm, dev, oracle, [200_003], 10, -0.3, 0.3, seed=21)
    try:
        best = np.inf
        with np.errstate(all="ignore"):
            for it in range(50):
                P.step(mode, pooled=(it % 2 == 1))
                P.compare(it, full=(it in (0, 1, 11, 49)))
                if it == 20 and mode == 3:
                    assert (P.rho != 0).all(), "all pairs accepted once the history is full"
                gmax = float(np.abs(P.gradient(P.x)[0]).max())
                if np.isfinite(gmax):
                    best = min(best, gmax)
        if mode == 3:
            # There is no termination test in the reference (lbfgs.go:245-301): once the
            # gradient reaches rounding level the curvature pairs are noise and later
            # iterations may wander; convergence is therefore judged on the best iterate.
            assert best < 1e-5, f"mode 3 must reach the minimiser on this problem (best |g| = {best})"
        if mode == 0:
            assert (P.rho == 0).all(), "the reference's statement order rejects every pair"
    finally:
        P.free()
        gm.lib.gm_lbfgs_set_mode(dev.h, 3)


@pytest.mark.parametrize("mode", [0, 3])
def test_lbfgs_ill_conditioned_as_configured(gm, dev, oracle, mode):
    """D log-uniform in [1e-2, 1e2], unit step, no line search (the configured
    problem, scaled to 1 M variables): the iteration blows up after a few steps
    in every mode; iterates must still match until and including the overflow."""
    gm.check(gm.lib.gm_lbfgs_set_mode(dev.h, mode), "mode")
    P = LbfgsProblem(gm, dev, oracle, [1_000_000], 10, -2.0, 2.0, seed=22)
    try:
        with np.errstate(all="ignore"):
            for it in range(50):
                P.step(mode)
                P.compare(it, full=False)
    finally:
        P.free()
        gm.lib.gm_lbfgs_set_mode(dev.h, 3)


def test_lbfgs_multi_tensor_short_history(gm, dev, oracle):
    """Several tensors (sizes not multiples of 4, one smaller than a chunk) and a
    3-slot history, so the circular index wraps many times."""
    gm.check(gm.lib.gm_lbfgs_set_mode(dev.h, 3), "mode")
    P = LbfgsProblem(gm, dev, oracle, [4097, 1, 70_001, 12_288], 3, -0.2, 0.2, seed=23)
    try:
        for it in range(20):
            P.step(3)
            P.compare(it, full=True)
    finally:
        P.free()


@pytest.mark.parametrize("shifts", [[1], [0, 0, 0, 2, 0, 1, 0]], ids=["all_off_by_one", "columns_disagree"])
def test_lbfgs_unaligned_buffers(gm, dev, oracle, shifts):
    """Buffers that do not start on a 16-byte boundary (every one shifted by one element,
    or only some columns of some tensors): the passes fall back to element-wise access
    with the same summation order, so every value stays bit-identical."""
    gm.check(gm.lib.gm_lbfgs_set_mode(dev.h, 3), "mode")
    P = LbfgsProblem(gm, dev, oracle, [4097, 3, 20_001, 8192], 4, -0.2, 0.2, seed=25, shifts=shifts)
    try:
        for it in range(9):
            P.step(3)
            P.compare(it, full=True)
    finally:
        P.free()


def test_lbfgs_single_slot_history(gm, dev, oracle):
    """history_size 1: the slot written (s[hi]) is also the previous slot."""
    P = LbfgsProblem(gm, dev, oracle, [10_001], 1, -0.2, 0.2, seed=24)
    try:
        for it in range(6):
            P.step(3)
            P.compare(it, full=True)
    finally:
        P.free()


def test_canonical_dot(gm, dev, oracle):
    O, L = oracle, gm.lib
    for n in (1, 5, 4095, 4096, 4097, 1_000_003):
        a = O.fill_normal(n, 0, 1, 31, n)
        b = O.fill_normal(n, 0, 1, 32, n)
        pa, pb = dev.to_device(a), dev.to_device(b)
        out = C.c_float()
        gm.check(L.gm_dot_canonical(dev.h, pa, pb, n, C.byref(out)), "dot")
        assert np.float32(out.value).view(np.uint32) == O.dot_canonical(a, b).view(np.uint32), f"n={n}"
        # unaligned operands take the element-wise loads but the same order
        if n > 8:
            gm.check(L.gm_dot_canonical(dev.h, pa + 4, pb + 4, n - 1, C.byref(out)), "dot")
            want = O.dot_canonical(np.ascontiguousarray(a[1:]), np.ascontiguousarray(b[1:]))
            assert np.float32(out.value).view(np.uint32) == want.view(np.uint32), f"unaligned n={n}"
        dev.free(pa)
        dev.free(pb)


def test_lbfgs_refuses_short_buffers(gm, dev):
    """A buffer the library allocated that is shorter than buffer_sizes says is refused
    before any kernel runs (a vector, a history slot, alpha)."""
    L = gm.lib
    n, m = 5000, 2
    big = lambda: dev.alloc(4 * n)
    x, g, old, d = big(), big(), big(), big()
    S, Y = [big() for _ in range(m)], [big() for _ in range(m)]
    RHO = [dev.alloc(4) for _ in range(m)]
    alpha, short = dev.alloc(4 * m), dev.alloc(4 * 100)
    step = C.c_float()

    def call(xx=x, ss=None, aa=alpha):
        return L.execute_lbfgs_step_cuda(dev.h, gm.uarray([xx]), gm.uarray([g]), gm.uarray([old]), gm.uarray([d]),
                                         gm.uarray(ss or S), gm.uarray(Y), gm.uarray(RHO), aa, 1, gm.iarray([4 * n]), m, 0, 0,
                                         1.0, 1e-4, 0.9, 20, 0.0, 0.0, C.byref(step))
    assert call() == 0, gm.last_error()
    assert call(xx=short) == -9 and "L-BFGS vector" in gm.last_error()
    assert call(ss=[S[0], short]) == -9 and "L-BFGS history" in gm.last_error()
    assert call(aa=dev.alloc(4)) == -9 and "L-BFGS alpha" in gm.last_error()
    assert call() == 0
    for p in [x, g, old, d, alpha, short] + S + Y + RHO:
        dev.free(p)


def test_lbfgs_argument_errors(gm, dev):
    L = gm.lib
    p = dev.alloc(64)
    one = gm.uarray([p])
    sz = gm.iarray([64])
    out = C.c_float()
    ok = [dev.h, one, one, one, one, one, one, one, p, 1, sz, 1, 0, 0, 1.0, 1e-4, 0.9, 20, 0.0, 0.0]
    bad_dev = list(ok); bad_dev[0] = 0
    assert L.execute_lbfgs_step_cuda(*bad_dev, C.byref(out)) == -1
    bad_count = list(ok); bad_count[12] = 2              # history_count > history_size
    assert L.execute_lbfgs_step_cuda(*bad_count, C.byref(out)) == -10
    nil = list(ok); nil[2] = gm.uarray([0])
    assert L.execute_lbfgs_step_cuda(*nil, C.byref(out)) == -4
    assert L.gm_lbfgs_set_mode(dev.h, 7) == -10
    dev.free(p)
