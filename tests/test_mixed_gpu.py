"""GPU parity of mixed-precision Adam (fp16 gradients, fp32 master weights,
device-resident dynamic loss scale) against the CPU oracle.

Bit-exact requirements: the loss-scale trajectory, the skip decisions, the
Adam step counter, master/m/v, and p16 == half_rn(master).
"""
import ctypes as C

import numpy as np
import pytest

import workloads as W

pytestmark = pytest.mark.gpu

LR, B1, B2, EPS, WD = 1e-3, 0.9, 0.999, 1e-8, 0.0


class PackedArenas:
    """Five flat arenas (g16, master, m, v, p16) with the tensors packed back to
    back, so tensor starts are generally not 16-byte aligned."""

    def __init__(self, gm, dev, sizes, lead=1):
        self.gm, self.dev, self.sizes = gm, dev, sizes
        self.offs = (np.concatenate([[0], np.cumsum(sizes)[:-1]]) + lead).astype(np.int64)
        self.total = int(sum(sizes)) + lead + 16
        L = gm.lib
        self.arena = L.gm_arena_create(dev.h, self.total * (2 + 4 + 4 + 4 + 2) + 5 * 256)
        assert self.arena, gm.last_error()
        self.eb = {"g": 2, "w": 4, "m": 4, "v": 4, "p": 2}
        self.base = {k: L.gm_arena_alloc(self.arena, self.total * self.eb[k]) for k in "gwmvp"}
        assert all(self.base.values()), gm.last_error()
        self.ptrs = {k: [self.base[k] + self.eb[k] * int(o) for o in self.offs] for k in "gwmvp"}
        self.list = dev.tensor_list([self.ptrs[k] for k in "gwmvp"], sizes, [2, 4, 4, 4, 2])

    def put(self, key, arrays):
        dt = np.uint16 if self.eb[key] == 2 else np.float32
        flat = np.zeros(self.total, dtype=dt)
        for o, a in zip(self.offs, arrays):
            flat[int(o):int(o) + a.size] = a
        self.dev.upload(self.base[key], flat)

    def get(self, key):
        dt = np.uint16 if self.eb[key] == 2 else np.float32
        flat = self.dev.to_host(self.base[key], self.total, dt)
        return [flat[int(o):int(o) + n].copy() for o, n in zip(self.offs, self.sizes)], flat

    def close(self):
        self.gm.lib.gm_tensor_list_destroy(self.list)
        self.gm.lib.gm_arena_destroy(self.arena)


def same_state(a, b):
    fields = ["scale", "growth", "backoff", "max_scale", "interval", "good_steps", "adam_t", "skipped", "last_overflow"]
    return all(getattr(a, f) == getattr(b, f) for f in fields)


def run_mixed(gm, dev, O, sizes, steps, interval, p_inject, check_every, seed=11, with_norm=False):
    L = gm.lib
    rng = np.random.default_rng(seed)
    master = [O.fill_uniform(n, -0.05, 0.05, seed, 50 + k) for k, n in enumerate(sizes)]
    m = [np.zeros(n, dtype=np.float32) for n in sizes]
    v = [np.zeros(n, dtype=np.float32) for n in sizes]
    p16 = [O.f32_to_f16(w) for w in master]
    st = O.new_loss_scale(interval=interval)
    A = PackedArenas(gm, dev, sizes)
    init = gm.LossScale(scale=st.scale, growth=st.growth, backoff=st.backoff, max_scale=st.max_scale,
                        interval=st.interval, good_steps=0, adam_t=0, skipped=0, last_overflow=0)
    mx = L.gm_mixed_create(dev.h, C.byref(init), B1, B2, 64)     # short table: exercises growth of the table
    assert mx, gm.last_error()
    if with_norm:
        gm.check(L.gm_mixed_enable_grad_norm(mx, 1), "enable grad norm")
    skips = 0
    scales = set()
    try:
        for key, arrs in (("w", master), ("m", m), ("v", v), ("p", p16)):
            A.put(key, arrs)
        for step in range(1, steps + 1):
            scale = np.float32(st.scale)
            g16 = []
            for n in sizes:
                z = rng.standard_normal(n, dtype=np.float32)
                g16.append(O.f32_to_f16(z * np.float32(1e-3) * scale))
            if rng.random() < p_inject:
                t = int(rng.integers(len(sizes)))
                e = int(rng.integers(sizes[t]))
                g16[t][e] = [0x7c00, 0xfc00, 0x7e00][int(rng.integers(3))]     # +inf, -inf or NaN
            A.put("g", g16)
            gm.check(L.gm_mixed_step_async(dev.h, mx, A.list, LR, EPS, WD), "mixed step")
            if with_norm:
                # the overflow-check pass also leaves sum((g16/scale)^2); float atomics, so relative
                got_ss = C.c_float()
                gm.check(L.gm_mixed_last_grad_sumsq(dev.h, mx, C.byref(got_ss)), "grad sumsq")
                want_ss = sum(O.sumsq_f16(g, 1.0 / float(scale)) for g in g16)
                if np.isfinite(want_ss):
                    assert abs(got_ss.value - want_ss) <= 1e-5 * want_ss, f"step {step}: {got_ss.value} vs {want_ss}"
                else:
                    assert not np.isfinite(got_ss.value), f"step {step}: overflow step must give a non-finite norm"
            skipped = O.mixed_adam_step(g16, master, m, v, p16, LR, B1, B2, EPS, WD, st)
            skips += skipped
            scales.add(float(st.scale))
            got = gm.LossScale()
            gm.check(L.gm_mixed_get_state(dev.h, mx, C.byref(got)), "get state")
            assert same_state(got, st), (
                f"step {step}: device scale={got.scale} good={got.good_steps} t={got.adam_t} skipped={got.skipped} "
                f"vs oracle scale={st.scale} good={st.good_steps} t={st.adam_t} skipped={st.skipped}")
            if step % check_every == 0 or step == steps or skipped:
                for key, want in (("w", master), ("m", m), ("v", v)):
                    got_list, _ = A.get(key)
                    for t, (a, b) in enumerate(zip(got_list, want)):
                        assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), f"step {step} {key}[{t}] differs"
                got_p, _ = A.get("p")
                got_w, _ = A.get("w")
                for t, (a, b) in enumerate(zip(got_p, p16)):
                    assert np.array_equal(a, b), f"step {step} p16[{t}] differs from the oracle"
                    assert np.array_equal(a, O.f32_to_f16(got_w[t])), f"step {step} p16[{t}] != half_rn(master)"
        # canaries: bytes between tensors were never written
        _, flat_m = A.get("m")
        mask = np.ones(A.total, dtype=bool)
        for o, n in zip(A.offs, sizes):
            mask[int(o):int(o) + n] = False
        assert not flat_m[mask].any(), "bytes outside the tensors were modified"
    finally:
        L.gm_mixed_destroy(mx)
        A.close()
    return skips, scales, st


def test_mixed_adam_ragged_500_steps(gm, dev, oracle):
    """48 ragged tensors (scaled-down sizes, same structure as the 25 M-parameter
    configuration), 500 steps, growth interval 100 and 2 % injected overflows so
    that growth, back-off and skipped steps all occur many times."""
    sizes = W.ragged_sizes(48, 393_217, 1024, 65536)
    skips, scales, st = run_mixed(gm, dev, oracle, sizes, 500, 100, 0.02, 50)
    assert skips >= 3, "the run must contain skipped steps"
    # the same run with the gradient norm taken in the check pass: nothing else may change
    skips_n, scales_n, st_n = run_mixed(gm, dev, oracle, sizes, 120, 100, 0.02, 40, with_norm=True)
    assert skips_n >= 1 and st_n.adam_t == 120 - skips_n
    assert len(scales) >= 3, "the scale must both grow and back off"
    assert st.adam_t == 500 - skips


def test_mixed_adam_reference_schedule(gm, dev, oracle):
    """Growth after 2000 clean steps and a 0.1 % injection rate, as configured in
    training/model_trainer.go:258-270; small tensors so 2100 steps stay cheap."""
    sizes = [1, 7, 9, 130, 4097, 33]
    skips, scales, st = run_mixed(gm, dev, oracle, sizes, 2100, 2000, 0.001, 300, seed=5)
    assert 131072.0 in scales or skips > 0


@pytest.mark.parametrize("case", ["inf_first", "nan_last", "neg_inf_middle"])
def test_overflow_anywhere_skips_everything(gm, dev, oracle, case):
    """One non-finite half anywhere (first element, last element of the last
    tensor, middle) must skip the whole step and leave every buffer untouched."""
    O, L = oracle, gm.lib
    sizes = [3, 2049, 70001, 5]
    A = PackedArenas(gm, dev, sizes)
    mx = L.gm_mixed_create(dev.h, None, B1, B2, 0)
    try:
        master = [O.fill_uniform(n, -1, 1, 3, k) for k, n in enumerate(sizes)]
        zeros = [np.zeros(n, dtype=np.float32) for n in sizes]
        p16 = [O.f32_to_f16(w) for w in master]
        for key, arrs in (("w", master), ("m", zeros), ("v", zeros), ("p", p16)):
            A.put(key, arrs)
        g16 = [O.f32_to_f16(O.fill_normal(n, 0, 1.0, 3, 10 + k)) for k, n in enumerate(sizes)]
        if case == "inf_first":
            g16[0][0] = 0x7c00
        elif case == "nan_last":
            g16[-1][-1] = 0x7fff
        else:
            g16[2][35000] = 0xfc00
        A.put("g", g16)
        before = {k: A.get(k)[1] for k in "wmvp"}
        gm.check(L.gm_mixed_step_async(dev.h, mx, A.list, LR, EPS, WD), "step")
        st = gm.LossScale()
        gm.check(L.gm_mixed_get_state(dev.h, mx, C.byref(st)), "state")
        assert (st.scale, st.good_steps, st.adam_t, st.skipped, st.last_overflow) == (32768.0, 0, 0, 1, 1)
        for k in "wmvp":
            assert np.array_equal(A.get(k)[1], before[k]), f"stream {k} changed on a skipped step"
        # the next clean step proceeds with the halved scale and t = 1
        g16 = [O.f32_to_f16(O.fill_normal(n, 0, 1.0, 3, 20 + k)) for k, n in enumerate(sizes)]
        A.put("g", g16)
        gm.check(L.gm_mixed_step_async(dev.h, mx, A.list, LR, EPS, WD), "step")
        gm.check(L.gm_mixed_get_state(dev.h, mx, C.byref(st)), "state")
        assert (st.scale, st.good_steps, st.adam_t, st.skipped, st.last_overflow) == (32768.0, 1, 1, 1, 0)
    finally:
        L.gm_mixed_destroy(mx)
        A.close()


def test_grad_norm_needs_enabling(gm, dev):
    L = gm.lib
    mx = L.gm_mixed_create(dev.h, None, B1, B2, 0)
    out = C.c_float()
    assert L.gm_mixed_last_grad_sumsq(dev.h, mx, C.byref(out)) == -10
    assert L.gm_mixed_enable_grad_norm(mx, 1) == 0
    assert L.gm_mixed_enable_grad_norm(0, 1) == -10
    L.gm_mixed_destroy(mx)


def test_mixed_state_set_get(gm, dev):
    L = gm.lib
    mx = L.gm_mixed_create(dev.h, None, B1, B2, 0)
    try:
        st = gm.LossScale()
        gm.check(L.gm_mixed_get_state(dev.h, mx, C.byref(st)), "get")
        assert (st.scale, st.growth, st.backoff, st.interval) == (65536.0, 2.0, 0.5, 2000)
        st.scale, st.good_steps, st.adam_t = 1024.0, 17, 40000
        gm.check(L.gm_mixed_set_state(dev.h, mx, C.byref(st)), "set")
        back = gm.LossScale()
        gm.check(L.gm_mixed_get_state(dev.h, mx, C.byref(back)), "get")
        assert (back.scale, back.good_steps, back.adam_t) == (1024.0, 17, 40000)
        bad = gm.LossScale(scale=-1.0, growth=2.0, backoff=0.5, max_scale=1.0, interval=1)
        assert L.gm_mixed_create(dev.h, C.byref(bad), B1, B2, 0) == 0
    finally:
        L.gm_mixed_destroy(mx)


def test_grad_sumsq(gm, dev, oracle):
    """Sum of squares of fp32 and of unscaled fp16 gradients; float atomics make
    the order free, so the check is relative (1e-5) against a double sum."""
    O, L = oracle, gm.lib
    sizes = [5, 4097, 100003]
    out = dev.alloc(256)
    try:
        g32 = [O.fill_normal(n, 0, 0.01, 9, k) for k, n in enumerate(sizes)]
        ptrs = [dev.to_device(g) for g in g32]
        lst = dev.tensor_list([ptrs], sizes, [4])
        gm.check(L.gm_grad_sumsq_async(dev.h, lst, 4, 1.0, out), "sumsq f32")
        got = float(dev.to_host(out, 1)[0])
        want = sum(O.sumsq_f32(g) for g in g32)
        assert abs(got - want) <= 1e-5 * want
        L.gm_tensor_list_destroy(lst)
        for p in ptrs:
            dev.free(p)
        g16 = [O.f32_to_f16(g * np.float32(65536.0)) for g in g32]
        ptrs = [dev.to_device(g) for g in g16]
        lst = dev.tensor_list([ptrs], sizes, [2])
        gm.check(L.gm_grad_sumsq_async(dev.h, lst, 2, 1.0 / 65536.0, out), "sumsq f16")
        got = float(dev.to_host(out, 1)[0])
        want = sum(O.sumsq_f16(g, 1.0 / 65536.0) for g in g16)
        assert abs(got - want) <= 1e-5 * want
        L.gm_tensor_list_destroy(lst)
        for p in ptrs:
            dev.free(p)
    finally:
        dev.free(out)


@pytest.mark.parametrize("seed", range(4))
def test_random_alignments_mixed(gm, dev, oracle, seed):
    """Seeded fuzz of the mixed-precision step: 1-10 tensors of 1-40,000 elements, each
    of the five streams of each tensor at a random element offset (shared by the streams
    of a tensor in 60 % of the lists, independent otherwise, which forces the
    element-wise path); four steps with an overflow injected in one of them; state,
    master weights, moments and fp16 parameters bit-exact, nothing written outside."""
    O, L = oracle, gm.lib
    rng = np.random.default_rng(500 + seed)
    special = [1, 7, 8, 9, 2047, 2048, 2049, 8191, 8192, 8193, 16385]
    nt = int(rng.integers(1, 11))
    sizes = [int(rng.choice(special)) if rng.random() < 0.5 else int(rng.integers(1, 40001)) for _ in range(nt)]
    keys, eb = "gwmvp", {"g": 2, "w": 4, "m": 4, "v": 4, "p": 2}
    dt = {k: (np.uint16 if eb[k] == 2 else np.float32) for k in keys}
    span = sum(sizes) + 16 * nt + 32
    shared = rng.random() < 0.6
    offs = {k: [0] * nt for k in keys}
    at = 8
    for t, n in enumerate(sizes):
        base = int(rng.integers(0, 8))
        for k in keys:
            offs[k][t] = at + (base if shared else int(rng.integers(0, 8)))
        at += n + 16
    host = {k: np.zeros(span, dt[k]) for k in keys}
    master = [O.fill_uniform(n, -0.05, 0.05, 31 + seed, 50 + t) for t, n in enumerate(sizes)]
    m = [np.zeros(n, np.float32) for n in sizes]
    v = [np.zeros(n, np.float32) for n in sizes]
    p16 = [O.f32_to_f16(w) for w in master]
    host["w"][:] = 3.0                                       # canary values between the tensors
    host["p"][:] = 0x1234
    for t, n in enumerate(sizes):
        host["w"][offs["w"][t]:offs["w"][t] + n] = master[t]
        host["p"][offs["p"][t]:offs["p"][t] + n] = p16[t]
    bufs = {k: dev.to_device(host[k]) for k in keys}
    lst = dev.tensor_list([[bufs[k] + eb[k] * offs[k][t] for t in range(nt)] for k in keys], sizes, [eb[k] for k in keys])
    st = O.new_loss_scale(interval=2)
    init = gm.LossScale(scale=st.scale, growth=st.growth, backoff=st.backoff, max_scale=st.max_scale,
                        interval=st.interval, good_steps=0, adam_t=0, skipped=0, last_overflow=0)
    mx = L.gm_mixed_create(dev.h, C.byref(init), B1, B2, 0)
    bad_step = int(rng.integers(1, 5))
    try:
        for step in range(1, 5):
            scale = np.float32(st.scale)
            g16 = [O.f32_to_f16(rng.standard_normal(n, dtype=np.float32) * np.float32(1e-3) * scale) for n in sizes]
            for a in g16:                                    # signed zeros, the smallest denormal half, the largest half
                a[::7] = 0x0000
                a[::13] = 0x8000
                a[3::17] = 0x0001
                a[5::19] = 0x7bff
            if step == bad_step:
                t = int(rng.integers(nt))
                g16[t][int(rng.integers(sizes[t]))] = 0x7e00
            for t, n in enumerate(sizes):
                host["g"][offs["g"][t]:offs["g"][t] + n] = g16[t]
            dev.upload(bufs["g"], host["g"])
            gm.check(L.gm_mixed_step_async(dev.h, mx, lst, LR, EPS, WD), "mixed step")
            skipped = O.mixed_adam_step(g16, master, m, v, p16, LR, B1, B2, EPS, WD, st)
            assert skipped == (1 if step == bad_step else 0)
            got = gm.LossScale()
            gm.check(L.gm_mixed_get_state(dev.h, mx, C.byref(got)), "state")
            assert same_state(got, st), f"seed {seed} step {step}"
            for k, arrs in (("w", master), ("m", m), ("v", v), ("p", p16)):
                for t, n in enumerate(sizes):
                    host[k][offs[k][t]:offs[k][t] + n] = arrs[t]
                dev_now = dev.to_host(bufs[k], span, dt[k])
                assert np.array_equal(dev_now.view(np.uint8), host[k].view(np.uint8)), (
                    f"seed {seed} step {step} stream {k}: sizes {sizes} offsets {offs[k]} shared={shared}")
    finally:
        L.gm_mixed_destroy(mx)
        L.gm_tensor_list_destroy(lst)
        for k in keys:
            dev.free(bufs[k])


def test_fp32_streams_on_16_but_not_32_byte_boundaries(gm, dev, oracle):
    """fp16 streams on a 16-byte boundary and fp32 streams 16 bytes past a 32-byte one:
    every stream is vector-aligned with no peel, yet the 256-bit accesses of the update
    kernel would be misaligned, so those tensors must take its 128-bit path.  One tensor
    in the usual packing (all streams at one element offset) rides along."""
    O, L = oracle, gm.lib
    sizes = [20_000, 8192 + 24, 3000]
    keys, eb = "gwmvp", {"g": 2, "w": 4, "m": 4, "v": 4, "p": 2}
    dt = {k: (np.uint16 if eb[k] == 2 else np.float32) for k in keys}
    span = sum(sizes) + 64 * len(sizes) + 64
    offs = {k: [] for k in keys}
    at = 16
    for t, n in enumerate(sizes):
        for k in keys:
            skew = 4 if (eb[k] == 4 and t < 2) else 0          # fp32 streams of tensors 0 and 1: +16 bytes
            offs[k].append(at + skew)
        at += (n + 63) // 16 * 16 + 16
    master = [O.fill_uniform(n, -0.05, 0.05, 71, 50 + t) for t, n in enumerate(sizes)]
    m = [np.zeros(n, np.float32) for n in sizes]
    v = [np.zeros(n, np.float32) for n in sizes]
    p16 = [O.f32_to_f16(w) for w in master]
    host = {k: np.zeros(span, dt[k]) for k in keys}
    for t, n in enumerate(sizes):
        host["w"][offs["w"][t]:offs["w"][t] + n] = master[t]
        host["p"][offs["p"][t]:offs["p"][t] + n] = p16[t]
    bufs = {k: dev.to_device(host[k]) for k in keys}
    for t in range(2):
        assert (bufs["g"] + 2 * offs["g"][t]) % 16 == 0 and (bufs["w"] + 4 * offs["w"][t]) % 32 == 16
    lst = dev.tensor_list([[bufs[k] + eb[k] * offs[k][t] for t in range(len(sizes))] for k in keys], sizes, [eb[k] for k in keys])
    st = O.new_loss_scale(interval=2000)
    mx = L.gm_mixed_create(dev.h, None, B1, B2, 0)
    rng = np.random.default_rng(3)
    try:
        for step in range(1, 4):
            g16 = [O.f32_to_f16(rng.standard_normal(n, dtype=np.float32) * np.float32(1e-3) * np.float32(st.scale)) for n in sizes]
            for t, n in enumerate(sizes):
                host["g"][offs["g"][t]:offs["g"][t] + n] = g16[t]
            dev.upload(bufs["g"], host["g"])
            gm.check(L.gm_mixed_step_async(dev.h, mx, lst, LR, EPS, WD), "mixed step")
            assert O.mixed_adam_step(g16, master, m, v, p16, LR, B1, B2, EPS, WD, st) == 0
            for k, arrs in (("w", master), ("m", m), ("v", v), ("p", p16)):
                for t, n in enumerate(sizes):
                    host[k][offs[k][t]:offs[k][t] + n] = arrs[t]
                got = dev.to_host(bufs[k], span, dt[k])
                assert np.array_equal(got.view(np.uint8), host[k].view(np.uint8)), f"step {step} stream {k}"
    finally:
        L.gm_mixed_destroy(mx)
        L.gm_tensor_list_destroy(lst)
        for k in keys:
            dev.free(bufs[k])


def test_resume_at_a_late_step_with_slow_betas(gm, dev, oracle):
    """A state created (or restored) at a step count far beyond the initial table, with
    betas whose corrections are still below 1 there: the bias corrections of the next
    steps must be those of that step count, not of the table's last entry."""
    O, L = oracle, gm.lib
    sizes = [4099, 33]
    b1, b2, t0 = 0.9999, 0.9999, 100_000
    for how in ("create", "set_state"):
        A = PackedArenas(gm, dev, sizes)
        st = O.new_loss_scale(adam_t=t0)
        init = gm.LossScale(scale=st.scale, growth=st.growth, backoff=st.backoff, max_scale=st.max_scale,
                            interval=st.interval, good_steps=0, adam_t=t0 if how == "create" else 0, skipped=0, last_overflow=0)
        mx = L.gm_mixed_create(dev.h, C.byref(init), b1, b2, 64)
        assert mx, gm.last_error()
        try:
            if how == "set_state":
                init.adam_t = t0
                gm.check(L.gm_mixed_set_state(dev.h, mx, C.byref(init)), "set state")
            master = [O.fill_uniform(n, -0.05, 0.05, 17, k) for k, n in enumerate(sizes)]
            m = [O.fill_normal(n, 0, 1e-3, 17, 10 + k) for k, n in enumerate(sizes)]
            v = [np.abs(O.fill_normal(n, 0, 1e-6, 17, 20 + k)) for k, n in enumerate(sizes)]
            p16 = [O.f32_to_f16(w) for w in master]
            for key, arrs in (("w", master), ("m", m), ("v", v), ("p", p16)):
                A.put(key, arrs)
            for step in range(3):
                g16 = [O.f32_to_f16(O.fill_normal(n, 0, 1e-3, 17, 100 * step + k) * np.float32(st.scale)) for k, n in enumerate(sizes)]
                A.put("g", g16)
                gm.check(L.gm_mixed_step_async(dev.h, mx, A.list, LR, EPS, WD), "step")
                O.mixed_adam_step(g16, master, m, v, p16, LR, b1, b2, EPS, WD, st)
            got = gm.LossScale()
            gm.check(L.gm_mixed_get_state(dev.h, mx, C.byref(got)), "state")
            assert same_state(got, st) and st.adam_t == t0 + 3
            bc = O.adam_scalars(b1, b2, t0 + 1)
            assert bc[0] < 1.0 and bc[1] < 1.0, "the case must sit where the corrections still matter"
            for key, want in (("w", master), ("m", m), ("v", v)):
                got_list, _ = A.get(key)
                for t, (a, b) in enumerate(zip(got_list, want)):
                    assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), f"{how}: {key}[{t}] differs"
        finally:
            L.gm_mixed_destroy(mx)
            A.close()


def test_set_state_validates_like_create(gm, dev):
    L = gm.lib
    mx = L.gm_mixed_create(dev.h, None, B1, B2, 0)
    try:
        ok = gm.LossScale(scale=1024.0, growth=2.0, backoff=0.5, max_scale=65536.0, interval=10, good_steps=0, adam_t=0,
                          skipped=0, last_overflow=0)
        assert L.gm_mixed_set_state(dev.h, mx, C.byref(ok)) == 0
        for field, value in (("max_scale", 0.0), ("growth", 0.5), ("backoff", 0.0), ("backoff", 1.5), ("scale", -1.0),
                             ("interval", 0), ("adam_t", -1), ("scale", float("inf"))):
            bad = gm.LossScale(scale=1024.0, growth=2.0, backoff=0.5, max_scale=65536.0, interval=10, good_steps=0,
                               adam_t=0, skipped=0, last_overflow=0)
            setattr(bad, field, value)
            assert L.gm_mixed_set_state(dev.h, mx, C.byref(bad)) == -10, field
            assert "invalid loss-scale state" in gm.last_error()
        assert L.gm_mixed_create(dev.h, C.byref(gm.LossScale(scale=1.0, growth=2.0, backoff=0.5, max_scale=0.5, interval=1)), B1, B2, 0) == 0
    finally:
        L.gm_mixed_destroy(mx)
