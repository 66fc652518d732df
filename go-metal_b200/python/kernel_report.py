#!/usr/bin/env python
"""Per-kernel throughput report for libgometal_cuda.so (CUDA-event timed).

    python go-metal_b200/python/kernel_report.py --case rules|mixed|lbfgs|small [--reps N] [--small]

Prints one JSON line per measured kernel: time per step, algorithmic GB/s
(bytes per parameter x parameters / time) and Gparams/s.  Inputs are seeded
and synthetic and larger than the 126 MB L2.  `--small` shrinks the problem
for profiler captures (nothing here is timed under a profiler).

  rules  every fp32 rule on 2^28 parameters in 64 tensors (2^26 with --small)
  mixed  mixed-precision Adam on 25,165,824 parameters in 48 ragged tensors
         packed back to back (tensor starts off the 16-byte boundary)
  lbfgs  L-BFGS, history 10, n = 10,000,000, once the history is full
  small  the two small models (MLP 101,770 parameters in 4 tensors, CNN 545,098 in
         8): latency of one step through the synchronous drop-in entry (host wall
         clock) and through the asynchronous entry (CUDA events, back to back)
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import gometal_cuda as gm  # noqa: E402

L = gm.lib


def emit(**kw):
    print(json.dumps(kw))
    sys.stdout.flush()


def timed(dev, fn, reps, warm=3):
    for _ in range(warm):
        fn()
    dev.sync()
    ms = C.c_float()
    gm.check(L.gm_timer_start(dev.h), "timer")
    for _ in range(reps):
        fn()
    gm.check(L.gm_timer_stop(dev.h, C.byref(ms)), "timer")
    return ms.value / reps


def fill(dev, ptr, n, scale, seed):
    pat = (np.random.default_rng(seed).standard_normal(1 << 22) * scale).astype(np.float32)
    for off in range(0, n, pat.size):
        k = min(pat.size, n - off)
        gm.check(L.gm_buffer_upload(dev.h, ptr + 4 * off, pat.ctypes.data, 4 * k), "upload")


def case_rules(dev, reps, small):
    n = 1 << (26 if small else 28)
    nt = 64
    per = n // nt
    names = ["w", "g", "s1", "s2", "s3"]
    buf = {k: dev.alloc(4 * n) for k in names}
    for k in names:
        gm.check(L.gm_buffer_zero(dev.h, buf[k], 4 * n), "zero")
    fill(dev, buf["w"], n, 0.05, 1)
    fill(dev, buf["g"], n, 0.01, 2)
    ptrs = {k: [buf[k] + 4 * per * t for t in range(nt)] for k in names}
    rules = [
        ("adam", gm.RULE_ADAM, ["w", "g", "s1", "s2"], 28, dict(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8)),
        ("nadam", gm.RULE_NADAM, ["w", "g", "s1", "s2"], 28, dict(lr=2e-3, beta1=0.9, beta2=0.999, eps=1e-8)),
        ("adadelta", gm.RULE_ADADELTA, ["w", "g", "s1", "s2"], 28, dict(beta1=0.9, eps=1e-6)),
        ("sgd_momentum", gm.RULE_SGD, ["w", "g", "s1"], 20, dict(lr=0.01, beta1=0.9)),
        ("rmsprop", gm.RULE_RMSPROP, ["w", "g", "s1"], 20, dict(lr=0.01, beta1=0.99, eps=1e-8)),
        ("adagrad", gm.RULE_ADAGRAD, ["w", "g", "s1"], 20, dict(lr=0.01, eps=1e-10)),
        ("sgd_plain", gm.RULE_SGD, ["w", "g"], 12, dict(lr=0.01, beta1=0.0)),
    ]
    for name, rule, streams, bpp, hp in rules:
        # fresh parameters and zero state for every rule: one rule's state is not a
        # valid state of the next (a negative first moment is no squared average)
        fill(dev, buf["w"], n, 0.05, 1)
        for k in ("s1", "s2", "s3"):
            gm.check(L.gm_buffer_zero(dev.h, buf[k], 4 * n), "zero")
        lst = dev.tensor_list([ptrs[k] for k in streams], [per] * nt)
        hy = gm.Hyper(step=1, **hp)
        state = {"t": 0}

        def one():
            state["t"] += 1
            hy.step = state["t"]
            gm.check(L.gm_step_async(dev.h, rule, lst, C.byref(hy)), name)

        ms = timed(dev, one, reps)
        emit(kernel=f"mta_apply_kernel<{name}>", params=n, ms=ms, bytes_per_param=bpp,
             gbs=bpp * n / ms / 1e6, gparams_s=n / ms / 1e6)
        L.gm_tensor_list_destroy(lst)
    for k in names:
        dev.free(buf[k])


def ragged_sizes(count, total, lo, hi, seed=0x5EED601D):
    rng = np.random.default_rng(seed)
    raw = np.exp(rng.uniform(np.log(lo), np.log(hi), size=count))
    sizes = np.maximum(lo, np.floor(raw * (total / raw.sum()))).astype(np.int64)
    sizes[sizes % 8 == 0] += 1
    sizes[int(np.argmax(sizes))] += int(total - sizes.sum())
    return [int(s) for s in sizes]


def case_mixed(dev, reps, small, scale_up=1, norm=False):
    # scale_up > 1: the same 48-tensor shape with every tensor that many times larger,
    # to separate the kernels' own rate from the ramp and tail of a 0.7 GB pass
    total_params = 25_165_824 * scale_up // (4 if small else 1)
    sizes = ragged_sizes(48, total_params, 4096 * scale_up, 4_194_304 * scale_up // (4 if small else 1))
    n = sum(sizes)
    total = n + 32
    eb = {"g": 2, "w": 4, "m": 4, "v": 4, "p": 2}
    base = {k: dev.alloc(total * eb[k]) for k in "gwmvp"}
    for k in "gwmvp":
        gm.check(L.gm_buffer_zero(dev.h, base[k], total * eb[k]), "zero")
    block = (np.random.default_rng(1).standard_normal(min(total, 1 << 25)).astype(np.float32) * 65.536).astype(np.float16)
    for lo in range(0, total, block.size):                       # one 32 Mi block repeated
        k = min(block.size, total - lo)
        gm.check(L.gm_buffer_upload(dev.h, base["g"] + 2 * lo, block.ctypes.data, 2 * k), "upload")
    offs = np.concatenate([[0], np.cumsum(sizes)[:-1]]).astype(np.int64) + 1
    ptrs = {k: [base[k] + eb[k] * int(o) for o in offs] for k in "gwmvp"}
    lst = dev.tensor_list([ptrs[k] for k in "gwmvp"], sizes, [2, 4, 4, 4, 2])
    mx = L.gm_mixed_create(dev.h, None, 0.9, 0.999, 0)
    if norm:                                                     # gradient norm taken by the overflow-check pass
        gm.check(L.gm_mixed_enable_grad_norm(mx, 1), "enable norm")
    ms = timed(dev, lambda: gm.check(L.gm_mixed_step_async(dev.h, mx, lst, 1e-3, 1e-8, 0.0), "mixed"), reps)
    st = gm.LossScale()
    gm.check(L.gm_mixed_get_state(dev.h, mx, C.byref(st)), "state")
    emit(kernel="mixed_check_kernel" + ("<norm>" if norm else "") + "+mixed_update_kernel", params=n, ms=ms, bytes_per_param=30,
         gbs=30 * n / ms / 1e6, gparams_s=n / ms / 1e6, scale=st.scale, adam_t=st.adam_t, skipped=st.skipped)
    L.gm_mixed_destroy(mx)
    L.gm_tensor_list_destroy(lst)
    for k in "gwmvp":
        dev.free(base[k])


def case_lbfgs(dev, reps, small):
    n = int(os.environ.get("GM_REPORT_LBFGS_ELEMENTS", 10_000_000 // (4 if small else 1)))
    m = 10
    z = lambda k: dev.to_device(np.zeros(k, np.float32)) if k < 4096 else _zeros(dev, k)
    x, g, old, d = (z(n) for _ in range(4))
    S = [z(n) for _ in range(m)]
    Y = [z(n) for _ in range(m)]
    RHO = [z(64) for _ in range(m)]
    ALPHA = z(64)
    rng = np.random.default_rng(2)
    D = (10 ** rng.uniform(-0.3, 0.3, n)).astype(np.float32)
    b = rng.standard_normal(n).astype(np.float32)
    xs = np.zeros(n, np.float32)
    hc = hi = 0
    walls = []
    for it in range(m + max(reps, 3)):
        dev.upload(g, (D * xs - b).astype(np.float32))
        step = C.c_float()
        dev.sync()
        t0 = time.perf_counter()
        rc = L.execute_lbfgs_step_cuda(dev.h, gm.uarray([x]), gm.uarray([g]), gm.uarray([old]), gm.uarray([d]), gm.uarray(S),
                                       gm.uarray(Y), gm.uarray(RHO), ALPHA, 1, gm.iarray([4 * n]), m, hc, hi, 1.0, 1e-4, 0.9,
                                       20, 0.0, 0.0, C.byref(step))
        dt = time.perf_counter() - t0
        gm.check(rc, "lbfgs")
        if hc == m:
            walls.append(dt * 1e3)
        hi, hc = (hi + 1) % m, min(hc + 1, m)
        xs = dev.to_host(x, n)
    ms = float(np.median(walls))
    bpe = 44 + 32 * m
    emit(kernel="lbfgs_axpy_dot_kernel x 21 + lbfgs_pass_kernel (one synchronous step)", elements=n, history=m, ms=ms,
         bytes_per_element=bpe, gbs=bpe * n / ms / 1e6, note="host wall clock around the synchronous drop-in entry")


def case_small(dev, reps, small):
    models = {"mlp_4_tensors": [100352, 128, 1280, 10],
              "cnn_8_tensors": [864, 32, 18432, 64, 524288, 128, 1280, 10]}
    for name, sizes in models.items():
        n = sum(sizes)
        bufs = {k: [_zeros(dev, s) for s in sizes] for k in "wgmv"}
        for p, s in zip(bufs["g"], sizes):
            dev.upload(p, (np.random.default_rng(s).standard_normal(s) * 0.01).astype(np.float32))
        arr = {k: gm.uarray(bufs[k]) for k in "wgmv"}
        sz = gm.iarray([4 * s for s in sizes])
        step = [0]

        def dropin():
            step[0] += 1
            gm.check(L.execute_adam_step_cuda(dev.h, arr["w"], arr["g"], arr["m"], arr["v"], len(sizes), sz,
                                              1e-3, 0.9, 0.999, 1e-8, 0.0, step[0]), "adam")

        for _ in range(10):
            dropin()
        t0 = time.perf_counter()
        for _ in range(max(reps, 200)):
            dropin()
        wall_us = (time.perf_counter() - t0) / max(reps, 200) * 1e6
        lst = dev.tensor_list([bufs[k] for k in "wgmv"], sizes)
        hy = gm.Hyper(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, step=1)

        def async_step():
            step[0] += 1
            hy.step = step[0]
            gm.check(L.gm_step_async(dev.h, gm.RULE_ADAM, lst, C.byref(hy)), "adam")

        ms = timed(dev, async_step, max(reps, 200), warm=10)
        emit(kernel=f"mta_apply_kernel<adam> {name}", params=n, dropin_sync_us_per_step=wall_us,
             async_us_per_step=ms * 1e3, bytes_per_step=28 * n,
             note="L2-resident and launch-bound; a bandwidth fraction is not meaningful at this size")
        L.gm_tensor_list_destroy(lst)
        for k in "wgmv":
            for p in bufs[k]:
                dev.free(p)


def case_sizes(dev, reps, small):
    """fp32 Adam on 16 equal tensors from 2^21 to 2^28 elements in all (2^24 at most with --small)."""
    rng = np.random.default_rng(1)
    block = 1 << 22
    fill = {"w": rng.uniform(-0.05, 0.05, block).astype(np.float32), "g": (rng.standard_normal(block) * 0.01).astype(np.float32),
            "m": (rng.standard_normal(block) * 0.001).astype(np.float32), "v": rng.uniform(1e-6, 1e-4, block).astype(np.float32)}
    for lg in range(21, (24 if small else 28) + 1):
        n, nt = 1 << lg, 16
        per = n // nt
        bufs = {k: dev.alloc(4 * n) for k in "wgmv"}
        for k in "wgmv":
            for lo in range(0, n, block):
                gm.check(L.gm_buffer_upload(dev.h, bufs[k] + 4 * lo, fill[k].ctypes.data, 4 * min(block, n - lo)), "upload")
        lst = dev.tensor_list([[bufs[k] + 4 * per * t for t in range(nt)] for k in "wgmv"], [per] * nt)
        hy = gm.Hyper(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, step=1)
        ms = timed(dev, lambda: gm.check(L.gm_step_async(dev.h, gm.RULE_ADAM, lst, C.byref(hy)), "adam"), reps)
        emit(kernel="mta_apply_kernel<adam>", elements=n, us=ms * 1e3, gbs=28 * n / ms / 1e6,
             chunks=L.gm_tensor_list_num_chunks(lst))
        L.gm_tensor_list_destroy(lst)
        for k in "wgmv":
            dev.free(bufs[k])


def case_convert(dev, reps, small):
    """Standalone fp32 <-> fp16 conversion (the drop-in convert_tensor_type entry, synchronous), 6 B/element."""
    n = 25_165_824 // (4 if small else 1)
    src = dev.to_device((np.random.default_rng(4).standard_normal(n) * 3).astype(np.float32))
    half, back = dev.alloc(2 * n), dev.alloc(4 * n)
    shape = gm.iarray([n])
    for name, a, b, st, dt_ in (("f32->f16", src, half, 0, 2), ("f16->f32", half, back, 2, 0)):
        walls = []
        for _ in range(max(reps, 5)):
            dev.sync()
            t0 = time.perf_counter()
            gm.check(L.convert_tensor_type_cuda(a, b, shape, 1, st, dt_, dev.h), "convert")
            walls.append((time.perf_counter() - t0) * 1e3)
        ms = float(np.median(walls))
        emit(kernel="convert " + name, elements=n, ms=ms, gbs=6 * n / ms / 1e6, note="host wall clock around the synchronous entry")
    for p in (src, half, back):
        dev.free(p)


def case_sumsq(dev, reps, small):
    """Stand-alone gradient sum of squares: 2^28 fp32 elements (4 B each) and 2^28 fp16 elements (2 B each)."""
    n, nt = (1 << 28) // (16 if small else 1), 16
    per = n // nt
    out = dev.alloc(256)
    for eb, name in ((4, "fp32"), (2, "fp16")):
        buf = dev.alloc(eb * n)
        fill(dev, buf, n * eb // 4, 0.01, 7)                     # any finite bit pattern will do for a timing
        if eb == 2:
            gm.check(L.gm_buffer_zero(dev.h, buf, eb * n), "zero")   # halves: zeros (an fp32 pattern may read as inf/NaN halves)
        lst = dev.tensor_list([[buf + eb * per * t for t in range(nt)]], [per] * nt, [eb])
        ms = timed(dev, lambda: gm.check(L.gm_grad_sumsq_async(dev.h, lst, eb, 1.0, out), "sumsq"), reps)
        emit(kernel=f"sumsq_kernel<{name}>", elements=n, ms=ms, gbs=eb * n / ms / 1e6)
        L.gm_tensor_list_destroy(lst)
        dev.free(buf)
    dev.free(out)


def _zeros(dev, k):
    p = dev.alloc(4 * k)
    gm.check(L.gm_buffer_zero(dev.h, p, 4 * k), "zero")
    return p


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", choices=["rules", "mixed", "mixed_norm", "mixed_x16", "lbfgs", "small", "sizes", "convert", "sumsq"], required=True)
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--small", action="store_true")
    args = ap.parse_args()
    dev = gm.Device(0)
    try:
        cases = {"sizes": case_sizes, "convert": case_convert, "sumsq": case_sumsq, "rules": case_rules, "mixed": case_mixed, "lbfgs": case_lbfgs, "small": case_small,
                 "mixed_x16": lambda d, r, sm: case_mixed(d, r, sm, scale_up=16),
                 "mixed_norm": lambda d, r, sm: case_mixed(d, r, sm, norm=True)}
        cases[args.case](dev, args.reps, args.small)
    finally:
        dev.close()


if __name__ == "__main__":
    main()
