"""Generates tests/golden/optimizer_steps.npz from the CPU oracle.

    python tests/golden/make_golden.py

The reference (go-metal) cannot run here -- its update rules execute inside
Apple's MPSGraph -- and its own tests hold no numeric result of an optimizer
step, so these vectors pin the oracle's *current* behaviour (and, through the
GPU tests, the CUDA kernels' behaviour) rather than the reference's output.
Inputs come from the oracle's seeded generators; every case is small.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402

SEED = 0x601D
N = 301          # not a multiple of 4: vector body, head and tail all occur
STEPS = 3


def grads(step, n=N):
    g = O.fill_normal(n, 0.0, 0.01, SEED, 10 + step)
    return O.scale_subset(g, 10, 100.0, SEED, 50 + step)


def main():
    out = {}
    w0 = O.fill_uniform(N, -0.3, 0.3, SEED, 1)
    out["w0"] = w0
    for s in range(1, STEPS + 1):
        out[f"g{s}"] = grads(s)
    z = lambda: np.zeros(N, np.float32)

    # Adam (with and without decay), NAdam
    for name, wd in (("adam", 0.0), ("adam_wd", 0.01)):
        w, m, v = w0.copy(), z(), z()
        for s in range(1, STEPS + 1):
            O.adam_step(w, out[f"g{s}"], m, v, 1e-3, 0.9, 0.999, 1e-8, wd, s)
        out[name + "_w"], out[name + "_m"], out[name + "_v"] = w, m, v
    w, m, v = w0.copy(), z(), z()
    for s in range(1, STEPS + 1):
        O.nadam_step(w, out[f"g{s}"], m, v, 0.002, 0.9, 0.999, 1e-8, 0.0, s)
    out["nadam_w"], out["nadam_m"], out["nadam_v"] = w, m, v

    # SGD: plain, momentum, Nesterov + decay
    w = w0.copy()
    for s in range(1, STEPS + 1):
        O.sgd_step(w, out[f"g{s}"], None, 0.01, 0.0, 0.0, 0)
    out["sgd_plain_w"] = w
    for name, nest, wd in (("sgd_mom", 0, 0.0), ("sgd_nesterov", 1, 1e-4)):
        w, mom = w0.copy(), z()
        for s in range(1, STEPS + 1):
            O.sgd_step(w, out[f"g{s}"], mom, 0.01, 0.9, wd, nest)
        out[name + "_w"], out[name + "_mom"] = w, mom

    # RMSProp: plain and centered+momentum
    w, sq = w0.copy(), z()
    for s in range(1, STEPS + 1):
        O.rmsprop_step(w, out[f"g{s}"], sq, None, None, 0.01, 0.99, 1e-8, 0.0, 0.0, False)
    out["rmsprop_w"], out["rmsprop_sq"] = w, sq
    w, sq, mom, ga = w0.copy(), z(), z(), z()
    for s in range(1, STEPS + 1):
        O.rmsprop_step(w, out[f"g{s}"], sq, mom, ga, 0.01, 0.99, 1e-8, 1e-3, 0.9, True, True)
    out["rmsprop_cm_w"], out["rmsprop_cm_sq"], out["rmsprop_cm_mom"], out["rmsprop_cm_gavg"] = w, sq, mom, ga

    # AdaGrad, AdaDelta
    w, sq = w0.copy(), z()
    for s in range(1, STEPS + 1):
        O.adagrad_step(w, out[f"g{s}"], sq, 0.01, 1e-10, 0.0)
    out["adagrad_w"], out["adagrad_sq"] = w, sq
    w, sq, up = w0.copy(), z(), z()
    for s in range(1, STEPS + 1):
        O.adadelta_step(w, out[f"g{s}"], sq, up, 0.9, 1e-6, 0.0)
    out["adadelta_w"], out["adadelta_sq"], out["adadelta_upd"] = w, sq, up

    # host scalars
    out["adam_scalars"] = np.array([O.adam_scalars(0.9, 0.999, t) for t in range(1, 21)], np.float32)
    out["nadam_mu"] = np.array([O.nadam_mu_next(0.9, t) for t in range(1, 21)], np.float32)

    # mixed precision: 2 tensors, 6 steps, growth every 2 clean steps, +inf injected at step 3
    sizes = [257, 64]
    master = [O.fill_uniform(n, -0.05, 0.05, SEED, 70 + k) for k, n in enumerate(sizes)]
    mm = [np.zeros(n, np.float32) for n in sizes]
    vv = [np.zeros(n, np.float32) for n in sizes]
    p16 = [O.f32_to_f16(a) for a in master]
    st = O.new_loss_scale(interval=2)
    traj = []
    for k in range(len(sizes)):
        out[f"mixed_master0_{k}"] = master[k].copy()
    for s in range(1, 7):
        g16 = [O.f32_to_f16(O.fill_normal(n, 0.0, 1e-3, SEED, 80 + 10 * s + k) * np.float32(st.scale))
               for k, n in enumerate(sizes)]
        if s == 3:
            g16[1][5] = 0x7c00
        for k in range(len(sizes)):
            out[f"mixed_g16_{s}_{k}"] = g16[k]
        O.mixed_adam_step(g16, master, mm, vv, p16, 1e-3, 0.9, 0.999, 1e-8, 0.0, st)
        traj.append([st.scale, st.good_steps, st.adam_t, st.skipped, st.last_overflow])
    out["mixed_traj"] = np.array(traj, np.float64)
    for k in range(len(sizes)):
        out[f"mixed_master_{k}"], out[f"mixed_m_{k}"], out[f"mixed_v_{k}"], out[f"mixed_p16_{k}"] = \
            master[k], mm[k], vv[k], p16[k]

    # canonical dot
    a = O.fill_normal(5000, 0, 1, SEED, 90)
    b = O.fill_normal(5000, 0, 1, SEED, 91)
    out["dot_a"], out["dot_b"] = a, b
    out["dot_value"] = np.array([O.dot_canonical(a, b), O.dot_sequential(a, b)], np.float32)

    # L-BFGS: n=300, history 3, 8 iterations, three modes
    n, hs = 300, 3
    D = O.fill_loguniform(n, -0.2, 0.2, SEED, 95)
    bb = O.fill_normal(n, 0, 1, SEED, 96)
    out["lbfgs_D"], out["lbfgs_b"] = D, bb
    for mode in (0, 1, 3):
        x, old, d = (np.zeros(n, np.float32) for _ in range(3))
        s_h = [[np.zeros(n, np.float32)] for _ in range(hs)]
        y_h = [[np.zeros(n, np.float32)] for _ in range(hs)]
        rho, alpha = np.zeros(hs, np.float32), np.zeros(hs, np.float32)
        hc = hi = 0
        rhos = []
        for _ in range(8):
            g = (D * x - bb).astype(np.float32)
            O.lbfgs_step([x], [g], [old], [d], s_h, y_h, rho, alpha, hs, hc, hi, 1.0, mode, 0)
            hi, hc = (hi + 1) % hs, min(hc + 1, hs)
            rhos.append(rho.copy())
        out[f"lbfgs_x_mode{mode}"] = x
        out[f"lbfgs_rho_mode{mode}"] = np.array(rhos, np.float32)

    path = os.path.join(HERE, "optimizer_steps.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
