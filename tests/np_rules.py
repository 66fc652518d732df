"""Second, independent restatement of the update rules in numpy float32.

numpy evaluates each float32 array operation with one IEEE rounding and never
fuses a multiply with an add, so these functions are a cross-check of the C
oracle's compile flags and statement order.  Operation order follows
cgo_bridge/bridge_optimizer.m (Adam :484-550, SGD :219-322, RMSProp :782-876,
AdaGrad :1480-1517, AdaDelta :1773-1843, NAdam :2114-2200).
"""
import math

import numpy as np

f32 = np.float32


def powf(base, exp):
    """libm powf via the oracle is the authority for host scalars; this helper
    only mirrors the call shape for readability in the tests."""
    return f32(math.pow(float(f32(base)), float(f32(exp))))


def adam(w, g, m, v, lr, b1, b2, eps, wd, bc1, bc2):
    lr, b1, b2, eps, wd, bc1, bc2 = map(f32, (lr, b1, b2, eps, wd, bc1, bc2))
    omb1, omb2 = f32(1) - b1, f32(1) - b2
    m2 = m * b1 + g * omb1
    v2 = v * b2 + (g * g) * omb2
    upd = (m2 / bc1) / (np.sqrt(v2 / bc2) + eps)
    if wd > 0:
        upd = upd + w * wd
    return w - upd * lr, m2, v2


def sgd(w, g, mom, lr, mu, wd, nesterov):
    lr, mu, wd = map(f32, (lr, mu, wd))
    gf = g + w * wd if wd > 0 else g
    if mu > 0 and mom is not None:
        m2 = mom * mu + gf
        step = lr * (mu * m2 + gf) if nesterov else lr * m2
        return w - step, m2
    return w - lr * gf, None


def rmsprop(w, g, sq, mom, gavg, lr, alpha, eps, wd, mu, centered):
    lr, alpha, eps, wd, mu = map(f32, (lr, alpha, eps, wd, mu))
    oma = f32(1) - alpha
    sq2 = sq * alpha + (g * g) * oma
    gavg2 = None
    if centered:
        gavg2 = gavg * alpha + g * oma
        denom = np.sqrt((sq2 - gavg2 * gavg2) + eps)
    else:
        denom = np.sqrt(sq2 + eps)
    upd = g / denom
    mom2 = None
    if mu > 0:
        mom2 = mom * mu + upd
        upd = mom2
    if wd > 0:
        upd = upd + w * wd
    return w - upd * lr, sq2, mom2, gavg2


def adagrad(w, g, sq, lr, eps, wd):
    lr, eps, wd = map(f32, (lr, eps, wd))
    gf = g + w * wd if wd > 0 else g
    sq2 = sq + gf * gf
    return w - (lr / (np.sqrt(sq2) + eps)) * gf, sq2


def adadelta(w, g, sq, upd, rho, eps, wd):
    rho, eps, wd = map(f32, (rho, eps, wd))
    omr = f32(1) - rho
    gf = g + w * wd if wd > 0 else g
    e2 = sq * rho + (gf * gf) * omr
    neg = -((np.sqrt(upd + eps) / np.sqrt(e2 + eps)) * gf)
    return w + neg, e2, upd * rho + (neg * neg) * omr


def nadam(w, g, m, v, lr, b1, b2, eps, wd, bc1, bc2, mu_next):
    lr, b1, b2, eps, wd, bc1, bc2, mu_next = map(f32, (lr, b1, b2, eps, wd, bc1, bc2, mu_next))
    omb1, omb2 = f32(1) - b1, f32(1) - b2
    m2 = m * b1 + g * omb1
    v2 = v * b2 + (g * g) * omb2
    v_hat = v2 / bc2
    m_bar = (m2 / bc1) * mu_next + (g / bc1) * (f32(1) - mu_next)
    upd = m_bar / (np.sqrt(v_hat) + eps)
    if wd > 0:
        upd = upd + w * wd
    return w - upd * lr, m2, v2


def dot_canonical(a, b):
    """The fixed summation order of the dot-product kernels, written with numpy
    array operations: chunks of 4096, 256 lanes walking (i*256+t)*4+k, an xor
    tree over each group of 32 lanes, eight group sums in order, then the chunk
    sums over 256 lanes with stride 256 and the same tree."""
    n = a.size
    nchunks = (n + 4095) // 4096
    pad = nchunks * 4096 - n
    prod = (a * b).astype(f32)
    valid = np.ones(n, dtype=bool)
    if pad:
        prod = np.concatenate([prod, np.zeros(pad, f32)])
        valid = np.concatenate([valid, np.zeros(pad, bool)])
    # element e of a chunk = (i*256 + t)*4 + k  ->  axes [chunk, i, t, k]
    prod = prod.reshape(nchunks, 4, 256, 4)
    valid = valid.reshape(nchunks, 4, 256, 4)
    lane = np.zeros((nchunks, 256), f32)
    for i in range(4):
        for k in range(4):
            lane = np.where(valid[:, i, :, k], lane + prod[:, i, :, k], lane)
    return _reduce_lanes(_reduce_partials_to_lanes(_tree(lane)))


def _tree(lane):
    """[rows, 256] lane values -> [rows] sums in the documented order."""
    rows = lane.shape[0]
    cur = lane.reshape(rows, 8, 32).copy()
    idx = np.arange(32)
    for off in (16, 8, 4, 2, 1):
        cur = cur + cur[:, :, idx ^ off]
    warp = cur[:, :, 0]
    total = warp[:, 0].copy()
    for wi in range(1, 8):
        total = total + warp[:, wi]
    return total.astype(f32)


def _reduce_partials_to_lanes(partials):
    lane = np.zeros(256, f32)
    count = partials.size
    rounds = (count + 255) // 256
    for r in range(rounds):
        seg = partials[r * 256:(r + 1) * 256]
        lane[:seg.size] = lane[:seg.size] + seg
    return lane


def _reduce_lanes(lane):
    return _tree(lane.reshape(1, 256))[0]


def sumsq_f16_layout(g16_list, heads, chunk, inv_scale):
    """Sum of (half * inv_scale)^2 in the order of the CUDA overflow-check pass, written
    with numpy array operations (see gmo_sumsq_f16_layout for the order in words)."""
    inv = f32(inv_scale)
    partials = []
    for g16, hd in zip(g16_list, heads):
        n = g16.size
        sq_all = (g16.view(np.float16).astype(f32) * inv).astype(f32)
        sq_all = (sq_all * sq_all).astype(f32)
        h = min(max(hd, 0), n)
        body = n - h
        nchunks = (body + chunk - 1) // chunk if body > 0 else 1
        for k in range(nchunks):
            b = min(h + k * chunk, n)
            e = min(b + chunk, n)
            lane = np.zeros(256, f32)
            if hd < 0:
                seg = sq_all[b:e]
                rounds = (seg.size + 255) // 256
                for r in range(rounds):
                    part = seg[r * 256:(r + 1) * 256]
                    lane[:part.size] = lane[:part.size] + part
            else:
                nvec = (e - b) >> 3
                vecs = sq_all[b:b + 8 * nvec].reshape(nvec, 8)
                rounds = (nvec + 255) // 256
                for r in range(rounds):
                    part = vecs[r * 256:(r + 1) * 256]
                    for j in range(8):
                        lane[:part.shape[0]] = lane[:part.shape[0]] + part[:, j]
                if k == 0 and h > 0:
                    lane[:h] = lane[:h] + sq_all[:h]
                tail = sq_all[b + 8 * nvec:e]
                lane[:tail.size] = lane[:tail.size] + tail
            partials.append(_tree(lane.reshape(1, 256))[0])
    return _reduce_lanes(_reduce_partials_to_lanes(np.array(partials, f32)))


def clip_coef(sumsq, max_norm):
    norm = np.sqrt(f32(sumsq)).astype(f32)
    coef = f32(max_norm) / f32(norm + f32(1e-6))
    return f32(coef) if coef < 1.0 else f32(1.0)
