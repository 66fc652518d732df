"""Seeded synthetic inputs shaped like the benchmark configurations.

Weights and gradients are produced by the oracle's counter-based generators on
the host and handed, bit for bit, to both the oracle and the CUDA library.
These stand in for real training tensors; no dataset is involved.
"""
import numpy as np

SEED = 0x5EED601D

# MLP 784->128->10 (Dense+bias, Dense+bias): 101,770 parameters.
MLP_SHAPES = [(784, 128), (128,), (128, 10), (10,)]
MLP_FAN_IN = [784, 0, 128, 0]
# CNN: Conv 3->32 k3, Conv 32->64 k3, Dense 4096->128, Dense 128->10: 545,098 parameters.
CNN_SHAPES = [(32, 3, 3, 3), (32,), (64, 32, 3, 3), (64,), (4096, 128), (128,), (128, 10), (10,)]
CNN_FAN_IN = [27, 0, 288, 0, 4096, 0, 128, 0]


def numel(shape):
    n = 1
    for s in shape:
        n *= s
    return n


def he_uniform_weights(O, shapes, fan_in, seed=SEED):
    """U(-L, L) with L = sqrt(6/fan_in); biases (fan_in 0) start at zero."""
    out = []
    for k, (shape, fi) in enumerate(zip(shapes, fan_in)):
        n = numel(shape)
        if fi == 0:
            out.append(np.zeros(n, dtype=np.float32))
        else:
            lim = float(np.sqrt(6.0 / fi))
            out.append(O.fill_uniform(n, -lim, lim, seed, 1000 + k))
    return out


def normal_grads(O, shapes, step, std=0.01, heavy_tail=False, seed=SEED):
    out = []
    for k, shape in enumerate(shapes):
        g = O.fill_normal(numel(shape), 0.0, std, seed, 100000 + step * 1000 + k)
        if heavy_tail:                      # 1 % of entries scaled x100
            O.scale_subset(g, 10, 100.0, seed, 200000 + step * 1000 + k)
        out.append(g)
    return out


def ragged_sizes(count, total, lo, hi, seed=SEED):
    """`count` log-uniform sizes in [lo, hi] summing to `total`, none a multiple of 8."""
    rng = np.random.default_rng(seed)
    raw = np.exp(rng.uniform(np.log(lo), np.log(hi), size=count))
    sizes = np.maximum(lo, np.floor(raw * (total / raw.sum()))).astype(np.int64)
    sizes[sizes % 8 == 0] += 1
    diff = int(total - sizes.sum())
    sizes[int(np.argmax(sizes))] += diff
    if sizes[int(np.argmax(sizes))] % 8 == 0:      # keep the sum, break the alignment
        j = int(np.argmax(sizes))
        k = (j + 1) % count
        sizes[j] -= 3
        sizes[k] += 3
        if sizes[k] % 8 == 0:
            sizes[k] -= 2
            sizes[j] += 2
    assert sizes.sum() == total and np.all(sizes > 0)
    return [int(s) for s in sizes]


def ulp_distance(a, b):
    """Distance in units of the last place between two float32 arrays (same sign regime)."""
    ia = a.view(np.int32).astype(np.int64)
    ib = b.view(np.int32).astype(np.int64)
    ia = np.where(ia < 0, np.int64(-2**31) - ia, ia)
    ib = np.where(ib < 0, np.int64(-2**31) - ib, ib)
    return np.abs(ia - ib)
