"""ctypes access to the CPU oracle (oracle/gm_oracle.c).

TEST INFRASTRUCTURE, NOT PRODUCT: imported only by tests/, by the smoke check
and by the benchmark's CPU-baseline leg and parity checks.  Parity unpinned -- the reference has
no golden vector for an optimizer step (see gm_oracle.h).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libgm_oracle.so")


def build(force: bool = False) -> str:
    """Compile the oracle with the committed Makefile (gcc only)."""
    src = os.path.join(_HERE, "gm_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)
             or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
             or os.path.getmtime(_LIB_PATH) < os.path.getmtime(os.path.join(_HERE, "gm_oracle.h")))
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-s"], check=True)
    return _LIB_PATH


class LossScale(C.Structure):
    _fields_ = [("scale", C.c_float), ("growth", C.c_float), ("backoff", C.c_float),
                ("max_scale", C.c_float), ("interval", C.c_int32), ("good_steps", C.c_int32),
                ("adam_t", C.c_int32), ("skipped", C.c_int32), ("last_overflow", C.c_int32)]


_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
_lib = None


def lib():
    global _lib
    if _lib is not None:
        return _lib
    L = C.CDLL(build())
    f, i, z = C.c_float, C.c_int, C.c_size_t
    L.gmo_adam_step.argtypes = [_f32p, _f32p, _f32p, _f32p, z, f, f, f, f, f, i]
    L.gmo_adam_step_mt.argtypes = [_f32p, _f32p, _f32p, _f32p, z, f, f, f, f, f, i, i]
    L.gmo_sgd_step.argtypes = [_f32p, _f32p, C.c_void_p, z, f, f, f, i]
    L.gmo_rmsprop_step.argtypes = [_f32p, _f32p, _f32p, C.c_void_p, C.c_void_p, z, f, f, f, f, f, i, i]
    L.gmo_adagrad_step.argtypes = [_f32p, _f32p, _f32p, z, f, f, f]
    L.gmo_adadelta_step.argtypes = [_f32p, _f32p, _f32p, _f32p, z, f, f, f]
    L.gmo_nadam_step.argtypes = [_f32p, _f32p, _f32p, _f32p, z, f, f, f, f, f, i]
    L.gmo_adam_scalars.argtypes = [f, f, i] + [C.POINTER(f)] * 4
    L.gmo_nadam_mu_next.argtypes = [f, i]
    L.gmo_nadam_mu_next.restype = f
    L.gmo_f32_to_f16.argtypes = [f]
    L.gmo_f32_to_f16.restype = C.c_uint16
    L.gmo_f16_to_f32.argtypes = [C.c_uint16]
    L.gmo_f16_to_f32.restype = f
    L.gmo_convert_f32_to_f16.argtypes = [_f32p, _u16p, z]
    L.gmo_convert_f16_to_f32.argtypes = [_u16p, _f32p, z]
    L.gmo_loss_scale_init.argtypes = [C.POINTER(LossScale)]
    L.gmo_f16_has_nonfinite.argtypes = [_u16p, z]
    L.gmo_f16_has_nonfinite.restype = i
    pp = C.POINTER(C.c_void_p)
    L.gmo_mixed_adam_step.argtypes = [i, C.POINTER(z), pp, pp, pp, pp, pp, f, f, f, f, f,
                                      C.POINTER(LossScale)]
    L.gmo_mixed_adam_step.restype = i
    L.gmo_dot_num_chunks.argtypes = [z]
    L.gmo_dot_num_chunks.restype = z
    L.gmo_dot_chunk_partials.argtypes = [_f32p, _f32p, z, _f32p]
    L.gmo_reduce_partials.argtypes = [_f32p, z]
    L.gmo_reduce_partials.restype = f
    L.gmo_dot_canonical.argtypes = [_f32p, _f32p, z]
    L.gmo_dot_canonical.restype = f
    L.gmo_dot_sequential.argtypes = [_f32p, _f32p, z]
    L.gmo_dot_sequential.restype = f
    L.gmo_sumsq_f32.argtypes = [_f32p, z]
    L.gmo_sumsq_f32.restype = C.c_double
    L.gmo_sumsq_f16.argtypes = [_u16p, z, f]
    L.gmo_sumsq_f16.restype = C.c_double
    L.gmo_lbfgs_step.argtypes = [i, C.POINTER(z), pp, pp, pp, pp, pp, pp, _f32p, _f32p,
                                 i, i, i, f, i, i, C.POINTER(f)]
    L.gmo_lbfgs_step.restype = i
    L.gmo_set_threads.argtypes = [i]
    L.gmo_get_threads.restype = i
    L.gmo_scale_to_f16.argtypes = [_f32p, f, _u16p, z]
    L.gmo_clip_coef.argtypes = [f, f]
    L.gmo_clip_coef.restype = f
    L.gmo_sumsq_canonical.argtypes = [i, C.POINTER(z), pp]
    L.gmo_sumsq_canonical.restype = f
    L.gmo_sumsq_f16_layout.argtypes = [i, C.POINTER(z), pp, C.POINTER(i), z, f]
    L.gmo_sumsq_f16_layout.restype = f
    L.gmo_mixed_adam_step_clipped.argtypes = [i, C.POINTER(z), pp, pp, pp, pp, pp, f, f, f, f, f,
                                              f, C.POINTER(i), z, C.POINTER(f), C.POINTER(f),
                                              C.POINTER(LossScale)]
    L.gmo_mixed_adam_step_clipped.restype = i
    L.gmo_hash64.argtypes = [C.c_uint64] * 3
    L.gmo_hash64.restype = C.c_uint64
    L.gmo_fill_uniform.argtypes = [_f32p, z, f, f, C.c_uint64, C.c_uint64]
    L.gmo_fill_normal.argtypes = [_f32p, z, f, f, C.c_uint64, C.c_uint64]
    L.gmo_scale_subset.argtypes = [_f32p, z, i, f, C.c_uint64, C.c_uint64]
    L.gmo_fill_loguniform.argtypes = [_f32p, z, f, f, C.c_uint64, C.c_uint64]
    _lib = L
    return L


def _ptr_array(arrays):
    arr = (C.c_void_p * len(arrays))()
    for k, a in enumerate(arrays):
        arr[k] = a.ctypes.data
    return arr


def _opt(a):
    return None if a is None else a.ctypes.data


def set_threads(n: int) -> None:
    """Threads for the independent elementwise loops (bit-identical results; default 1)."""
    lib().gmo_set_threads(int(n))


def all_cores() -> int:
    return max(1, min(64, os.cpu_count() or 1))


# ---- elementwise rules (flat float32 arrays, updated in place) ----

def adam_step(w, g, m, v, lr, beta1, beta2, eps, wd, step, threads=1):
    if threads > 1:
        lib().gmo_adam_step_mt(w, g, m, v, w.size, lr, beta1, beta2, eps, wd, step, threads)
    else:
        lib().gmo_adam_step(w, g, m, v, w.size, lr, beta1, beta2, eps, wd, step)


def sgd_step(w, g, mom, lr, momentum, wd, nesterov):
    lib().gmo_sgd_step(w, g, _opt(mom), w.size, lr, momentum, wd, int(nesterov))


def rmsprop_step(w, g, sq, mom, gavg, lr, alpha, eps, wd, momentum, centered, persist_aux=True):
    lib().gmo_rmsprop_step(w, g, sq, _opt(mom), _opt(gavg), w.size, lr, alpha, eps, wd, momentum,
                           int(centered), int(persist_aux))


def adagrad_step(w, g, sq, lr, eps, wd):
    lib().gmo_adagrad_step(w, g, sq, w.size, lr, eps, wd)


def adadelta_step(w, g, sq, upd, rho, eps, wd):
    lib().gmo_adadelta_step(w, g, sq, upd, w.size, rho, eps, wd)


def nadam_step(w, g, m, v, lr, beta1, beta2, eps, wd, step):
    lib().gmo_nadam_step(w, g, m, v, w.size, lr, beta1, beta2, eps, wd, step)


def adam_scalars(beta1, beta2, step):
    out = [C.c_float() for _ in range(4)]
    lib().gmo_adam_scalars(beta1, beta2, step, *[C.byref(o) for o in out])
    return tuple(np.float32(o.value) for o in out)


def nadam_mu_next(beta1, step):
    return np.float32(lib().gmo_nadam_mu_next(beta1, step))


# ---- fp16 ----

def f32_to_f16(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().gmo_convert_f32_to_f16(x.reshape(-1), out.reshape(-1), x.size)
    return out


def f16_to_f32(h):
    h = np.ascontiguousarray(h, dtype=np.uint16)
    out = np.empty(h.shape, dtype=np.float32)
    lib().gmo_convert_f16_to_f32(h.reshape(-1), out.reshape(-1), h.size)
    return out


def scale_to_f16(x, factor):
    """half(x * factor), the product rounded to float32 first."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().gmo_scale_to_f16(x.reshape(-1), float(factor), out.reshape(-1), x.size)
    return out


# ---- mixed precision ----

def new_loss_scale(**kw):
    st = LossScale()
    lib().gmo_loss_scale_init(C.byref(st))
    for k, val in kw.items():
        setattr(st, k, val)
    return st


def mixed_adam_step(g16, master, m, v, p16, lr, beta1, beta2, eps, wd, state):
    n = len(g16)
    numel = (C.c_size_t * n)(*[a.size for a in master])
    return lib().gmo_mixed_adam_step(n, numel, _ptr_array(g16), _ptr_array(master), _ptr_array(m),
                                     _ptr_array(v), _ptr_array(p16), lr, beta1, beta2, eps, wd,
                                     C.byref(state))


def mixed_adam_step_clipped(g16, master, m, v, p16, lr, beta1, beta2, eps, wd, max_norm, head, chunk, state):
    """Returns (skipped, sumsq, coef); head = per-tensor element offsets of the device layout."""
    n = len(g16)
    numel = (C.c_size_t * n)(*[a.size for a in master])
    heads = (C.c_int * n)(*[int(h) for h in head])
    ss, cf = C.c_float(), C.c_float()
    skipped = lib().gmo_mixed_adam_step_clipped(n, numel, _ptr_array(g16), _ptr_array(master), _ptr_array(m),
                                                _ptr_array(v), _ptr_array(p16), lr, beta1, beta2, eps, wd,
                                                max_norm, heads, chunk, C.byref(ss), C.byref(cf), C.byref(state))
    return skipped, np.float32(ss.value), np.float32(cf.value)


def clip_coef(sumsq, max_norm):
    return np.float32(lib().gmo_clip_coef(float(sumsq), float(max_norm)))


def sumsq_canonical(tensors):
    n = len(tensors)
    numel = (C.c_size_t * n)(*[a.size for a in tensors])
    return np.float32(lib().gmo_sumsq_canonical(n, numel, _ptr_array(tensors)))


def sumsq_f16_layout(g16, head, chunk, inv_scale):
    n = len(g16)
    numel = (C.c_size_t * n)(*[a.size for a in g16])
    heads = (C.c_int * n)(*[int(h) for h in head])
    return np.float32(lib().gmo_sumsq_f16_layout(n, numel, _ptr_array(g16), heads, chunk, float(inv_scale)))


# ---- reductions ----

def dot_canonical(a, b):
    return np.float32(lib().gmo_dot_canonical(a, b, a.size))


def dot_sequential(a, b):
    return np.float32(lib().gmo_dot_sequential(a, b, a.size))


def sumsq_f32(g):
    return lib().gmo_sumsq_f32(g, g.size)


def sumsq_f16(g, inv_scale):
    return lib().gmo_sumsq_f16(g, g.size, inv_scale)


# ---- L-BFGS ----

def lbfgs_step(w, g, old_g, direction, s, y, rho, alpha, history_size, history_count,
               history_index, initial_step, mode, order=0):
    """w/g/old_g/direction: lists of arrays (one per tensor); s/y: [slot][tensor]."""
    nt = len(w)
    numel = (C.c_size_t * nt)(*[a.size for a in w])
    s_flat = [s[k][t] for k in range(history_size) for t in range(nt)]
    y_flat = [y[k][t] for k in range(history_size) for t in range(nt)]
    step = C.c_float()
    rc = lib().gmo_lbfgs_step(nt, numel, _ptr_array(w), _ptr_array(g), _ptr_array(old_g),
                              _ptr_array(direction), _ptr_array(s_flat), _ptr_array(y_flat),
                              rho, alpha, history_size, history_count, history_index,
                              initial_step, mode, order, C.byref(step))
    return rc, step.value


# ---- generators ----

def fill_uniform(n, lo, hi, seed, stream):
    out = np.empty(n, dtype=np.float32)
    lib().gmo_fill_uniform(out, n, lo, hi, seed, stream)
    return out


def fill_normal(n, mean, std, seed, stream):
    out = np.empty(n, dtype=np.float32)
    lib().gmo_fill_normal(out, n, mean, std, seed, stream)
    return out


def scale_subset(a, per_mille, factor, seed, stream):
    lib().gmo_scale_subset(a, a.size, per_mille, factor, seed, stream)
    return a


def fill_loguniform(n, lo_exp10, hi_exp10, seed, stream):
    out = np.empty(n, dtype=np.float32)
    lib().gmo_fill_loguniform(out, n, lo_exp10, hi_exp10, seed, stream)
    return out
