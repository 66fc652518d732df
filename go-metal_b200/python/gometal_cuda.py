"""ctypes binding of libgometal_cuda.so for the test-suite and the benchmark.

This module only declares the C ABI of include/gometal_cuda.h and adds small
numpy conveniences; it contains no arithmetic.  Importing it loads the shared
library and raises if the library has not been built -- there is no fallback.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "lib", "libgometal_cuda.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python go-metal_b200/build.py` "
        "(there is no CPU or PyTorch fallback for the optimizer step)")

lib = C.CDLL(LIB_PATH)

u, i, f, i64, vp = C.c_size_t, C.c_int, C.c_float, C.c_int64, C.c_void_p
up = C.POINTER(C.c_size_t)      # uintptr_t*
ip = C.POINTER(C.c_int)


class Hyper(C.Structure):
    _fields_ = [("lr", f), ("beta1", f), ("beta2", f), ("eps", f), ("weight_decay", f),
                ("momentum", f), ("nesterov", i), ("centered", i), ("step", i)]


class LossScale(C.Structure):
    _fields_ = [("scale", f), ("growth", f), ("backoff", f), ("max_scale", f),
                ("interval", C.c_int32), ("good_steps", C.c_int32), ("adam_t", C.c_int32),
                ("skipped", C.c_int32), ("last_overflow", C.c_int32)]


RULE_SGD, RULE_ADAM, RULE_RMSPROP, RULE_ADAGRAD, RULE_ADADELTA, RULE_NADAM = range(6)

_SIGS = {
    # part 1
    "create_cuda_device": (u, []),
    "destroy_cuda_device": (None, [u]),
    "create_command_queue": (u, [u]),
    "release_command_queue": (None, [u]),
    "allocate_cuda_buffer": (u, [u, i, i]),
    "deallocate_cuda_buffer": (None, [u]),
    "zero_cuda_buffer": (i, [u, u, i]),
    "copy_data_to_cuda_buffer": (i, [u, vp, i]),
    "copy_float32_array_to_cuda_buffer": (i, [u, vp, i]),
    "copy_int32_array_to_cuda_buffer": (i, [u, vp, i]),
    "copy_cuda_buffer_to_float32_array": (i, [u, vp, i]),
    "copy_cuda_buffer_to_int32_array": (i, [u, vp, i]),
    "convert_tensor_type_cuda": (i, [u, u, ip, i, i, i, u]),
    "execute_sgd_step_cuda": (i, [u, up, up, up, i, ip, f, f, f, i, i]),
    "execute_adam_step_cuda": (i, [u, up, up, up, up, i, ip, f, f, f, f, f, i]),
    "execute_adam_step_cuda_pooled": (i, [u, up, up, up, up, i, ip, f, f, f, f, f, i, u]),
    "execute_rmsprop_step_cuda": (i, [u, up, up, up, up, up, i, ip, f, f, f, f, f, C.c_bool, i]),
    "execute_adagrad_step_cuda": (i, [u, up, up, up, i, ip, f, f, f]),
    "execute_adagrad_step_cuda_pooled": (i, [u, up, up, up, i, ip, f, f, f, u]),
    "execute_adadelta_step_cuda": (i, [u, up, up, up, up, i, ip, f, f, f]),
    "execute_adadelta_step_cuda_pooled": (i, [u, up, up, up, up, i, ip, f, f, f, u]),
    "execute_nadam_step_cuda": (i, [u, up, up, up, up, i, ip, f, f, f, f, f, i]),
    "execute_lbfgs_step_cuda": (i, [u, up, up, up, up, up, up, up, u, i, ip, i, i, i, f, f, f, i, f, f,
                                    C.POINTER(f)]),
    "execute_lbfgs_step_cuda_pooled": (i, [u, up, up, up, up, up, up, up, u, i, ip, i, i, i, f, f, f, i, f,
                                           f, u, C.POINTER(f)]),
    # part 2
    "gm_last_error": (C.c_char_p, []),
    "gm_version": (C.c_char_p, []),
    "gm_device_create": (u, [i]),
    "gm_device_ordinal": (i, [u]),
    "gm_device_sm_count": (i, [u]),
    "gm_device_stream": (u, [u]),
    "gm_device_synchronize": (i, [u]),
    "gm_device_synchronize_timeout": (i, [u, i]),
    "gm_device_launch_count": (i64, [u]),
    "gm_buffer_alloc": (u, [u, i64]),
    "gm_buffer_free": (None, [u]),
    "gm_buffer_size": (i64, [u]),
    "gm_buffer_zero": (i, [u, u, i64]),
    "gm_buffer_upload": (i, [u, u, vp, i64]),
    "gm_buffer_download": (i, [u, u, vp, i64]),
    "gm_arena_create": (u, [u, i64]),
    "gm_arena_alloc": (u, [u, i64]),
    "gm_arena_base": (u, [u]),
    "gm_arena_capacity": (i64, [u]),
    "gm_arena_used": (i64, [u]),
    "gm_arena_reset": (None, [u]),
    "gm_arena_destroy": (None, [u]),
    "gm_host_alloc_pinned": (vp, [i64]),
    "gm_host_free_pinned": (None, [vp]),
    "gm_buffer_upload_async": (i, [u, u, vp, i64]),
    "gm_buffer_download_async": (i, [u, u, vp, i64]),
    "gm_tensor_list_create": (u, [u, i, i, C.POINTER(up), C.POINTER(i64), ip]),
    "gm_tensor_list_destroy": (None, [u]),
    "gm_tensor_list_total": (i64, [u]),
    "gm_tensor_list_num_chunks": (i, [u]),
    "gm_tensor_list_chunk_elems": (i, [u]),
    "gm_tensor_list_head": (i, [u, i]),
    "gm_grad_clip_coef_async": (i, [u, u, f, u]),
    "gm_step_clipped_async": (i, [u, i, u, C.POINTER(Hyper), u]),
    "gm_step_with_clip_async": (i, [u, i, u, C.POINTER(Hyper), f]),
    "gm_last_clip": (i, [u, C.POINTER(f)]),
    "gm_step_async": (i, [u, i, u, C.POINTER(Hyper)]),
    "gm_step_timed": (i, [u, i, u, C.POINTER(Hyper), C.POINTER(f)]),
    "gm_step_host": (i, [u, i, u, C.POINTER(Hyper), vp, vp, i]),
    "gm_mixed_create": (u, [u, C.POINTER(LossScale), f, f, i]),
    "gm_mixed_destroy": (None, [u]),
    "gm_mixed_step_async": (i, [u, u, u, f, f, f]),
    "gm_mixed_get_state": (i, [u, u, C.POINTER(LossScale)]),
    "gm_mixed_set_state": (i, [u, u, C.POINTER(LossScale)]),
    "gm_mixed_state_device_ptr": (u, [u]),
    "gm_mixed_enable_grad_norm": (i, [u, i]),
    "gm_mixed_last_grad_sumsq": (i, [u, u, C.POINTER(f)]),
    "gm_mixed_set_clip": (i, [u, f]),
    "gm_mixed_last_clip": (i, [u, u, C.POINTER(f), C.POINTER(f)]),
    "gm_grad_sumsq_async": (i, [u, u, i, f, u]),
    "gm_lbfgs_set_mode": (i, [u, i]),
    "gm_dot_canonical": (i, [u, u, u, i64, C.POINTER(f)]),
    "gm_dot_canonical_static": (i, [u, u, i64, u, u]),
    "gm_zero1_unique_id": (i, [vp]),
    "gm_zero1_create": (u, [u, vp, i, i]),
    "gm_zero1_destroy": (None, [u]),
    "gm_zero1_allgather_async": (i, [u, u, i64, i]),
    "gm_zero1_adam_step_async": (i, [u, u, C.POINTER(Hyper), u, i64]),
    "gm_zero1_step_async": (i, [u, i, u, C.POINTER(Hyper), u, i64]),
    "gm_zero1_rank": (i, [u]),
    "gm_zero1_world": (i, [u]),
    "gm_zero1_ipc_handle": (i, [u, u, vp]),
    "gm_zero1_open_peers": (i, [u, vp]),
    "gm_zero1_adam_push_step_async": (i, [u, u, C.POINTER(Hyper)]),
    "gm_zero1_adam_push_step_host": (i, [u, u, C.POINTER(Hyper), vp, vp, i]),
    "gm_zero1_adam_dma_step_async": (i, [u, u, C.POINTER(Hyper), i]),
    "gm_zero1_mixed_step_async": (i, [u, u, u, f, f, f, u, i64]),
    "gm_zero1_reduce_scatter_async": (i, [u, u, i64, i]),
    "gm_zero1_ipc_handle_slot": (i, [u, i, u, vp]),
    "gm_zero1_open_peers_slot": (i, [u, i, vp]),
    "gm_zero1_mixed_push_step_async": (i, [u, u, u, f, f, f]),
    "gm_selftest_const_div": (i, [u, f, C.POINTER(C.c_uint64), C.POINTER(C.c_uint32), ip]),
    "gm_selftest_barrier_timeout": (i, [u, C.c_longlong, ip]),
    "gm_device_set_tuning": (i, [u, C.c_char_p, C.c_longlong]),
    "gm_device_get_tuning": (C.c_longlong, [u, C.c_char_p]),
    "gm_timer_start": (i, [u]),
    "gm_timer_stop": (i, [u, C.POINTER(f)]),
}

MISSING = []
for _name, (_res, _args) in _SIGS.items():
    try:
        _fn = getattr(lib, _name)
    except AttributeError:
        MISSING.append(_name)
        continue
    _fn.restype = _res
    _fn.argtypes = _args


class GmError(RuntimeError):
    pass


def last_error() -> str:
    return lib.gm_last_error().decode("utf-8", "replace")


def check(rc: int, what: str = "call") -> None:
    if rc != 0:
        raise GmError(f"{what} failed with code {rc}: {last_error()}")


def uarray(values) -> "C.Array":
    """uintptr_t[] from an iterable of addresses."""
    values = list(values)
    return (C.c_size_t * len(values))(*values)


def iarray(values) -> "C.Array":
    values = list(values)
    return (C.c_int * len(values))(*values)


class Device:
    """Owns one device handle (create_cuda_device / gm_device_create)."""

    def __init__(self, ordinal: int | None = None):
        self.h = lib.create_cuda_device() if ordinal is None else lib.gm_device_create(ordinal)
        if not self.h:
            raise GmError(f"no CUDA device: {last_error()}")

    def close(self):
        if self.h:
            lib.destroy_cuda_device(self.h)
            self.h = 0

    def sync(self):
        check(lib.gm_device_synchronize(self.h), "synchronize")

    def alloc(self, nbytes: int) -> int:
        p = lib.gm_buffer_alloc(self.h, nbytes)
        if not p:
            raise GmError(f"allocation of {nbytes} bytes failed: {last_error()}")
        return p

    def free(self, p: int):
        lib.gm_buffer_free(p)

    def upload(self, p: int, a: np.ndarray):
        a = np.ascontiguousarray(a)
        check(lib.gm_buffer_upload(self.h, p, a.ctypes.data, a.nbytes), "upload")

    def download(self, p: int, a: np.ndarray):
        assert a.flags["C_CONTIGUOUS"]
        check(lib.gm_buffer_download(self.h, p, a.ctypes.data, a.nbytes), "download")

    def to_device(self, a: np.ndarray) -> int:
        a = np.ascontiguousarray(a)
        p = self.alloc(max(a.nbytes, 1))
        if a.nbytes:
            self.upload(p, a)
        return p

    def to_host(self, p: int, n: int, dtype=np.float32) -> np.ndarray:
        out = np.empty(n, dtype=dtype)
        if n:
            self.download(p, out)
        return out

    def tensor_list(self, streams, numel, elem_bytes=None) -> int:
        """streams: list (per stream) of lists of device addresses."""
        ns, nt = len(streams), len(numel)
        arrays = [uarray(s) for s in streams]
        outer = (up * ns)(*[C.cast(a, up) for a in arrays])
        n64 = (i64 * nt)(*numel)
        eb = iarray(elem_bytes) if elem_bytes is not None else None
        h = lib.gm_tensor_list_create(self.h, ns, nt, outer, n64, eb)
        if not h:
            raise GmError(f"tensor list creation failed: {last_error()}")
        return h

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
