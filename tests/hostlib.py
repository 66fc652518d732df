"""ctypes access to libgometal_host.so (the C++ mirror of go-metal's optimizer
host side) for the tests; builds the library and the recording fake backend on
first use."""
import ctypes as C
import importlib.util
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HERE = os.path.dirname(os.path.abspath(__file__))
FAKE = os.path.join(HERE, "_build", "libfake_backend.so")
CUDA = os.path.join(ROOT, "go-metal_b200", "lib", "libgometal_cuda.so")

SGD, ADAM, ADAM_POOLED, RMSPROP, ADAGRAD, ADADELTA, NADAM, LBFGS = range(8)
MIXED_STEP, LIST_CREATE, LIST_DESTROY, MIXED_CREATE, MIXED_DESTROY = range(8, 13)


class LossScaleC(C.Structure):
    """Layout of gm_loss_scale_t."""
    _fields_ = [("scale", C.c_float), ("growth", C.c_float), ("backoff", C.c_float), ("max_scale", C.c_float),
                ("interval", C.c_int32), ("good_steps", C.c_int32), ("adam_t", C.c_int32), ("skipped", C.c_int32),
                ("last_overflow", C.c_int32)]


def build_fake():
    src = os.path.join(HERE, "fake_backend.c")
    if not os.path.exists(FAKE) or os.path.getmtime(FAKE) < os.path.getmtime(src):
        os.makedirs(os.path.dirname(FAKE), exist_ok=True)
        subprocess.run(["gcc", "-O1", "-fPIC", "-shared", "-o", FAKE, src], check=True)
    return FAKE


def load_host():
    spec = importlib.util.spec_from_file_location("gm_host_build", os.path.join(ROOT, "go-metal_b200", "host", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    H = C.CDLL(mod.build())
    u, i, d, f, vp, s = C.c_size_t, C.c_int, C.c_double, C.c_float, C.c_void_p, C.c_char_p
    ip = C.POINTER(C.c_int)
    sig = {
        "gmh_last_error": (s, []), "gmh_init": (i, [s]), "gmh_device_create": (u, []), "gmh_device_destroy": (None, [u]),
        "gmh_mm_create": (vp, [u]), "gmh_mm_destroy": (None, [vp]), "gmh_mm_use_arena": (i, [vp, C.c_int64]), "gmh_mm_allocate": (u, [vp, i]),
        "gmh_mm_release": (None, [vp, u]), "gmh_mm_tracked_size": (i, [vp, u]), "gmh_find_pool_size": (i, [i]),
        "gmh_calculate_max_pool_size": (i, [i]), "gmh_mm_stats": (i, [vp, i, ip, ip, ip]),
        "gmh_extract_buffer_index": (i, [s]), "gmh_calculate_tensor_size": (i, [ip, i]),
        "gmh_state_new": (vp, [s]), "gmh_state_destroy": (None, [vp]), "gmh_state_type": (s, [vp]),
        "gmh_state_set_float64": (None, [vp, s, d]), "gmh_state_set_bool": (None, [vp, s, i]),
        "gmh_state_set_uint64": (None, [vp, s, C.c_uint64]), "gmh_state_get_param": (i, [vp, s, C.POINTER(d)]),
        "gmh_extract_float32_param": (f, [vp, s, f]), "gmh_extract_bool_param": (i, [vp, s, i]),
        "gmh_extract_uint64_param": (C.c_uint64, [vp, s, C.c_uint64]), "gmh_validate_state_type": (i, [s, vp]),
        "gmh_pow": (C.c_float, [C.c_float, C.c_float]),
        "gmh_state_to_json": (s, [vp]), "gmh_state_from_json": (vp, [s]),
        "gmh_state_add_tensor": (None, [vp, s, s, vp, i]), "gmh_state_num_tensors": (i, [vp]),
        "gmh_state_tensor_name": (s, [vp, i]), "gmh_state_tensor_type": (s, [vp, i]), "gmh_state_tensor_numel": (i, [vp, i]),
        "gmh_state_tensor_shape0": (i, [vp, i]), "gmh_state_tensor_data": (None, [vp, i, vp]),
        "gmh_optimizer_create": (vp, [s, C.POINTER(d), i, ip, ip, i, vp, u]), "gmh_optimizer_destroy": (None, [vp]),
        "gmh_optimizer_set_weight_buffers": (i, [vp, C.POINTER(u), i]), "gmh_optimizer_step": (i, [vp, C.POINTER(u), i, f]),
        "gmh_optimizer_step_count": (C.c_uint64, [vp]), "gmh_optimizer_update_lr": (i, [vp, f]), "gmh_optimizer_lr": (f, [vp]),
        "gmh_optimizer_type": (s, [vp]), "gmh_optimizer_set_command_pool": (None, [vp, u]), "gmh_optimizer_cleanup": (None, [vp]),
        "gmh_optimizer_stat": (d, [vp, s]), "gmh_optimizer_get_state": (vp, [vp]), "gmh_optimizer_load_state": (i, [vp, vp]),
        "gmh_mixed_init_master": (i, [vp, i, vp, i]), "gmh_mixed_read_master": (i, [vp, i, vp, i]),
        "gmh_mixed_loss_scale": (i, [vp, vp]),
        "gmh_mixed_set_clip": (i, [vp, f]), "gmh_mixed_last_clip": (i, [vp, C.POINTER(f), C.POINTER(f)]),
        "gmh_lbfgs_history": (i, [vp, ip, ip]), "gmh_lbfgs_read_rho": (i, [vp, vp, i]),
        "gmh_sched_create": (vp, [i, i, d, d, s]), "gmh_sched_destroy": (None, [vp]), "gmh_sched_get_lr": (d, [vp, i, i, d]),
        "gmh_sched_step": (d, [vp, d, d]), "gmh_sched_name": (s, [vp]), "gmh_apply_scheduler": (i, [vp, vp, i, i, d]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(H, name)
        fn.restype, fn.argtypes = res, args
    return H


def err(H):
    return H.gmh_last_error().decode()


def make_optimizer(H, kind, cfg, shapes, mm, device):
    flat = [d for sh in shapes for d in sh]
    nd = [len(sh) for sh in shapes]
    cfg_arr = (C.c_double * max(len(cfg), 1))(*cfg)
    return H.gmh_optimizer_create(kind.encode(), cfg_arr, len(cfg), (C.c_int * max(len(flat), 1))(*flat),
                                  (C.c_int * max(len(nd), 1))(*nd), len(shapes), mm, device)


def uarr(vals):
    vals = list(vals)
    return (C.c_size_t * max(len(vals), 1))(*vals)
