"""The C-ABI library loads on a machine without a GPU and exports every symbol
that include/gometal_cuda.h declares; nothing here launches device work."""
import ctypes as C
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PREFIXES = ("gm_", "execute_", "create_", "destroy_", "release_", "allocate_", "deallocate_", "zero_",
            "copy_", "convert_")


def declared_functions():
    text = open(os.path.join(ROOT, "include", "gometal_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"^\s*#.*$", "", text, flags=re.M)
    names = set(re.findall(r"\b([a-z][a-z_0-9]+)\s*\(", text))
    return sorted(n for n in names if n.startswith(PREFIXES))


def test_header_declares_the_dropin_surface():
    names = declared_functions()
    # one replacement per reference entry of bridge_optimizer.h / bridge_memory.h on this path
    for want in ["execute_sgd_step_cuda", "execute_adam_step_cuda", "execute_adam_step_cuda_pooled",
                 "execute_rmsprop_step_cuda", "execute_adagrad_step_cuda", "execute_adagrad_step_cuda_pooled",
                 "execute_adadelta_step_cuda", "execute_adadelta_step_cuda_pooled", "execute_nadam_step_cuda",
                 "execute_lbfgs_step_cuda", "execute_lbfgs_step_cuda_pooled", "allocate_cuda_buffer",
                 "deallocate_cuda_buffer", "zero_cuda_buffer", "copy_float32_array_to_cuda_buffer",
                 "copy_cuda_buffer_to_float32_array", "convert_tensor_type_cuda", "create_cuda_device",
                 "destroy_cuda_device", "create_command_queue", "release_command_queue"]:
        assert want in names
    assert len(names) >= 70


def test_library_exports_every_declared_symbol(gm):
    missing = [n for n in declared_functions() if not hasattr(gm.lib, n)]
    assert not missing, f"declared in the header but not exported: {missing}"
    assert not gm.MISSING
    unbound = sorted(set(declared_functions()) - set(gm._SIGS))
    assert not unbound, f"declared in the header but absent from the ctypes binding: {unbound}"


def test_no_silent_cpu_path(gm):
    """Without a visible GPU the device constructor returns 0 and says why;
    with one it returns a handle.  Either way nothing computes on the CPU."""
    import torch
    h = gm.lib.gm_device_create(0)
    if torch.cuda.is_available():
        assert h != 0
        gm.lib.destroy_cuda_device(h)
    else:
        assert h == 0
        assert "no CPU path" in gm.last_error()
        one = gm.uarray([4096])
        rc = gm.lib.execute_adam_step_cuda(0, one, one, one, one, 1, gm.iarray([16]), 1e-3, 0.9, 0.999, 1e-8, 0.0, 1)
        assert rc == -1


def test_product_code_never_touches_the_oracle():
    """Only tests/, __graft_entry__.smoke() and bench.py's CPU legs may use oracle/."""
    pkg = os.path.join(ROOT, "go-metal_b200")
    offenders = []
    for dirpath, _, files in os.walk(pkg):
        if os.path.basename(dirpath) in ("build", "lib", "__pycache__"):
            continue
        for name in files:
            if name.endswith((".py", ".cu", ".cuh", ".h", ".hpp", ".cpp", ".go", ".c")):
                text = open(os.path.join(dirpath, name), errors="replace").read()
                if re.search(r"\boracle\b|gm_oracle|gmo_", text):
                    offenders.append(os.path.join(dirpath, name))
    assert not offenders, offenders
