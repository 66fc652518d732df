"""gm_dot_canonical_static: the dot product for hosts that cannot allocate.

Some users of this library hand all of HBM to their own arenas, or run a
training loop that must never stall on cudaMalloc/cudaFree (both synchronise
the whole device).  For them the library carries its reduction scratch as a
built-in device array, and this entry uses it instead of allocated buffers.
The file is named so that pytest collects it last.

Checked here, through the C ABI: the result has the same bits as the existing
gm_dot_canonical entry (this suite's tolerance for dot products is bit
equality), on two calls in a row that share the built-in array, for aligned
and unaligned operands; sizes beyond the built-in limit are refused.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

LIMIT = 67_108_864      # GM_DOT_STATIC_MAX_ELEMENTS


def reference_dot(gm, dev, pa, pb, n):
    out = C.c_float()
    gm.check(gm.lib.gm_dot_canonical(dev.h, pa, pb, n, C.byref(out)), "gm_dot_canonical")
    return np.float32(out.value)


def static_dot(gm, dev, pa, pb, n, pout):
    stream = gm.lib.gm_device_stream(dev.h)
    gm.check(gm.lib.gm_dot_canonical_static(pa, pb, n, pout, stream), "gm_dot_canonical_static")
    return dev.to_host(pout, 1)[0]          # waits for the stream, then copies the float


def test_static_dot_matches_allocating_entry_twice_in_a_row(gm, dev, oracle):
    O = oracle
    pout = dev.alloc(256)
    try:
        # two different problems back to back: the second call finds the first
        # call's chunk sums still in the built-in array and must not be affected
        # 5,000,003 elements = 1,221 chunks: more chunks than CTAs (each CTA loops) and more than
        # 256 (the last CTA's lanes each add several chunk sums)
        cases = [(1_000_003, 41), (70_001, 42), (1_000_003, 41), (5, 43), (4096, 44), (5_000_003, 45)]
        for n, seed in cases:
            a = O.fill_normal(n, 0, 1, seed, 1)
            b = O.fill_normal(n, 0, 1, seed, 2)
            pa, pb = dev.to_device(a), dev.to_device(b)
            want = reference_dot(gm, dev, pa, pb, n)
            got1 = static_dot(gm, dev, pa, pb, n, pout)
            got2 = static_dot(gm, dev, pa, pb, n, pout)
            assert got1.view(np.uint32) == want.view(np.uint32), f"n={n}: first call {got1} vs {want}"
            assert got2.view(np.uint32) == want.view(np.uint32), f"n={n}: second call {got2} vs {want}"
            assert want.view(np.uint32) == O.dot_canonical(a, b).view(np.uint32)
            if n > 8:                           # operands off the 16-byte boundary
                want_u = reference_dot(gm, dev, pa + 4, pb + 4, n - 1)
                got_u = static_dot(gm, dev, pa + 4, pb + 4, n - 1, pout)
                assert got_u.view(np.uint32) == want_u.view(np.uint32), f"unaligned n={n}"
            dev.free(pa)
            dev.free(pb)
    finally:
        dev.free(pout)


def test_static_dot_at_its_size_limit(gm, dev, oracle):
    """n = GM_DOT_STATIC_MAX_ELEMENTS exactly: every slot of the built-in array is used (two
    256 MB operands); one element more is refused in the test below."""
    torch = pytest.importorskip("torch")
    O = oracle
    n = LIMIT
    gen = torch.Generator(device="cuda")
    gen.manual_seed(46)
    a = torch.empty(n, dtype=torch.float32, device="cuda").normal_(0.0, 1.0, generator=gen)
    b = torch.empty(n, dtype=torch.float32, device="cuda").normal_(0.0, 1.0, generator=gen)
    torch.cuda.synchronize()
    pout = dev.alloc(256)
    try:
        want = reference_dot(gm, dev, a.data_ptr(), b.data_ptr(), n)
        for _ in range(2):
            got = static_dot(gm, dev, a.data_ptr(), b.data_ptr(), n, pout)
            assert got.view(np.uint32) == want.view(np.uint32), f"{got} vs {want}"
        O.set_threads(O.all_cores())
        try:
            cpu = O.dot_canonical(a.cpu().numpy(), b.cpu().numpy())
        finally:
            O.set_threads(1)
        assert want.view(np.uint32) == cpu.view(np.uint32)
    finally:
        dev.free(pout)
        del a, b
        torch.cuda.empty_cache()


def test_static_dot_refuses_what_it_cannot_hold(gm, dev):
    L = gm.lib
    p = dev.alloc(256)
    try:
        assert L.gm_dot_canonical_static(p, p, LIMIT + 1, p, 0) == -9
        assert "exceed" in gm.last_error()
        assert L.gm_dot_canonical_static(p, p, 0, p, 0) == -9
        assert L.gm_dot_canonical_static(0, p, 4, p, 0) == -4
        assert L.gm_dot_canonical_static(p, p, 4, 0, 0) == -4
    finally:
        dev.free(p)
