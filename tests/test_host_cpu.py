"""Host-side logic of the optimizer package (C++ mirror of optimizer/*.go,
memory/manager.go, training/scheduler.go) against the known-answer tables the
reference's own tests hold, driven through a recording fake backend: no GPU,
no arithmetic.  Each test names the reference test it restates."""
import ctypes as C

import numpy as np
import pytest

import hostlib as HL


@pytest.fixture(scope="module")
def H():
    lib = HL.load_host()
    assert lib.gmh_init(HL.build_fake().encode()) == 0, HL.err(lib)
    return lib


@pytest.fixture(scope="module")
def fake():
    F = C.CDLL(HL.build_fake())
    F.fake_last_float.restype = C.c_float
    return F


@pytest.fixture()
def env(H, fake):
    fake.fake_reset()
    dev = H.gmh_device_create()
    mm = H.gmh_mm_create(dev)
    yield H, fake, mm, dev
    H.gmh_mm_destroy(mm)


# ---------------- helper tables ----------------

def test_extract_buffer_index_table(H):
    """optimizer/state_helpers_test.go:310-376"""
    table = {"momentum_0": 0, "variance_5": 5, "squared_grad_avg_10": 10, "momentum": -1, "momentum_abc": -1,
             "": -1, "_": -1, "momentum_buffer_5": 5, "momentum_-1": -1, "momentum_999": 999}
    for name, want in table.items():
        assert H.gmh_extract_buffer_index(name.encode()) == want, name


def test_calculate_tensor_size_table(H):
    """optimizer/state_helpers_test.go:206-258"""
    for shape, want in [([], 1), ([10], 10), ([10, 20], 200), ([5, 10, 20], 1000), ([2, 3, 4, 5], 120), ([1], 1), ([0], 0)]:
        arr = (C.c_int * max(len(shape), 1))(*shape)
        assert H.gmh_calculate_tensor_size(arr, len(shape)) == want


def test_extract_params_follow_json_float64_convention(H):
    """optimizer/state_helpers_test.go:11-163: numbers are read only when they are
    float64 (what JSON decoding produces); bools only when bool; else the default."""
    st = H.gmh_state_new(b"Adam")
    H.gmh_state_set_float64(st, b"learning_rate", 0.01)
    H.gmh_state_set_bool(st, b"nesterov", 1)
    H.gmh_state_set_float64(st, b"step_count", 42.0)
    H.gmh_state_set_uint64(st, b"as_uint", 7)
    assert abs(H.gmh_extract_float32_param(st, b"learning_rate", 0.5) - 0.01) < 1e-9
    assert H.gmh_extract_float32_param(st, b"missing", 0.5) == 0.5
    assert H.gmh_extract_float32_param(st, b"nesterov", 0.25) == 0.25          # wrong kind -> default
    assert H.gmh_extract_bool_param(st, b"nesterov", 0) == 1
    assert H.gmh_extract_bool_param(st, b"learning_rate", 1) == 1              # wrong kind -> default
    assert H.gmh_extract_uint64_param(st, b"step_count", 0) == 42
    assert H.gmh_extract_uint64_param(st, b"as_uint", 3) == 3                  # uint64 is not float64 -> default
    assert H.gmh_validate_state_type(b"Adam", st) == 0
    assert H.gmh_validate_state_type(b"SGD", st) != 0
    assert HL.err(H) == "state type mismatch: expected SGD, got Adam"          # interface.go:79-84
    H.gmh_state_destroy(st)


def test_pow_table(H):
    """adam_test.go:282-308."""
    for x, y, want in [(5.0, 0.0, 1.0), (5.0, 1.0, 5.0), (3.0, 2.0, 9.0), (2.0, 3.0, 8.0), (-2.0, 2.0, 4.0),
                       (1.5, 2.0, 2.25)]:
        assert H.gmh_pow(x, y) == want, (x, y)


def test_pool_tier_tables(H):
    """memory/memory_test.go:215-266"""
    for size, want in [(100, 1024), (1024, 1024), (5000, 16384), (100000000, 100000000)]:
        assert H.gmh_find_pool_size(size) == want
    for size, want in [(1024, 100), (4096, 100), (16384, 50), (65536, 50), (262144, 20), (1048576, 20),
                       (4194304, 20), (16777216, 20), (67108864, 15)]:
        assert H.gmh_calculate_max_pool_size(size) == want


def test_memory_manager_reuses_and_caps(env):
    """memory/manager.go:20-98, 289-317: buffers come back from the tier's free
    list; a tier refuses to grow past its cap; AllocateBuffer then returns nil."""
    H, fake, mm, dev = env
    a = H.gmh_mm_allocate(mm, 3000)
    assert a and H.gmh_mm_tracked_size(mm, a) == 4096 and fake.fake_allocs() == 1
    H.gmh_mm_release(mm, a)
    b = H.gmh_mm_allocate(mm, 4000)
    assert b == a and fake.fake_allocs() == 1                   # reused, no new device allocation
    av, al, mx = C.c_int(), C.c_int(), C.c_int()
    assert H.gmh_mm_stats(mm, 4096, C.byref(av), C.byref(al), C.byref(mx)) == 0
    assert (av.value, al.value, mx.value) == (0, 1, 100)
    big = [H.gmh_mm_allocate(mm, 70_000_000) for _ in range(3)]      # beyond the last tier: exact size, own pool
    assert all(big) and H.gmh_mm_tracked_size(mm, big[0]) == 70_000_000
    held = [H.gmh_mm_allocate(mm, 20_000_000) for _ in range(16)]    # 64 MB tier holds 15
    assert all(held[:15]) and held[15] == 0
    assert H.gmh_mm_allocate(mm, 0) == 0 and H.gmh_mm_allocate(mm, -5) == 0
    for p in big + held[:15] + [b]:
        H.gmh_mm_release(mm, p)
    H.gmh_mm_release(mm, 0)                                          # nil is ignored


def test_memory_manager_on_a_flat_arena(H, fake):
    """The arena-backed pool: one flat 256-byte-aligned arena instead of per-tier device
    allocations.  The reference's tier caps (100 buffers of 1 KB) no longer bind, only the
    arena's size; released buffers are reused; nothing is allocated from or returned to the
    device one by one; the arena goes when the manager goes."""
    fake.fake_reset()
    dev = H.gmh_device_create()
    plain = H.gmh_mm_create(dev)
    held = [H.gmh_mm_allocate(plain, 1000) for _ in range(101)]
    assert all(held[:100]) and held[100] == 0                         # manager.go:210-224: the 1 KB tier holds 100
    for p in held[:100]:
        H.gmh_mm_release(plain, p)
    assert H.gmh_mm_use_arena(plain, 1 << 20) != 0 and "before the first allocation" in HL.err(H)
    H.gmh_mm_destroy(plain)

    fake.fake_reset()
    mm = H.gmh_mm_create(dev)
    assert H.gmh_mm_use_arena(mm, 0) != 0
    assert H.gmh_mm_use_arena(mm, 160 * 1024) == 0, HL.err(H)
    assert H.gmh_mm_use_arena(mm, 160 * 1024) != 0 and "already has an arena" in HL.err(H)
    assert fake.fake_arenas_live() == 1
    bufs = [H.gmh_mm_allocate(mm, 1000) for _ in range(150)]
    assert all(bufs) and fake.fake_allocs() == 0                      # carved from the arena, no device allocation
    assert all(p % 256 == 0 for p in bufs) and bufs[1] - bufs[0] == 1024 and H.gmh_mm_tracked_size(mm, bufs[5]) == 1024
    more = [H.gmh_mm_allocate(mm, 1024) for _ in range(11)]
    assert all(more[:10]) and more[10] == 0                           # 160 KB hold exactly 160 buffers of 1 KB
    H.gmh_mm_release(mm, bufs[7])
    assert H.gmh_mm_allocate(mm, 900) == bufs[7] and fake.fake_frees() == 0     # reused from the tier's free list
    o = HL.make_optimizer(H, "Adam", [], [[8]], mm, dev)
    assert not o and "failed to allocate" in HL.err(H)                # arena full: the constructor fails cleanly
    H.gmh_mm_destroy(mm)
    assert fake.fake_arenas_live() == 0 and fake.fake_frees() == 0


# ---------------- constructors ----------------

SHAPES = [[784, 128], [128], [128, 10], [10]]


def test_default_configs_reach_the_bridge(env):
    """Default*Config values (adam_test.go:129-154, sgd_test.go:13-39, rmsprop_test.go:19-52,
    adagrad_test.go:210-245, adadelta_test.go:235-269, nadam_test.go:298-320) arrive at the C entry unchanged."""
    H, fake, mm, dev = env
    w = HL.uarr([0x10, 0x20, 0x30, 0x40])
    want = {
        "Adam": (HL.ADAM, [0.001, 0.9, 0.999, 1e-8, 0.0]),
        "SGD": (HL.SGD, [0.01, 0.0, 0.0]),
        "RMSProp": (HL.RMSPROP, [0.01, 0.99, 1e-8, 0.0, 0.0]),
        "AdaGrad": (HL.ADAGRAD, [0.01, 1e-10, 0.0]),
        "AdaDelta": (HL.ADADELTA, [0.95, 1e-6, 0.0]),
        "Nadam": (HL.NADAM, [0.002, 0.9, 0.999, 1e-8, 0.0]),
    }
    for kind, (slot, scalars) in want.items():
        o = HL.make_optimizer(H, kind, [], SHAPES, mm, dev)
        assert o, HL.err(H)
        assert H.gmh_optimizer_set_weight_buffers(o, w, 4) == 0
        assert H.gmh_optimizer_step(o, w, 4, 0.0) == 0, HL.err(H)
        assert fake.fake_calls(slot) == 1
        for i, v in enumerate(scalars):
            assert fake.fake_last_float(i) == np.float32(v), (kind, i)
        assert fake.fake_last_int(2) == 4
        H.gmh_optimizer_destroy(o)


def test_constructor_validation_messages(env):
    """sgd_test.go:94-178, nadam_test.go:153-296, adadelta_test.go:144-233, lbfgs_test.go:101-162"""
    H, fake, mm, dev = env
    cases = [
        ("SGD", [-0.1], "learning rate cannot be negative: -0.100000"),
        ("SGD", [0.01, -0.5], "momentum cannot be negative: -0.500000"),
        ("SGD", [0.01, 1.5], "momentum cannot be greater than 1.0: 1.500000"),
        ("SGD", [0.01, 0.9, -1.0], "weight decay cannot be negative: -1.000000"),
        ("Nadam", [0.0], "learning rate must be positive, got 0.000000"),
        ("Nadam", [0.002, 1.0], "beta1 must be in [0, 1), got 1.000000"),
        ("Nadam", [0.002, 0.9, -0.1], "beta2 must be in [0, 1), got -0.100000"),
        ("Nadam", [0.002, 0.9, 0.999, 0.0], "epsilon must be positive, got 0.000000e+00"),
        ("Nadam", [0.002, 0.9, 0.999, 1e-8, -1.0], "weight decay must be non-negative, got -1.000000"),
        ("AdaDelta", [0.0], "rho must be in range (0, 1), got 0.000000"),
        ("AdaDelta", [1.0], "rho must be in range (0, 1), got 1.000000"),
        ("LBFGS", [0], "history size must be positive, got 0"),
    ]
    for kind, cfg, msg in cases:
        assert not HL.make_optimizer(H, kind, cfg, SHAPES, mm, dev)
        assert HL.err(H) == msg
    for kind in ("SGD", "Adam", "RMSProp", "AdaGrad", "AdaDelta", "Nadam", "LBFGS"):
        assert not HL.make_optimizer(H, kind, [], SHAPES, None, dev) and HL.err(H) == "memory manager cannot be nil"
        assert not HL.make_optimizer(H, kind, [], SHAPES, mm, 0) and HL.err(H) == "device cannot be nil"
        assert not HL.make_optimizer(H, kind, [], [], mm, dev) and HL.err(H) == "no weight shapes provided"


def test_allocation_failure_cleans_up(env):
    """adam.go:98-136: a failed allocation releases what was already taken."""
    H, fake, mm, dev = env
    fake.fake_fail_alloc_after(3)
    assert not HL.make_optimizer(H, "Adam", [], SHAPES, mm, dev)
    assert "failed to allocate" in HL.err(H) and "buffer for weight 1" in HL.err(H)
    fake.fake_fail_alloc_after(-1)
    o = HL.make_optimizer(H, "Adam", [], SHAPES, mm, dev)        # the three released buffers are reused
    assert o and fake.fake_allocs() <= 8
    H.gmh_optimizer_destroy(o)


def test_state_buffer_counts(env):
    """adam_test.go:248-251 and rmsprop_test.go:238-358: TotalBufferSize = state slots x sum of tensor bytes;
    SGD without momentum and plain RMSProp allocate nothing extra."""
    H, fake, mm, dev = env
    total = sum(int(np.prod(s)) for s in SHAPES) * 4
    for kind, cfg, slots in [("Adam", [], 2), ("Nadam", [], 2), ("AdaDelta", [], 2), ("AdaGrad", [], 1), ("SGD", [], 0),
                             ("SGD", [0.01, 0.9], 1), ("RMSProp", [], 1), ("RMSProp", [0.01, 0.99, 1e-8, 0, 0.9, 0], 2),
                             ("RMSProp", [0.01, 0.99, 1e-8, 0, 0.9, 1], 3), ("RMSProp", [0.01, 0.99, 1e-8, 0, 0.0, 1], 2)]:
        o = HL.make_optimizer(H, kind, cfg, SHAPES, mm, dev)
        assert o, HL.err(H)
        assert H.gmh_optimizer_stat(o, b"TotalBufferSize") == slots * total, (kind, cfg)
        assert H.gmh_optimizer_stat(o, b"NumWeights") == 4
        H.gmh_optimizer_destroy(o)


# ---------------- Step / SetWeightBuffers / LR ----------------

def test_step_counter_and_length_checks(env):
    """adam.go:160-234: SetWeightBuffers and Step reject wrong lengths; the counter is bumped before the bridge call
    and passed to it; a failing bridge call is reported with its code."""
    H, fake, mm, dev = env
    o = HL.make_optimizer(H, "Adam", [], SHAPES, mm, dev)
    w = HL.uarr([1, 2, 3, 4])
    assert H.gmh_optimizer_set_weight_buffers(o, w, 3) != 0
    assert HL.err(H) == "expected 4 weight buffers, got 3"
    assert H.gmh_optimizer_set_weight_buffers(o, w, 4) == 0
    assert H.gmh_optimizer_step(o, w, 2, 0.0) != 0
    assert HL.err(H) == "gradient buffers length (2) doesn't match weight buffers length (4)"
    assert H.gmh_optimizer_step_count(o) == 0
    for k in range(1, 4):
        assert H.gmh_optimizer_step(o, w, 4, 0.0) == 0
        assert H.gmh_optimizer_step_count(o) == k and fake.fake_last_int(1) == k
    assert fake.fake_last_int(4) == 784 * 128 * 4                       # byte sizes, as in adam.go:100
    fake.fake_next_return(-4)
    assert H.gmh_optimizer_step(o, w, 4, 0.0) != 0
    assert HL.err(H).startswith("Adam step execution failed: Adam step failed with error code: -4")
    H.gmh_optimizer_set_command_pool(o, 0x2000)                         # pooled entry once a pool is set
    assert H.gmh_optimizer_step(o, w, 4, 0.0) == 0 and fake.fake_calls(HL.ADAM_POOLED) == 1
    H.gmh_optimizer_destroy(o)


def test_update_learning_rate_and_scheduler_hook(env):
    """adam.go:254-256 stores the value for the next step; adadelta.go:222-225 ignores it;
    lbfgs.go:330-332 refuses; model_trainer.go:1476-1582 feeds scheduler output (float64 -> float32)."""
    H, fake, mm, dev = env
    w = HL.uarr([1, 2, 3, 4])
    o = HL.make_optimizer(H, "Adam", [], SHAPES, mm, dev)
    H.gmh_optimizer_set_weight_buffers(o, w, 4)
    assert H.gmh_optimizer_update_lr(o, 0.5) == 0 and H.gmh_optimizer_lr(o) == 0.5
    H.gmh_optimizer_step(o, w, 4, 0.0)
    assert fake.fake_last_float(0) == 0.5
    sched = H.gmh_sched_create(0, 2, 0.1, 0.0, b"")
    for epoch, want in [(0, 0.1), (2, 0.01), (4, 0.001)]:
        assert H.gmh_apply_scheduler(sched, o, epoch, 0, 0.1) == 0
        H.gmh_optimizer_step(o, w, 4, 0.0)
        assert fake.fake_last_float(0) == np.float32(0.1 * 0.1 ** (epoch // 2))
        assert abs(fake.fake_last_float(0) - want) < 1e-8
    H.gmh_sched_destroy(sched)
    H.gmh_optimizer_destroy(o)
    d = HL.make_optimizer(H, "AdaDelta", [], SHAPES, mm, dev)
    assert H.gmh_optimizer_update_lr(d, 0.5) == 0 and H.gmh_optimizer_lr(d) == 0.0
    H.gmh_optimizer_destroy(d)
    l = HL.make_optimizer(H, "LBFGS", [3], [[50]], mm, dev)
    assert H.gmh_optimizer_update_lr(l, 0.5) != 0
    assert HL.err(H) == "L-BFGS does not use a fixed learning rate; it uses line search"      # lbfgs_test.go:549
    H.gmh_optimizer_destroy(l)


def test_lbfgs_history_bookkeeping(env):
    """lbfgs.go:245-301: the circular index advances and the count saturates at HistorySize;
    the previous loss is handed to the next call."""
    H, fake, mm, dev = env
    o = HL.make_optimizer(H, "LBFGS", [3], [[50], [7]], mm, dev)
    assert o, HL.err(H)
    w = HL.uarr([1, 2])
    assert H.gmh_optimizer_set_weight_buffers(o, w, 2) == 0
    cnt, idx = C.c_int(), C.c_int()
    seen = []
    for k in range(5):
        assert H.gmh_optimizer_step(o, w, 2, float(10 - k)) == 0
        assert (fake.fake_last_int(0), fake.fake_last_int(2)) == (3, 2)
        seen.append((fake.fake_last_int(1), fake.fake_last_int(3), fake.fake_last_float(1), fake.fake_last_float(2)))
        H.gmh_lbfgs_history(o, C.byref(cnt), C.byref(idx))
    assert [s[:2] for s in seen] == [(0, 0), (1, 1), (2, 2), (3, 0), (3, 1)]       # (count, index) passed to the bridge
    assert [s[2:] for s in seen] == [(10.0, 0.0), (9.0, 10.0), (8.0, 9.0), (7.0, 8.0), (6.0, 7.0)]
    assert (cnt.value, idx.value) == (3, 2) and H.gmh_optimizer_step_count(o) == 5
    # (2m+2) vectors per weight + m rho + 1 alpha (lbfgs.go:113-190)
    assert fake.fake_allocs() == (2 * 3 + 2) * 2 + 3 + 1
    H.gmh_optimizer_destroy(o)


# ---------------- GetState / LoadState ----------------

def test_state_structure_and_round_trip(env):
    """adam.go:333-452 and the *GetStateStructure / *LoadStateValidation tests: names "<kind>_<i>", flat [numel] shapes,
    state types, error texts for a wrong type, a bad index and a size mismatch."""
    H, fake, mm, dev = env
    shapes = [[6], [2, 3]]
    o = HL.make_optimizer(H, "RMSProp", [0.01, 0.99, 1e-8, 0.0, 0.9, 1], shapes, mm, dev)
    st = H.gmh_optimizer_get_state(o)
    assert st and H.gmh_state_type(st) == b"RMSProp"
    names = [(H.gmh_state_tensor_name(st, i).decode(), H.gmh_state_tensor_type(st, i).decode(),
              H.gmh_state_tensor_shape0(st, i)) for i in range(H.gmh_state_num_tensors(st))]
    assert names == [("squared_grad_avg_0", "squared_grad_avg", 6), ("squared_grad_avg_1", "squared_grad_avg", 6),
                     ("momentum_0", "momentum", 6), ("momentum_1", "momentum", 6),
                     ("gradient_avg_0", "gradient_avg", 6), ("gradient_avg_1", "gradient_avg", 6)]
    val = C.c_double()
    assert H.gmh_state_get_param(st, b"step_count", C.byref(val)) == 2 and val.value == 0       # stored as uint64
    assert H.gmh_state_get_param(st, b"centered", C.byref(val)) == 1 and val.value == 1
    assert H.gmh_state_get_param(st, b"alpha", C.byref(val)) == 3 and abs(val.value - 0.99) < 1e-6
    H.gmh_state_destroy(st)

    # a checkpoint as JSON decoding would deliver it: float64 numbers
    new = H.gmh_state_new(b"RMSProp")
    H.gmh_state_set_float64(new, b"learning_rate", 0.25)
    H.gmh_state_set_float64(new, b"alpha", 0.5)
    H.gmh_state_set_float64(new, b"step_count", 17.0)
    data = np.arange(6, dtype=np.float32) + 1
    H.gmh_state_add_tensor(new, b"momentum_1", b"momentum", data.ctypes.data, 6)
    assert H.gmh_optimizer_load_state(o, new) == 0, HL.err(H)
    assert H.gmh_optimizer_lr(o) == 0.25 and H.gmh_optimizer_step_count(o) == 17
    back = H.gmh_optimizer_get_state(o)
    got = np.zeros(6, np.float32)
    H.gmh_state_tensor_data(back, 3, got.ctypes.data)                    # momentum_1
    assert np.array_equal(got, data)
    H.gmh_state_destroy(back)
    H.gmh_state_destroy(new)

    wrong = H.gmh_state_new(b"Adam")
    assert H.gmh_optimizer_load_state(o, wrong) != 0 and HL.err(H) == "state type mismatch: expected RMSProp, got Adam"
    H.gmh_state_destroy(wrong)
    for name, stype, n, msg in [(b"momentum_7", b"momentum", 6, "invalid buffer index in tensor name: momentum_7"),
                                (b"momentum", b"momentum", 6, "invalid buffer index in tensor name: momentum"),
                                (b"momentum_0", b"momentum", 5, "data size mismatch for momentum_0: expected 6 elements, got 5"),
                                (b"variance_0", b"variance", 6, "unknown state type: variance")]:
        bad = H.gmh_state_new(b"RMSProp")
        H.gmh_state_add_tensor(bad, name, stype, data.ctypes.data, n)
        assert H.gmh_optimizer_load_state(o, bad) != 0 and HL.err(H) == msg
        H.gmh_state_destroy(bad)
    # step_count stored as uint64 (what GetState itself produces) is accepted too
    u = H.gmh_state_new(b"RMSProp")
    H.gmh_state_set_uint64(u, b"step_count", 99)
    assert H.gmh_optimizer_load_state(o, u) == 0 and H.gmh_optimizer_step_count(o) == 99
    H.gmh_state_destroy(u)
    H.gmh_optimizer_cleanup(o)
    assert H.gmh_optimizer_stat(o, b"TotalBufferSize") == 0
    H.gmh_optimizer_destroy(o)


def test_mixed_adam_host_logic(env):
    """The mixed-precision optimizer type: defaults of training/model_trainer.go:258-270 reach the backend,
    the tensor list has the five streams (g16, master, m, v, p16) and is rebuilt only when a pointer changes,
    the checkpoint payload carries the loss-scale fields and survives a float64 (JSON) round trip."""
    H, fake, mm, dev = env
    shapes = [[4, 3], [5]]
    o = HL.make_optimizer(H, "MixedAdam", [], shapes, mm, dev)
    assert o, HL.err(H)
    assert H.gmh_optimizer_type(o) == b"MixedAdam" and abs(H.gmh_optimizer_lr(o) - 0.001) < 1e-9
    assert fake.fake_calls(HL.MIXED_CREATE) == 1 and fake.fake_allocs() == 6          # master, m, v per weight
    assert H.gmh_optimizer_stat(o, b"TotalBufferSize") == 3 * (12 + 5) * 4
    ls = HL.LossScaleC()
    assert H.gmh_mixed_loss_scale(o, C.byref(ls)) == 0
    assert (ls.scale, ls.growth, ls.backoff, ls.interval, ls.max_scale) == (65536.0, 2.0, 0.5, 2000, 16777216.0)

    w16 = [H.gmh_mm_allocate(mm, 24), H.gmh_mm_allocate(mm, 10)]
    g16 = [H.gmh_mm_allocate(mm, 24), H.gmh_mm_allocate(mm, 10)]
    assert H.gmh_optimizer_step(o, HL.uarr(g16), 2, 0.0) != 0 and "weight buffer 0 is nil" in HL.err(H)
    assert H.gmh_optimizer_set_weight_buffers(o, HL.uarr(w16[:1]), 1) != 0
    assert H.gmh_optimizer_set_weight_buffers(o, HL.uarr(w16), 2) == 0
    assert H.gmh_optimizer_step(o, HL.uarr(g16[:1]), 1, 0.0) != 0
    assert HL.err(H) == "gradient buffers length (1) doesn't match weight buffers length (2)"
    for _ in range(3):
        assert H.gmh_optimizer_step(o, HL.uarr(g16), 2, 0.0) == 0, HL.err(H)
    assert fake.fake_calls(HL.MIXED_STEP) == 3 and fake.fake_calls(HL.LIST_CREATE) == 1
    assert (fake.fake_list_streams(), fake.fake_list_tensors()) == (5, 2)
    assert [fake.fake_list_elem_bytes(s) for s in range(5)] == [2, 4, 4, 4, 2]
    assert abs(fake.fake_last_float(0) - 0.001) < 1e-9 and abs(fake.fake_last_float(3) - 1e-8) < 1e-12
    g16b = [g16[1], g16[0]]
    g16b[1] = H.gmh_mm_allocate(mm, 24)
    assert H.gmh_optimizer_step(o, HL.uarr([g16b[1], g16[1]]), 2, 0.0) == 0
    assert fake.fake_calls(HL.LIST_CREATE) == 2 and fake.fake_calls(HL.LIST_DESTROY) == 1   # new gradient buffer: new list
    assert H.gmh_optimizer_step_count(o) == 4
    fake.fake_next_return(-8)
    assert H.gmh_optimizer_step(o, HL.uarr([g16b[1], g16[1]]), 2, 0.0) != 0
    assert "MixedAdam step failed with error code: -8" in HL.err(H)

    master = np.arange(12, dtype=np.float32) / 8
    assert H.gmh_mixed_init_master(o, 0, master.ctypes.data, 12) == 0
    assert H.gmh_mixed_init_master(o, 0, master.ctypes.data, 11) != 0
    assert HL.err(H) == "data size mismatch for master_0: expected 12 elements, got 11"
    st = H.gmh_optimizer_get_state(o)
    assert st and H.gmh_state_type(st) == b"MixedAdam"
    names = [H.gmh_state_tensor_name(st, i).decode() for i in range(H.gmh_state_num_tensors(st))]
    assert names == ["master_0", "master_1", "momentum_0", "momentum_1", "variance_0", "variance_1"]
    got = np.zeros(12, np.float32)
    H.gmh_state_tensor_data(st, 0, got.ctypes.data)
    assert np.array_equal(got, master)
    val = C.c_double()
    kinds = {}
    for key in (b"loss_scale", b"growth_factor", b"backoff_factor", b"max_loss_scale", b"growth_interval", b"good_steps",
                b"skipped_steps", b"adam_step", b"step_count", b"learning_rate"):
        kinds[key] = (H.gmh_state_get_param(st, key, C.byref(val)), val.value)
    assert kinds[b"loss_scale"] == (3, 65536.0) and kinds[b"growth_interval"] == (2, 2000.0)
    assert kinds[b"adam_step"] == (2, 4.0) and kinds[b"step_count"] == (2, 5.0) and kinds[b"good_steps"] == (2, 4.0)
    H.gmh_state_destroy(st)

    # resume into a fresh optimizer from a payload whose numbers are all float64, as after JSON
    o2 = HL.make_optimizer(H, "MixedAdam", [], shapes, mm, dev)
    new = H.gmh_state_new(b"MixedAdam")
    for key, v in ((b"loss_scale", 1024.0), (b"good_steps", 77.0), (b"skipped_steps", 3.0), (b"adam_step", 40.0),
                   (b"step_count", 43.0), (b"learning_rate", 0.5), (b"growth_interval", 100.0)):
        H.gmh_state_set_float64(new, key, v)
    H.gmh_state_add_tensor(new, b"master_0", b"master", master.ctypes.data, 12)
    assert H.gmh_optimizer_load_state(o2, new) == 0, HL.err(H)
    assert H.gmh_mixed_loss_scale(o2, C.byref(ls)) == 0
    assert (ls.scale, ls.good_steps, ls.skipped, ls.adam_t, ls.interval, ls.growth) == (1024.0, 77, 3, 40, 100, 2.0)
    assert H.gmh_optimizer_step_count(o2) == 43 and H.gmh_optimizer_lr(o2) == 0.5
    got[:] = 0
    assert H.gmh_mixed_read_master(o2, 0, got.ctypes.data, 12) == 0 and np.array_equal(got, master)
    H.gmh_state_set_float64(new, b"beta1", 0.5)
    assert H.gmh_optimizer_load_state(o2, new) != 0 and "beta1/beta2 of the saved state" in HL.err(H)
    H.gmh_state_destroy(new)
    wrong = H.gmh_state_new(b"Adam")
    assert H.gmh_optimizer_load_state(o2, wrong) != 0 and HL.err(H) == "state type mismatch: expected MixedAdam, got Adam"
    H.gmh_state_destroy(wrong)
    for cfg, msg in (([0.001, 0.9, 0.999, 1e-8, 0, 0.0], "initial loss scale must be positive"),
                     ([0.001, 0.9, 0.999, 1e-8, 0, 65536, 0.5], "growth factor must be at least 1"),
                     ([0.001, 0.9, 0.999, 1e-8, 0, 65536, 2, 1.0], "backoff factor must be in (0, 1)"),
                     ([0.001, 0.9, 0.999, 1e-8, 0, 65536, 2, 0.5, 0], "growth interval must be positive")):
        assert not HL.make_optimizer(H, "MixedAdam", cfg, shapes, mm, dev) and msg in HL.err(H)
    H.gmh_optimizer_destroy(o)
    H.gmh_optimizer_destroy(o2)
    assert fake.fake_calls(HL.MIXED_DESTROY) == 2


def test_checkpoint_json_round_trip(env):
    """checkpoints/checkpoint.go:74-86: field names of the payload; after a JSON round trip
    every parameter number is a float64 (what Go's decoder hands to LoadState) and every
    tensor value has the bits it was saved with -- denormals, -0 and extremes included."""
    import json
    H, fake, mm, dev = env
    shapes = [[5], [2, 2]]
    o = HL.make_optimizer(H, "Adam", [], shapes, mm, dev)
    data = np.array([1.0, -0.0, 1e-42, 3.4028235e38, 0.1], np.float32)
    src = H.gmh_state_new(b"Adam")
    H.gmh_state_set_uint64(src, b"step_count", 12345678901)
    H.gmh_state_set_bool(src, b"nesterov", 1)
    H.gmh_state_set_float64(src, b"learning_rate", 0.001)
    H.gmh_state_add_tensor(src, b"momentum_0", b"momentum", data.ctypes.data, 5)
    H.gmh_state_add_tensor(src, b"variance_1", b"variance", (data[:4] * np.float32(0.5)).ctypes.data, 4)
    text = H.gmh_state_to_json(src)
    assert text, HL.err(H)
    doc = json.loads(text.decode())
    assert set(doc) == {"type", "parameters", "state_data"} and doc["type"] == "Adam"
    assert doc["parameters"] == {"learning_rate": 0.001, "nesterov": True, "step_count": 12345678901}
    assert [sorted(t) for t in doc["state_data"]] == [["data", "name", "shape", "state_type"]] * 2
    assert doc["state_data"][0]["shape"] == [5] and doc["state_data"][0]["state_type"] == "momentum"
    back = H.gmh_state_from_json(text)
    assert back, HL.err(H)
    val = C.c_double()
    assert H.gmh_state_get_param(back, b"step_count", C.byref(val)) == 0 and val.value == 12345678901.0   # float64 now
    assert H.gmh_state_get_param(back, b"nesterov", C.byref(val)) == 1 and val.value == 1.0
    assert H.gmh_state_get_param(back, b"learning_rate", C.byref(val)) == 0 and val.value == 0.001
    got = np.zeros(5, np.float32)
    H.gmh_state_tensor_data(back, 0, got.ctypes.data)
    assert np.array_equal(got.view(np.uint32), data.view(np.uint32))
    assert H.gmh_state_tensor_name(back, 1) == b"variance_1" and H.gmh_state_tensor_shape0(back, 1) == 4
    # the decoded payload loads: step_count arrives as float64, tensors land in the buffers
    assert H.gmh_optimizer_load_state(o, back) == 0, HL.err(H)
    assert H.gmh_optimizer_step_count(o) == 12345678901
    # what a Go writer produces loads too: other key order, whitespace, an unknown field, null slices
    go_text = (b'{ "state_data": [ {"state_type": "variance", "data": [0.25, 1e-3], "shape": [2], "name": "variance_0", "x": [1, {"y": null}]} ],'
               b' "extra": "ignored", "parameters": {"beta1": 0.9, "step_count": 7, "note": "text"}, "type": "Adam" }')
    g = H.gmh_state_from_json(go_text)
    assert g, HL.err(H)
    assert H.gmh_state_type(g) == b"Adam" and H.gmh_state_num_tensors(g) == 1 and H.gmh_state_tensor_numel(g, 0) == 2
    assert H.gmh_state_get_param(g, b"note", C.byref(val)) == -1
    empty = H.gmh_state_from_json(b'{"type":"SGD","parameters":{},"state_data":null}')
    assert empty and H.gmh_state_num_tensors(empty) == 0
    for bad in (b"", b"{", b'{"type":"Adam"} x', b'{"type":5}', b'{"state_data":[{"data":[1,}]}'):
        assert not H.gmh_state_from_json(bad) and "invalid checkpoint JSON" in HL.err(H)
    # json.Marshal refuses NaN and infinities; so does the encoder
    nan = H.gmh_state_new(b"Adam")
    H.gmh_state_add_tensor(nan, b"momentum_0", b"momentum", np.array([np.nan], np.float32).ctypes.data, 1)
    assert not H.gmh_state_to_json(nan) and "unsupported value" in HL.err(H)
    for st in (src, back, g, empty, nan):
        H.gmh_state_destroy(st)
    H.gmh_optimizer_destroy(o)


# ---------------- schedulers ----------------

def test_scheduler_tables(H):
    """training/scheduler_test.go:8-109"""
    s = H.gmh_sched_create(0, 2, 0.1, 0.0, b"")
    for epoch, want in [(0, 0.1), (1, 0.1), (2, 0.01), (3, 0.01), (4, 0.001), (5, 0.001), (6, 0.0001)]:
        assert abs(H.gmh_sched_get_lr(s, epoch, 0, 0.1) - want) <= 1e-8
    assert H.gmh_sched_name(s) == b"StepLR"
    H.gmh_sched_destroy(s)
    s = H.gmh_sched_create(1, 0, 0.9, 0.0, b"")
    for epoch, want in [(0, 0.1), (1, 0.09), (2, 0.081), (3, 0.0729), (4, 0.06561), (5, 0.059049)]:
        assert abs(H.gmh_sched_get_lr(s, epoch, 0, 0.1) - want) <= 1e-8
    assert H.gmh_sched_name(s) == b"ExponentialLR"
    H.gmh_sched_destroy(s)
    s = H.gmh_sched_create(2, 5, 0.0001, 0.0, b"")
    for epoch, want in [(0, 0.01), (5, 0.0001), (2, 0.006580)]:
        assert abs(H.gmh_sched_get_lr(s, epoch, 0, 0.01) - want) <= 1e-6
    assert H.gmh_sched_get_lr(s, 10, 0, 0.01) == 0.0001 and H.gmh_sched_name(s) == b"CosineAnnealingLR"
    H.gmh_sched_destroy(s)
    s = H.gmh_sched_create(3, 2, 0.5, 0.01, b"min")
    lr = H.gmh_sched_step(s, 1.0, 0.1)
    assert lr == 0.1
    lr = H.gmh_sched_step(s, 0.98, lr)
    assert lr == 0.1
    lr = H.gmh_sched_step(s, 0.99, lr)
    assert lr == 0.1
    lr = H.gmh_sched_step(s, 0.99, lr)
    assert lr == 0.05 and H.gmh_sched_name(s) == b"ReduceLROnPlateau" and H.gmh_sched_get_lr(s, 0, 0, 0.1) == 0.05
    H.gmh_sched_destroy(s)
    s = H.gmh_sched_create(4, 0, 0.0, 0.0, b"")
    assert H.gmh_sched_get_lr(s, 9, 9, 0.3) == 0.3 and H.gmh_sched_name(s) == b"ConstantLR"
    H.gmh_sched_destroy(s)
    # out-of-range constructor arguments fall back to the defaults (scheduler.go:27-36)
    s = H.gmh_sched_create(0, 0, 1.5, 0.0, b"")
    assert abs(H.gmh_sched_get_lr(s, 30, 0, 1.0) - 0.1) < 1e-12 and H.gmh_sched_get_lr(s, 29, 0, 1.0) == 1.0
    H.gmh_sched_destroy(s)
