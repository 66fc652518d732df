#!/usr/bin/env python
"""Benchmark of the optimizer-step hot path.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Headline workload (all N): fp32 Adam (lr 1e-3, betas 0.9/0.999, eps 1e-8, no decay)
on 1,073,741,824 parameters in 256 flat tensors of 4,194,304, He-uniform weights
and N(0, 0.01^2) gradients generated on the device from a fixed seed.  One step =
one pass of the update over all parameters.  At N > 1 the optimizer state and the
gradients are sharded ZeRO-1 style (rank r owns tensors [r*256/N, (r+1)*256/N))
and every step ends with the exchange of the updated fp32 parameters over
NVLink, so the total work is fixed (strong scaling).

`value` is timed with CUDA events on the stream the kernels are launched on,
inputs resident in HBM, max over ranks.  After the timed region (and outside it)
every rank compares a strided sample of its whole parameter arena with the CPU
oracle replayed over the same steps: `parity_check`.  `e2e` times the host-buffer
entry: every step copies that step's gradients from pinned host memory to the
device and the updated parameters back inside the timed region, pipelined slice
by slice.  At N = 1 a `workloads` block adds the other configurations, device
timed: mixed-precision Adam (25.2 M parameters, 48 ragged tensors), L-BFGS
(n = 10^7, history 10) and the other fp32 rules on 2^28 parameters.

`--impl reference` times the CPU restatement of the reference's Adam rule
(the oracle; the reference itself needs Apple Metal) on the host cores.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "go-metal_b200", "python"))
sys.path.insert(0, ROOT)

METRIC = "optimizer_step_throughput"
UNIT = "Gparams/s"
NUM_TENSORS = 256               # --tensors shrinks this for profiler captures only
TENSOR_ELEMS = 4_194_304
TOTAL = NUM_TENSORS * TENSOR_ELEMS
BYTES_PER_PARAM = 28            # read w,g,m,v (16) + write w,m,v (12)
SEED = 0x5EED601D
LR, B1, B2, EPS, WD = 1e-3, 0.9, 0.999, 1e-8, 0.0
WORKLOAD = "fp32 Adam, 2^30 params in 256 flat tensors of 4 Mi (config 4), ZeRO-1 over N GPUs"
# Both arms print exactly this object as `config`.
CONFIG = {"workload": WORKLOAD, "rule": "adam", "lr": LR, "beta1": B1, "beta2": B2, "eps": EPS, "weight_decay": WD,
          "params": 256 * TENSOR_ELEMS, "tensors": 256, "seed": SEED}
CPU_SAMPLE = 1 << 26            # parameters per CPU step (1/16 of the workload)
NVLINK_NOMINAL_GBS = 900.0      # per direction per GPU
NVLINK_MEASURED_GBS = 770.0     # peer copy measured on this pool, per direction


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def ncu_traffic_record():
    """DRAM bytes of one launch of the headline kernel from the committed ncu capture."""
    path = os.path.join(ROOT, "profiles", "adam_fp32_traffic.json")
    try:
        with open(path) as fh:
            return json.load(fh)
    except Exception:
        return None


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for name, bit in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": []}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


# ---------------------------------------------------------------------------
# CPU arm: the oracle timed on the host cores
# ---------------------------------------------------------------------------
def cpu_adam_rate(steps: int, warmup: int, sample_elems: int, budget_s: float | None, threads: int | None = None):
    """Returns (Gparams/s, threads used, steps_run, seconds_per_step)."""
    import numpy as np
    from oracle import oracle as O
    cores = threads or os.cpu_count() or 1
    n = sample_elems
    lim = float(np.sqrt(6.0 / 4096.0))
    O.set_threads(cores)
    w = O.fill_uniform(n, -lim, lim, SEED, 1)
    g = O.fill_normal(n, 0.0, 0.01, SEED, 2)
    O.set_threads(1)
    m = np.zeros(n, dtype=np.float32)
    v = np.zeros(n, dtype=np.float32)
    m.fill(0.0)                       # np.zeros maps pages lazily: touch them so that no timed step pays the page faults
    v.fill(0.0)
    step = 0
    for _ in range(warmup):
        step += 1
        O.adam_step(w, g, m, v, LR, B1, B2, EPS, WD, step, threads=cores)
    t0 = time.perf_counter()
    done = 0
    for _ in range(steps):
        step += 1
        O.adam_step(w, g, m, v, LR, B1, B2, EPS, WD, step, threads=cores)
        done += 1
        if budget_s is not None and time.perf_counter() - t0 > budget_s:
            break
    dt = time.perf_counter() - t0
    return n * done / dt / 1e9, cores, done, dt / done


def cpu_sample_text(done: int) -> str:
    return (f"{done} Adam steps over a {CPU_SAMPLE}-parameter slice (1/16 of the workload; same rule, same "
            "hyper-parameters), pthread split over all host cores")


def go_transcription_rate(sample_elems: int):
    """Times the Go twin of the oracle (oracle/go) when a Go toolchain is on PATH."""
    import shutil
    import subprocess
    if shutil.which("go") is None:
        return "no Go toolchain on this host; the C restatement stands in"
    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle", "go")
    try:
        out = subprocess.run(["go", "run", "./cmd/gmoracle_bench", "-n", str(sample_elems), "-steps", "3"],
                             cwd=here, capture_output=True, text=True, timeout=240, check=True).stdout
        return json.loads(out.strip().splitlines()[-1])
    except Exception as exc:                                   # a broken toolchain must not cost the bench line
        return f"go run failed: {exc}"


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    rate, cores, done, per_step = cpu_adam_rate(args.steps, args.warmup, CPU_SAMPLE, None)
    line = {
        "impl": "reference", "metric": METRIC, "value": rate, "unit": UNIT, "n_gpus": args.gpus,
        "steps": done, "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": dict(CONFIG),
        "cpu_baseline": {"value": rate, "unit": UNIT, "cores": cores, "kind": "port", "sample": cpu_sample_text(done),
                         "go_transcription": go_transcription_rate(CPU_SAMPLE)},
        "e2e": {"value": rate, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU restatement of the reference's Adam rule (oracle); the reference itself needs Apple Metal",
    }
    print(json.dumps(line))
    return 0


# ---------------------------------------------------------------------------
# GPU arm: the other configurations, device timed (N = 1)
# ---------------------------------------------------------------------------
def _event_timed(gm, dev, fn, reps, warm=3):
    L = gm.lib
    for _ in range(warm):
        fn()
    dev.sync()
    ms = C.c_float()
    gm.check(L.gm_timer_start(dev.h), "timer")
    for _ in range(reps):
        fn()
    gm.check(L.gm_timer_stop(dev.h, C.byref(ms)), "timer")
    return ms.value / reps


def _entry(name, params, ms, algorithmic_bpp, dram_bpp, dram_basis, peak, **extra):
    gbs_dram = dram_bpp * params / ms / 1e6
    d = {"name": name, "params": params, "ms": ms, "gparams_s": params / ms / 1e6,
         "algorithmic_bytes": algorithmic_bpp * params, "dram_bytes": dram_bpp * params, "dram_basis": dram_basis,
         "dram_gbs": gbs_dram, "frac": gbs_dram / peak}
    d.update(extra)
    return d


def workload_mixed(gm, dev, torch, peak, reps, clip=False):
    """Mixed-precision Adam on 25,165,824 parameters in 48 ragged tensors packed back to back;
    clip: with global-norm clipping (the norm is formed by the overflow-check pass)."""
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from workloads import ragged_sizes
    L = gm.lib
    sizes = ragged_sizes(48, 25_165_824, 4096, 4_194_304)
    n = sum(sizes)
    total = n + 32
    gen = torch.Generator(device="cuda")
    gen.manual_seed(SEED + 30)
    g16 = (torch.empty(total, dtype=torch.float32, device="cuda").normal_(0.0, 1e-3 * 65536.0, generator=gen)).to(torch.float16)
    w = torch.empty(total, dtype=torch.float32, device="cuda").uniform_(-0.05, 0.05, generator=gen)
    m = torch.zeros(total, dtype=torch.float32, device="cuda")
    v = torch.zeros(total, dtype=torch.float32, device="cuda")
    p16 = w.to(torch.float16)
    offs = np.concatenate([[0], np.cumsum(sizes)[:-1]]).astype(np.int64) + 1     # tensor starts off the 16-byte boundary
    eb = [2, 4, 4, 4, 2]
    ptrs = [[a.data_ptr() + e * int(o) for o in offs] for a, e in zip((g16, w, m, v, p16), eb)]
    lst = dev.tensor_list(ptrs, sizes, eb)
    init = gm.LossScale(scale=65536.0, growth=2.0, backoff=0.5, max_scale=16777216.0, interval=1 << 30,
                        good_steps=0, adam_t=0, skipped=0, last_overflow=0)    # the scale stays at 65536 while timing
    mx = L.gm_mixed_create(dev.h, C.byref(init), B1, B2, 0)
    if not mx:
        raise SystemExit("mixed state: " + gm.last_error())
    if clip:
        gm.check(L.gm_mixed_set_clip(mx, 0.1), "clip")         # ||g|| is about 1e-3 * sqrt(25.2 M) = 5: every step is clipped
    torch.cuda.synchronize()
    ms = _event_timed(gm, dev, lambda: gm.check(L.gm_mixed_step_async(dev.h, mx, lst, LR, EPS, WD), "mixed"), reps)
    st = gm.LossScale()
    gm.check(L.gm_mixed_get_state(dev.h, mx, C.byref(st)), "state")
    L.gm_mixed_destroy(mx)
    L.gm_tensor_list_destroy(lst)
    del g16, w, m, v, p16
    name = "mixed-precision Adam, 25,165,824 params in 48 ragged tensors (config 3)"
    if clip:
        name += " with global-norm clipping"
    return _entry(name, n, ms, 30, 28,
                  "28 B/param: fp16 gradients once (the update re-reads them from L2), master/m/v read and "
                  "written, fp16 parameters written; ncu measured 705 MB per step = 28.0 B/param", peak,
                  kernels="mixed_check_kernel + mixed_update_kernel", steps_timed=reps, clean_steps=int(st.adam_t),
                  skipped_steps=int(st.skipped))


def workload_lbfgs(gm, dev, torch, peak, reps):
    """L-BFGS, n = 10,000,000, history 10: one iteration once the history is full."""
    import numpy as np
    L = gm.lib
    n, m = 10_000_000, 10
    z = lambda k: torch.zeros(k, dtype=torch.float32, device="cuda")
    x, g, old, d = (z(n) for _ in range(4))
    S, Y = [z(n) for _ in range(m)], [z(n) for _ in range(m)]
    RHO, ALPHA = [z(64) for _ in range(m)], z(64)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(SEED + 50)
    D = torch.pow(10.0, torch.empty(n, dtype=torch.float32, device="cuda").uniform_(-0.3, 0.3, generator=gen))
    b = torch.empty(n, dtype=torch.float32, device="cuda").normal_(0.0, 1.0, generator=gen)
    P = lambda ts: gm.uarray([t.data_ptr() for t in ts])
    hc = hi = 0
    times = []
    ms = C.c_float()
    step = C.c_float()
    for it in range(m + reps):
        torch.mul(D, x, out=g)                                 # gradient of the quadratic, outside the timed part
        g.sub_(b)
        torch.cuda.synchronize()
        gm.check(L.gm_timer_start(dev.h), "timer")
        rc = L.execute_lbfgs_step_cuda(dev.h, P([x]), P([g]), P([old]), P([d]), P(S), P(Y), P(RHO), ALPHA.data_ptr(), 1,
                                       gm.iarray([4 * n]), m, hc, hi, 1.0, 1e-4, 0.9, 20, 0.0, 0.0, C.byref(step))
        gm.check(rc, "lbfgs")
        gm.check(L.gm_timer_stop(dev.h, C.byref(ms)), "timer")
        if hc == m:
            times.append(ms.value)
        hi, hc = (hi + 1) % m, min(hc + 1, m)
    accepted = int(sum(1 for r in RHO if float(r[0]) != 0.0))
    med = float(np.median(times))
    del x, g, old, d, S, Y, RHO, ALPHA, D, b
    # bytes that must cross DRAM with the direction vector kept on chip: g 4; each of the 2h loop passes reads
    # two history vectors (8h + 8h); the final pass reads x, g, old_g, s_prev and writes x, old_g, s, y (32)
    must = 4 + 16 * m + 32
    return _entry("L-BFGS iteration, n = 10,000,000, history 10 full (config 5; working mode)", n, med, 44 + 32 * m, must,
                  f"{must} B/element: what has to cross DRAM if the direction vector never left the chip "
                  "(history vectors do not fit L2, so each is read once per loop); the kernels' own ncu "
                  "DRAM traffic is 198 B/element", peak,
                  kernels=f"{2 * m + 1} x lbfgs_axpy_dot_kernel + lbfgs_pass_kernel", iterations_timed=len(times),
                  pairs_accepted=accepted, timing="CUDA events around the synchronous drop-in entry, median")


def workload_rules(gm, dev, torch, peak, reps):
    L = gm.lib
    n, nt = 1 << 28, 64
    per = n // nt
    gen = torch.Generator(device="cuda")
    gen.manual_seed(SEED + 20)
    bufs = {k: torch.zeros(n, dtype=torch.float32, device="cuda") for k in ("w", "g", "s1", "s2")}
    bufs["g"].normal_(0.0, 0.01, generator=gen)
    ptrs = {k: [a.data_ptr() + 4 * per * t for t in range(nt)] for k, a in bufs.items()}
    rules = [
        ("NAdam", gm.RULE_NADAM, ["w", "g", "s1", "s2"], 28, dict(lr=2e-3, beta1=0.9, beta2=0.999, eps=1e-8)),
        ("AdaDelta", gm.RULE_ADADELTA, ["w", "g", "s1", "s2"], 28, dict(beta1=0.9, eps=1e-6)),
        ("SGD with momentum", gm.RULE_SGD, ["w", "g", "s1"], 20, dict(lr=0.01, beta1=0.9)),
        ("RMSProp", gm.RULE_RMSPROP, ["w", "g", "s1"], 20, dict(lr=0.01, beta1=0.99, eps=1e-8)),
        ("AdaGrad", gm.RULE_ADAGRAD, ["w", "g", "s1"], 20, dict(lr=0.01, eps=1e-10)),
    ]
    out = []
    # fp32 Adam with global-norm clipping: the fixed-order norm pass (4 B/param) and the clipped step (28)
    bufs["w"].uniform_(-0.05, 0.05, generator=gen)
    lst = dev.tensor_list([ptrs[k] for k in ("w", "g", "s1", "s2")], [per] * nt)
    hy = gm.Hyper(lr=LR, beta1=B1, beta2=B2, eps=EPS, step=1)
    cnt = {"t": 0}

    def clipped():
        cnt["t"] += 1
        hy.step = cnt["t"]
        gm.check(L.gm_step_with_clip_async(dev.h, gm.RULE_ADAM, lst, C.byref(hy), 1.0), "clipped adam")

    ms = _event_timed(gm, dev, clipped, reps)
    out.append(_entry("Adam with global-norm clipping, fp32, 2^28 params in 64 tensors", n, ms, 32, 32,
                      "gradients read twice (norm pass, then the step): 4 + 28 B/param", peak,
                      kernels="sumsq_canonical_kernel + mta_apply_kernel<AdamRule, clip>", steps_timed=reps))
    L.gm_tensor_list_destroy(lst)
    for name, rule, streams, bpp, hp in rules:
        bufs["w"].uniform_(-0.05, 0.05, generator=gen)         # one rule's state is not a valid state of the next
        bufs["s1"].zero_()
        bufs["s2"].zero_()
        torch.cuda.synchronize()
        lst = dev.tensor_list([ptrs[k] for k in streams], [per] * nt)
        hy = gm.Hyper(step=1, **hp)
        state = {"t": 0}

        def one():
            state["t"] += 1
            hy.step = state["t"]
            gm.check(L.gm_step_async(dev.h, rule, lst, C.byref(hy)), name)

        ms = _event_timed(gm, dev, one, reps)
        out.append(_entry(f"{name}, fp32, 2^28 params in 64 tensors", n, ms, bpp, bpp,
                          "every stream is read once and every written stream written once", peak,
                          kernels="mta_apply_kernel", steps_timed=reps))
        L.gm_tensor_list_destroy(lst)
    del bufs
    return out


def workload_small(gm, dev, torch, reps):
    """The two small configurations: everything is L2-resident, so the figure is microseconds per
    step, not bandwidth.  Config 1: Adam on the 101,770-parameter MLP (4 tensors); config 2: the
    five other rules on the 545,098-parameter CNN (8 tensors)."""
    L = gm.lib
    gen = torch.Generator(device="cuda")
    gen.manual_seed(SEED + 40)
    out = []

    def make(sizes, streams):
        n = sum(sizes)
        bufs = [torch.zeros(n, dtype=torch.float32, device="cuda") for _ in range(streams)]
        bufs[0].uniform_(-0.05, 0.05, generator=gen)
        bufs[1].normal_(0.0, 0.01, generator=gen)
        offs = [sum(sizes[:k]) for k in range(len(sizes))]
        return bufs, [[b.data_ptr() + 4 * o for o in offs] for b in bufs]

    mlp = [784 * 128, 128, 128 * 10, 10]
    cnn = [864, 32, 18432, 64, 524288, 128, 1280, 10]
    cases = [("config 1: Adam, MLP, 101,770 params in 4 tensors", gm.RULE_ADAM, mlp, 4,
              dict(lr=LR, beta1=B1, beta2=B2, eps=EPS)),
             ("config 2: SGD with momentum, CNN, 545,098 params in 8 tensors", gm.RULE_SGD, cnn, 3, dict(lr=0.01, beta1=0.9)),
             ("config 2: RMSProp", gm.RULE_RMSPROP, cnn, 3, dict(lr=0.01, beta1=0.99, eps=1e-8)),
             ("config 2: AdaGrad", gm.RULE_ADAGRAD, cnn, 3, dict(lr=0.01, eps=1e-10)),
             ("config 2: AdaDelta", gm.RULE_ADADELTA, cnn, 4, dict(beta1=0.9, eps=1e-6)),
             ("config 2: NAdam", gm.RULE_NADAM, cnn, 4, dict(lr=2e-3, beta1=0.9, beta2=0.999, eps=1e-8))]
    for name, rule, sizes, streams, hp in cases:
        bufs, ptrs = make(sizes, streams)
        lst = dev.tensor_list(ptrs, sizes)
        hy = gm.Hyper(step=1, **hp)
        state = {"t": 0}

        def one():
            state["t"] += 1
            hy.step = state["t"]
            gm.check(L.gm_step_async(dev.h, rule, lst, C.byref(hy)), name)

        n_async = max(reps, 20) * 10
        us_async = _event_timed(gm, dev, one, n_async) * 1e3
        # the same step, synchronous: returns with the results in the buffers, as the reference's entry does
        for _ in range(3):
            one(); dev.sync()
        t0 = time.perf_counter()
        for _ in range(n_async):
            one(); dev.sync()
        us_sync = (time.perf_counter() - t0) / n_async * 1e6
        out.append({"name": name, "params": sum(sizes), "us_per_step_back_to_back": us_async,
                    "us_per_step_synchronous": us_sync, "steps_timed": n_async,
                    "note": "L2-resident: latency-bound, one launch per step"})
        L.gm_tensor_list_destroy(lst)
        del bufs
    return out


def run_only(args):
    """Profiler captures: one of the other configurations alone, a few repetitions, one JSON line."""
    import torch
    import gometal_cuda as gm
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; the optimizer step has no CPU path")
    torch.cuda.set_device(0)
    dev = gm.Device(0)
    peak, _ = measured_peak_gbs()
    fn = {"mixed": workload_mixed, "mixed_clip": lambda *a: workload_mixed(*a, clip=True), "lbfgs": workload_lbfgs,
          "rules": workload_rules, "small": lambda gm_, dev_, torch_, peak_, reps_: workload_small(gm_, dev_, torch_, reps_)}[args.only]
    out = fn(gm, dev, torch, peak, max(args.steps, 1))
    dev.close()
    print(json.dumps({"only": args.only, "result": out}))
    return 0


def mixed_scaling_case(gm, dev, torch, dist, zero1, rank, world, steps, exchange_wanted):
    """Second scaling case: mixed-precision Adam on the headline's 2^30 parameters (256 flat
    tensors of 4 Mi), master weights, moments and fp16 gradients sharded over the ranks, the
    fp16 parameter arena exchanged every step (2 B/param instead of 4).  Strong scaling.
    Returns the block for the JSON line (rank 0) or None."""
    import numpy as np
    L = gm.lib
    per_rank = 256 // world
    shard = per_rank * TENSOR_ELEMS
    total = 256 * TENSOR_ELEMS
    first = rank * per_rank
    gen = torch.Generator(device="cuda")
    gen.manual_seed(SEED + 77)
    p16 = torch.empty(total, dtype=torch.float32, device="cuda").uniform_(-0.05, 0.05, generator=gen).to(torch.float16)
    master = p16[first * TENSOR_ELEMS: first * TENSOR_ELEMS + shard].to(torch.float32)
    gen.manual_seed(SEED + 78 + rank)
    g16 = torch.empty(shard, dtype=torch.float32, device="cuda").normal_(0.0, 1e-3 * 65536.0, generator=gen).to(torch.float16)
    m = torch.zeros(shard, dtype=torch.float32, device="cuda")
    v = torch.zeros(shard, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    tp = lambda a, eb, off=0: [a.data_ptr() + eb * (off + t) * TENSOR_ELEMS for t in range(per_rank)]
    lst = dev.tensor_list([tp(g16, 2), tp(master, 4), tp(m, 4), tp(v, 4), tp(p16, 2, first)], [TENSOR_ELEMS] * per_rank, [2, 4, 4, 4, 2])
    init = gm.LossScale(scale=65536.0, growth=2.0, backoff=0.5, max_scale=16777216.0, interval=1 << 30,
                        good_steps=0, adam_t=0, skipped=0, last_overflow=0)
    mx = L.gm_mixed_create(dev.h, C.byref(init), B1, B2, 0)
    if not mx:
        raise SystemExit("mixed state: " + gm.last_error())
    exchange = "none"
    if world > 1:
        exchange = "push" if exchange_wanted in ("push", "dma") else "nccl"
        if exchange == "push":
            mine_h = (C.c_ubyte * 64)()
            rc = L.gm_zero1_ipc_handle_slot(zero1, 1, p16.data_ptr(), mine_h)
            ok = torch.tensor([1 if rc == 0 else 0], device="cuda")
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if int(ok.item()) == 0:
                exchange = "nccl"
            else:
                mine_t = torch.tensor(list(bytes(mine_h)), dtype=torch.uint8, device="cuda")
                all_t = [torch.empty_like(mine_t) for _ in range(world)]
                dist.all_gather(all_t, mine_t)
                blob = bytes(b for tt in all_t for b in tt.cpu().tolist())
                gm.check(L.gm_zero1_open_peers_slot(zero1, 1, (C.c_ubyte * len(blob))(*blob)), "open peers (fp16 arena)")

    # the sample the parity check follows, taken before any step
    edge = np.concatenate([np.arange(0, 64), np.arange(shard - 64, shard)])
    idx_np = np.unique(np.concatenate([np.arange(0, total, 4099)] + [edge + r * shard for r in range(world)])).astype(np.int64)
    owner = idx_np // shard
    sel = owner == rank
    mine = torch.from_numpy(idx_np[sel] - rank * shard).cuda()
    pos = torch.from_numpy(np.nonzero(sel)[0]).cuda()

    def gather_samples(values_i32):
        buf = torch.zeros(idx_np.size, dtype=torch.int32, device="cuda")
        buf[pos] = values_i32
        if dist is not None:
            dist.all_reduce(buf, op=dist.ReduceOp.SUM)
        return buf.cpu().numpy()

    g_s = gather_samples(g16[mine].view(torch.int16).to(torch.int32)).astype(np.uint16)
    w_s = gather_samples(master[mine].view(torch.int32)).view(np.float32).copy()

    def step():
        if world == 1:
            gm.check(L.gm_mixed_step_async(dev.h, mx, lst, LR, EPS, WD), "mixed step")
        elif exchange == "push":
            gm.check(L.gm_zero1_mixed_push_step_async(zero1, mx, lst, LR, EPS, WD), "zero1 mixed push step")
        else:
            gm.check(L.gm_zero1_mixed_step_async(zero1, mx, lst, LR, EPS, WD, p16.data_ptr(), shard), "zero1 mixed step")

    def sync_all():
        dev.sync()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()

    def max_ranks(x):
        if dist is None:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    done = 0
    for _ in range(3):
        step()
        done += 1
    sync_all()
    ms = C.c_float()
    gm.check(L.gm_timer_start(dev.h), "timer")
    for _ in range(steps):
        step()
        done += 1
    gm.check(L.gm_timer_stop(dev.h, C.byref(ms)), "timer")
    sync_all()
    step_ms = max_ranks(float(ms.value)) / steps

    # parity: the sampled fp16 parameters of the whole arena on every rank, and the owner's master weights
    from oracle import oracle as O
    st = O.new_loss_scale(interval=1 << 30)
    m_s, v_s, p_s = np.zeros_like(w_s), np.zeros_like(w_s), np.zeros(w_s.size, np.uint16)
    for _ in range(done):
        O.mixed_adam_step([g_s], [w_s], [m_s], [v_s], [p_s], LR, B1, B2, EPS, WD, st)
    got_p = p16[torch.from_numpy(idx_np).cuda()].view(torch.int16).cpu().numpy().view(np.uint16)
    ok = bool(np.array_equal(got_p, p_s)) and bool(np.array_equal(master[mine].cpu().numpy().view(np.uint32), w_s[sel].view(np.uint32)))
    flag = torch.tensor([1 if ok else 0], device="cuda")
    if dist is not None:
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)

    update_ms = step_ms
    if world > 1:
        gm.check(L.gm_timer_start(dev.h), "timer")
        for _ in range(steps):
            gm.check(L.gm_mixed_step_async(dev.h, mx, lst, LR, EPS, WD), "mixed step")
        gm.check(L.gm_timer_stop(dev.h, C.byref(ms)), "timer")
        sync_all()
        update_ms = max_ranks(float(ms.value)) / steps
    L.gm_mixed_destroy(mx)
    L.gm_tensor_list_destroy(lst)
    sync_all()
    peak, peak_kind = measured_peak_gbs()
    bytes_in = 2 * (total - shard)
    out = {
        "workload": "mixed-precision Adam, 2^30 params in 256 flat tensors of 4 Mi, state sharded over N GPUs, fp16 parameters exchanged",
        "exchange": exchange, "ms_per_step": step_ms, "gparams_s": total / step_ms / 1e6, "steps": steps,
        "update_only_ms_per_step": update_ms,
        "update_dram_gbs": 28 * shard / update_ms / 1e6, "update_frac": 28 * shard / update_ms / 1e6 / peak, "peak_source": f"of {peak_kind}",
        "dram_basis": "28 B/param (fp16 gradients once, master/m/v read and written, fp16 parameters written)",
        "exchange_bytes_in_per_gpu": bytes_in,
        "exchange_gbs_in_per_gpu": bytes_in / step_ms / 1e6 if world > 1 else 0.0,
        "exchange_floor_ms_at_770": bytes_in / NVLINK_MEASURED_GBS / 1e6,
        "parity_check": {"ranks": world, "sampled": int(idx_np.size), "steps_replayed": done, "ok": bool(int(flag.item()) == 1)},
    }
    del p16, master, g16, m, v
    torch.cuda.empty_cache()
    return out if rank == 0 else None


def run_workloads(gm, dev, torch, reps):
    peak, peak_kind = measured_peak_gbs()
    entries = [workload_mixed(gm, dev, torch, peak, max(reps, 20))]
    torch.cuda.empty_cache()
    entries.append(workload_mixed(gm, dev, torch, peak, max(reps, 20), clip=True))
    torch.cuda.empty_cache()
    entries.append(workload_lbfgs(gm, dev, torch, peak, max(reps // 2, 8)))
    torch.cuda.empty_cache()
    entries.extend(workload_rules(gm, dev, torch, peak, max(reps // 2, 10)))
    torch.cuda.empty_cache()
    small = workload_small(gm, dev, torch, reps)
    return {"peak_gbs": peak, "peak_source": f"of {peak_kind}", "timing": "CUDA events on the launching stream, after warm-up; "
            "every list is larger than the 126 MB L2", "entries": entries, "small_configs": small}


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
def run_gpu(args):
    import numpy as np
    import torch
    import gometal_cuda as gm
    L = gm.lib
    global NUM_TENSORS, TOTAL
    if args.tensors != NUM_TENSORS:
        NUM_TENSORS = args.tensors
        TOTAL = NUM_TENSORS * TENSOR_ELEMS

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; the optimizer step has no CPU path")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    dev = gm.Device(local)
    per_rank_tensors = NUM_TENSORS // world
    shard_elems = per_rank_tensors * TENSOR_ELEMS
    first = rank * per_rank_tensors

    # --- arenas (torch is used for device memory and the random fills only) ---
    gen = torch.Generator(device="cuda")
    gen.manual_seed(SEED)                               # same weights on every rank
    lim = (6.0 / 4096.0) ** 0.5
    w_arena = torch.empty(TOTAL, dtype=torch.float32, device="cuda").uniform_(-lim, lim, generator=gen)
    gen.manual_seed(SEED + 1 + rank)
    grads = [torch.empty(shard_elems, dtype=torch.float32, device="cuda").normal_(0.0, 0.01, generator=gen)
             for _ in range(2)]                         # two gradient sets, alternated step by step
    m_arena = torch.zeros(shard_elems, dtype=torch.float32, device="cuda")
    v_arena = torch.zeros(shard_elems, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()

    def tensor_ptrs(base, offset_tensors=0):
        return [base + 4 * (offset_tensors + t) * TENSOR_ELEMS for t in range(per_rank_tensors)]

    w_ptrs = tensor_ptrs(w_arena.data_ptr(), first)
    m_ptrs = tensor_ptrs(m_arena.data_ptr())
    v_ptrs = tensor_ptrs(v_arena.data_ptr())
    g_ptrs = [tensor_ptrs(g.data_ptr()) for g in grads]
    numel = [TENSOR_ELEMS] * per_rank_tensors
    lists = [dev.tensor_list([w_ptrs, gp, m_ptrs, v_ptrs], numel) for gp in g_ptrs]

    # --- the sample the parity check follows: a stride over the whole arena plus both ends of every shard ---
    edge = np.concatenate([np.arange(0, 64), np.arange(shard_elems - 64, shard_elems)])
    idx_np = np.unique(np.concatenate([np.arange(0, TOTAL, 4099)] + [edge + r * shard_elems for r in range(world)])).astype(np.int64)
    idx = torch.from_numpy(idx_np).cuda()
    w0_sample = w_arena[idx].cpu().numpy()              # before any step
    owner = idx_np // shard_elems
    mine = torch.from_numpy(idx_np[owner == rank] - rank * shard_elems).cuda()

    zero1 = 0
    exchange = "none"
    if world > 1:
        uid = (C.c_ubyte * 128)()
        if rank == 0:
            gm.check(L.gm_zero1_unique_id(uid), "nccl unique id")
        t = torch.tensor(list(bytes(uid)), dtype=torch.uint8, device="cuda")
        dist.broadcast(t, 0)
        uid = (C.c_ubyte * 128)(*t.cpu().tolist())
        zero1 = L.gm_zero1_create(dev.h, uid, rank, world)
        if not zero1:
            raise SystemExit("ZeRO-1 group creation failed: " + gm.last_error())
        exchange = args.exchange
        if exchange in ("push", "dma"):
            mine_h = (C.c_ubyte * 64)()
            rc = L.gm_zero1_ipc_handle(zero1, w_arena.data_ptr(), mine_h)
            # torch may have carved the arena out of a larger segment, which cannot be exported to
            # the peers; every rank then takes the NCCL all-gather instead
            ok = torch.tensor([1 if rc == 0 else 0], device="cuda")
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if int(ok.item()) == 0:
                exchange = "nccl"
                if rank == 0:
                    print(f"peer mapping unavailable ({gm.last_error()}); using the NCCL all-gather", file=sys.stderr)
        if exchange in ("push", "dma"):
            mine_t = torch.tensor(list(bytes(mine_h)), dtype=torch.uint8, device="cuda")
            all_t = [torch.empty_like(mine_t) for _ in range(world)]
            dist.all_gather(all_t, mine_t)
            blob = bytes(b for tt in all_t for b in tt.cpu().tolist())
            gm.check(L.gm_zero1_open_peers(zero1, (C.c_ubyte * len(blob))(*blob)), "open peers")

    hyper = gm.Hyper(lr=LR, beta1=B1, beta2=B2, eps=EPS, weight_decay=WD, step=0)
    step_no = [0]

    def one_step():
        step_no[0] += 1
        hyper.step = step_no[0]
        lst = lists[step_no[0] % 2]
        if world == 1:
            gm.check(L.gm_step_async(dev.h, gm.RULE_ADAM, lst, C.byref(hyper)), "adam step")
        elif exchange == "push":
            gm.check(L.gm_zero1_adam_push_step_async(zero1, lst, C.byref(hyper)), "zero1 push step")
        elif exchange == "dma":
            gm.check(L.gm_zero1_adam_dma_step_async(zero1, lst, C.byref(hyper), args.slices), "zero1 dma step")
        else:
            gm.check(L.gm_zero1_adam_step_async(zero1, lst, C.byref(hyper), w_arena.data_ptr(), shard_elems),
                     "zero1 step")

    def barrier():
        dev.sync()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()

    def max_over_ranks(x: float) -> float:
        if dist is None:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        one_step()
    barrier()

    # --- timed region: K steps, CUDA events on the launching stream ---
    sampler = ClockSampler(local)
    launches_before = L.gm_device_launch_count(dev.h)
    sampler.start()
    gm.check(L.gm_timer_start(dev.h), "timer")
    for _ in range(args.steps):
        one_step()
    ms = C.c_float()
    gm.check(L.gm_timer_stop(dev.h, C.byref(ms)), "timer")
    clocks = sampler.stop()
    launches = L.gm_device_launch_count(dev.h) - launches_before
    barrier()
    total_ms = max_over_ranks(float(ms.value))
    ms_per_step = total_ms / args.steps
    value = TOTAL / (ms_per_step * 1e-3) / 1e9

    # --- parity: the sampled elements of the WHOLE arena on every rank against the oracle, outside the timed region ---
    parity = None
    if not args.no_parity_check:
        from oracle import oracle as O
        steps_done = step_no[0]
        g_samples = []
        for gset in grads:                                      # every rank contributes the samples it owns (exact: int32 sum with zeros)
            buf = torch.zeros(idx.numel(), dtype=torch.int32, device="cuda")
            buf[torch.from_numpy(np.nonzero(owner == rank)[0]).cuda()] = gset[mine].view(torch.int32)
            if dist is not None:
                dist.all_reduce(buf, op=dist.ReduceOp.SUM)
            g_samples.append(buf.view(torch.float32).cpu().numpy())
        ws, ms_o, vs_o = w0_sample.copy(), np.zeros_like(w0_sample), np.zeros_like(w0_sample)
        for s in range(1, steps_done + 1):
            O.adam_step(ws, g_samples[s % 2], ms_o, vs_o, LR, B1, B2, EPS, WD, s)
        got_w = w_arena[idx].cpu().numpy()
        sel = owner == rank
        ok_w = bool(np.array_equal(got_w.view(np.uint32), ws.view(np.uint32)))
        ok_m = bool(np.array_equal(m_arena[mine].cpu().numpy().view(np.uint32), ms_o[sel].view(np.uint32)))
        ok_v = bool(np.array_equal(v_arena[mine].cpu().numpy().view(np.uint32), vs_o[sel].view(np.uint32)))
        flag = torch.tensor([1 if (ok_w and ok_m and ok_v) else 0], device="cuda")
        if dist is not None:
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        parity = {"ranks": world, "sampled": int(idx.numel()), "steps_replayed": steps_done, "ok": bool(int(flag.item()) == 1),
                  "what": "bit equality of the sampled parameters of the whole arena on every rank (and of the "
                          "owner's m and v) with the CPU oracle replayed over the same steps"}
        if not parity["ok"] and rank == 0:
            print("PARITY CHECK FAILED", file=sys.stderr)

    # --- update-only timing at N > 1 (the part the HBM roofline applies to) ---
    update_ms = ms_per_step
    if world > 1:
        gm.check(L.gm_timer_start(dev.h), "timer")
        for _ in range(args.steps):
            step_no[0] += 1
            hyper.step = step_no[0]
            gm.check(L.gm_step_async(dev.h, gm.RULE_ADAM, lists[step_no[0] % 2], C.byref(hyper)), "adam step")
        gm.check(L.gm_timer_stop(dev.h, C.byref(ms)), "timer")
        update_ms = max_over_ranks(float(ms.value)) / args.steps
        barrier()

    peak, peak_kind = measured_peak_gbs()
    achieved = BYTES_PER_PARAM * shard_elems / (update_ms * 1e-3) / 1e9
    rec = ncu_traffic_record()
    traffic = None
    if rec is not None:
        traffic = rec["dram_bytes_per_param"] * shard_elems
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": traffic, "traffic_source": (rec or {}).get("source"), "peak_source": f"of {peak_kind}",
                "kernel": "mta_apply_kernel<AdamRule>", "algorithmic_bytes_per_launch": BYTES_PER_PARAM * shard_elems,
                "kernel_ms": update_ms, "frac_of_8TBs_nominal": achieved / 8000.0}

    scaling_detail = None
    if world > 1:
        # the same update on the whole workload on one GPU, measured here so that the efficiency of the update
        # phase needs no number from another run
        full_ms = None
        if not args.no_full_update:
            gf = torch.empty(TOTAL, dtype=torch.float32, device="cuda").normal_(0.0, 0.01, generator=gen)
            mf = torch.zeros(TOTAL, dtype=torch.float32, device="cuda")
            vf = torch.zeros(TOTAL, dtype=torch.float32, device="cuda")
            wf = torch.empty(TOTAL, dtype=torch.float32, device="cuda").uniform_(-lim, lim, generator=gen)
            ptr_all = lambda a: [a.data_ptr() + 4 * t * TENSOR_ELEMS for t in range(NUM_TENSORS)]
            lf = dev.tensor_list([ptr_all(wf), ptr_all(gf), ptr_all(mf), ptr_all(vf)], [TENSOR_ELEMS] * NUM_TENSORS)
            hf = gm.Hyper(lr=LR, beta1=B1, beta2=B2, eps=EPS, weight_decay=WD, step=0)
            cnt = [0]

            def full_step():
                cnt[0] += 1
                hf.step = cnt[0]
                gm.check(L.gm_step_async(dev.h, gm.RULE_ADAM, lf, C.byref(hf)), "adam step")

            full_ms = max_over_ranks(_event_timed(gm, dev, full_step, 5))
            L.gm_tensor_list_destroy(lf)
            del gf, mf, vf, wf
            torch.cuda.empty_cache()
            barrier()
        bytes_in = 4 * (TOTAL - shard_elems)
        gbs_in = bytes_in / (ms_per_step * 1e-3) / 1e9
        scaling_detail = {
            "exchange": exchange,
            "update_only_ms_per_step": update_ms,
            "one_gpu_update_ms_measured_here": full_ms,
            "update_phase_efficiency": (full_ms / (world * update_ms)) if full_ms else None,
            "exchange_bytes_in_per_gpu": bytes_in,
            "exchange_gbs_in_per_gpu": gbs_in,
            "exchange_frac_of_900_nominal": gbs_in / NVLINK_NOMINAL_GBS,
            "exchange_frac_of_770_measured_peer_copy": gbs_in / NVLINK_MEASURED_GBS,
            "exchange_floor_ms_at_770": bytes_in / NVLINK_MEASURED_GBS / 1e6,
            "bound": "NVLink ingress: every GPU must receive 4*(N-1)/N bytes per parameter",
        }

    # --- end to end: host buffers through the host-buffer entries ---
    e2e = None
    if not args.skip_e2e:
        e2e_steps = max(10, min(args.steps, 20))
        host_g = torch.empty(shard_elems, dtype=torch.float32).pin_memory()
        host_g.copy_(grads[0].cpu())
        host_w = torch.empty(shard_elems, dtype=torch.float32).pin_memory()
        sizes = gm.iarray([4 * TENSOR_ELEMS] * per_rank_tensors)
        arr = {k: gm.uarray(p) for k, p in (("w", w_ptrs), ("g", g_ptrs[0]), ("m", m_ptrs), ("v", v_ptrs))}
        shard_bytes = 4 * shard_elems
        w_shard_ptr = w_arena.data_ptr() + 4 * first * TENSOR_ELEMS
        use_push_host = world > 1 and exchange == "push"

        def e2e_step_dropin():
            # upload, synchronous drop-in entry, download: nothing overlaps
            step_no[0] += 1
            gm.check(L.gm_buffer_upload_async(dev.h, grads[0].data_ptr(), host_g.data_ptr(), shard_bytes), "h2d")
            rc = L.execute_adam_step_cuda(dev.h, arr["w"], arr["g"], arr["m"], arr["v"], per_rank_tensors, sizes,
                                          LR, B1, B2, EPS, WD, step_no[0])
            gm.check(rc, "execute_adam_step_cuda")
            if world > 1:
                gm.check(L.gm_zero1_allgather_async(zero1, w_arena.data_ptr(), shard_elems, 4), "all-gather")
            gm.check(L.gm_buffer_download_async(dev.h, w_shard_ptr, host_w.data_ptr(), shard_bytes), "d2h")
            dev.sync()

        def e2e_step_host():
            # the host-buffer entry: upload, update (and exchange) and download pipelined slice by slice
            step_no[0] += 1
            hyper.step = step_no[0]
            if use_push_host:
                gm.check(L.gm_zero1_adam_push_step_host(zero1, lists[0], C.byref(hyper), host_g.data_ptr(), host_w.data_ptr(),
                                                        args.host_slices), "gm_zero1_adam_push_step_host")
                return
            gm.check(L.gm_step_host(dev.h, gm.RULE_ADAM, lists[0], C.byref(hyper), host_g.data_ptr(), host_w.data_ptr(),
                                    args.host_slices), "gm_step_host")
            if world > 1:
                gm.check(L.gm_zero1_allgather_async(zero1, w_arena.data_ptr(), shard_elems, 4), "all-gather")
                dev.sync()

        def time_e2e(fn, steps):
            fn()
            barrier()
            t0 = time.perf_counter()
            for _ in range(steps):
                fn()
            dt = max_over_ranks(time.perf_counter() - t0)
            barrier()
            return dt / steps

        # the floor of any host-buffer step: the same two copies, both directions at once, no kernel
        up, down = torch.cuda.Stream(), torch.cuda.Stream()
        g_dev = grads[0][:shard_elems]
        w_dev = w_arena[first * TENSOR_ELEMS: first * TENSOR_ELEMS + shard_elems]
        scratch_w = torch.empty_like(host_w).pin_memory()

        def copies_only():
            with torch.cuda.stream(up):
                g_dev.copy_(host_g, non_blocking=True)
            with torch.cuda.stream(down):
                scratch_w.copy_(w_dev, non_blocking=True)
            torch.cuda.synchronize()

        dropin_s = time_e2e(e2e_step_dropin, 3)
        e2e_s = time_e2e(e2e_step_host, e2e_steps)
        copy_s = time_e2e(copies_only, 5)
        del scratch_w
        api = ("gm_zero1_adam_push_step_host" if use_push_host else "gm_step_host" + (" + NCCL all-gather" if world > 1 else ""))
        e2e = {"value": TOTAL / e2e_s / 1e9, "unit": UNIT, "h2d_bytes_per_step": shard_bytes,
               "d2h_bytes_per_step": shard_bytes, "steps": e2e_steps, "ms_per_step": e2e_s * 1e3,
               "api": f"{api} (pinned host gradients in, updated parameters out, {args.host_slices} pipelined slices)",
               "copy_floor": {"ms_per_step": copy_s * 1e3,
                              "note": "the step's two host<->device copies alone, concurrent, no kernel; at N > 1 all "
                                      "ranks share the box's host<->device bandwidth, which is what bounds this leg"},
               "unpipelined": {"value": TOTAL / dropin_s / 1e9, "ms_per_step": dropin_s * 1e3, "steps": 3,
                               "api": "upload + execute_adam_step_cuda (synchronous drop-in entry) + download"}}

    for lst in lists:
        L.gm_tensor_list_destroy(lst)
    lists = []
    del grads, m_arena, v_arena, w_arena
    torch.cuda.empty_cache()

    workloads = None
    if world == 1 and not args.no_workloads and NUM_TENSORS == 256:
        workloads = run_workloads(gm, dev, torch, args.steps)
    mixed_case = None
    if not args.no_workloads and NUM_TENSORS == 256:
        mixed_case = mixed_scaling_case(gm, dev, torch, dist, zero1, rank, world, args.steps, exchange)

    line = None
    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            rate, cores, done, per = cpu_adam_rate(50, 1, CPU_SAMPLE, 12.0)
            one, _, done1, _ = cpu_adam_rate(4, 1, CPU_SAMPLE // 4, 3.0, threads=1)
            cpu = {"value": rate, "unit": UNIT, "cores": cores, "kind": "port", "sample": cpu_sample_text(done),
                   "single_thread": {"value": one, "unit": UNIT,
                                     "sample": f"{done1} steps over {CPU_SAMPLE // 4} parameters, one thread"}}
        cfg = dict(CONFIG)
        if NUM_TENSORS != 256:
            cfg["workload"] = f"REDUCED for profiling: {NUM_TENSORS} tensors"
            cfg["params"], cfg["tensors"] = TOTAL, NUM_TENSORS
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": cfg,
            "details": {"parallelism": f"zero1x{world}", "exchange": exchange,
                        "l2": "inputs (>= 2 GiB per rank) far exceed the 126 MB L2; no flush needed",
                        "hbm_gbs_algorithmic": BYTES_PER_PARAM * TOTAL / (ms_per_step * 1e-3) / 1e9},
            "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches), "roofline": roofline,
            "parity_check": parity, "cpu_baseline": cpu,
        }
        if scaling_detail is not None:
            line["zero1"] = scaling_detail
            line["update_only_ms_per_step"] = update_ms
        if workloads is not None:
            line["workloads"] = workloads
        if mixed_case is not None:
            line["zero1_mixed"] = mixed_case
    if zero1:
        L.gm_zero1_destroy(zero1)
    dev.close()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if line is not None:
        print(json.dumps(line))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--exchange", choices=["nccl", "push", "dma"], default="push")
    ap.add_argument("--slices", type=int, default=8, help="slices of the shard for --exchange dma")
    ap.add_argument("--host-slices", type=int, default=64, help="pipeline depth of the host-buffer step (e2e)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-workloads", action="store_true", help="leave out the block of other configurations (N = 1)")
    ap.add_argument("--no-parity-check", action="store_true")
    ap.add_argument("--no-full-update", action="store_true", help="N > 1: skip the one-GPU update timing behind update_phase_efficiency")
    ap.add_argument("--skip-e2e", action="store_true", help="profiling runs: leave out the host-buffer leg")
    ap.add_argument("--tensors", type=int, default=256,
                    help="profiling runs only: fewer 4 Mi tensors than the 256 of the workload")
    ap.add_argument("--only", choices=["mixed", "mixed_clip", "lbfgs", "rules", "small"],
                    help="profiling runs only: time one of the other configurations alone for --steps repetitions")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.only:
        return run_only(args)
    return run_gpu(args)


if __name__ == "__main__":
    sys.exit(main())
