#!/usr/bin/env python
"""Benchmark of the optimizer-step hot path.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Workload (all N): fp32 Adam (lr 1e-3, betas 0.9/0.999, eps 1e-8, no decay) on
1,073,741,824 parameters in 256 flat tensors of 4,194,304, He-uniform weights
and N(0, 0.01^2) gradients generated on the device from a fixed seed.  One
step = one pass of the update over all parameters.  At N > 1 the optimizer
state and the gradients are sharded ZeRO-1 style (rank r owns tensors
[r*256/N, (r+1)*256/N)) and every step ends with the exchange of the updated
fp32 parameters over NVLink, so the total work is fixed (strong scaling).

`value` is timed with CUDA events on the stream the kernels are launched on,
inputs resident in HBM, max over ranks.  `e2e` times the host-buffer entry
(gm_step_host): every step copies that step's gradients from pinned host
memory to the device and the updated parameters back to pinned host memory
inside the timed region, pipelined slice by slice; the same step through the
synchronous drop-in entry with plain copies is reported beside it.

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
# dram__bytes_read.sum + dram__bytes_write.sum of one mta_apply_kernel<AdamRule> launch,
# measured on a 16-tensor launch and scaled by the tensor count (traffic is proportional to it).
TRAFFIC_BYTES_PER_LAUNCH = 16 * (1.07389e9 + 0.75180e9)   # ncu, 16-tensor case: 1.074 GB read + 0.752 GB written, x16


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


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
def cpu_adam_rate(steps: int, warmup: int, sample_elems: int, budget_s: float | None):
    """Returns (Gparams/s, cores, steps_run, seconds_per_step)."""
    import numpy as np
    from oracle import oracle as O
    cores = os.cpu_count() or 1
    n = sample_elems
    lim = float(np.sqrt(6.0 / 4096.0))
    w = O.fill_uniform(n, -lim, lim, SEED, 1)
    g = O.fill_normal(n, 0.0, 0.01, SEED, 2)
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
    sample = 1 << 26
    rate, cores, done, per_step = cpu_adam_rate(args.steps, args.warmup, sample, None)
    line = {
        "impl": "reference", "metric": METRIC, "value": rate, "unit": UNIT, "n_gpus": args.gpus,
        "steps": done, "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": f"{sample} of {TOTAL} params per step"},
        "cpu_baseline": {"value": rate, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"{done} Adam steps over a {sample}-parameter slice (same rule, same "
                                   "hyper-parameters), pthread split over all host cores",
                         "go_transcription": go_transcription_rate(sample)},
        "e2e": {"value": rate, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU restatement of the reference's Adam rule (oracle); the reference itself needs Apple Metal",
    }
    print(json.dumps(line))
    return 0


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
def run_gpu(args):
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
            mine = (C.c_ubyte * 64)()
            rc = L.gm_zero1_ipc_handle(zero1, w_arena.data_ptr(), mine)
            # torch may have carved the arena out of a larger segment, which cannot be exported to
            # the peers; every rank then takes the NCCL all-gather instead
            ok = torch.tensor([1 if rc == 0 else 0], device="cuda")
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if int(ok.item()) == 0:
                exchange = "nccl"
                if rank == 0:
                    print(f"peer mapping unavailable ({gm.last_error()}); using the NCCL all-gather", file=sys.stderr)
        if exchange in ("push", "dma"):
            mine_t = torch.tensor(list(bytes(mine)), dtype=torch.uint8, device="cuda")
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

    for _ in range(max(args.warmup, 3)):
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

    # update-only timing at N > 1 (the part the HBM roofline applies to)
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
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": TRAFFIC_BYTES_PER_LAUNCH * shard_elems / (256 * TENSOR_ELEMS), "peak_source": f"of {peak_kind}",
                "kernel": "mta_apply_kernel<AdamRule>", "algorithmic_bytes_per_launch": BYTES_PER_PARAM * shard_elems,
                "kernel_ms": update_ms, "frac_of_8TBs_nominal": achieved / 8000.0}

    # --- end to end: host buffers through the drop-in entry ---
    if args.skip_e2e:
        return _finish(args, gm, L, dev, dist, lists, zero1, rank, world, value, ms_per_step, update_ms, clocks,
                       launches, roofline, None, exchange, shard_elems)
    e2e_steps = min(args.steps, 3)
    host_g = torch.empty(shard_elems, dtype=torch.float32).pin_memory()
    host_g.copy_(grads[0].cpu())
    host_w = torch.empty(shard_elems, dtype=torch.float32).pin_memory()
    sizes = gm.iarray([4 * TENSOR_ELEMS] * per_rank_tensors)
    arr = {k: gm.uarray(p) for k, p in (("w", w_ptrs), ("g", g_ptrs[0]), ("m", m_ptrs), ("v", v_ptrs))}
    shard_bytes = 4 * shard_elems
    w_shard_ptr = w_arena.data_ptr() + 4 * first * TENSOR_ELEMS

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
        # the host-buffer entry: upload, update and download pipelined slice by slice
        step_no[0] += 1
        hyper.step = step_no[0]
        gm.check(L.gm_step_host(dev.h, gm.RULE_ADAM, lists[0], C.byref(hyper), host_g.data_ptr(), host_w.data_ptr(),
                                args.host_slices), "gm_step_host")
        if world > 1:
            gm.check(L.gm_zero1_allgather_async(zero1, w_arena.data_ptr(), shard_elems, 4), "all-gather")
            dev.sync()

    def time_e2e(fn):
        fn()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            fn()
        dt = max_over_ranks(time.perf_counter() - t0)
        barrier()
        return dt

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

    dropin_s = time_e2e(e2e_step_dropin)
    e2e_s = time_e2e(e2e_step_host)
    copy_s = time_e2e(copies_only)
    del scratch_w
    e2e = {"value": TOTAL * e2e_steps / e2e_s / 1e9, "unit": UNIT, "h2d_bytes_per_step": shard_bytes,
           "d2h_bytes_per_step": shard_bytes, "steps": e2e_steps, "ms_per_step": e2e_s / e2e_steps * 1e3,
           "api": f"gm_step_host (pinned host gradients in, updated parameters out, {args.host_slices} pipelined slices)",
           "copy_floor": {"ms_per_step": copy_s / e2e_steps * 1e3,
                          "note": "the step's two host<->device copies alone, concurrent, no kernel"},
           "unpipelined": {"value": TOTAL * e2e_steps / dropin_s / 1e9, "ms_per_step": dropin_s / e2e_steps * 1e3,
                           "api": "upload + execute_adam_step_cuda (synchronous drop-in entry) + download"}}

    return _finish(args, gm, L, dev, dist, lists, zero1, rank, world, value, ms_per_step, update_ms, clocks,
                   launches, roofline, e2e, exchange, shard_elems)


def _finish(args, gm, L, dev, dist, lists, zero1, rank, world, value, ms_per_step, update_ms, clocks, launches,
            roofline, e2e, exchange, shard_elems):
    line = None
    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            rate, cores, done, per = cpu_adam_rate(50, 1, 1 << 26, 12.0)
            cpu = {"value": rate, "unit": UNIT, "cores": cores, "kind": "port",
                   "sample": f"{done} Adam steps over a {1 << 26}-parameter slice of the workload, "
                             "pthread split over all host cores"}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD if NUM_TENSORS == 256 else f"REDUCED for profiling: {NUM_TENSORS} tensors",
                       "params": TOTAL, "tensors": NUM_TENSORS,
                       "parallelism": f"zero1x{world}", "exchange": exchange,
                       "l2": "inputs (>= 2 GiB per rank) far exceed the 126 MB L2; no flush needed",
                       "hbm_gbs_algorithmic": BYTES_PER_PARAM * TOTAL / (ms_per_step * 1e-3) / 1e9},
            "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches), "roofline": roofline,
            "cpu_baseline": cpu,
        }
        if world > 1:
            line["update_only_ms_per_step"] = update_ms
            line["exchange_bytes_in_per_gpu"] = 4 * (TOTAL - shard_elems)
    for lst in lists:
        L.gm_tensor_list_destroy(lst)
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
    ap.add_argument("--skip-e2e", action="store_true", help="profiling runs: leave out the host-buffer leg")
    ap.add_argument("--tensors", type=int, default=256,
                    help="profiling runs only: fewer 4 Mi tensors than the 256 of the workload")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    return run_gpu(args)


if __name__ == "__main__":
    sys.exit(main())
