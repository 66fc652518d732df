"""One rank of the multi-GPU ZeRO-1 parity check (launched by
tests/test_zero1_multigpu.py through torch.distributed.run).

Every rank keeps the full parameter arena, updates its own shard with the CUDA
library and exchanges parameters: with the NCCL all-gather path, the fused
update+push kernel, the copy-engine path and the push path fed from host
buffers; after each step every rank's arena must equal, bit for bit, the
oracle's update of ALL tensors.
"""
import ctypes as C
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "go-metal_b200", "python"))
import gometal_cuda as gm  # noqa: E402
import zero1_plan as ZP  # noqa: E402
from oracle import oracle as O  # noqa: E402

T, E, STEPS = 16, 100_003, 4          # tensor starts are not 16-byte aligned inside the arena
LR, B1, B2, EPS, WD = 1e-3, 0.9, 0.999, 1e-8, 0.0


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    L = gm.lib
    dev = gm.Device(local)
    plan = ZP.make_plan(T, E, world, rank)

    uid = (C.c_ubyte * 128)()
    if rank == 0:
        gm.check(L.gm_zero1_unique_id(uid), "unique id")
    t = torch.tensor(list(bytes(uid)), dtype=torch.uint8, device="cuda")
    dist.broadcast(t, 0)
    uid = (C.c_ubyte * 128)(*t.cpu().tolist())
    z = L.gm_zero1_create(dev.h, uid, rank, world)
    assert z, gm.last_error()
    assert L.gm_zero1_rank(z) == rank and L.gm_zero1_world(z) == world

    # GM_TEST_EXCHANGES narrows the run to some exchange paths (and leaves out the mixed-precision
    # and reduce-scatter parts): used to repeat the push path under its other store orders.
    only = os.environ.get("GM_TEST_EXCHANGES")
    exchanges = tuple(only.split(",")) if only else ("nccl", "push", "dma", "push_host")
    for exchange in exchanges:
        w0 = O.fill_uniform(T * E, -0.1, 0.1, 91, 1)
        full, fm, fv = w0.copy(), np.zeros(T * E, np.float32), np.zeros(T * E, np.float32)
        arena = dev.to_device(w0)
        dg = dev.alloc(4 * plan.shard_elems)
        dm = dev.to_device(np.zeros(plan.shard_elems, np.float32))
        dv = dev.to_device(np.zeros(plan.shard_elems, np.float32))
        w_ptrs = [arena + 4 * plan.tensor_offset(k) for k in plan.owned]
        loc = lambda base: [base + 4 * plan.local_offset(k) for k in plan.owned]
        lst = dev.tensor_list([w_ptrs, loc(dg), loc(dm), loc(dv)], [E] * plan.tensors_per_rank)
        if exchange in ("push", "dma", "push_host"):
            mine = (C.c_ubyte * 64)()
            # an address inside the allocation cannot be exported: the peers would map the
            # allocation's first byte and store at the wrong offset
            assert L.gm_zero1_ipc_handle(z, arena + 256, mine) == -10, "interior pointer must be refused"
            gm.check(L.gm_zero1_ipc_handle(z, arena, mine), "ipc handle")
            mine_t = torch.tensor(list(bytes(mine)), dtype=torch.uint8, device="cuda")
            all_t = [torch.empty_like(mine_t) for _ in range(world)]
            dist.all_gather(all_t, mine_t)
            blob = bytes(b for tt in all_t for b in tt.cpu().tolist())
            gm.check(L.gm_zero1_open_peers(z, (C.c_ubyte * len(blob))(*blob)), "open peers")
            dist.barrier()
            # a shard list whose parameters are not in the exported arena must be refused, not run
            stray = dev.alloc(4 * plan.shard_elems)
            bad = dev.tensor_list([loc(stray), loc(dg), loc(dm), loc(dv)], [E] * plan.tensors_per_rank)
            hy0 = gm.Hyper(lr=LR, beta1=B1, beta2=B2, eps=EPS, weight_decay=WD, step=1)
            assert L.gm_zero1_adam_push_step_async(z, bad, C.byref(hy0)) == -10, "tensor outside the arena must be refused"
            assert L.gm_zero1_adam_dma_step_async(z, bad, C.byref(hy0), 2) == -10
            L.gm_tensor_list_destroy(bad)
            dev.free(stray)
        for step in range(1, STEPS + 1):
            grads = [O.fill_normal(E, 0.0, 0.01, 91, 1000 * step + k) for k in range(T)]
            shard_g = np.concatenate([grads[k] for k in plan.owned])
            if exchange != "push_host":
                dev.upload(dg, shard_g)
            dist.barrier()                       # nobody pushes into an arena that is still being read
            hy = gm.Hyper(lr=LR, beta1=B1, beta2=B2, eps=EPS, weight_decay=WD, step=step)
            if exchange == "nccl":
                gm.check(L.gm_zero1_adam_step_async(z, lst, C.byref(hy), arena, plan.shard_elems), "zero1 step")
            elif exchange == "push":
                gm.check(L.gm_zero1_adam_push_step_async(z, lst, C.byref(hy)), "zero1 push step")
            elif exchange == "dma":
                gm.check(L.gm_zero1_adam_dma_step_async(z, lst, C.byref(hy), 3), "zero1 dma step")
            else:
                # gradients come from host memory and the rank's new parameters go back to it, in 3 slices
                host_w = np.empty(plan.shard_elems, np.float32)
                gm.check(L.gm_zero1_adam_push_step_host(z, lst, C.byref(hy), shard_g.ctypes.data, host_w.ctypes.data, 3),
                         "zero1 push step with host buffers")
            dev.sync()
            for k in range(T):
                a = k * E
                ws, ms, vs = (np.ascontiguousarray(x[a:a + E]) for x in (full, fm, fv))
                O.adam_step(ws, grads[k], ms, vs, LR, B1, B2, EPS, WD, step)
                full[a:a + E], fm[a:a + E], fv[a:a + E] = ws, ms, vs
            got = dev.to_host(arena, T * E)
            bad = np.flatnonzero(got.view(np.uint32) != full.view(np.uint32))
            assert bad.size == 0, (f"rank {rank} {exchange} step {step}: {bad.size} parameters differ, first at "
                                   f"{bad[0]} (tensor {bad[0] // E})")
            if exchange == "push_host":
                want_w = full[plan.shard_offset:plan.shard_offset + plan.shard_elems]
                assert np.array_equal(host_w.view(np.uint32), want_w.view(np.uint32)), f"rank {rank}: downloaded shard differs"
            got_m = dev.to_host(dm, plan.shard_elems)
            want_m = fm[plan.shard_offset:plan.shard_offset + plan.shard_elems]
            assert np.array_equal(got_m.view(np.uint32), want_m.view(np.uint32)), f"rank {rank}: m differs"
            dist.barrier()
        L.gm_tensor_list_destroy(lst)
        dist.barrier()
        for p in (dg, dm, dv):
            dev.free(p)
        if exchange == "nccl":
            dev.free(arena)
        # the pushed arena stays mapped by the peers until the group is destroyed
    if not only:
        other_rule_zero1(L, dev, z, plan, rank)
        mixed_zero1(L, dev, z, plan, rank, "nccl")
        mixed_zero1(L, dev, z, plan, rank, "push")
        reduce_scatter(L, dev, z, plan, rank, world)
    dist.barrier()
    L.gm_zero1_destroy(z)
    dist.barrier()
    dev.close()
    dist.destroy_process_group()
    print(f"rank {rank} ok")


def other_rule_zero1(L, dev, z, plan, rank):
    """The sharded step is not Adam's alone: NAdam through the rule-generic entry (update of the
    shard, then the all-gather), every rank's whole arena against the oracle."""
    w0 = O.fill_uniform(T * E, -0.1, 0.1, 93, 1)
    full, fm, fv = w0.copy(), np.zeros(T * E, np.float32), np.zeros(T * E, np.float32)
    arena = dev.to_device(w0)
    dg = dev.alloc(4 * plan.shard_elems)
    dm = dev.to_device(np.zeros(plan.shard_elems, np.float32))
    dv = dev.to_device(np.zeros(plan.shard_elems, np.float32))
    w_ptrs = [arena + 4 * plan.tensor_offset(k) for k in plan.owned]
    loc = lambda base: [base + 4 * plan.local_offset(k) for k in plan.owned]
    lst = dev.tensor_list([w_ptrs, loc(dg), loc(dm), loc(dv)], [E] * plan.tensors_per_rank)
    for step in range(1, 4):
        grads = [O.fill_normal(E, 0.0, 0.01, 93, 1000 * step + k) for k in range(T)]
        dev.upload(dg, np.concatenate([grads[k] for k in plan.owned]))
        hy = gm.Hyper(lr=2e-3, beta1=B1, beta2=B2, eps=EPS, weight_decay=WD, step=step)
        gm.check(L.gm_zero1_step_async(z, gm.RULE_NADAM, lst, C.byref(hy), arena, plan.shard_elems), "zero1 NAdam step")
        dev.sync()
        for k in range(T):
            a = k * E
            ws, ms, vs = (np.ascontiguousarray(x[a:a + E]) for x in (full, fm, fv))
            O.nadam_step(ws, grads[k], ms, vs, 2e-3, B1, B2, EPS, WD, step)
            full[a:a + E], fm[a:a + E], fv[a:a + E] = ws, ms, vs
        got = dev.to_host(arena, T * E)
        bad = np.flatnonzero(got.view(np.uint32) != full.view(np.uint32))
        assert bad.size == 0, f"rank {rank} NAdam step {step}: {bad.size} parameters differ, first at {bad[0]}"
        dist.barrier()
    L.gm_tensor_list_destroy(lst)
    for p in (dg, dm, dv, arena):
        dev.free(p)


def reduce_scatter(L, dev, z, plan, rank, world):
    """Gradient hand-off: small-integer-valued gradients make the cross-rank sum exact
    whatever order NCCL adds in, so the shard can be compared bit for bit."""
    n = T * E
    mine = ((np.arange(n, dtype=np.int64) * (rank + 3)) % 17 - 8).astype(np.float32)
    arena = dev.to_device(mine)
    gm.check(L.gm_zero1_reduce_scatter_async(z, arena, plan.shard_elems, 4), "reduce-scatter")
    got = dev.to_host(arena, n)[plan.shard_offset:plan.shard_offset + plan.shard_elems]
    idx = np.arange(plan.shard_offset, plan.shard_offset + plan.shard_elems, dtype=np.int64)
    want = np.zeros(plan.shard_elems, np.float32)
    for r in range(world):
        want += ((idx * (r + 3)) % 17 - 8).astype(np.float32)
    assert np.array_equal(got, want), f"rank {rank}: reduce-scattered gradient shard differs"
    dev.free(arena)


def mixed_zero1(L, dev, z, plan, rank, exchange):
    """Mixed-precision Adam with sharded fp16 gradients: an overflow in ONE rank's shard
    must make every rank skip; states, master shards and the gathered fp16 arena
    must equal the oracle's run over all tensors.  exchange: the fp16 parameters travel by
    the NCCL all-gather or by peer stores from inside the update kernel."""
    world = dist.get_world_size()
    sizes = [E] * T
    master = [O.fill_uniform(E, -0.05, 0.05, 93, k) for k in range(T)]
    mm = [np.zeros(E, np.float32) for _ in range(T)]
    vv = [np.zeros(E, np.float32) for _ in range(T)]
    p16 = [O.f32_to_f16(a) for a in master]
    st = O.new_loss_scale(interval=2)
    own = list(plan.owned)
    p16_arena = dev.to_device(np.concatenate(p16))
    d_master = dev.to_device(np.concatenate([master[k] for k in own]))
    d_m = dev.to_device(np.zeros(plan.shard_elems, np.float32))
    d_v = dev.to_device(np.zeros(plan.shard_elems, np.float32))
    d_g = dev.alloc(2 * plan.shard_elems)
    loc = lambda base, eb: [base + eb * plan.local_offset(k) for k in own]
    p_ptrs = [p16_arena + 2 * plan.tensor_offset(k) for k in own]
    lst = dev.tensor_list([loc(d_g, 2), loc(d_master, 4), loc(d_m, 4), loc(d_v, 4), p_ptrs], [E] * len(own), [2, 4, 4, 4, 2])
    init = gm.LossScale(scale=st.scale, growth=st.growth, backoff=st.backoff, max_scale=st.max_scale, interval=2,
                        good_steps=0, adam_t=0, skipped=0, last_overflow=0)
    mx = L.gm_mixed_create(dev.h, C.byref(init), B1, B2, 0)
    assert mx, gm.last_error()
    if exchange == "push":
        mine = (C.c_ubyte * 64)()
        assert L.gm_zero1_ipc_handle_slot(z, 2, p16_arena, mine) == -10, "only slots 0 and 1 exist"
        gm.check(L.gm_zero1_ipc_handle_slot(z, 1, p16_arena, mine), "ipc handle (fp16 arena)")
        mine_t = torch.tensor(list(bytes(mine)), dtype=torch.uint8, device="cuda")
        all_t = [torch.empty_like(mine_t) for _ in range(world)]
        dist.all_gather(all_t, mine_t)
        blob = bytes(b for tt in all_t for b in tt.cpu().tolist())
        gm.check(L.gm_zero1_open_peers_slot(z, 1, (C.c_ubyte * len(blob))(*blob)), "open peers (fp16 arena)")
        dist.barrier()
    for step in range(1, 6):
        g16 = [O.f32_to_f16(O.fill_normal(E, 0.0, 1e-3, 93, 100 * step + k) * np.float32(st.scale)) for k in range(T)]
        if step == 2:
            g16[0][17] = 0x7c00                  # +inf in rank 0's shard only
        dev.upload(d_g, np.concatenate([g16[k] for k in own]))
        dist.barrier()
        if exchange == "push":
            gm.check(L.gm_zero1_mixed_push_step_async(z, mx, lst, LR, EPS, WD), "zero1 mixed push step")
        else:
            gm.check(L.gm_zero1_mixed_step_async(z, mx, lst, LR, EPS, WD, p16_arena, plan.shard_elems), "zero1 mixed step")
        O.mixed_adam_step(g16, master, mm, vv, p16, LR, B1, B2, EPS, WD, st)
        got = gm.LossScale()
        gm.check(L.gm_mixed_get_state(dev.h, mx, C.byref(got)), "state")
        assert (got.scale, got.good_steps, got.adam_t, got.skipped, got.last_overflow) == \
               (st.scale, st.good_steps, st.adam_t, st.skipped, st.last_overflow), f"rank {rank} step {step}: state differs"
        arena = dev.to_host(p16_arena, T * E, np.uint16)
        assert np.array_equal(arena, np.concatenate(p16)), f"rank {rank} step {step}: gathered fp16 parameters differ"
        shard = dev.to_host(d_master, plan.shard_elems)
        want = np.concatenate([master[k] for k in own])
        assert np.array_equal(shard.view(np.uint32), want.view(np.uint32)), f"rank {rank} step {step}: master shard differs"
        dist.barrier()
    assert st.skipped == 1
    L.gm_mixed_destroy(mx)
    L.gm_tensor_list_destroy(lst)
    dist.barrier()
    for p in (d_master, d_m, d_v, d_g) + (() if exchange == "push" else (p16_arena,)):
        dev.free(p)                              # a pushed arena stays mapped by the peers until the group is destroyed


if __name__ == "__main__":
    main()
