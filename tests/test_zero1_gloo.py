"""CPU test of the N>1 path: two gloo ranks run the ZeRO-1 partition plan, each
updates its shard with the oracle (standing in for the kernel) and the shards
are exchanged with an in-place all-gather; the result must equal the
single-process update bit for bit."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "go-metal_b200", "python"))
import zero1_plan as ZP  # noqa: E402


def test_plan_arithmetic():
    p = ZP.make_plan(256, 4_194_304, 8, 3)
    assert (p.first_tensor, p.tensors_per_rank, p.shard_elems) == (96, 32, 32 * 4_194_304)
    assert p.shard_offset == 96 * 4_194_304 and list(p.owned)[0] == 96 and list(p.owned)[-1] == 127
    assert p.local_offset(97) == 4_194_304 and p.tensor_offset(97) == 97 * 4_194_304
    assert ZP.exchange_bytes_in(p) == 4 * (2 ** 30) * 7 // 8
    covered = []
    for r in range(8):
        covered += list(ZP.make_plan(256, 10, 8, r).owned)
    assert covered == list(range(256))
    # sharded checkpoint bookkeeping
    p1 = ZP.make_plan(4, 3, 2, 1)
    shard = {"type": "Adam", "parameters": {"beta1": 0.9}, "state_data": [
        {"name": "momentum_0", "shape": [3], "data": [1, 2, 3], "state_type": "momentum"},
        {"name": "variance_1", "shape": [3], "data": [4, 5, 6], "state_type": "variance"}]}
    g = ZP.shard_state_to_global(shard, p1)
    assert [t["name"] for t in g["state_data"]] == ["momentum_2", "variance_3"]
    assert ZP.global_state_to_shard(g, p1) == shard
    assert ZP.global_state_to_shard(g, ZP.make_plan(4, 3, 2, 0))["state_data"] == []
    with pytest.raises(ValueError, match="invalid buffer index"):
        ZP.shard_state_to_global({"type": "Adam", "parameters": {}, "state_data": [{"name": "momentum", "data": []}]}, p1)
    with pytest.raises(ValueError, match="more than one shard"):
        ZP.merge_shard_states([g, g])
    with pytest.raises(ValueError, match="disagree"):
        ZP.merge_shard_states([g, dict(g, parameters={"beta1": 0.8}, state_data=[])])
    with pytest.raises(ValueError):
        ZP.make_plan(10, 4, 4, 0)               # uneven split
    with pytest.raises(ValueError):
        ZP.make_plan(8, 4, 2, 2)
    with pytest.raises(IndexError):
        p.local_offset(5)
    one = ZP.make_plan(4, 7, 1, 0)
    assert one.shard_elems == 28 and ZP.exchange_bytes_in(one) == 0


WORKER = r'''
import os, sys
import numpy as np
import torch
import torch.distributed as dist
sys.path.insert(0, os.environ["GM_ROOT"])
sys.path.insert(0, os.path.join(os.environ["GM_ROOT"], "go-metal_b200", "python"))
import zero1_plan as ZP
from oracle import oracle as O

dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
T, E, STEPS = 8, 1001, 4
plan = ZP.make_plan(T, E, world, rank)
w = O.fill_uniform(T * E, -0.1, 0.1, 77, 1)                 # same full arena on every rank
full = w.copy()
m = np.zeros(plan.shard_elems, np.float32)
v = np.zeros(plan.shard_elems, np.float32)
fm, fv = np.zeros(T * E, np.float32), np.zeros(T * E, np.float32)
for step in range(1, STEPS + 1):
    grads = {t: O.fill_normal(E, 0.0, 0.01, 77, 100 * step + t) for t in range(T)}
    for t in plan.owned:                                     # this rank's shard only
        a, b = plan.tensor_offset(t), plan.local_offset(t)
        ws = np.ascontiguousarray(w[a:a + E]); ms = np.ascontiguousarray(m[b:b + E]); vs = np.ascontiguousarray(v[b:b + E])
        O.adam_step(ws, grads[t], ms, vs, 1e-3, 0.9, 0.999, 1e-8, 0.0, step)
        w[a:a + E], m[b:b + E], v[b:b + E] = ws, ms, vs
    # in-place all-gather: rank r contributes arena[r*count:(r+1)*count]
    tw = torch.from_numpy(w)
    parts = list(tw.split(plan.shard_elems))
    dist.all_gather(parts, parts[rank].clone())
    for t in range(T):                                       # single-process reference
        a = t * E
        ws = np.ascontiguousarray(full[a:a + E]); ms = np.ascontiguousarray(fm[a:a + E]); vs = np.ascontiguousarray(fv[a:a + E])
        O.adam_step(ws, grads[t], ms, vs, 1e-3, 0.9, 0.999, 1e-8, 0.0, step)
        full[a:a + E], fm[a:a + E], fv[a:a + E] = ws, ms, vs
    assert np.array_equal(w.view(np.uint32), full.view(np.uint32)), f"rank {rank} step {step}: arena differs"
# sharded checkpoint: every rank's payload (local tensor numbers) -> one global payload on
# every rank -> cut back per rank; it must equal the single-process payload and round-trip
def payload(mm, vv, count):
    data = [{"name": f"momentum_{i}", "shape": [E], "data": mm[i * E:(i + 1) * E].tolist(), "state_type": "momentum"} for i in range(count)]
    data += [{"name": f"variance_{i}", "shape": [E], "data": vv[i * E:(i + 1) * E].tolist(), "state_type": "variance"} for i in range(count)]
    return {"type": "Adam", "parameters": {"learning_rate": 1e-3, "beta1": 0.9, "step_count": STEPS}, "state_data": data}
mine = ZP.shard_state_to_global(payload(m, v, plan.tensors_per_rank), plan)
gathered = [None] * world
dist.all_gather_object(gathered, mine)
merged = ZP.merge_shard_states(gathered[::-1])                 # order of arrival must not matter
assert merged == payload(fm, fv, T), f"rank {rank}: merged checkpoint differs from the single-process one"
back = ZP.global_state_to_shard(merged, plan)
assert back == payload(m, v, plan.tensors_per_rank), f"rank {rank}: shard cut from the checkpoint differs"
dist.barrier()
dist.destroy_process_group()
print(f"rank {rank} ok")
'''


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def test_two_gloo_ranks_match_single_process(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, GM_ROOT=ROOT, OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()), str(script)]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert "rank 0 ok" in out.stdout and "rank 1 ok" in out.stdout
