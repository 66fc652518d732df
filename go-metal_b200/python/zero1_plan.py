"""Host-side ZeRO-1 partition plan: which tensors of a flat parameter arena a
rank updates, and where its shard sits for the in-place all-gather.

Pure integer arithmetic shared by bench.py, the multi-GPU worker and the CPU
(gloo) tests; there is no compute here.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Zero1Plan:
    world: int
    rank: int
    num_tensors: int
    tensor_elems: int
    first_tensor: int        # first tensor this rank owns
    tensors_per_rank: int
    shard_elems: int         # elements this rank updates (= count per rank of the all-gather)
    shard_offset: int        # element offset of the shard inside the full arena

    @property
    def owned(self) -> range:
        return range(self.first_tensor, self.first_tensor + self.tensors_per_rank)

    def tensor_offset(self, t: int) -> int:
        """Element offset of tensor t inside the full arena (tensors are packed back to back)."""
        if not 0 <= t < self.num_tensors:
            raise IndexError(f"tensor {t} outside [0, {self.num_tensors})")
        return t * self.tensor_elems

    def local_offset(self, t: int) -> int:
        """Element offset of owned tensor t inside this rank's gradient/state arenas."""
        if t not in self.owned:
            raise IndexError(f"tensor {t} is not owned by rank {self.rank}")
        return (t - self.first_tensor) * self.tensor_elems


def make_plan(num_tensors: int, tensor_elems: int, world: int, rank: int) -> Zero1Plan:
    """Rank r owns tensors [r*T/R, (r+1)*T/R).  The in-place all-gather needs every
    rank to contribute the same count, so T must divide evenly."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} for world {world}")
    if num_tensors < 1 or tensor_elems < 1:
        raise ValueError("need at least one tensor with at least one element")
    if num_tensors % world:
        raise ValueError(f"{num_tensors} tensors do not divide evenly over {world} ranks")
    per = num_tensors // world
    return Zero1Plan(world=world, rank=rank, num_tensors=num_tensors, tensor_elems=tensor_elems,
                     first_tensor=rank * per, tensors_per_rank=per, shard_elems=per * tensor_elems,
                     shard_offset=rank * per * tensor_elems)


def exchange_bytes_in(plan: Zero1Plan, elem_bytes: int = 4) -> int:
    """Bytes every rank receives per step: all shards but its own."""
    return elem_bytes * (plan.num_tensors * plan.tensor_elems - plan.shard_elems)


# ---- sharded checkpoints -------------------------------------------------------------
#
# Under ZeRO-1 a rank's optimizer holds state only for the tensors it owns, numbered from
# zero ("momentum_0" is the first tensor of the shard).  A checkpoint is one payload for
# the whole model (optimizer/interface.go:47-51: Type, Parameters, StateData with names
# "<state type>_<tensor index>"), so the shard payloads are renumbered to global tensor
# indices and concatenated on save, and cut back per rank on load.  Payloads here are
# plain dicts with the JSON field names of checkpoints/checkpoint.go:74-86.

def _split_name(name: str) -> tuple[str, int]:
    kind, _, idx = name.rpartition("_")
    if not kind or not idx.isdigit():
        raise ValueError(f"invalid buffer index in tensor name: {name}")
    return kind, int(idx)


def shard_state_to_global(state: dict, plan: Zero1Plan) -> dict:
    """One rank's payload with its tensors renamed to global tensor indices."""
    out = {"type": state["type"], "parameters": dict(state["parameters"]), "state_data": []}
    for t in state["state_data"]:
        kind, local = _split_name(t["name"])
        if not 0 <= local < plan.tensors_per_rank:
            raise ValueError(f"{t['name']}: rank {plan.rank} owns {plan.tensors_per_rank} tensors")
        out["state_data"].append(dict(t, name=f"{kind}_{plan.first_tensor + local}"))
    return out


def merge_shard_states(states: list[dict]) -> dict:
    """Payloads of all ranks (already global, any order) -> one payload, tensors grouped by
    state type and ordered by tensor index like a single-process GetState.  The scalar
    parameters must agree across ranks: they are replicated, not sharded."""
    if not states:
        raise ValueError("no shard payloads")
    first = states[0]
    for s in states[1:]:
        if s["type"] != first["type"]:
            raise ValueError(f"state type mismatch: expected {first['type']}, got {s['type']}")
        if s["parameters"] != first["parameters"]:
            raise ValueError("ranks disagree on the replicated optimizer parameters")
    tensors, order = {}, []
    for s in states:
        for t in s["state_data"]:
            kind, idx = _split_name(t["name"])
            if kind not in order:
                order.append(kind)
            if (kind, idx) in tensors:
                raise ValueError(f"{t['name']} appears in more than one shard")
            tensors[(kind, idx)] = t
    merged = [tensors[key] for key in sorted(tensors, key=lambda k: (order.index(k[0]), k[1]))]
    return {"type": first["type"], "parameters": dict(first["parameters"]), "state_data": merged}


def global_state_to_shard(state: dict, plan: Zero1Plan) -> dict:
    """The part of a whole-model payload that one rank loads, renumbered from zero."""
    out = {"type": state["type"], "parameters": dict(state["parameters"]), "state_data": []}
    for t in state["state_data"]:
        kind, idx = _split_name(t["name"])
        if idx in plan.owned:
            out["state_data"].append(dict(t, name=f"{kind}_{idx - plan.first_tensor}"))
    return out

