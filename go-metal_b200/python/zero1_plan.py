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
