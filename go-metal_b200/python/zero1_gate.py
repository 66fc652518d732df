"""Host-side step gate for the sharded (ZeRO-1) step: failure detection without a GPU fault.

A sharded step ends in a collective (the parameter exchange and its closing one-word
all-reduce).  A rank that never enters that collective -- it crashed, it left, its host
thread is stuck -- would leave every other rank waiting inside it for ever.  The gate
makes that visible on the host BEFORE a rank launches its step: every rank announces the
step it is about to run in a key-value store (any torch.distributed store: TCPStore,
FileStore), then waits, with a deadline, until all peers have announced the same step.  A
peer that said good-bye (`leave`) or that stays silent past the deadline raises PeerLost on
the others, which then skip the launch and tear the group down in an orderly way; no
kernel or collective is in flight when that happens.  For steps already launched the
library offers the bounded wait gm_device_synchronize_timeout (GM_ERR_TIMEOUT).

The reference has nothing comparable (it is single-device: cgo_bridge/bridge_optimizer.m
only maps exceptions to return codes, :353-356).
"""
from __future__ import annotations

import time
from datetime import timedelta


class PeerLost(RuntimeError):
    """Raised by StepGate.arrive when some peers cannot take part in the step."""

    def __init__(self, step: int, missing, left):
        self.step, self.missing, self.left = step, sorted(missing), sorted(left)
        what = []
        if self.left:
            what.append(f"ranks {self.left} left the group")
        if self.missing:
            what.append(f"ranks {self.missing} did not announce step {step} in time")
        super().__init__("; ".join(what))


class StepGate:
    def __init__(self, store, rank: int, world: int, timeout_s: float = 10.0, prefix: str = "gm_gate", poll_s: float = 0.005):
        if not (0 <= rank < world):
            raise ValueError(f"rank {rank} outside [0, {world})")
        if timeout_s <= 0:
            raise ValueError("timeout must be positive")
        self.store, self.rank, self.world = store, rank, world
        self.timeout_s, self.prefix, self.poll_s = timeout_s, prefix, poll_s

    def _key(self, step: int, rank: int) -> str:
        return f"{self.prefix}/step/{step}/{rank}"

    def _left_key(self, rank: int) -> str:
        return f"{self.prefix}/left/{rank}"

    def _has(self, key: str) -> bool:
        return bool(self.store.check([key]))

    def _scan(self, step: int, waiting):
        """(still waiting, of those: known to have left); a store that cannot be reached any
        more (its host is gone) counts as every awaited peer missing."""
        try:
            waiting = {r for r in waiting if not self._has(self._key(step, r))}
            left = {r for r in waiting if self._has(self._left_key(r))}
            return waiting, left, True
        except Exception:
            return set(waiting), set(), False

    def arrive(self, step: int) -> None:
        """Announce `step` and wait until every peer has announced it too.  Raises PeerLost
        as soon as a peer is known to have left, or when the deadline passes."""
        waiting = set(range(self.world)) - {self.rank}
        try:
            self.store.set(self._key(step, self.rank), "1")
        except Exception:
            raise PeerLost(step, waiting, set()) from None
        deadline = time.monotonic() + self.timeout_s
        while True:
            waiting, left, reachable = self._scan(step, waiting)
            if left or not reachable:
                raise PeerLost(step, waiting - left, left)
            if not waiting:
                return
            if time.monotonic() >= deadline:
                raise PeerLost(step, waiting, set())
            time.sleep(self.poll_s)

    def leave(self) -> None:
        """Say good-bye: peers waiting at the gate learn of it at once instead of timing out.
        Call it between steps, with none of this rank's kernels or collectives in flight."""
        self.store.set(self._left_key(self.rank), "1")

    def wait_keys(self, keys, timeout_s: float) -> bool:
        """Convenience for callers that use the same store for other rendezvous."""
        try:
            self.store.wait(list(keys), timedelta(seconds=timeout_s))
            return True
        except Exception:
            return False
