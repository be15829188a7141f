"""Host-side failure detection for batch-sharded runs: ranks announce each step in a key-value store, and nobody
launches a step's collectives before every rank has announced it.

The reference has no counterpart (one device, no ranks).  The realize path's only exchange is the gradient all-reduce,
and an all-reduce that a rank never joins keeps the others' GPUs spinning.  So the survivors should learn of a missing
rank on the host, BEFORE they launch: a rank that leaves says so (``leave``), a rank that died simply stops
announcing and the others' ``check`` runs into its deadline.  Either way ``check`` raises ``RankLost`` and the caller
stops stepping with nothing in flight.  (Under this sits the C side's own net: collectives and the host waits behind
them run against a wall-clock deadline, after which the communicator is aborted; see ormi_b200/csrc/comm.cu.)

The store is anything with torch.distributed.Store's ``add`` / ``set`` / ``get`` / ``check`` / ``delete_key``
(TCPStore, FileStore, a process group's own store).  One ``check`` costs a couple of store round trips; ``every``
spaces them out.
"""
from __future__ import annotations

import time


class RankLost(RuntimeError):
    """A rank left, or did not announce the step within the deadline."""


class StepGuard:
    def __init__(self, store, rank: int, world: int, timeout_s: float = 10.0, every: int = 1, prefix: str = "ormi_b200/guard"):
        self.store, self.rank, self.world = store, rank, world
        self.timeout_s, self.every, self.prefix = timeout_s, max(1, every), prefix

    def _key(self, step: int) -> str:
        return f"{self.prefix}/step/{step}"

    def leave(self):
        """This rank stops stepping (between steps, nothing of its own in flight): the others' next check raises at once."""
        self.store.set(f"{self.prefix}/left/{self.rank}", b"1")

    def _gone(self):
        keys = [f"{self.prefix}/left/{r}" for r in range(self.world) if r != self.rank]
        return [r for r, k in zip([r for r in range(self.world) if r != self.rank], keys) if self.store.check([k])]

    def check(self, step: int):
        """Call before launching step `step`: returns once every rank has announced it; raises RankLost otherwise."""
        if step % self.every:
            return
        arrived = self.store.add(self._key(step), 1)
        deadline = time.monotonic() + self.timeout_s
        pause = 0.0002
        while arrived < self.world:
            gone = self._gone()
            if gone:
                raise RankLost(f"rank(s) {gone} left before step {step}")
            if time.monotonic() > deadline:
                raise RankLost(f"only {arrived} of {self.world} ranks announced step {step} within {self.timeout_s} s")
            time.sleep(pause)
            pause = min(pause * 2, 0.01)
            arrived = self.store.add(self._key(step), 0)
        if self.rank == 0 and step >= 2 * self.every:
            try:
                self.store.delete_key(self._key(step - 2 * self.every))
            except Exception:
                pass        # a store without delete_key just keeps a few bytes per step
