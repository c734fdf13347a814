"""Peer liveness over the rendezvous store: ranks learn on the host that a peer has left.

Every rank publishes ``live/{rank} = "<step>:<wall time>"`` before a step (and ``"exit:<reason>"`` when it leaves through
teardown or an exception). ``check()`` reads the peers' entries before the step's first collective and raises
``PeerLost`` when a peer announced its exit or has been silent for longer than the timeout; ``diagnose(exc)`` turns
the error of a collective that ran into the process-group timeout into the same ``PeerLost`` when the store shows why.
Nothing here touches a GPU: a rank only ever leaves between steps, with none of its kernels or collectives in flight,
and the survivors find out before their next launch or through the (short) process-group timeout.
The reference has no failure detection beyond ``mp.spawn(join=True)`` (``scripts/train.py:233-237``).
"""
from __future__ import annotations

import time
from typing import List, Optional, Tuple

import torch.distributed as dist


class PeerLost(RuntimeError):
    def __init__(self, rank: int, reason: str):
        super().__init__(f"rank {rank} is gone: {reason}")
        self.rank, self.reason = rank, reason


def default_store():
    """The store the default process group was created with (None when not distributed)."""
    if not dist.is_available() or not dist.is_initialized():
        return None
    try:
        return dist.distributed_c10d._get_default_store()
    except Exception:
        return None


class PeerLiveness:
    def __init__(self, store, rank: int, world: int, timeout_s: float = 60.0, prefix: str = "live"):
        self.store, self.rank, self.world, self.timeout_s, self.prefix = store, rank, world, float(timeout_s), prefix
        self._exited = False

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self, step: int) -> None:
        self.store.set(self._key(self.rank), f"{step}:{time.time():.3f}")

    def mark_exit(self, reason: str = "finished") -> None:
        if not self._exited:
            self._exited = True
            try:
                self.store.set(self._key(self.rank), f"exit:{reason}")
            except Exception:
                pass                      # the store host may already be gone; nothing left to tell

    def peers(self) -> List[Tuple[int, Optional[str]]]:
        out = []
        for r in range(self.world):
            if r == self.rank:
                continue
            key = self._key(r)
            try:
                val = self.store.get(key).decode() if self.store.check([key]) else None
            except Exception as ex:       # the store itself is unreachable: its host rank is gone
                raise PeerLost(0, f"rendezvous store unreachable ({ex!r})")
            out.append((r, val))
        return out

    def check(self) -> None:
        now = time.time()
        for r, val in self.peers():
            if val is None:
                continue                  # has not reached its first step yet
            if val.startswith("exit:"):
                raise PeerLost(r, val[5:])
            try:
                t = float(val.split(":", 1)[1])
            except (IndexError, ValueError):
                continue
            if now - t > self.timeout_s:
                raise PeerLost(r, f"no heartbeat for {now - t:.1f} s")

    def diagnose(self, exc: BaseException) -> BaseException:
        """After a failed collective: PeerLost when the store explains it, else the original error."""
        try:
            self.check()
        except PeerLost as lost:
            lost.__cause__ = exc
            return lost
        return exc
