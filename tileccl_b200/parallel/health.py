"""Host-side failure detection between steps: heartbeats and a leave notice in the
``torch.distributed`` store.

The fused kernels wait on one another across GPUs, so a rank that is gone must be noticed on the
host *before* the next launch (a launch whose peer never arrives only comes back when its bounded
device wait runs out).  Every rank calls :meth:`PeerHealth.beat` after a step and
:meth:`PeerHealth.check` before the next one: a peer that posted :meth:`leave`, or whose heartbeat
is older than the time-out, raises :class:`PeerFailure` on everybody else, who can then shut down or
re-form the group without having queued a kernel that would wait for the missing rank.

The reference's counterpart is the ``failed`` flag of its shared blob that lets ranks bail out of
the host barrier (comm_comp/ipc_multiproc.cuh:74-85,138-142); the native launcher here keeps that
form (csrc/runtime/launcher.cpp), this is the form for torchrun-started ranks.
"""
from __future__ import annotations

import time

import torch.distributed as dist


class PeerFailure(RuntimeError):
    def __init__(self, rank: int, why: str):
        self.rank, self.why = rank, why
        super().__init__(f"rank {rank} is gone: {why}")


class PeerHealth:
    def __init__(self, store=None, rank: int | None = None, world: int | None = None, prefix: str = "tileccl/health"):
        if store is None:
            if not dist.is_initialized():
                raise RuntimeError("PeerHealth needs torch.distributed (or an explicit store)")
            store = dist.distributed_c10d._get_default_store()
        self.store = store
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world is None else world
        self.prefix = prefix
        self.step = 0
        self.beat()

    def _key(self, what: str, r: int) -> str:
        return f"{self.prefix}/{what}/{r}"

    def beat(self) -> None:
        """Records 'alive, finished step N' with a wall-clock stamp."""
        self.step += 1
        self.store.set(self._key("beat", self.rank), f"{self.step}:{time.time():.3f}")

    def leave(self, why: str = "left") -> None:
        """Announces an orderly departure (call between steps, with no kernel or collective in flight)."""
        self.store.set(self._key("left", self.rank), why)

    def check(self, timeout_s: float = 10.0) -> None:
        """Raises :class:`PeerFailure` if a peer left or has not beaten for ``timeout_s`` seconds."""
        now = time.time()
        for r in range(self.world):
            if r == self.rank:
                continue
            if self.store.check([self._key("left", r)]):
                raise PeerFailure(r, self.store.get(self._key("left", r)).decode())
            if self.store.check([self._key("beat", r)]):
                stamp = float(self.store.get(self._key("beat", r)).decode().split(":")[1])
                if now - stamp > timeout_s:
                    raise PeerFailure(r, f"no heartbeat for {now - stamp:.1f} s")
            # a peer that has not beaten yet is still starting up: the rendezvous time-out covers that
