"""Host-side failure detection.

Every rank publishes ``(step, wall clock)`` to the process group's key-value store on a background
thread; each rank watches the others and declares a peer dead when its heartbeat is older than the
timeout. The trainer asks between steps (never while kernels or collectives are in flight), so a
lost rank surfaces as a Python exception before the next launch instead of a collective that
blocks until the process-group timeout. Recovery is restart-from-latest-checkpoint, driven by the
launcher. Device-side waits are bounded separately (status word written by the kernels).
(The reference has only the process-group timeout and resume-on-restart:
ironcore/parallel/parallel.py:68, ironcore/trainer.py:209-219.)"""

from __future__ import annotations

import threading
import time
from typing import Dict, List, Optional

import torch.distributed as dist


class RankFailure(RuntimeError):
    def __init__(self, ranks: List[int], ages: Dict[int, float]):
        self.ranks, self.ages = ranks, ages
        super().__init__("ranks without a recent heartbeat: " + ", ".join(f"{r} ({ages[r]:.1f}s)" for r in ranks))


class Heartbeat:
    def __init__(self, interval_s: float = 1.0, timeout_s: float = 60.0, store=None, rank: Optional[int] = None,
                 world_size: Optional[int] = None, prefix: str = "icb_hb", clock=time.time):
        self.interval_s, self.timeout_s, self.prefix, self.clock = interval_s, timeout_s, prefix, clock
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world_size is None else world_size
        if store is None:
            from torch.distributed.distributed_c10d import _get_default_store

            store = _get_default_store()
        self.store = store
        self.step = -1
        self._stop = threading.Event()
        self._thread = None
        self._publish()
        if interval_s > 0:
            self._thread = threading.Thread(target=self._run, name="icb-heartbeat", daemon=True)
            self._thread.start()

    def _key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def _publish(self):
        self.store.set(self._key(self.rank), f"{self.step}:{self.clock():.3f}")

    def _run(self):
        while not self._stop.wait(self.interval_s):
            try:
                self._publish()
            except Exception:
                return

    def beat(self, step: int):
        self.step = step
        self._publish()

    def peer_ages(self) -> Dict[int, float]:
        now = self.clock()
        ages = {}
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                raw = self.store.get(self._key(r)).decode()
                ages[r] = now - float(raw.split(":")[1])
            except Exception:
                ages[r] = float("inf")
        return ages

    def dead_peers(self) -> List[int]:
        return sorted(r for r, age in self.peer_ages().items() if age > self.timeout_s)

    def raise_if_peer_dead(self):
        ages = self.peer_ages()
        dead = sorted(r for r, age in ages.items() if age > self.timeout_s)
        if dead:
            raise RankFailure(dead, ages)

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)
