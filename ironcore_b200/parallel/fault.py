"""Host-side failure detection.

Every rank publishes ``(step, beat counter)`` to the process group's key-value store on a background
thread; each rank watches the others and declares a peer dead when that peer's counter has not moved
for longer than the timeout, measured on the watcher's own clock (clocks of different hosts are never
compared, and a key that is not there yet is probed with ``check`` instead of a blocking ``get``). A rank that
leaves on purpose (an exception in its training loop) publishes a tombstone first, which its peers read as a
failure at once, without waiting for the timeout. The trainer asks between steps (never while kernels or collectives are in flight), so a
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
        self._seq = 0
        self._seen: Dict[int, tuple] = {}       # peer -> (last counter value, local time it was first seen)
        self._born = self.clock()
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._thread = None
        self._publish()
        if interval_s > 0:
            self._thread = threading.Thread(target=self._run, name="icb-heartbeat", daemon=True)
            self._thread.start()

    def _key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def _publish(self):
        if getattr(self, "_left", False):
            return
        self._seq += 1
        self.store.set(self._key(self.rank), f"{self.step}:{self._seq}")

    def _run(self):
        while not self._stop.wait(self.interval_s):
            try:
                self._publish()
                self.peer_ages()        # keep the "last change" times current between the trainer's questions
            except Exception:
                return

    def beat(self, step: int):
        self.step = step
        self._publish()

    def leave(self, reason: str = "") -> None:
        """Tell the peers that this rank stops taking part (call between steps, with nothing of this rank in
        flight): its record becomes a tombstone that ``raise_if_peer_dead`` on the other ranks reports at once."""
        self._stop.set()
        self._left = True
        try:
            self.store.set(self._key(self.rank), f"{self.step}:left:{reason[:200]}")
        except Exception:   # the store lives on rank 0: if that is gone there is nobody left to tell
            pass

    def _read(self, rank: int) -> Optional[str]:
        """The peer's record, or None when it has not published yet. Never blocks on a missing key."""
        key = self._key(rank)
        check = getattr(self.store, "check", None)
        try:
            if check is not None and not check([key]):
                return None
            raw = self.store.get(key)
        except Exception:
            return None
        return raw.decode() if isinstance(raw, (bytes, bytearray)) else str(raw)

    def peer_steps(self) -> Dict[int, int]:
        """Last optimizer step each peer reported (-1 before its first step or when it never published)."""
        out = {}
        for r in range(self.world):
            if r != self.rank:
                raw = self._read(r)
                out[r] = int(raw.split(":")[0]) if raw else -1
        return out

    def peer_ages(self) -> Dict[int, float]:
        """Seconds, on this rank's clock, since each peer's beat counter last changed (since this watcher
        started, for a peer that never published)."""
        ages = {}
        for r in range(self.world):
            if r == self.rank:
                continue
            raw = self._read(r)
            now = self.clock()
            if raw is None:
                ages[r] = now - self._born
                continue
            if raw.split(":")[1:2] == ["left"]:
                ages[r] = float("inf")
                continue
            with self._lock:
                seen = self._seen.get(r)
                if seen is None or seen[0] != raw:
                    self._seen[r] = (raw, now)
                    ages[r] = 0.0
                else:
                    ages[r] = now - seen[1]
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
