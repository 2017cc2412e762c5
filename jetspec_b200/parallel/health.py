"""Host-side failure detection for multi-process runs.

The reference has no rank-failure handling (its multi-GPU mode is independent data-parallel replicas,
``bench/engine/tps_walltime.py:178-203``).  The fused collectives of this framework make ranks wait for one
another inside kernels, so a peer that died must be noticed ON THE HOST, between steps, before the next launch:

* :class:`Heartbeat` - every rank posts ``(step, wall time)`` and an optional error string to a key-value store
  (``torch.distributed.TCPStore`` or any object with ``set``/``get``); :meth:`Heartbeat.check` raises
  :class:`PeerFailure` when a peer reported an error, or has not advanced within ``timeout`` seconds.
* :class:`MailboxModel` - an executable model of the device mailbox protocol of :mod:`.handoff` (payload words,
  then a release-store of a round number; the reader waits, bounded, for the round number).  Tests inject a
  lost or delayed flag write here and check that the bounded wait reports a status instead of waiting forever -
  the same contract the device kernels implement with their status word.
"""
from __future__ import annotations

import json
import time
from typing import Callable, Optional


class PeerFailure(RuntimeError):
    def __init__(self, rank: int, why: str):
        super().__init__(f"rank {rank}: {why}")
        self.rank, self.why = rank, why


class DictStore:
    """In-process stand-in for a TCPStore (tests, single-process runs)."""

    def __init__(self):
        self._d: dict = {}

    def set(self, key: str, value) -> None:
        self._d[key] = value if isinstance(value, bytes) else str(value).encode()

    def get(self, key: str) -> bytes:
        return self._d[key]

    def check(self, keys) -> bool:
        return all(k in self._d for k in keys)


class Heartbeat:
    """``beat()`` after every step; ``check()`` before launching the next one."""

    def __init__(self, store, rank: int, world: int, timeout: float = 30.0, prefix: str = "hb",
                 clock: Callable[[], float] = time.time):
        self.store, self.rank, self.world = store, int(rank), int(world)
        self.timeout, self.prefix, self.clock = float(timeout), prefix, clock
        self.step = 0
        self._seen: dict = {}            # rank -> (step, local time it was first seen at that step)
        self.beat()

    def _key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def beat(self, error: Optional[str] = None) -> None:
        self.store.set(self._key(self.rank), json.dumps({"step": self.step, "t": self.clock(), "error": error}))
        self.step += 1

    def fail(self, error: str) -> None:
        """Tell the peers this rank is going down (call from an exception handler)."""
        self.beat(error=error)

    def _read(self, rank: int) -> Optional[dict]:
        try:
            if hasattr(self.store, "check") and not self.store.check([self._key(rank)]):
                return None
            return json.loads(bytes(self.store.get(self._key(rank))).decode())
        except Exception:
            return None

    def check(self) -> None:
        now = self.clock()
        for r in range(self.world):
            if r == self.rank:
                continue
            rec = self._read(r)
            if rec is None:
                first = self._seen.setdefault(r, (-1, now))
                if now - first[1] > self.timeout:
                    raise PeerFailure(r, f"never reported within {self.timeout:.0f} s")
                continue
            if rec.get("error"):
                raise PeerFailure(r, str(rec["error"]))
            last = self._seen.get(r)
            if last is None or last[0] != rec["step"]:
                self._seen[r] = (rec["step"], now)
            elif now - last[1] > self.timeout:
                raise PeerFailure(r, f"no progress for {now - last[1]:.1f} s (stuck at step {rec['step']})")


# ----------------------------------------------------------------------------- mailbox protocol model
OK, TIMEOUT = 0, 4          # the status codes of the device kernels (4 = waited for a flag another GPU should write)


class MailboxModel:
    """One direction of the handoff: ``push(words)`` writes the payload then release-stores round ``n``;
    ``wait(limit)`` polls for round ``n`` at most ``limit`` times and returns ``(status, payload)``.

    ``drop_flag`` / ``delay_polls`` inject the two failures a peer store can suffer from the reader's
    point of view: the flag never arrives, or it arrives late.
    """

    def __init__(self):
        self.payload: list = []
        self.flag = 0
        self.round_push = 0
        self.round_wait = 0
        self.drop_flag = False
        self.delay_polls = 0
        self._pending: Optional[int] = None

    def push(self, words) -> None:
        self.payload = list(words)
        self.round_push += 1
        if self.drop_flag:
            return
        if self.delay_polls > 0:
            self._pending = self.round_push
        else:
            self.flag = self.round_push

    def wait(self, limit: int = 1000):
        want = self.round_wait + 1
        for _ in range(limit):
            if self._pending is not None:
                if self.delay_polls == 0:
                    self.flag, self._pending = self._pending, None
                else:
                    self.delay_polls -= 1
            if self.flag >= want:
                self.round_wait = want
                return OK, list(self.payload)
        self.round_wait = want          # the device kernel advances its round number on a timeout as well
        return TIMEOUT, None
