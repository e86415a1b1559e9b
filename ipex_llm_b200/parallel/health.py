"""Host-side failure detection for multi-rank jobs: heartbeats through the rendezvous store.

The reference has no failure detection beyond timeouts of its launchers (a ``ddp_timeout`` in
python/llm/src/ipex_llm/transformers/training_patch.py:127, the queue timeout of the FastAPI server,
``RANK_WAIT_TIME`` in the AutoTP example).  On a shared GPU machine a rank that disappears must be noticed on the
host, *between* steps and before the next kernel or collective is launched, because a kernel that waits for a
peer that is gone can only time out.  ``RankMonitor`` gives every rank three cheap operations on the process
group's key-value store (no collective, no GPU work):

* ``beat(step)``   publish "I have finished step ``step``" with a wall-clock stamp;
* ``leave()``      publish "I am leaving on purpose" (call it between steps, with nothing in flight);
* ``check()``      raise ``PeerLostError`` when a peer has left, or has not beaten for ``timeout`` seconds.

A training / decoding loop calls ``beat`` after each step and ``check`` before the next launch.  Ranks that die
without calling ``leave`` (an exception, a kill) are caught by the staleness rule.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional

import torch.distributed as dist


class PeerLostError(RuntimeError):
    """A peer rank left the job or stopped responding.  ``ranks`` lists them, ``reason`` maps rank -> text."""

    def __init__(self, reason: Dict[int, str]):
        self.reason = dict(reason)
        self.ranks = sorted(reason)
        super().__init__("lost peer rank(s): " + ", ".join(f"{r} ({reason[r]})" for r in self.ranks))


class RankMonitor:
    def __init__(self, store=None, rank: Optional[int] = None, world_size: Optional[int] = None,
                 timeout: float = 30.0, prefix: str = "ipex_llm/health", clock=time.time):
        if store is None:
            store = dist.distributed_c10d._get_default_store()
        self.store = store
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world_size is None else world_size
        self.timeout = float(timeout)
        self.prefix = prefix
        self.clock = clock
        self._started = clock()
        self.beat(-1)

    def _key(self, kind: str, rank: int) -> str:
        return f"{self.prefix}/{kind}/{rank}"

    def beat(self, step: int):
        self.store.set(self._key("beat", self.rank), f"{int(step)}:{self.clock():.3f}")

    def leave(self, why: str = "left"):
        self.store.set(self._key("left", self.rank), why)

    def _get(self, key: str) -> Optional[str]:
        try:
            if hasattr(self.store, "check") and not self.store.check([key]):
                return None
            v = self.store.get(key)
            return v.decode() if isinstance(v, bytes) else str(v)
        except Exception:  # noqa: BLE001 - a store without `check` raises on a missing key
            return None

    def peers(self) -> Dict[int, dict]:
        """Last published state of every rank: ``{rank: {"step", "age", "left"}}`` (age in seconds, None = never)."""
        now = self.clock()
        out = {}
        for r in range(self.world):
            beat = self._get(self._key("beat", r))
            left = self._get(self._key("left", r))
            step, age = None, None
            if beat is not None:
                s, stamp = beat.split(":")
                step, age = int(s), max(0.0, now - float(stamp))
            out[r] = {"step": step, "age": age, "left": left}
        return out

    def lost(self) -> Dict[int, str]:
        bad = {}
        now = self.clock()
        for r, st in self.peers().items():
            if r == self.rank:
                continue
            if st["left"] is not None:
                bad[r] = f"left: {st['left']}"
            elif st["age"] is None:
                if now - self._started > self.timeout:
                    bad[r] = f"never reported within {self.timeout:.0f} s"
            elif st["age"] > self.timeout:
                bad[r] = f"no heartbeat for {st['age']:.1f} s (last step {st['step']})"
        return bad

    def check(self):
        bad = self.lost()
        if bad:
            raise PeerLostError(bad)

    def wait_for_step(self, step: int, poll: float = 0.05) -> List[int]:
        """Block until every peer has reported ``step`` (or raise ``PeerLostError``): a host-side rendezvous that a
        loop can use instead of entering a collective blindly."""
        while True:
            self.check()
            st = self.peers()
            if all(v["step"] is not None and v["step"] >= step for r, v in st.items() if r != self.rank):
                return [v["step"] for v in st.values()]
            time.sleep(poll)
