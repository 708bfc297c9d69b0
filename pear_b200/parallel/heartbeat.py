"""Host-side failure detection between steps.

World size is fixed (no elastic resize, as upstream), but a rank that died must be noticed BEFORE the survivors launch
kernels that wait on it: every rank publishes a heartbeat (step number + wall time) in a ``torch.distributed`` store
after each step and checks its peers' before the next launch. A peer whose heartbeat is older than ``timeout_s``, or
that announced its departure, raises ``PeerLost`` on the host; nothing on the device ever waits for a dead rank (and
device-side waits are bounded anyway).
"""

from __future__ import annotations

import json
import time
from typing import Optional


class PeerLost(RuntimeError):
    def __init__(self, ranks: list[int], reason: str):
        super().__init__(f"ranks {ranks} lost: {reason}")
        self.ranks = ranks


class Heartbeat:
    def __init__(self, store, rank: int, world: int, timeout_s: float = 30.0, prefix: str = "hb"):
        self.store, self.rank, self.world, self.timeout_s, self.prefix = store, rank, world, timeout_s, prefix
        self.beat(step=-1)

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self, step: int, leaving: bool = False) -> None:
        self.store.set(self._key(self.rank), json.dumps({"step": step, "time": time.time(), "leaving": leaving}))

    def leave(self, step: int) -> None:
        """Announce a clean departure between steps (no kernel or collective of this rank is in flight)."""
        self.beat(step, leaving=True)

    def peers(self) -> dict[int, Optional[dict]]:
        out: dict[int, Optional[dict]] = {}
        for r in range(self.world):
            try:
                if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                    out[r] = None
                    continue
                out[r] = json.loads(self.store.get(self._key(r)))
            except Exception:  # noqa: BLE001 - an unreachable store entry counts as no heartbeat
                out[r] = None
        return out

    def check(self, min_step: Optional[int] = None) -> None:
        """Raise ``PeerLost`` unless every peer is alive (and has reached ``min_step`` when given)."""
        now = time.time()
        gone, absent, stale, behind = [], [], [], []
        for r, hb in self.peers().items():
            if r == self.rank:
                continue
            if hb is None:
                absent.append(r)
            elif hb.get("leaving"):
                gone.append(r)
            elif now - hb["time"] > self.timeout_s:
                stale.append(r)
            elif min_step is not None and hb["step"] < min_step:
                behind.append(r)
        if gone:
            raise PeerLost(gone, "left the job")
        if absent:
            raise PeerLost(absent, "never joined")
        if stale:
            raise PeerLost(stale, f"no heartbeat for more than {self.timeout_s}s")
        if behind:
            raise PeerLost(behind, f"still before step {min_step}")

    def wait_all(self, step: int, poll_s: float = 0.05) -> None:
        """Block (on the host) until every peer reached ``step``; raises ``PeerLost`` instead of waiting for a dead one."""
        deadline = time.time() + self.timeout_s
        while True:
            try:
                self.check(min_step=step)
                return
            except PeerLost as e:
                if not ("still before" in str(e) or "never joined" in str(e)) or time.time() > deadline:
                    raise
            time.sleep(poll_s)
