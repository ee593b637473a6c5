"""Host-side failure detection for multi-process jobs: every rank touches a heartbeat file from a daemon thread; any
rank can ask whether its peers are still beating *before* it enters a collective that would otherwise wait for the
process-group timeout.  Recovery is a restart from the last checkpoint (``resume_from_checkpoint``).

Nothing here touches a GPU: a rank that has stopped (crashed, been killed, exited) is noticed through the file system.
The reference bounds hangs only by ``ddp_timeout`` (transformers TrainingArguments) and by the heartbeat of the async
rollout worker (trl/experimental/async_grpo/async_rollout_worker.py:972-1053)."""
from __future__ import annotations

import os
import threading
import time


class PeerFailure(RuntimeError):
    pass


class RankWatchdog:
    def __init__(self, directory: str, rank: int, world: int, interval_s: float = 1.0, stale_after_s: float = 30.0):
        self.dir, self.rank, self.world = directory, rank, world
        self.interval, self.stale_after = interval_s, stale_after_s
        os.makedirs(directory, exist_ok=True)
        self._stop = threading.Event()
        self._thread = None
        self.started_at = time.time()

    def _path(self, r: int) -> str:
        return os.path.join(self.dir, f"heartbeat_rank{r}")

    def beat(self) -> None:
        with open(self._path(self.rank), "w") as f:
            f.write(f"{time.time():.3f}\n")

    def start(self) -> "RankWatchdog":
        self.beat()
        self._thread = threading.Thread(target=self._loop, name="trl-b200-watchdog", daemon=True)
        self._thread.start()
        return self

    def _loop(self):
        while not self._stop.wait(self.interval):
            self.beat()

    def stale_peers(self) -> list[int]:
        now, bad = time.time(), []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                age = now - os.path.getmtime(self._path(r))
            except OSError:
                age = now - self.started_at  # never seen: give it the start-up grace period
            if age > self.stale_after:
                bad.append(r)
        return bad

    def check_peers(self) -> None:
        bad = self.stale_peers()
        if bad:
            raise PeerFailure(f"rank {self.rank}: no heartbeat from rank(s) {bad} for more than {self.stale_after:.0f} s; "
                              "restart the job with resume_from_checkpoint")

    def stop(self, remove: bool = True) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=self.interval + 1)
        if remove:
            try:
                os.remove(self._path(self.rank))
            except OSError:
                pass
