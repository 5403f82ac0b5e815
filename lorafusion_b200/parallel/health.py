"""Host-side failure detection for multi-rank runs: heartbeats and failure notes in a
``torch.distributed`` key-value store.

The fused kernels wait on flags that other ranks set; every such wait is bounded and ends in an
error status (``ops/_native.check_device_errors``), but a rank that is already gone should be
noticed BEFORE the next launch rather than by a 10-second device timeout.  Each rank therefore

* publishes a heartbeat counter from a background thread (``hb/<rank>``),
* publishes its progress from the training loop itself (``prog/<rank>``, one tick per pipeline
  slot or step -- a main thread stuck in a collective keeps its heartbeat thread alive, so
  liveness alone cannot show a stall),
* publishes a note when its step raised (``failed/<rank>`` = message), and
* calls :meth:`HealthMonitor.check` between steps AND between the microbatch slots of a
  schedule (``PipelineRuntime``), which raises :class:`PeerFailure` if a peer left a failure
  note, its heartbeat has not advanced for ``timeout`` seconds, or (with
  ``progress_timeout``) its progress counter has stood still for that long.

A rank only ever leaves between steps, with none of its kernels or collectives in flight.  The
reference has no failure handling (an out-of-memory run is found by grepping the log,
``benchmarks_paper/scripts/run_single.sh:366-370``).  Works with any store (TCPStore of the
default process group, FileStore, HashStore for single-process tests).
"""

from __future__ import annotations

import threading
import time
from typing import Callable, Optional


class PeerFailure(RuntimeError):
    def __init__(self, ranks, reasons):
        self.ranks, self.reasons = list(ranks), dict(reasons)
        super().__init__("peer failure: " + ", ".join(f"rank {r}: {self.reasons.get(r, 'no heartbeat')}"
                                                      for r in self.ranks))


class HealthMonitor:
    def __init__(self, store, rank: int, world: int, *, interval: float = 0.5, timeout: float = 5.0,
                 prefix: str = "lf_health", clock: Callable[[], float] = time.monotonic,
                 progress_timeout: Optional[float] = None):
        self.store, self.rank, self.world = store, rank, world
        self.interval, self.timeout, self.prefix = interval, timeout, prefix
        self.progress_timeout = progress_timeout
        self.clock = clock
        self._beat = 0
        self._progress = 0
        self._last_progress: dict[int, tuple[int, float]] = {}
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._last_seen: dict[int, tuple[int, float]] = {}
        self._started_at = clock()

    # ------------------------------------------------------------------ publishing
    def _key(self, kind: str, rank: int) -> str:
        return f"{self.prefix}/{kind}/{rank}"

    def beat(self) -> None:
        self._beat += 1
        self.store.set(self._key("hb", self.rank), str(self._beat))

    def progress(self) -> None:
        """Called from the training loop: publish that this rank's main thread moved on."""
        self._progress += 1
        self.store.set(self._key("prog", self.rank), str(self._progress))

    def start(self) -> "HealthMonitor":
        self.beat()

        def loop():
            while not self._stop.wait(self.interval):
                try:
                    self.beat()
                except Exception:  # the store is gone: nothing left to tell
                    return

        self._thread = threading.Thread(target=loop, name="lf-heartbeat", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1.0)
            self._thread = None

    def report_failure(self, message: str) -> None:
        """Tell the peers that this rank cannot go on (called from an ``except`` block)."""
        self.store.set(self._key("failed", self.rank), message[:500] or "failed")

    def leave(self) -> None:
        """Orderly exit between steps: peers see it as a failure note, not as a silent stop."""
        self.report_failure("left the job")
        self.stop()

    # ------------------------------------------------------------------ checking
    def _get(self, key: str) -> Optional[str]:
        try:
            if not self.store.check([key]):
                return None
            return self.store.get(key).decode()
        except Exception:
            return None

    def failed_peers(self) -> dict:
        """``{rank: reason}`` of peers that reported a failure or stopped beating."""
        now = self.clock()
        bad = {}
        for r in range(self.world):
            if r == self.rank:
                continue
            note = self._get(self._key("failed", r))
            if note is not None:
                bad[r] = note
                continue
            hb = self._get(self._key("hb", r))
            if hb is None:
                if now - self._started_at > self.timeout:
                    bad[r] = "never joined"
                continue
            count = int(hb)
            seen = self._last_seen.get(r)
            if seen is None or seen[0] != count:
                self._last_seen[r] = (count, now)
            elif now - seen[1] > self.timeout:
                bad[r] = f"no heartbeat for {now - seen[1]:.1f}s"
                continue
            if self.progress_timeout is not None:
                pg = self._get(self._key("prog", r))
                if pg is not None:
                    seen = self._last_progress.get(r)
                    if seen is None or seen[0] != int(pg):
                        self._last_progress[r] = (int(pg), now)
                    elif now - seen[1] > self.progress_timeout:
                        bad[r] = f"alive but no progress for {now - seen[1]:.1f}s"
        return bad

    def check(self) -> None:
        bad = self.failed_peers()
        if bad:
            raise PeerFailure(sorted(bad), bad)

    def guarded(self, step_fn: Callable, *args, **kwargs):
        """Check the peers, run one step, and leave a failure note if the step raises."""
        self.check()
        try:
            return step_fn(*args, **kwargs)
        except Exception as e:  # noqa: BLE001 - every failure is reported, then re-raised
            self.report_failure(f"{type(e).__name__}: {e}")
            raise
