"""Host-side failure detection for one-process-per-GPU jobs.

The reference has none: a rank that dies leaves the others inside a collective until the library's time-out
(keras/src/backend/torch/trainer.py:83-92 relies on NCCL defaults).  Here every rank runs a small thread that

* increments its own heartbeat counter in the job's c10d key-value store every ``interval_s`` seconds, and
* reads the other ranks' counters; a counter that has not moved for ``timeout_s`` seconds, or a rank that announced its
  departure (``leave``) or an exception (``report_failure``), marks that rank as failed.

``check()`` raises ``RankFailure`` on the host *between* steps, before the next kernel or collective is launched, so no GPU
ever waits for a peer that is known to be gone; waits that are already on the device are bounded on their own (see
``collectives``).  ``FailureDetection`` is the callback that wires this into ``fit`` (combine it with ``BackupAndRestore`` to
restart from the last saved epoch).
"""

import atexit
import threading
import time

import torch.distributed as dist

from keras_b200.parallel import process_groups


class RankFailure(RuntimeError):
    """One or more ranks of the job stopped responding, left or reported an exception."""

    def __init__(self, ranks, reasons):
        self.ranks = sorted(ranks)
        self.reasons = dict(reasons)
        detail = ", ".join(f"rank {r}: {self.reasons.get(r, 'no heartbeat')}" for r in self.ranks)
        super().__init__(f"Lost {len(self.ranks)} rank(s) of the job ({detail}).")


def _default_store():
    from torch.distributed import distributed_c10d

    return distributed_c10d._get_default_store()


_ACTIVE = []


def explain_collective_error(exc, wait_s=3.0):
    """Called when a library collective raised: if a running watchdog knows (or learns within ``wait_s``) of a lost rank, raise
    ``RankFailure`` naming it, chained to the library's error; otherwise return so the caller re-raises the original."""
    for wd in list(_ACTIVE):
        failed = wd.wait_for_failure(wait_s)
        if failed:
            raise RankFailure(failed.keys(), failed) from exc


class RankWatchdog:
    def __init__(self, interval_s=0.5, timeout_s=10.0, store=None, rank=None, world_size=None, prefix="kb200_wd"):
        self.interval_s = float(interval_s)
        self.timeout_s = float(timeout_s)
        self.store = store if store is not None else _default_store()
        self.rank = process_groups.rank() if rank is None else int(rank)
        self.world = process_groups.world_size() if world_size is None else int(world_size)
        self.prefix = prefix
        self._failed = {}
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._beating = True
        self._thread = None
        self._last_seen = {}

    # -- keys ---------------------------------------------------------------------------------------
    def _hb(self, r):
        return f"{self.prefix}/hb/{r}"

    def _gone(self, r):
        return f"{self.prefix}/gone/{r}"

    # -- life cycle ---------------------------------------------------------------------------------
    def start(self):
        if self._thread is not None:
            return self
        self.store.add(self._hb(self.rank), 1)
        now = time.monotonic()
        self._last_seen = {r: (None, now) for r in range(self.world) if r != self.rank}
        self._thread = threading.Thread(target=self._run, name="kb200-rank-watchdog", daemon=True)
        self._thread.start()
        _ACTIVE.append(self)
        atexit.register(self.stop)  # the thread must not outlive the store's client at interpreter shutdown
        return self

    def stop(self):
        if self in _ACTIVE:
            _ACTIVE.remove(self)
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval_s + 1.0)
            self._thread = None

    def pause_heartbeat(self):
        """Stop publishing this rank's heartbeat (the thread keeps watching): what a wedged process looks like from outside."""
        self._beating = False

    def leave(self, reason="left the job"):
        """Announce an orderly departure (call between steps, with no collective in flight) and stop."""
        self.store.set(self._gone(self.rank), str(reason))
        self.stop()

    def report_failure(self, exc):
        """Publish an exception raised on this rank so that the others abort at their next check."""
        self.store.set(self._gone(self.rank), f"{type(exc).__name__}: {exc}"[:500])

    # -- watching ----------------------------------------------------------------------------------
    def _poll_once(self):
        now = time.monotonic()
        if self._beating:
            self.store.add(self._hb(self.rank), 1)
        for r in list(self._last_seen):
            if r in self._failed:
                continue
            if self.store.check([self._gone(r)]):
                reason = self.store.get(self._gone(r)).decode(errors="ignore")
                with self._lock:
                    self._failed[r] = reason
                continue
            count = self.store.add(self._hb(r), 0)
            last_count, last_time = self._last_seen[r]
            if count != last_count:
                self._last_seen[r] = (count, now)
            elif now - last_time > self.timeout_s:
                with self._lock:
                    self._failed[r] = f"no heartbeat for {now - last_time:.1f} s"

    def _run(self):
        while not self._stop.is_set():
            try:
                self._poll_once()
            except Exception as e:  # the store itself went away: the job's first rank is gone
                with self._lock:
                    self._failed.setdefault(0, f"key-value store unreachable ({type(e).__name__})")
                return
            self._stop.wait(self.interval_s)

    # -- queries -----------------------------------------------------------------------------------
    def failed_ranks(self):
        with self._lock:
            return dict(self._failed)

    def check(self):
        """Raise ``RankFailure`` if any rank is known to be lost.  Cheap: reads local state only."""
        failed = self.failed_ranks()
        if failed:
            raise RankFailure(failed.keys(), failed)

    def wait_for_failure(self, timeout_s):
        """Block up to ``timeout_s`` for a failure to be detected; returns the dict of failed ranks (possibly empty)."""
        end = time.monotonic() + timeout_s
        while time.monotonic() < end:
            failed = self.failed_ranks()
            if failed:
                return failed
            time.sleep(min(0.05, self.interval_s))
        return self.failed_ranks()
