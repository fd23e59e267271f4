"""Host watchdog of an expert-parallel group.

The reference leaves time limits of collectives to its runtime: operators carry an `_op_exec_never_timeout` attribute
(python/torchair/scope/__init__.py:47-72) and the barrier operator a `time_out` input
(python/torchair/_ge_concrete_graph/ge_converter/custom/distribute_barrier.py:4-19).  Here the exchange is a set of
torch.distributed collectives ('nccl' transport) or this library's kernels over peer memory ('peer' transport, whose
device waits are bounded by themselves), and the host needs two things the process group does not give it in time:

* to learn that a peer is gone BEFORE enqueueing a collective that would wait for it.  Every rank's watchdog thread
  writes a heartbeat counter into the rendezvous store and reads the others'; a peer whose counter has not moved for
  `timeout_s` marks the group failed, and the next dispatch / combine raises EpGroupFailed without launching anything;
* to notice an exchange that was enqueued and does not finish.  After the collectives of a step the caller hands the
  watchdog a CUDA event; the thread polls it (cudaEventQuery, no synchronisation) and, when it is still pending after
  `timeout_s`, marks the group failed and asks the backend to abort its communicator, which ends the pending kernels
  with an error instead of leaving the stream blocked.

Nothing here touches a GPU except the event queries and the abort call of the process group's own backend.
"""
from __future__ import annotations

import threading
import time
from typing import Callable, Dict, List, Optional, Tuple


class EpGroupFailed(RuntimeError):
    """A rank of the expert-parallel group stopped answering, or an exchange did not finish in time."""


class EpWatchdog:
    def __init__(self, name: str, store, rank: int, world: int, interval_s: float = 0.5, timeout_s: float = 10.0,
                 abort: Optional[Callable[[], None]] = None, clock: Callable[[], float] = time.monotonic):
        if not (0 <= rank < world):
            raise ValueError("rank must be in [0, world)")
        if interval_s <= 0 or timeout_s <= interval_s:
            raise ValueError("need 0 < interval_s < timeout_s")
        self.name, self.store, self.rank, self.world = name, store, rank, world
        self.interval_s, self.timeout_s = float(interval_s), float(timeout_s)
        self._abort = abort
        self._clock = clock
        self._failure: Optional[str] = None
        self._beat = 0
        self._seen: Dict[int, Tuple[Optional[bytes], float]] = {}
        self._pending: List[Tuple[object, float, str]] = []
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.aborted = False

    # ---- the part the hot path sees: one attribute read, one list append ---------------------------------------------
    def check(self) -> None:
        f = self._failure
        if f is not None:
            raise EpGroupFailed(f"expert-parallel group {self.name!r}: {f}")

    def watch(self, event, what: str) -> None:
        """event: an object with query() -> bool (a recorded torch.cuda.Event)."""
        with self._lock:
            self._pending.append((event, self._clock(), what))

    @property
    def failure(self) -> Optional[str]:
        return self._failure

    # ---- the thread ------------------------------------------------------------------------------------------------------
    def _key(self, r: int) -> str:
        return f"tab_ep_watchdog/{self.name}/{r}"

    def start(self) -> "EpWatchdog":
        if self._thread is not None:
            return self
        now = self._clock()
        self._seen = {r: (None, now) for r in range(self.world) if r != self.rank}
        self.store.set(self._key(self.rank), str(self._beat))
        self._thread = threading.Thread(target=self._run, name=f"tab-ep-watchdog-{self.name}", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        """Stops the heartbeat (the peers' watchdogs will report this rank after their timeout)."""
        self._stop.set()
        t, self._thread = self._thread, None
        if t is not None:
            t.join(timeout=5.0)

    def _run(self) -> None:
        while not self._stop.wait(self.interval_s):
            try:
                self.poll_once()
            except Exception as exc:             # the store itself went away: the rendezvous host is gone
                self._fail(f"the rendezvous store failed: {exc}")
                return
            if self._failure is not None:
                return

    def poll_once(self) -> None:
        """One round of the thread's work (public so that a test can drive it with a fake clock)."""
        now = self._clock()
        self._beat += 1
        self.store.set(self._key(self.rank), str(self._beat))
        for r, (last, since) in list(self._seen.items()):
            key = self._key(r)
            value = self.store.get(key) if self.store.check([key]) else None
            if value != last:
                self._seen[r] = (value, now)
            elif now - since > self.timeout_s:
                self._fail(f"rank {r} has not been heard from for {now - since:.1f} s (limit {self.timeout_s:.1f} s)")
                return
        with self._lock:
            pending, self._pending = self._pending, []
        keep = []
        for event, since, what in pending:
            if event.query():
                continue
            if now - since > self.timeout_s:
                self._fail(f"{what} was enqueued {now - since:.1f} s ago and has not finished (limit {self.timeout_s:.1f} s)",
                           abort=True)
                return
            keep.append((event, since, what))
        if keep:
            with self._lock:
                self._pending = keep + self._pending

    def _fail(self, why: str, abort: bool = False) -> None:
        if self._failure is None:
            self._failure = why
        if abort and self._abort is not None and not self.aborted:
            self.aborted = True
            try:
                self._abort()
            except Exception as exc:
                self._failure += f"; aborting the communicator failed: {exc}"


def backend_abort(process_group, device) -> Callable[[], None]:
    """The abort call of the group's backend for `device`, or a no-op where the backend has none (gloo)."""
    def run():
        try:
            backend = process_group._get_backend(device)
        except Exception:
            return
        for attr in ("abort", "_abort", "_shutdown"):
            fn = getattr(backend, attr, None)
            if callable(fn):
                fn()
                return
    return run
