"""Failure detection and recovery for multi-rank training, all of it on the host.

* ``Heartbeat``: every rank publishes ``(step, wall time)`` in a ``torch.distributed`` store after each step and, before
  it launches the next one, looks at its peers: a rank that announced its departure, or whose last beat is older than
  ``timeout_s``, raises ``PeerLost`` on everyone else, before they enter a collective that could no longer complete.
* ``StatusWatchdog``: a thread that polls the device status word (the word in which kernels with bounded waits record a
  time-out) and the completion of the step's last CUDA event; the training thread calls ``check()`` and gets a typed
  ``CollectiveTimeout`` / ``StepHung`` instead of finding out from diverged replicas. The sources are callables, so
  the logic is testable without a GPU.
* ``run_elastic``: a supervisor that starts one process per rank; when a rank exits with ``EXIT_PEER_LOST`` or dies, it
  stops the remaining ranks (by their own process ids), and starts all ranks again. The workers resume from
  ``latest_checkpoint()``; a resumed run continues bit for bit like an uninterrupted one (checkpoints are published by
  rename, so a reader never sees a half-written one: io/checkpoint.py).

The reference trains on one device and has no recovery loop; what is kept from it is the atomic checkpoint publish
(scirust-sciagent/src/cuda_model.rs:1812-1856) and the resume-equals-uninterrupted contract
(scirust-sciagent/tests/cuda_parity.rs:223). A rank leaves only between steps, with none of its collectives in flight.
"""
from __future__ import annotations

import multiprocessing as mp
import threading
import time

EXIT_PEER_LOST = 75          # EX_TEMPFAIL: "try again": the supervisor restarts the job


class PeerLost(RuntimeError):
    def __init__(self, rank: int, why: str):
        super().__init__(f"rank {rank} is gone: {why}")
        self.rank, self.why = rank, why


class StepHung(RuntimeError):
    pass


class Heartbeat:
    """``store`` is any ``torch.distributed`` store (TCPStore, FileStore, HashStore) shared by the ranks."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 30.0, prefix: str = "hb"):
        self.store, self.rank, self.world, self.timeout_s, self.prefix = store, rank, world, timeout_s, prefix

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self, step: int) -> None:
        self.store.set(self._key(self.rank), f"{step} {time.time():.3f}")

    def leave(self, why: str = "left") -> None:
        """Announce a departure between steps (the polite form: nothing of this rank is in flight)."""
        self.store.set(self._key(self.rank), f"-1 {time.time():.3f} {why}")

    def check_peers(self, min_step: int = -1) -> None:
        """Raise ``PeerLost`` if a peer has left or has not beaten for ``timeout_s``; ``min_step``: a peer whose last
        beat is older than this step is given until the timeout, not treated as lost at once."""
        now = time.time()
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                    continue                      # has not started beating yet
                raw = self.store.get(self._key(r)).decode()
            except Exception as e:  # noqa: BLE001  the store itself is gone: the rank hosting it died
                raise PeerLost(r, f"store unreachable: {e}") from None
            parts = raw.split(" ", 2)
            step, t = int(parts[0]), float(parts[1])
            if step < 0:
                raise PeerLost(r, parts[2] if len(parts) > 2 else "left")
            if now - t > self.timeout_s:
                raise PeerLost(r, f"no heartbeat for {now - t:.1f}s (last step {step})")


class StatusWatchdog:
    """Polls ``read_status() -> int`` (0 = fine) and ``step_done() -> bool`` every ``interval_s``. A non-zero status is
    kept as ``CollectiveTimeout``; a step that stays unfinished for ``hang_s`` as ``StepHung``. ``check()`` re-raises
    in the caller's thread; ``on_error(exc)`` (optional) runs in the watchdog thread, e.g. to tell the peers."""

    def __init__(self, read_status, step_done=None, interval_s: float = 0.5, hang_s: float = 120.0, on_error=None):
        self.read_status, self.step_done = read_status, step_done
        self.interval_s, self.hang_s, self.on_error = interval_s, hang_s, on_error
        self.error = None
        self._armed_at = None
        self._stop = threading.Event()
        self._thread = None

    def start(self) -> "StatusWatchdog":
        self._thread = threading.Thread(target=self._run, name="status-watchdog", daemon=True)
        self._thread.start()
        return self

    def arm(self) -> None:
        """A step has been queued: start its hang clock."""
        self._armed_at = time.time()

    def disarm(self) -> None:
        self._armed_at = None

    def _fail(self, exc) -> None:
        if self.error is None:
            self.error = exc
            if self.on_error is not None:
                try:
                    self.on_error(exc)
                except Exception:  # noqa: BLE001
                    pass

    def _run(self) -> None:
        from ..ops._lib import CollectiveTimeout
        while not self._stop.wait(self.interval_s):
            try:
                code = int(self.read_status())
            except Exception as e:  # noqa: BLE001
                self._fail(e)
                return
            if code != 0:
                self._fail(CollectiveTimeout(code))
                return
            if self._armed_at is not None and self.step_done is not None:
                if self.step_done():
                    self._armed_at = None
                elif time.time() - self._armed_at > self.hang_s:
                    self._fail(StepHung(f"the step queued {time.time() - self._armed_at:.0f}s ago has not finished"))
                    return

    def check(self) -> None:
        if self.error is not None:
            raise self.error

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)


def cuda_watchdog(device, interval_s: float = 0.5, hang_s: float = 120.0, on_error=None) -> StatusWatchdog:
    """Watchdog over the device status word of ``device``. The word is mirrored into pinned host memory by an
    asynchronous copy on a side stream each poll, so polling never blocks the training stream; ``mark_step()``
    records the event whose completion the hang clock watches."""
    import torch

    from ..ops import _lib
    word = _lib.status_word(device)
    host = torch.zeros(1, dtype=torch.int32).pin_memory()
    side = torch.cuda.Stream(device=device)
    state = {"event": None}

    def read_status():
        with torch.cuda.stream(side):
            host.copy_(word, non_blocking=True)
        side.synchronize()
        return int(host[0])

    def step_done():
        ev = state["event"]
        return ev is None or ev.query()

    wd = StatusWatchdog(read_status, step_done, interval_s, hang_s, on_error)

    def mark_step():
        ev = torch.cuda.Event()
        ev.record()
        state["event"] = ev
        wd.arm()
    wd.mark_step = mark_step
    return wd


def _entry(worker, rank, world, attempt, args):
    import sys
    try:
        code = worker(rank, world, attempt, *args)
    except PeerLost:
        code = EXIT_PEER_LOST
    sys.exit(int(code or 0))


def run_elastic(worker, world: int, args=(), max_restarts: int = 3, poll_s: float = 0.1, grace_s: float = 20.0):
    """Run ``worker(rank, world, attempt, *args) -> exit code`` as ``world`` processes until all exit 0. If a rank
    exits non-zero, the others are given ``grace_s`` to notice (heartbeat) and leave by themselves, then terminated
    by process id, and the whole job is started again with ``attempt + 1``. Returns the list of per-attempt exit
    codes; raises ``RuntimeError`` after ``max_restarts`` failed attempts."""
    ctx = mp.get_context("spawn")
    history = []
    for attempt in range(max_restarts + 1):
        procs = [ctx.Process(target=_entry, args=(worker, r, world, attempt, args)) for r in range(world)]
        for p in procs:
            p.start()
        failed_at = None
        while any(p.is_alive() for p in procs):
            time.sleep(poll_s)
            if failed_at is None and any((not p.is_alive()) and p.exitcode != 0 for p in procs):
                failed_at = time.time()
            if failed_at is not None and time.time() - failed_at > grace_s:
                for p in procs:
                    if p.is_alive():
                        p.terminate()          # exactly the processes this supervisor started
        for p in procs:
            p.join()
        codes = [p.exitcode for p in procs]
        history.append(codes)
        if all(c == 0 for c in codes):
            return history
    raise RuntimeError(f"job failed {max_restarts + 1} times: exit codes {history}")
