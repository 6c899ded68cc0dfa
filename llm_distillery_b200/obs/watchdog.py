"""Failure detection between ranks on the host: heartbeats + a watchdog.

The reference has none: a stuck inference worker stalls the supervisor's poll loop forever
(classes/teacher/model.py:57-60) and recovery is "run it again" (the SHA sync collects only what is missing,
collect_and_finetune.py:211-291). Here every rank

* writes a heartbeat record ``{rank, step, phase, time}`` into a small file under a directory that all ranks of
  the node see (``/dev/shm`` by default) - from a daemon thread every ``interval`` seconds, and with the current step
  at every step boundary (``beat``);
* runs a watchdog thread that reads the other ranks' records; a rank whose record is older than ``timeout`` seconds,
  or that has said goodbye with ``phase = "failed"``, is reported.

The training / collection loop calls ``check()`` between steps, i.e. with none of its kernels or collectives in
flight: on a reported failure it raises ``RankFailure`` BEFORE the next launch, so that no kernel ever waits for a
peer that is gone; the caller saves its state and leaves. Device-side waits are bounded independently of this (they
report through the device error word, ``ops._lib.take_device_error``), so a failure that slips through between two
checks costs one time-out, not a hung GPU.

A clean exit marks the record ``phase = "done"``: finished ranks are never reported.
"""
from __future__ import annotations

import json
import os
import tempfile
import threading
import time


class RankFailure(RuntimeError):
    def __init__(self, ranks, reason: str):
        super().__init__(f"rank(s) {sorted(ranks)} {reason}")
        self.ranks = sorted(ranks)


def default_dir(run_id: str) -> str:
    base = "/dev/shm" if os.path.isdir("/dev/shm") and os.access("/dev/shm", os.W_OK) else tempfile.gettempdir()
    return os.path.join(base, f"b200_heartbeat_{run_id}")


class Heartbeat:
    def __init__(self, directory: str, rank: int, world: int, interval: float = 1.0, timeout: float = 30.0,
                 stall_timeout: float | None = None, clock=time.time, start_threads: bool = True, on_failure=None,
                 grace: float | None = None):
        """``timeout``: a peer whose record is older than this is gone (its process died). ``stall_timeout``: a peer
        that is alive but has not called ``beat`` for this long while training / collecting is hung (None: off).
        ``on_failure(failed: dict)``: called ONCE from the watchdog thread when a failure has been known for
        ``grace`` seconds (default 2 x timeout) and the main thread has not reacted through ``check()`` - the
        escalation for a main thread that is itself stuck inside a collective."""
        self.dir, self.rank, self.world = directory, rank, world
        self.interval, self.timeout, self.clock = interval, timeout, clock
        self.stall_timeout, self.on_failure = stall_timeout, on_failure
        self.grace = 2.0 * timeout if grace is None else grace
        self._first_failure_at = None
        self._handled = False
        self._step_time = clock()
        os.makedirs(directory, exist_ok=True)
        self.step = 0
        self.phase = "init"
        self.failed: dict[int, str] = {}
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._threads: list[threading.Thread] = []
        self._started = clock()
        self._write()
        if start_threads:
            for fn in (self._beat_loop, self._watch_loop):
                t = threading.Thread(target=fn, daemon=True, name=f"hb-{fn.__name__}")
                t.start()
                self._threads.append(t)

    # ------------------------------------------------------------------ writer side
    def _path(self, rank: int) -> str:
        return os.path.join(self.dir, f"rank{rank}.json")

    def _write(self) -> None:
        rec = {"rank": self.rank, "step": self.step, "phase": self.phase, "time": self.clock(),
               "step_time": self._step_time, "pid": os.getpid()}
        tmp = self._path(self.rank) + f".tmp{os.getpid()}"
        with open(tmp, "w", encoding="utf-8") as f:
            json.dump(rec, f)
        os.replace(tmp, self._path(self.rank))      # readers never see a half-written record

    def beat(self, step: int | None = None, phase: str | None = None) -> None:
        with self._lock:
            if step is not None:
                self.step = step
            if phase is not None:
                self.phase = phase
            self._step_time = self.clock()
            self._write()

    def _beat_loop(self) -> None:
        while not self._stop.wait(self.interval):
            with self._lock:
                if self.phase not in ("done", "failed"):
                    self._write()

    # ------------------------------------------------------------------ reader side
    def read(self, rank: int) -> dict | None:
        try:
            with open(self._path(rank), encoding="utf-8") as f:
                return json.load(f)
        except (OSError, ValueError):
            return None

    def scan(self) -> dict[int, str]:
        """One pass over the peers' records; returns {rank: reason} of ranks considered failed (sticky)."""
        now = self.clock()
        for r in range(self.world):
            if r == self.rank or r in self.failed:
                continue
            rec = self.read(r)
            if rec is not None and float(rec.get("time", 0.0)) < self._started - self.timeout:
                rec = None      # left over from an earlier run with the same id: that rank has not started yet
            if rec is None:
                if now - self._started > self.timeout:
                    self.failed[r] = "never wrote a heartbeat"
            elif rec.get("phase") == "failed":
                self.failed[r] = "reported a failure"
            elif rec.get("phase") != "done" and now - float(rec.get("time", 0.0)) > self.timeout:
                self.failed[r] = f"stopped beating {now - float(rec['time']):.1f} s ago at step {rec.get('step')}"
            elif (self.stall_timeout is not None and rec.get("phase") in ("train", "collect")
                  and now - float(rec.get("step_time", now)) > self.stall_timeout):
                self.failed[r] = f"made no progress for {now - float(rec['step_time']):.1f} s at step {rec.get('step')}"
        if self.failed and self._first_failure_at is None:
            self._first_failure_at = now
        return dict(self.failed)

    def _watch_loop(self) -> None:
        while not self._stop.wait(self.interval):
            failed = self.scan()
            if (failed and self.on_failure is not None and not self._handled
                    and self.clock() - self._first_failure_at > self.grace):
                self._handled = True
                self.on_failure(failed)

    def check(self) -> None:
        """Call between steps (nothing of this rank in flight). Raises RankFailure if a peer is gone."""
        failed = self.scan()
        if failed:
            self._handled = True
            r = sorted(failed)
            raise RankFailure(r, "; ".join(f"rank {k}: {failed[k]}" for k in r))

    # ------------------------------------------------------------------ shutdown
    def close(self, phase: str = "done") -> None:
        self._stop.set()
        with self._lock:
            self.phase = phase
            try:
                self._write()
            except OSError:
                pass
        for t in self._threads:
            t.join(timeout=2 * self.interval + 1.0)


def from_env(rank: int, world: int, **kw) -> Heartbeat | None:
    """Heartbeat for a torchrun job (run id = MASTER_PORT + TORCHELASTIC_RUN_ID), or None for a single process."""
    if world <= 1:
        return None
    run_id = f"{os.environ.get('TORCHELASTIC_RUN_ID', 'run')}_{os.environ.get('MASTER_PORT', '0')}"
    return Heartbeat(default_dir(run_id), rank, world, **kw)
