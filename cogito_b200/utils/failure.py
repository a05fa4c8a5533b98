"""Failure detection and restart for multi-rank jobs.

Detection is host-side and happens between steps: every rank publishes a heartbeat (a counter
and a wall-clock stamp) in the job's key-value store; before a step a rank checks its peers and
raises ``RankFailure`` instead of entering a collective that can no longer complete.  A rank
that leaves does so between steps, with no kernel or collective in flight.  Device-side waits
of this library are bounded and report through the status word (``ops._lib.read_status``), so a
peer that vanished mid-kernel ends the kernel with an error code, not a hang; ``check_device``
folds that into the same exception.  As a last line a short process-group timeout turns a
stuck collective into an error.

Recovery: ``run_with_restarts`` calls the training function; on ``RankFailure`` the survivors
tear the process group down, agree on the new world through the store, re-initialise and call
the function again, which resumes from the last checkpoint (see ``io.checkpoint``).

The reference has no failure handling: the results of its NCCL calls are ignored
(src/pipeline/pipeline.c:111,126, src/pipeline/tensor_parallel.c:68,100), CUDA errors are turned
into a string and the function returns (src/cuda/cg_cuda.c:33-49), and its error enumeration
(include/cogito.h:47-53) has no code for a timeout.
"""
from __future__ import annotations

import threading
import time


class RankFailure(RuntimeError):
    def __init__(self, dead, reason=""):
        super().__init__(f"ranks {sorted(dead)} stopped responding {reason}".strip())
        self.dead = sorted(dead)


class Heartbeat:
    """Publishes this rank's liveness and watches the others.

    store: a ``torch.distributed`` store (TCPStore / FileStore / HashStore) or any object with
    ``set(key, bytes)`` and ``get(key)``; a beat is written every ``interval`` seconds by a
    daemon thread; a peer counts as dead when its last beat is older than ``timeout`` seconds or
    when it has announced its exit."""

    def __init__(self, store, rank: int, world: int, interval: float = 0.5, timeout: float = 5.0, prefix: str = "hb", clock=time.time):
        self.store, self.rank, self.world = store, rank, world
        self.interval, self.timeout, self.prefix, self.clock = interval, timeout, prefix, clock
        self._stop = threading.Event()
        self._thread = None
        self.beats = 0

    def _key(self, r):
        return f"{self.prefix}/{r}"

    def beat(self):
        self.beats += 1
        self.store.set(self._key(self.rank), f"{self.beats} {self.clock():.3f} alive")

    def announce_exit(self):
        self.store.set(self._key(self.rank), f"{self.beats} {self.clock():.3f} exit")

    def start(self):
        self.beat()
        if self.interval > 0:
            def loop():
                while not self._stop.wait(self.interval):
                    try:
                        self.beat()
                    except Exception:
                        return
            self._thread = threading.Thread(target=loop, daemon=True)
            self._thread.start()
        return self

    def stop(self, announce: bool = True):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1)
        if announce:
            try:
                self.announce_exit()
            except Exception:
                pass

    def dead_ranks(self, wait_for_first: bool = True):
        now = self.clock()
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                raw = self.store.get(self._key(r))
            except Exception:
                raw = None
            if raw is None:
                if not wait_for_first:
                    dead.append(r)
                continue
            text = raw.decode() if isinstance(raw, (bytes, bytearray)) else str(raw)
            _, stamp, state = text.split()
            if state == "exit" or now - float(stamp) > self.timeout:
                dead.append(r)
        return dead

    def check(self):
        dead = self.dead_ranks()
        if dead:
            raise RankFailure(dead)

    def guard(self, fn, *args, **kw):
        """Runs a collective.  A peer that left while this rank was already inside it shows up as a
        transport error (connection reset, timeout) rather than as a stale heartbeat: on such an error
        wait up to ``timeout`` + 1 s for the heartbeats to name the dead ranks and raise ``RankFailure``
        with them; if every peer is alive the original error is raised."""
        try:
            return fn(*args, **kw)
        except RankFailure:
            raise
        except Exception as e:
            end = time.time() + self.timeout + 1.0
            while True:
                dead = self.dead_ranks()
                if dead:
                    raise RankFailure(dead) from e
                if time.time() >= end:
                    raise
                time.sleep(min(0.1, max(self.interval, 0.01)))


def check_device():
    """Raise when a kernel of this library reported a bounded wait that ran out."""
    import torch
    if not torch.cuda.is_available():
        return
    from ..ops import _lib
    code, where, block, aux = _lib.read_status()
    if code != 0:
        raise RankFailure([], f"(device status code={code} where={where} block={block} aux={aux})")


def run_with_restarts(fn, make_group, max_restarts: int = 3, on_restart=None):
    """fn(world_info) runs the training loop and returns its result; make_group(attempt, dead)
    (re)creates the process group for the surviving ranks and returns ``world_info`` (whatever
    fn needs: rank, world size, heartbeat...), or None when this rank is not part of the new
    world.  Restarts at most ``max_restarts`` times."""
    dead, attempt = [], 0
    while True:
        info = make_group(attempt, dead)
        if info is None:
            return None
        try:
            return fn(info)
        except RankFailure as e:
            attempt += 1
            dead = e.dead
            if on_restart is not None:
                on_restart(attempt, e)
            if attempt > max_restarts:
                raise
