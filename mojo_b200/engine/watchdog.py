"""Failure detection for the engine loop, all of it on the host.

`Watchdog`   a thread per worker that watches the iteration heartbeat of its own process: when no step finishes
             within the limit it marks the worker unhealthy, dumps the Python stacks and calls `on_stall`.
`Heartbeat`  cross-rank liveness through a key-value store (`torch.distributed.TCPStore` / `FileStore` / any
             object with set/get): every rank publishes `(step, wall time)` after each step, or the word "left"
             when it leaves on purpose; `check()` raises `WorkerLost` before the next launch when a peer is
             stale or gone. A rank leaves only between steps, with none of its kernels or collectives in flight.
`recover()`  the recovery policy: abort what is running, re-queue every unfinished request so that it is
             recomputed from its prompt plus the tokens it had already produced. No elastic resize.
"""
from __future__ import annotations

import faulthandler
import sys
import threading
import time


class WorkerLost(RuntimeError):
    def __init__(self, ranks, reason: str):
        super().__init__(f"worker rank(s) {ranks} {reason}")
        self.ranks = list(ranks)
        self.reason = reason


class Watchdog:
    def __init__(self, limit_s: float = 60.0, on_stall=None, poll_s: float | None = None, dump_stacks: bool = True):
        self.limit_s = limit_s
        self.on_stall = on_stall
        self.poll_s = poll_s if poll_s is not None else min(1.0, limit_s / 4)
        self.dump_stacks = dump_stacks
        self.healthy = True
        self.stalls = 0
        self.last_step = -1
        self._last_beat = time.monotonic()
        self._busy = False
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None

    def start(self) -> "Watchdog":
        self._thread = threading.Thread(target=self._run, name="b2-watchdog", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)

    def begin_step(self) -> None:
        self._busy = True
        self._last_beat = time.monotonic()

    def end_step(self, step: int) -> None:
        self._busy = False
        self.last_step = step
        self._last_beat = time.monotonic()
        self.healthy = True

    def seconds_since_beat(self) -> float:
        return time.monotonic() - self._last_beat

    def _run(self) -> None:
        reported = False
        while not self._stop.wait(self.poll_s):
            stalled = self._busy and self.seconds_since_beat() > self.limit_s
            if stalled and not reported:
                reported = True
                self.healthy = False
                self.stalls += 1
                if self.dump_stacks:
                    faulthandler.dump_traceback(file=sys.stderr, all_threads=True)
                if self.on_stall is not None:
                    self.on_stall(self)
            elif not stalled:
                reported = False


class Heartbeat:
    def __init__(self, store, rank: int, world_size: int, limit_s: float = 30.0, prefix: str = "b2hb"):
        self.store, self.rank, self.world, self.limit_s, self.prefix = store, rank, world_size, limit_s, prefix
        self.beat(-1)

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self, step: int) -> None:
        self.store.set(self._key(self.rank), f"{step}:{time.time():.6f}")

    def leave(self) -> None:
        self.store.set(self._key(self.rank), "left")

    def _read(self, r: int):
        try:
            raw = self.store.get(self._key(r))
        except Exception:  # noqa: BLE001 - a key that was never written
            return None
        return raw.decode() if isinstance(raw, (bytes, bytearray)) else str(raw)

    def peers(self) -> dict:
        """rank -> ("left", None) | ("alive" | "stale" | "unknown", step)."""
        now, out = time.time(), {}
        for r in range(self.world):
            v = self._read(r)
            if v is None:
                out[r] = ("unknown", None)
            elif v == "left":
                out[r] = ("left", None)
            else:
                step, _, t = v.partition(":")
                out[r] = ("alive" if now - float(t) <= self.limit_s else "stale", int(step))
        return out

    def check(self) -> None:
        """Call before each launch: raises `WorkerLost` when a peer has left or stopped beating."""
        st = self.peers()
        gone = [r for r, (s, _) in st.items() if s == "left" and r != self.rank]
        if gone:
            raise WorkerLost(gone, "left the job")
        stale = [r for r, (s, _) in st.items() if s == "stale" and r != self.rank]
        if stale:
            raise WorkerLost(stale, f"sent no heartbeat for more than {self.limit_s:.1f} s")


def recover(engine) -> list[int]:
    """Re-queue every unfinished request of `engine` for recomputation: its new prompt is the old prompt plus the
    tokens already produced, its token budget shrinks by the same amount, and its KV pages are released. Returns
    the re-queued request ids (same ids, so callers that stream by id keep working)."""
    if hasattr(engine, "discard_inflight"):
        engine.discard_inflight()      # a pipelined engine may have a step in flight whose tokens were never booked
    redo = []
    for rid, st in list(engine.requests.items()):
        if st.finished:
            continue
        prompt = list(engine.prompt_of(rid)) + list(st.output_ids)
        engine.scheduler.abort(rid)
        redo.append((rid, prompt, st))
    for rid, prompt, st in redo:
        remaining = max(1, st.params.max_tokens - len(st.output_ids))
        engine.readmit(rid, prompt, remaining, st)
    return [r for r, _, _ in redo]
