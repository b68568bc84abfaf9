"""Host-side fault injection. Faults are made on the host or among CPU ranks, never on a GPU: a rank that raises,
sleeps, skips a launch or leaves between steps; a dropped signal in the CPU-rank simulator.

The spec is a colon-separated string, usually from the `B2_FAULT` environment variable:

    raise:rank=1:step=3           rank 1 raises InjectedFault at the start of step 3
    raise_after:rank=1:step=3     rank 1 raises InjectedFault at the end of step 3, after its launches and collectives
                                  have completed (what a kernel status error looks like to the host)
    delay:rank=0:step=2:ms=500    rank 0 sleeps 500 ms before step 2
    skip_launch:rank=2:step=5     rank 2 does not launch step 5 (the engine runs the scheduler but not the model)
    leave:rank=3:step=4           rank 3 announces that it is leaving and exits its loop before step 4
    drop_signal:rank=1:step=7     only meaningful to the CPU-rank simulator (`symm_sim_run`)

`FaultInjector.before_step(step)` and `after_execute(step)` are the hooks the engine loop calls.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass

KINDS = ("raise", "raise_after", "delay", "skip_launch", "leave", "drop_signal")


class InjectedFault(RuntimeError):
    """Raised by a `raise:` fault spec."""


class RankLeaving(Exception):
    """Raised by a `leave:` fault spec: the rank must stop between steps, with nothing in flight."""


@dataclass
class FaultSpec:
    kind: str
    rank: int = 0
    step: int = 0
    ms: int = 0

    def __str__(self) -> str:
        s = f"{self.kind}:rank={self.rank}:step={self.step}"
        return s + (f":ms={self.ms}" if self.ms else "")


def parse(spec: str | None) -> FaultSpec | None:
    if not spec or spec == "none":
        return None
    parts = spec.split(":")
    if parts[0] not in KINDS:
        raise ValueError(f"unknown fault kind {parts[0]!r} (one of {', '.join(KINDS)})")
    f = FaultSpec(parts[0])
    for p in parts[1:]:
        key, _, val = p.partition("=")
        if key not in ("rank", "step", "ms") or not val.isdigit():
            raise ValueError(f"malformed fault field {p!r} in {spec!r}")
        setattr(f, key, int(val))
    return f


def from_env() -> FaultSpec | None:
    return parse(os.environ.get("B2_FAULT"))


class FaultInjector:
    """Applies one fault spec to the rank that owns it."""

    def __init__(self, spec: FaultSpec | str | None, rank: int):
        self.spec = parse(spec) if isinstance(spec, str) else spec
        self.rank = rank
        self.fired = False

    def _mine(self, step: int) -> bool:
        s = self.spec
        return s is not None and not self.fired and s.rank == self.rank and s.step == step

    def after_execute(self, step: int) -> None:
        """Called when the step's device work has been issued and its results read back."""
        if self.spec is not None and self.spec.kind == "raise_after" and self._mine(step):
            self.fired = True
            raise InjectedFault(f"injected fault on rank {self.rank} after step {step}")

    def before_step(self, step: int) -> bool:
        """Returns True when this step's launch must be skipped. May sleep or raise, according to the spec."""
        if not self._mine(step) or self.spec.kind == "raise_after":
            return False
        self.fired = True
        kind = self.spec.kind
        if kind == "raise":
            raise InjectedFault(f"injected fault on rank {self.rank} at step {step}")
        if kind == "leave":
            raise RankLeaving(f"rank {self.rank} leaves before step {step}")
        if kind == "delay":
            time.sleep(self.spec.ms / 1e3)
            return False
        return kind == "skip_launch"
