"""Five-body solar system, dt = 0.01 (reference: examples/nbody.mojo:26-205). Five bodies are no work for a GPU, so
this runs in the C++ host runtime. 50 million steps must end at energy -0.1690599 (nbody.mojo:183-186)."""
from __future__ import annotations

import ctypes
import sys
import time

from ._lib import lib


def run(steps: int, dt: float = 0.01):
    e0 = ctypes.c_double()
    e1 = lib().b2_ex_nbody(steps, dt, ctypes.byref(e0))
    return e0.value, e1


def main() -> None:
    steps = int(sys.argv[1]) if len(sys.argv) > 1 else 50_000_000
    t0 = time.perf_counter()
    e0, e1 = run(steps)
    print(f"energy before {e0:.9f}, after {steps} steps {e1:.9f}  ({time.perf_counter() - t0:.2f} s)")
    if steps == 50_000_000:
        assert abs(e1 - (-0.1690599)) < 1e-6


if __name__ == "__main__":
    main()
