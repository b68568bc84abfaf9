"""Run every example in turn: `python -m mojo_b200.examples [name ...]`.

The counterpart of the reference's `examples/run-examples.sh` (it runs each program with a RUN line through lit,
examples/lit.cfg.py:19-56). Each example checks its kernel against a CPU restatement before it prints timings, so a
clean run of this module is the examples' integration test. Without a CUDA device only the host-side examples run
(n-body; the others are reported as skipped). Exit status 1 if any example failed."""
from __future__ import annotations

import importlib
import sys
import time
import traceback

EXAMPLES = ("deviceinfo", "matmul", "mandelbrot", "nbody", "reduce", "life", "raytrace")
HOST_ONLY = ("nbody",)


def main(argv=None) -> int:
    import torch

    names = list(argv if argv is not None else sys.argv[1:]) or list(EXAMPLES)
    unknown = [n for n in names if n not in EXAMPLES]
    if unknown:
        print(f"unknown example(s) {unknown}; available: {', '.join(EXAMPLES)}", file=sys.stderr)
        return 2
    have_gpu = torch.cuda.is_available()
    failed = []
    for name in names:
        if not have_gpu and name not in HOST_ONLY:
            print(f"== {name}: skipped (needs a CUDA device)")
            continue
        print(f"== {name}", flush=True)
        t0 = time.perf_counter()
        saved = sys.argv
        sys.argv = [f"mojo_b200.examples.{name}"]     # the examples read their own options from sys.argv: give them none
        try:
            importlib.import_module(f"mojo_b200.examples.{name}").main()
        except Exception:  # noqa: BLE001  (report and go on with the next example)
            traceback.print_exc()
            failed.append(name)
        finally:
            sys.argv = saved
        print(f"   ({time.perf_counter() - t0:.1f} s)", flush=True)
    if failed:
        print(f"FAILED: {', '.join(failed)}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
