"""Mandelbrot escape-time kernel, 960x960, 200 iterations over [-2, 0.6] x [-1.5, 1.5] (reference:
examples/mandelbrot.mojo:24-69). Output is an int32 iteration-count buffer on the device; the reference's plotting
is dropped. Oracle and timed CPU baseline: the same recurrence in numpy."""
from __future__ import annotations

import time

import ctypes

import numpy as np
import torch

from ._lib import lib, ptr, stream, time_cuda

ROWS = COLS = 960
MAX_ITERS = 200
MIN_X, MAX_X, MIN_Y, MAX_Y = -2.0, 0.6, -1.5, 1.5


def gpu() -> torch.Tensor:
    out = torch.empty(ROWS, COLS, dtype=torch.int32, device="cuda")
    assert lib().b2_ex_mandelbrot(ptr(out), ROWS, COLS, MAX_ITERS, *(ctypes.c_float(v) for v in (MIN_X, MAX_X, MIN_Y, MAX_Y)), stream()) == 0
    return out


def cpu() -> np.ndarray:
    f = np.float32
    cx = (f(MIN_X) + np.arange(COLS, dtype=f) * f((f(MAX_X) - f(MIN_X)) / f(COLS)))[None, :].repeat(ROWS, 0)
    cy = (f(MIN_Y) + np.arange(ROWS, dtype=f) * f((f(MAX_Y) - f(MIN_Y)) / f(ROWS)))[:, None].repeat(COLS, 1)
    x = np.zeros_like(cx); y = np.zeros_like(cx)
    iters = np.zeros(cx.shape, np.int32)
    alive = np.ones(cx.shape, bool)
    for _ in range(MAX_ITERS):
        y2 = y * y
        ynew = x * (y + y) + cy
        inside = (x * x + y2) <= 4
        xnew = x * x + (cx - y2)
        alive &= inside
        iters += alive
        x = np.where(alive, xnew, x); y = np.where(alive, ynew, y)
    return iters


def main() -> None:
    import ctypes  # noqa: F401

    t0 = time.perf_counter()
    want = cpu()
    cpu_ms = (time.perf_counter() - t0) * 1e3
    got = gpu().cpu().numpy()
    mism = (got != want).mean()
    assert mism < 5e-3, f"{mism:.4%} of pixels differ"   # fma contraction moves a few boundary pixels (0.21 % measured)
    ms = time_cuda(gpu)
    print(f"mandelbrot {ROWS}x{COLS}, {MAX_ITERS} iters: CPU numpy {cpu_ms:.1f} ms, GPU {ms * 1e3:.1f} us, speed-up {cpu_ms / ms:.0f}x, "
          f"{(got == MAX_ITERS).sum()} pixels in the set")


if __name__ == "__main__":
    main()
