"""Conway's Game of Life on a 1024x1024 torus (reference: examples/life/gridv2.mojo:97-125, benchmark
examples/life/benchmark.mojo:22-62). One generation = one stencil kernel; the reference's pygame window
(examples/life/lifev2.mojo:29-83) is left out: no graphics stack exists here, the grid stays a device buffer."""
from __future__ import annotations

import time

import numpy as np
import torch

from ._lib import lib, ptr, stream, time_cuda


def evolve_gpu(grid: torch.Tensor) -> torch.Tensor:
    nxt = torch.empty_like(grid)
    assert lib().b2_ex_life(ptr(grid), ptr(nxt), grid.shape[0], grid.shape[1], stream()) == 0
    return nxt


def evolve_cpu(g: np.ndarray) -> np.ndarray:
    n = sum(np.roll(np.roll(g, dr, 0), dc, 1) for dr in (-1, 0, 1) for dc in (-1, 0, 1) if (dr, dc) != (0, 0))
    return ((n | g) == 3).astype(np.uint8)


def main() -> None:
    rng = np.random.default_rng(0)
    g = (rng.random((1024, 1024)) < 0.5).astype(np.uint8)
    gd = torch.from_numpy(g).cuda()
    cur_cpu, cur_gpu = g, gd
    t0 = time.perf_counter()
    for _ in range(10):
        cur_cpu = evolve_cpu(cur_cpu)
    cpu_ms = (time.perf_counter() - t0) * 1e3 / 10
    for _ in range(10):
        cur_gpu = evolve_gpu(cur_gpu)
    assert np.array_equal(cur_gpu.cpu().numpy(), cur_cpu)
    ms = time_cuda(lambda: evolve_gpu(gd))
    print(f"life 1024x1024: CPU numpy {cpu_ms:.2f} ms/gen, GPU {ms * 1e3:.1f} us/gen, live cells after 10 gens: {int(cur_cpu.sum())}")


if __name__ == "__main__":
    main()
