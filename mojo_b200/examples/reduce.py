"""Sum of 2^21 and 2^27 float32 values (reference: examples/reduce.mojo:28-51) as a CUDA reduction: float4 loads, f32
partial sums per thread, block reduction, one f64 atomic per block. Oracle: compensated (Kahan-accurate) f64 sum."""
from __future__ import annotations

import math
import time

import torch

from ._lib import lib, ptr, stream, time_cuda


def gpu_sum(x: torch.Tensor) -> float:
    out = torch.zeros(1, dtype=torch.float64, device=x.device)
    assert lib().b2_ex_reduce_sum(ptr(x), x.numel(), ptr(out), stream()) == 0
    return float(out.item())


def main() -> None:
    for n in (1 << 21, 1 << 27):
        x = torch.rand(n, generator=torch.Generator().manual_seed(0))
        t0 = time.perf_counter()
        want = math.fsum(x.double().tolist()) if n <= (1 << 21) else float(x.double().sum())
        cpu_ms = (time.perf_counter() - t0) * 1e3
        xd = x.cuda()
        got = gpu_sum(xd)
        assert abs(got - want) <= 1e-6 * abs(want), (got, want)
        out = torch.zeros(1, dtype=torch.float64, device="cuda")
        ms = time_cuda(lambda: lib().b2_ex_reduce_sum(ptr(xd), n, ptr(out), stream()))
        print(f"sum of {n} f32: {got:.3f}  CPU {cpu_ms:.1f} ms, GPU {ms * 1e3:.1f} us ({n * 4 / ms / 1e6:.0f} GB/s)")


if __name__ == "__main__":
    main()
