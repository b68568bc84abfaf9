"""Matmul walk-through (reference: examples/matmul.mojo:103-280, a CPU tutorial from naive loops to tiled+parallel):
the GPU steps are naive (one thread per output) -> shared-memory tiles -> the tcgen05/TMEM GEMM of this library.
Every variant is checked against the naive CPU product, like `test_all` in the reference (matmul.mojo:330-356)."""
from __future__ import annotations

import time

import torch

from .. import ops
from ._lib import lib, ptr, stream, time_cuda

M, N, K = 512, 4096, 512   # the reference's problem size


def gpu_variant(a: torch.Tensor, b: torch.Tensor, variant: int) -> torch.Tensor:
    c = torch.empty(a.shape[0], b.shape[1], dtype=torch.float32, device=a.device)
    rc = lib().b2_ex_matmul(ptr(a), ptr(b), ptr(c), a.shape[0], b.shape[1], a.shape[1], variant, stream())
    assert rc == 0
    return c


def tensor_core(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return ops.linear(a.bfloat16(), b.t().contiguous().bfloat16())


def main() -> None:
    g = torch.Generator().manual_seed(0)
    a, b = torch.rand(M, K, generator=g), torch.rand(K, N, generator=g)
    t0 = time.perf_counter()
    want = a @ b
    cpu_ms = (time.perf_counter() - t0) * 1e3
    ad, bd = a.cuda(), b.cuda()
    flops = 2.0 * M * N * K
    print(f"CPU (torch, fp32): {cpu_ms:8.3f} ms  {flops / cpu_ms / 1e6:9.1f} GFLOP/s")
    for name, fn, tol in (("naive", lambda: gpu_variant(ad, bd, 0), 1e-3), ("tiled smem", lambda: gpu_variant(ad, bd, 1), 1e-3),
                          ("tcgen05 bf16", lambda: tensor_core(ad, bd), 1.5)):
        torch.testing.assert_close(fn().float().cpu(), want, atol=tol, rtol=2e-2)
        ms = time_cuda(fn)
        print(f"GPU {name:12s}: {ms:8.3f} ms  {flops / ms / 1e6:9.1f} GFLOP/s")


if __name__ == "__main__":
    main()
