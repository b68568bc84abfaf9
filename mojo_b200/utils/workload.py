"""Synthetic serving workloads: Poisson arrivals, uniform prompt/output lengths, uniform-random token ids.
Everything derives from one seed so every rank of a tensor-parallel job builds the identical trace."""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass
class SyntheticRequest:
    arrival: float          # seconds after the start of the trace
    prompt: np.ndarray      # int32 token ids
    max_tokens: int


def poisson_trace(n: int, rate: float, prompt_range=(128, 2048), output_range=(64, 512), vocab: int = 128256,
                  seed: int = 0) -> list[SyntheticRequest]:
    """`n` requests with exponential inter-arrival times of mean 1/rate (rate <= 0: all arrive at t = 0)."""
    rng = np.random.default_rng(seed)
    gaps = rng.exponential(1.0 / rate, size=n) if rate > 0 else np.zeros(n)
    t = np.cumsum(gaps)
    out = []
    for i in range(n):
        pl = int(rng.integers(prompt_range[0], prompt_range[1] + 1))
        ol = int(rng.integers(output_range[0], output_range[1] + 1))
        out.append(SyntheticRequest(float(t[i]), rng.integers(0, vocab, size=pl, dtype=np.int32), ol))
    return out


def fixed_batch(n: int, prompt_len: int, output_len: int, vocab: int, seed: int = 0) -> list[SyntheticRequest]:
    rng = np.random.default_rng(seed)
    return [SyntheticRequest(0.0, rng.integers(0, vocab, size=prompt_len, dtype=np.int32), output_len) for _ in range(n)]
