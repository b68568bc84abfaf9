"""Measured configuration tables for the bf16 tcgen05 GEMM.

The analytic rule in the kernel picks a good configuration for most shapes, but near tile-count boundaries the
best tile width, split-K factor or stream-K choice is decided by effects it does not model (L2 sharing between
CTAs, the wave tail). `tune()` times every valid configuration of one weight shape at a set of token counts with
CUDA events, on rotating weight copies larger than L2 (in serving a layer's weights are always cold), and records
the winner per token-count bucket; `lookup()` is what `ops.linear` / `ops.linear_swiglu` consult when the caller
passes no explicit configuration. Host-side only: the table is consulted before launch, so it works under
CUDA-graph capture. Tuning itself must not run under capture.
"""
from __future__ import annotations

import bisect

import torch

EPI_NONE, EPI_ADD_RESIDUAL, EPI_SWIGLU = 0, 1, 2
PAIR_CONFIG = 1 << 28
L2_BYTES = 126 << 20

# (N, K, epilogue, device index) -> (sorted list of bucket upper bounds, configs)
_TABLE: dict[tuple, tuple[list, list]] = {}
enabled = True


def _encode(swap: bool, bn: int, splits: int = 1, stream_k: bool = False) -> int:
    return (int(swap) << 30) | (int(stream_k) << 29) | ((1 if stream_k else splits) << 16) | bn


def describe(config: int) -> str:
    if config == 0:
        return "auto"
    if config & PAIR_CONFIG:
        return f"CTA pair 256x{(config & 0xffff) or 256}"
    return f"{'swap' if (config >> 30) & 1 else 'normal'} bn={config & 0xffff} splits={(config >> 16) & 0xff}" + (" stream-k" if (config >> 29) & 1 else "")


def candidates(M: int, N: int, K: int, epilogue: int) -> list[int]:
    """Every configuration the kernel accepts for this shape that is not obviously wasteful."""
    num_kb = (K + 63) // 64
    out = []

    def ws_ok(tiles, splits, bn):
        return tiles <= 65536 and tiles * splits * bn * 128 * 4 <= (64 << 20)

    if M <= 256:
        for bn in (16, 32, 64, 128, 256):
            if bn * 4 < M or (bn >= 2 * M and bn > 16):
                continue
            tiles = ((N + 127) // 128) * ((M + bn - 1) // bn)
            for sp in (1, 2, 4, 8):
                if sp > 1 and (num_kb // sp < 4 or not ws_ok(tiles, sp, bn)):
                    continue
                out.append(_encode(True, bn, sp))
            if M <= bn and num_kb >= 8 and tiles % 148 != 0:
                out.append(_encode(True, bn, 1, True))
    if M > 64 and N % 8 == 0:
        for bn in (64, 96, 128, 160, 192, 224, 256):
            if epilogue == EPI_SWIGLU and bn < 32:
                continue
            tiles = ((M + 127) // 128) * ((N + bn - 1) // bn)
            for sp in (1, 2, 4):
                if sp > 1 and (num_kb // sp < 4 or not ws_ok(tiles, sp, bn) or tiles * sp > 4 * 148):
                    continue
                out.append(_encode(False, bn, sp))
    if M >= 192 and N >= 256 and N % 8 == 0 and epilogue != EPI_ADD_RESIDUAL:
        out.append(PAIR_CONFIG | 256)   # 256 x 256 tiles on CTA pairs
        out.append(PAIR_CONFIG | 128)   # 256 x 128
    return out


def _time(fn, iters: int) -> float:
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    fn()
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    e.synchronize()
    return s.elapsed_time(e) / iters


def tune(N: int, K: int, epilogue: int, token_counts, device=None, iters: int = 3, weight: torch.Tensor | None = None) -> dict:
    """Time all candidates for weight shape [N, K] at each token count; fill the lookup table. Returns
    {M: (config, microseconds, microseconds of the analytic rule's choice)}."""
    from .. import _ext
    from . import _launch_gemm as _launch
    from . import _state

    C = _ext.require()
    if not isinstance(device, torch.device):
        device = torch.device("cuda", torch.cuda.current_device())
    st = _state.get(device)
    copies = max(2, min(16, (2 * L2_BYTES) // (N * K * 2) + 1))
    ws = [weight] if weight is not None else []
    while len(ws) < copies:
        ws.append(torch.randn(N, K, device=device, dtype=torch.bfloat16) * 0.02)
    n_out = N // 2 if epilogue == EPI_SWIGLU else N
    report = {}
    bounds, configs = [], []
    for M in sorted(set(int(m) for m in token_counts)):
        x = torch.randn(M, K, device=device, dtype=torch.bfloat16)
        y = torch.empty(M, n_out, device=device, dtype=torch.bfloat16)
        res = torch.zeros(M, n_out, device=device, dtype=torch.bfloat16) if epilogue == EPI_ADD_RESIDUAL else None
        turn = [0]

        def run(cfg):
            w = ws[turn[0] % len(ws)]
            turn[0] += 1
            _launch(C, x, w, y, res, epilogue, cfg, st)

        best_cfg, best_t = 0, _time(lambda: run(0), iters)
        t_auto = best_t
        for cfg in candidates(M, N, K, epilogue):
            t = _time(lambda: run(cfg), iters)
            if t < best_t * 0.98:  # prefer the analytic choice on a tie
                best_cfg, best_t = cfg, t
        bounds.append(M)
        configs.append(best_cfg)
        report[M] = (best_cfg, best_t * 1e3, t_auto * 1e3)
    _TABLE[(N, K, epilogue, device.index or 0)] = (bounds, configs)
    return report


def lookup(M: int, N: int, K: int, epilogue: int, device_index: int = 0) -> int:
    """Configuration of the smallest tuned token count >= M (0 = let the kernel's own rule decide)."""
    if not enabled:
        return 0
    entry = _TABLE.get((N, K, epilogue, device_index))
    if entry is None:
        return 0
    bounds, configs = entry
    i = bisect.bisect_left(bounds, M)
    if i >= len(bounds):
        return 0
    # a bucket far above M was tuned for a different tile count: only trust near neighbours
    if bounds[i] > 2 * M and bounds[i] - M > 128:
        return 0
    return configs[i]


def clear() -> None:
    _TABLE.clear()


def default_token_counts(max_tokens: int, decode_buckets=()) -> list[int]:
    ms = set(int(b) for b in decode_buckets)
    ms.update(m for m in (1, 2, 4, 8, 16, 32, 64, 128, 192, 256) if m <= max_tokens)
    m = 384
    while m <= max_tokens:
        ms.add(m)
        m += 128
    return sorted(ms)
