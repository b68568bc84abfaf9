"""Per-device scratch owned by the op layer: the status word every kernel reports into, the split-K GEMM
workspace and the split-KV attention workspace. Allocated once per device on first use."""
from __future__ import annotations

import torch

from .. import _ext

STATUS_CODES = {0: "OK", 1: "TIMEOUT", 2: "ASSERT", 3: "OUT_OF_BOUNDS", 4: "BAD_ARGUMENT", 5: "TOO_LARGE"}
STATUS_SITES = {
    0: "none", 1: "gemm.full", 2: "gemm.empty", 3: "gemm.tmem_full", 4: "gemm.tmem_empty", 5: "gemm.drain",
    6: "gemm.split_k", 7: "peer.signal", 8: "grid.barrier", 9: "ag.chunk", 10: "rs.tile", 11: "ep.count",
    12: "attention", 13: "kv.index", 14: "sampling", 15: "test",
}

GEMM_WORKSPACE_BYTES = 96 << 20
ATTN_WORKSPACE_BYTES = 64 << 20


class KernelError(RuntimeError):
    """A device-side check failed or a bounded wait ran out; the CUDA context is still usable."""

    def __init__(self, code: int, site: int, block: int, thread: int, a: int, b: int):
        self.code, self.site, self.block, self.thread, self.a, self.b = code, site, block, thread, a, b
        super().__init__(
            f"kernel reported {STATUS_CODES.get(code, code)} at {STATUS_SITES.get(site, site)} "
            f"(block {block}, thread {thread}, a={a}, b={b})"
        )


class _DeviceState:
    def __init__(self, device: torch.device):
        self.status = torch.zeros(8, dtype=torch.int32, device=device)
        self.gemm_ws = torch.zeros(GEMM_WORKSPACE_BYTES // 4, dtype=torch.int32, device=device)
        self.attn_ws = torch.empty(ATTN_WORKSPACE_BYTES // 4, dtype=torch.float32, device=device)
        # per (sequence, kv head) arrival counters of the split decode attention (self-resetting; zero between launches)
        self.attn_counters = torch.zeros(1 << 18, dtype=torch.int32, device=device)


_states: dict[int, _DeviceState] = {}


def get(device: torch.device) -> _DeviceState:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    st = _states.get(idx)
    if st is None:
        _ext.require()
        st = _DeviceState(torch.device("cuda", idx))
        _states[idx] = st
    return st


def check_status(device: torch.device | None = None, reset: bool = True) -> None:
    """Read the status word (synchronises the device) and raise KernelError if a kernel recorded a problem."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    st = get(device)
    words = st.status.cpu()
    code = int(words[0])
    if code == 0:
        return
    a = (int(words[5]) << 32) | (int(words[4]) & 0xFFFFFFFF)
    b = (int(words[7]) << 32) | (int(words[6]) & 0xFFFFFFFF)
    if reset:
        st.status.zero_()
        st.gemm_ws[: 65536].zero_()  # split-K counters may be left mid-count by an aborted kernel
        st.attn_counters.zero_()
    raise KernelError(code, int(words[1]), int(words[2]), int(words[3]), a, b)
