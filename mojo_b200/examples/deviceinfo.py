"""Print what the runtime sees of the machine (reference: examples/deviceinfo.mojo:38-80 prints CPU features): GPU name,
compute capability, SMs, shared memory, L2, memory, clocks, peer access and NVLS multicast support."""
from __future__ import annotations

from .. import _ext


def main() -> None:
    C = _ext.require()
    import torch

    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    print(f"visible CUDA devices: {n}")
    for d in range(n):
        caps = C.device_caps(d)
        print(f"device {d}: {caps.get('name')}")
        for k in ("cc_major", "cc_minor", "sm_count", "smem_per_block_optin", "l2_bytes", "total_mem", "clock_khz", "mem_clock_khz",
                  "can_map_peer", "multicast_supported", "max_cluster"):
            print(f"  {k:22s} {caps.get(k)}")
        ok = caps.get("cc_major") == 10 and caps.get("cc_minor") == 0
        print(f"  sm_100a kernels usable : {ok}")


if __name__ == "__main__":
    main()
