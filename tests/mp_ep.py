"""Multi-GPU worker: expert-parallel MoE (dispatch / grouped GEMM / combine kernels) against the dense fp32 reference.
Every rank owns E / world experts and its own tokens (different counts per rank, one rank with none at all)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mojo_b200 import ops  # noqa: E402
from mojo_b200.ops import reference as ref  # noqa: E402
from mojo_b200.parallel import init_distributed  # noqa: E402
from mojo_b200.parallel.ep import EPComm  # noqa: E402


def main():
    info = init_distributed("cuda")
    rank, world, dev = info.rank, info.world_size, info.device
    E, k, H, F = 16 * world if world <= 4 else 64, 4, 512, 256
    ep = EPComm(info, E, H, F, k, max_tokens=256, timeout_s=10.0)
    g = torch.Generator().manual_seed(0)   # identical on all ranks
    wg = (torch.randn(E, F, H, generator=g) * 0.05).bfloat16()
    wu = (torch.randn(E, F, H, generator=g) * 0.05).bfloat16()
    wd = (torch.randn(E, H, F, generator=g) * 0.05).bfloat16()
    e0, el = rank * (E // world), E // world
    w_il = torch.stack([ref.interleave_gate_up(wg[e], wu[e]) for e in range(e0, e0 + el)]).to(dev)
    wd_l = wd[e0:e0 + el].contiguous().to(dev)
    for it, counts in enumerate([[37, 50, 5, 64, 1, 2, 3, 4], [0, 200, 17, 0, 9, 9, 9, 9], [128] * 8]):
        T = counts[rank]
        gr = torch.Generator().manual_seed(100 + 10 * it + rank)
        x = torch.randn(T, H, generator=gr).bfloat16()
        logits = torch.stack([torch.randperm(E, generator=gr) for _ in range(T)]).float().mul(0.125).sub(E / 16).bfloat16() if T else torch.zeros(0, E).bfloat16()
        shared = torch.randn(T, H, generator=gr).bfloat16()
        got = ep.moe(x.to(dev), logits.to(dev), w_il, wd_l, shared.to(dev), norm_topk=False, route_scale=1.0)
        torch.cuda.synchronize()
        ops.check_status(dev)
        if T:
            w_ref, id_ref = ref.moe_route(logits, k)
            want = ref.moe_forward(x, torch.cat([wg, wu], dim=1), wd, w_ref, id_ref) + shared.float()
            err = (got.float().cpu() - want).abs().max().item()
            assert err <= 0.03 * want.abs().max().item() + 0.03, f"rank {rank} iter {it}: err {err}"
    # nothing, local or from a peer, may have written past the end of the symmetric region
    torch.cuda.synchronize()
    dist.barrier()
    assert ep.region.check_guard() == 0, f"rank {rank}: {ep.region.check_guard()} byte(s) of the guard band after the symmetric region were overwritten"
    dist.barrier()
    if rank == 0:
        print(f"EP_OK {world}", flush=True)
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
