"""Multi-GPU worker: standalone symmetric-memory collectives against torch.distributed (NCCL) results.
Prints `COLL_OK <world>` on rank 0 when every check passed."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mojo_b200 import ops  # noqa: E402
from mojo_b200.parallel import init_distributed  # noqa: E402
from mojo_b200.parallel.coll import SymmCollectives  # noqa: E402


def main():
    info = init_distributed("cuda")
    rank, tp, dev = info.rank, info.world_size, info.device
    coll = SymmCollectives(info, max_bytes=4 << 20, timeout_s=5.0, nvls=os.environ.get("B2_TEST_NVLS", "0") == "1")

    def mk(shape, seed):
        g = torch.Generator(device="cpu").manual_seed(seed)
        return torch.randn(*shape, generator=g).bfloat16().to(dev)

    def close(a, b, what):
        err = (a.float() - b.float()).abs().max().item()
        ref = b.float().abs().max().item()
        assert err <= 0.02 * ref + 0.03, f"{what}: max err {err} (ref max {ref}) on rank {rank}"

    algos = ["one_shot", "two_shot"] + (["nvls"] if coll.mc_ptr else [])
    for i, n in enumerate([8, 1000, 4096 * 7 + 3, 1 << 20]):
        x = mk((n,), 10 * i + rank)
        want = x.float().clone()
        dist.all_reduce(want)
        for algo in algos:
            for rep in range(3):  # repeated launches exercise both buffer halves and the epochs
                y = coll.all_reduce(x, algo=algo)
                close(y, want, f"all_reduce n={n} {algo} rep={rep}")
        ys = [coll.all_reduce(x, algo="one_shot") for _ in range(2)]
        assert torch.equal(ys[0], ys[1]), "one-shot all-reduce must be deterministic"
    torch.cuda.synchronize()
    ops.check_status(dev)

    for i, rows in enumerate([tp, tp * 16, tp * 256]):
        x = mk((rows, 512), 500 + 10 * i + rank)
        want = x.float().clone()
        dist.all_reduce(want)
        r = rows // tp
        close(coll.reduce_scatter(x), want[rank * r:(rank + 1) * r], f"reduce_scatter rows={rows}")
        g = coll.all_gather(x[:r].contiguous())
        parts = [torch.empty_like(x[:r]) for _ in range(tp)]
        dist.all_gather(parts, x[:r].contiguous())
        assert torch.equal(g, torch.stack(parts)), f"all_gather rows={r}"
    torch.cuda.synchronize()
    ops.check_status(dev)

    # all-reduce + residual add + RMSNorm in one kernel, against the separate ops
    from mojo_b200.ops import reference

    for i, (rows, hidden) in enumerate([(1, 512), (37, 4096), (256, 8192), (130, 1024)]):
        part = mk((rows, hidden), 700 + 10 * i + rank)
        res0 = mk((rows, hidden), 760 + i)
        wn = mk((hidden,), 780 + i) * 0.1 + 1.0
        want_sum = part.float().clone()
        dist.all_reduce(want_sum)
        h = want_sum.bfloat16()
        want_x, want_res = reference.rms_norm(h.cpu(), wn.cpu(), 1e-5, res0.clone().cpu())
        for rep in range(2):
            res = res0.clone()
            coll.staging_view((rows, hidden)).copy_(part)
            x, res_out = coll.all_reduce_rmsnorm_staged((rows, hidden), wn, 1e-5, res)
            torch.cuda.synchronize()
            close(res_out, want_res.to(dev), f"fused all-reduce+norm residual {rows}x{hidden}")
            close(x, want_x.to(dev), f"fused all-reduce+norm output {rows}x{hidden}")
            # every rank must hold the same bits (greedy decoding takes the arg-max of what follows on every rank)
            mine = torch.cat([x.reshape(-1), res_out.reshape(-1)]).view(torch.int16).to(torch.int32)
            lo, hi = mine.clone(), mine.clone()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX)
            assert torch.equal(lo, hi), f"fused all-reduce+norm {rows}x{hidden}: ranks hold different bits"
    ops.check_status(dev)

    # all-to-all with per-peer row counts (zero rows to some peers)
    max_rows, row = 64, 256
    for it in range(3):
        blocks = mk((tp, max_rows, row), 900 + 10 * it + rank)
        send = [(rank * 7 + j * 3 + it) % (max_rows + 1) if (rank + j + it) % 3 else 0 for j in range(tp)]
        recv, counts = coll.all_to_all(blocks, send)
        torch.cuda.synchronize()
        all_send = [None] * tp
        dist.all_gather_object(all_send, send)
        for s in range(tp):
            n = all_send[s][rank]
            assert int(counts[s]) == n, f"all_to_all count from {s}: {int(counts[s])} != {n}"
            g = torch.Generator(device="cpu").manual_seed(900 + 10 * it + s)
            src = torch.randn(tp, max_rows, row, generator=g).bfloat16()
            assert torch.equal(recv[s, :n].cpu(), src[rank, :n]), f"all_to_all rows from {s}"
    ops.check_status(dev)

    # vocabulary-parallel greedy sampling, with ties across ranks (smallest global index wins)
    S, v_local = 37, 1000
    full = torch.randn(S, v_local * tp, generator=torch.Generator().manual_seed(7)).bfloat16()
    full[3, 17] = 9.0
    full[3, v_local * (tp - 1) + 5] = 9.0
    full[4, v_local * (tp - 1) + 999] = 11.0
    shard = full[:, rank * v_local:(rank + 1) * v_local].contiguous().to(dev)
    for rep in range(3):
        tok = coll.vocab_argmax(shard)
        torch.cuda.synchronize()
        want = torch.argmax(full.float(), dim=-1)
        vals = full.float().gather(1, tok.cpu().view(-1, 1)).view(-1)
        assert torch.equal(vals, full.float().max(dim=-1).values), "vocab_argmax picked a non-maximal logit"
        assert tok[3].item() == 17 and tok[4].item() == v_local * (tp - 1) + 999, tok[:6]
        assert (tok.cpu() == want).float().mean() > 0.9
    ops.check_status(dev)

    # the same collectives replayed from a CUDA graph
    x = mk((4096,), 2000 + rank)
    want = x.float().clone()
    dist.all_reduce(want)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        coll.all_reduce(x)
        coll.all_reduce(x)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    dist.barrier()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        a = coll.all_reduce(x, algo="one_shot")
        b = coll.all_reduce(a, algo="two_shot").clone()
    for _ in range(4):
        g.replay()
    torch.cuda.synchronize()
    close(a, want, "graph all_reduce")
    want_b = a.float().clone()
    dist.all_reduce(want_b)
    close(b, want_b, "graph chained all_reduce")
    ops.check_status(dev)

    # nothing, local or from a peer, may have written past the end of the symmetric region
    torch.cuda.synchronize()
    dist.barrier()
    assert coll.region.check_guard() == 0, f"rank {rank}: {coll.region.check_guard()} byte(s) of the guard band after the symmetric region were overwritten"
    dist.barrier()
    if rank == 0:
        print(f"COLL_OK {tp} nvls={int(bool(coll.mc_ptr))} heap={coll.region.backend}", flush=True)
    from mojo_b200.parallel.dist import shutdown

    shutdown()


if __name__ == "__main__":
    main()
