"""Multi-GPU worker (launched by torch.distributed.run): fused tensor-parallel kernels against NCCL + fp32 matmul.
Prints one line `TP_FUSED_OK <world>` on rank 0 when every check passed."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mojo_b200 import ops  # noqa: E402
from mojo_b200.parallel import init_distributed  # noqa: E402
from mojo_b200.parallel.fused import FusedTPComm  # noqa: E402


def main():
    info = init_distributed("cuda")
    rank, tp, dev = info.rank, info.world_size, info.device
    hidden = 2048
    # B2_TEST_NVLS=1: the reductions run in the NVLink switch (multimem). The default, plain peer loads and stores, is the
    # form the timeout section below runs on: waits that are made to run out belong to the path without multicast.
    nvls = os.environ.get("B2_TEST_NVLS", "0") == "1"
    comm = FusedTPComm(info, max_tokens=2048, hidden=hidden, timeout_s=5.0, nvls=nvls)
    comm.barrier()
    torch.cuda.synchronize()
    ops.check_status(dev)

    def mk(shape, seed, scale=1.0):
        g = torch.Generator(device="cpu").manual_seed(seed)
        return (torch.randn(*shape, generator=g) * scale).bfloat16().to(dev)

    def close(a, b, what):
        err = (a.float() - b.float()).abs().max().item()
        ref = b.float().abs().max().item()
        assert err <= 0.02 * ref + 0.05, f"{what}: max err {err} (ref max {ref}) on rank {rank}"

    def progress(what):
        # one line per finished section on stderr: tells which section a failure belongs to
        torch.cuda.synchronize()
        print(f"[rank {rank}] ok: {what}", file=sys.stderr, flush=True)

    k_local = 512
    # ---- GEMM -> all-reduce and -> reduce-scatter (row-parallel: every rank has its own K shard) ----
    for i, M in enumerate([8, 64, 136, 512, 1024, 16, 2048]):
        N = hidden if M != 136 else 1024
        x = mk((M, k_local), 100 + 10 * i + rank)
        w = mk((N, k_local), 200 + 10 * i + rank, 0.05)
        res = mk((M, N), 300 + i)
        want = x.float() @ w.float().t()
        dist.all_reduce(want)
        y = comm.linear_all_reduce(x, w)
        close(y, want, f"all-reduce M={M}")
        y2 = comm.linear_all_reduce(x, w, residual=res)
        close(y2, want + res.float(), f"all-reduce+residual M={M}")
        if M % tp == 0:
            r = M // tp
            y3 = comm.linear_reduce_scatter(x, w, residual=res[rank * r:(rank + 1) * r].contiguous())
            close(y3, (want + res.float())[rank * r:(rank + 1) * r], f"reduce-scatter M={M}")
        progress(f"row-parallel M={M}")
    torch.cuda.synchronize()
    ops.check_status(dev)
    progress("row-parallel GEMM + all-reduce / reduce-scatter")

    # ---- back-to-back launches without host syncs (epochs + double buffering) ----
    x = mk((256, k_local), 1000 + rank)
    w = mk((hidden, k_local), 2000 + rank, 0.05)
    want = x.float() @ w.float().t()
    dist.all_reduce(want)
    outs = []
    for _ in range(12):
        outs.append(comm.linear_all_reduce(x, w).clone())
    torch.cuda.synchronize()
    for o in outs:
        close(o, want, "back-to-back all-reduce")
    ops.check_status(dev)
    progress("back-to-back launches")

    # ---- all-gather -> GEMM (column-parallel: every rank has its own rows of X and its own N shard) ----
    for i, M in enumerate([tp * 4, tp * 32, 512, 2048]):
        K, n_local = hidden, 768
        r = M // tp
        x_full = mk((M, K), 3000 + i)            # same on all ranks
        w = mk((n_local, K), 4000 + 10 * i + rank, 0.05)
        want = x_full.float() @ w.float().t()
        for rep in range(3):
            comm.gather_input(M, K).copy_(x_full[rank * r:(rank + 1) * r])
            y = comm.all_gather_linear(w, M)
            close(y, want, f"all-gather GEMM M={M} rep={rep}")
        comm.gather_input(M, K).copy_(x_full[rank * r:(rank + 1) * r])
        full = comm.all_gather_rows(M, K)
        torch.cuda.synchronize()
        assert torch.equal(full, x_full), f"standalone all-gather M={M}"
        progress(f"all-gather M={M}")
    torch.cuda.synchronize()
    ops.check_status(dev)
    progress("all-gather GEMM")

    # ---- the same launches replayed from a CUDA graph ----
    x = mk((64, k_local), 5000 + rank)
    w = mk((hidden, k_local), 6000 + rank, 0.05)
    want = x.float() @ w.float().t()
    dist.all_reduce(want)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        comm.linear_all_reduce(x, w)
        comm.linear_all_reduce(x, w)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        comm.begin_graph()
        a = comm.linear_all_reduce(x, w)
        b = comm.linear_all_reduce(a[:, :k_local].contiguous(), w)
    for _ in range(5):
        g.replay()
    torch.cuda.synchronize()
    close(a, want, "graph replay all-reduce")
    want_b = a[:, :k_local].float() @ w.float().t()
    dist.all_reduce(want_b)
    close(b, want_b, "graph replay chained all-reduce")
    ops.check_status(dev)
    progress("graph replay")

    # ---- the two-launch form: GEMM writing into the all-reduce kernel's input buffer, one-shot and two-shot ----
    comm.ar_mode = "split"
    for i, M in enumerate([8, 64, 512, 2048]):
        x = mk((M, k_local), 6500 + 10 * i + rank)
        w = mk((hidden, k_local), 6600 + 10 * i + rank, 0.05)
        want = x.float() @ w.float().t()
        dist.all_reduce(want)
        for rep in range(3):
            close(comm.linear_all_reduce(x, w), want, f"split all-reduce M={M} rep={rep}")
    comm.ar_mode = "auto"
    rep = comm.tune_all_reduce(hidden, k_local, [16, 256, 1024])
    assert set(rep) == {16, 256, 1024} and all(a > 0 and b > 0 for a, b in rep.values())
    close(comm.linear_all_reduce(x, w), want, "all-reduce after tuning")
    torch.cuda.synchronize()
    ops.check_status(dev)
    progress("split all-reduce")

    # ---- block-scaled fp8 GEMM -> all-reduce / reduce-scatter ----
    from mojo_b200.ops import reference

    for i, M in enumerate([8, 48, 256, 1024]):
        N = hidden
        x8 = mk((M, k_local), 7000 + 10 * i + rank)
        w8 = mk((N, k_local), 7500 + 10 * i + rank, 0.05)
        res = mk((M, N), 7900 + i)
        xq, xs = ops.quant_e4m3(x8)
        wq, ws = reference.quant_e4m3_128x128(w8)
        want8 = reference.linear_fp8_block(xq, xs, wq, ws).float()
        dist.all_reduce(want8)
        for rep in range(2):
            y = comm.linear_fp8_all_reduce((xq, xs), wq, ws, residual=res if rep else None)
            close(y, want8 + res.float() if rep else want8, f"fp8 all-reduce M={M} rep={rep}")
        if M % tp == 0:
            r = M // tp
            y3 = comm.linear_fp8_reduce_scatter(x8, wq, ws)
            close(y3, want8[rank * r:(rank + 1) * r], f"fp8 reduce-scatter M={M}")
    torch.cuda.synchronize()
    ops.check_status(dev)
    progress("fp8 GEMM + all-reduce / reduce-scatter")

    # ---- fp8 all-gather -> GEMM: every rank quantises its own rows straight into the gathered buffer ----
    for i, M in enumerate([tp * 4, tp * 24, 512, 2048]):
        K, n_local = 2048, 768
        r = M // tp
        x_full = mk((M, K), 8000 + i)
        w8 = mk((n_local, K), 8100 + 10 * i + rank, 0.05)
        wq, ws = reference.quant_e4m3_128x128(w8)
        xq_full, xs_full = ops.quant_e4m3(x_full)
        want8 = reference.linear_fp8_block(xq_full, xs_full, wq, ws).float()
        for rep in range(3):
            q_view, s_view = comm.gather_input_fp8(M, K)
            ops.quant_e4m3(x_full[rank * r:(rank + 1) * r].contiguous(), out_q=q_view, out_s=s_view)
            y = comm.all_gather_linear_fp8(wq, ws, M)
            close(y, want8, f"fp8 all-gather GEMM M={M} rep={rep}")
    torch.cuda.synchronize()
    ops.check_status(dev)
    progress("fp8 all-gather GEMM")

    # ---- timeout path: a wait nobody satisfies returns a TIMEOUT status and leaves the context usable ----
    if not nvls:
        flag = torch.zeros(1, dtype=torch.int32, device=dev)
        comm.C.wait_flag(flag, 1, 50_000_000, comm.status)
        torch.cuda.synchronize()
        try:
            ops.check_status(dev)
            raise AssertionError("expected a TIMEOUT status")
        except ops.KernelError as e:
            assert e.code == 1 and e.site == 15, e
        y = comm.linear_all_reduce(x, w)
        torch.cuda.synchronize()
        close(y, want, "all-reduce after a timeout")
        ops.check_status(dev)
        progress("timeout path")
    # nothing, local or from a peer, may have written past the end of the symmetric region
    torch.cuda.synchronize()
    dist.barrier()
    assert comm.region.check_guard() == 0, f"rank {rank}: {comm.region.check_guard()} byte(s) of the guard band after the symmetric region were overwritten"
    if comm._coll is not None:
        assert comm._coll.region.check_guard() == 0, f"rank {rank}: collective staging region overran"
    dist.barrier()
    if rank == 0:
        print(f"TP_FUSED_OK {tp} nvls={int(bool(comm.mc_ptr))}", flush=True)
    from mojo_b200.parallel.dist import shutdown

    shutdown()


if __name__ == "__main__":
    main()
