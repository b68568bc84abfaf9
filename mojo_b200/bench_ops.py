"""Standalone sweep of the fused tensor-parallel ops against the separate matmul + NCCL pattern.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m mojo_b200.bench_ops [--sizes 64,256,1024,4096,16384] [--cols 8192] [--inner 28672] [--out result.json]

For every M:
  gemm_rs   Y = reduce_scatter(X[M, K/tp] W[N, K/tp]^T)       fused kernel  vs  torch.matmul + reduce_scatter_tensor
  gemm_ar   Y = all_reduce(...)                               fused kernel  vs  torch.matmul + all_reduce
  ag_gemm   Y = all_gather(X_r[M/tp, K_ag]) W[N_ag/tp, K_ag]^T  fused kernel  vs  all_gather_into_tensor + torch.matmul
            in two shapes: the model's column-parallel GEMM (K_ag = 8192, N_ag = 28672) and the same operands as the
            reduce-scatter rows (K_ag = 28672, N_ag = 8192)
Times are CUDA-event durations on the launching stream after warm-up, max over ranks. The roofline of an op is the
slower of its FLOPs at the GEMM peak and its bytes over NVLink at the per-direction link bandwidth. Both denominators
are inputs: `--peak-tflops` / `--hbm-gbs` name the machine's measured GEMM and copy rates, and the link bandwidth is
either given (`--nvlink-gbs`) or measured here first, with the library's own peer loads and stores (`p2p_probe`).

    ... -m mojo_b200.bench_ops --probe-only        prints the link probe table (uni- and bidirectional, push and pull,
                                                   ring and all-to-all, 1 MB ... 256 MB) and exits
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

from . import ops
from .parallel import init_distributed
from .parallel.fused import FusedTPComm

FALLBACK_TFLOPS = 1590.0     # used (and labelled "fallback") when --peak-tflops is not given
FALLBACK_HBM_GBS = 6650.0
NVLINK_GBS = 0.0             # set in main(): --nvlink-gbs or the probe's result


def timed(fn, iters: int, warm: int, info) -> float:
    """Median-free simple mean over `iters` back-to-back launches, microseconds, max over ranks."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ops.check_status(info.device)   # a wait that ran out in the warm-up ends the sweep here, not after every timed launch
    if info.world_size > 1:
        dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) * 1e3 / iters], device=info.device)
    if info.world_size > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def probe_nvlink(info, sizes=(1 << 20, 8 << 20, 64 << 20, 256 << 20), iters: int = 10) -> dict:
    """Measure peer bandwidth with the library's own peer stores (push) and loads (pull). GB/s are per direction per GPU:
    bytes a sending GPU moved / time, max-over-ranks time. Patterns: one sender to its neighbour (one direction of one
    GPU pair), every rank to its neighbour (each GPU sends and receives at once), every rank to every peer."""
    from .parallel.coll import SymmCollectives

    tp = info.world_size
    coll = SymmCollectives(info, max_bytes=max(sizes), timeout_s=10.0)
    table = []
    for nbytes in sizes:
        row = {"bytes": nbytes}
        for name, n_peers, senders in (("one_pair", 1, 1), ("ring", 1, None), ("all_to_all", tp - 1, None)):
            for pull in (False, True):
                key = f"{name}_{'pull' if pull else 'push'}"
                if n_peers < 1 or (name == "all_to_all" and tp == 2):
                    continue
                us = timed(lambda: coll.p2p_probe(nbytes, n_peers, senders, pull), iters, 2, info)
                row[key + "_gbs"] = round(nbytes * n_peers / (us * 1e-6) / 1e9, 1)
        table.append(row)
    best = max(v for k, v in table[-1].items() if k.endswith("_gbs"))
    return {"tp": tp, "rows": table, "per_direction_gbs": best}


def fp8_sweep(a, info, comm, ms, peak_bf16) -> None:  # noqa: C901
    """Block-scaled fp8 variant of the sweep. The unfused arm is this library's own fp8 GEMM followed by the NCCL
    collective (torch has no block-scaled fp8 matmul to stand in for the library GEMM). There is no measured fp8
    GEMM peak on file: the compute roof uses twice the measured bf16 peak, the ratio of the nominal figures."""
    from .ops import reference

    tp, rank, dev = info.world_size, info.rank, info.device
    k_local, n_ag_local = a.inner // tp, a.cols_ag // tp
    peak = 2.0 * peak_bf16
    rows = []
    for M in ms:
        Mp = (M + tp - 1) // tp * tp
        x = torch.randn(Mp, k_local, device=dev).bfloat16()
        xq, xs = ops.quant_e4m3(x)
        wq, ws = reference.quant_e4m3_128x128(torch.randn(a.cols, k_local, device=dev) * 0.02)
        y_full = torch.empty(Mp, a.cols, device=dev, dtype=torch.bfloat16)
        y_shard = torch.empty(Mp // tp, a.cols, device=dev, dtype=torch.bfloat16)

        def base_rs():
            ops.linear_fp8((xq, xs), wq, ws, out=y_full)
            if tp > 1:
                dist.reduce_scatter_tensor(y_shard, y_full)

        t_base_rs = timed(base_rs, a.iters, 3, info)
        t_rs = timed(lambda: comm.linear_fp8_reduce_scatter((xq, xs), wq, ws), a.iters, 3, info)
        t_gemm = timed(lambda: ops.linear_fp8((xq, xs), wq, ws, out=y_full), a.iters, 3, info)
        flops = 2.0 * Mp * a.cols * k_local
        rs_bytes = (tp - 1) / tp * Mp * a.cols * 2
        roof_rs = max(flops / (peak * 1e6), rs_bytes / (NVLINK_GBS * 1e3))
        # all-gather GEMM: quantised rows + scales are gathered
        xfull = torch.randn(Mp, a.inner_ag, device=dev).bfloat16()
        waq, was = reference.quant_e4m3_128x128(torch.randn(n_ag_local, a.inner_ag, device=dev) * 0.02)
        r = Mp // tp
        x_r = xfull[rank * r:(rank + 1) * r].contiguous()
        xq_r, xs_r = ops.quant_e4m3(x_r)
        xq_all = torch.empty(Mp, a.inner_ag, device=dev, dtype=torch.float8_e4m3fn)
        xs_all = torch.empty(Mp, a.inner_ag // 128, device=dev, dtype=torch.float32)
        y_ag = torch.empty(Mp, n_ag_local, device=dev, dtype=torch.bfloat16)

        def base_ag():
            if tp > 1:
                dist.all_gather_into_tensor(xq_all.view(torch.uint8), xq_r.view(torch.uint8))
                dist.all_gather_into_tensor(xs_all, xs_r)
            else:
                xq_all.copy_(xq_r)
                xs_all.copy_(xs_r)
            ops.linear_fp8((xq_all, xs_all), waq, was, out=y_ag)

        def fused_ag():
            qv, sv = comm.gather_input_fp8(Mp, a.inner_ag)
            qv.copy_(xq_r)
            sv.copy_(xs_r)
            comm.all_gather_linear_fp8(waq, was, Mp, out=y_ag)

        t_base_ag = timed(base_ag, a.iters, 3, info)
        t_ag = timed(fused_ag, a.iters, 3, info)
        flops_ag = 2.0 * Mp * n_ag_local * a.inner_ag
        ag_bytes = (tp - 1) / tp * Mp * (a.inner_ag + a.inner_ag // 32)
        roof_ag = max(flops_ag / (peak * 1e6), ag_bytes / (NVLINK_GBS * 1e3))
        torch.cuda.synchronize()
        ops.check_status(dev)
        row = {
            "M": M, "tp": tp, "N": a.cols, "K_local": k_local, "dtype": "fp8 block-scaled", "gemm_only_us": round(t_gemm, 1),
            "gemm_rs": {"fused_us": round(t_rs, 1), "gemm_nccl_us": round(t_base_rs, 1), "roofline_us": round(roof_rs, 1),
                        "pct_roofline": round(100 * roof_rs / t_rs, 1)},
            "ag_gemm": {"fused_us": round(t_ag, 1), "all_gather_gemm_us": round(t_base_ag, 1), "roofline_us": round(roof_ag, 1),
                        "pct_roofline": round(100 * roof_ag / t_ag, 1), "N_local": n_ag_local, "K": a.inner_ag},
        }
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
    if rank == 0 and a.out:
        json.dump({"peak_tflops_assumed_fp8": peak, "nvlink_gbs": NVLINK_GBS, "nvlink_source": a.nvlink_source, "rows": rows}, open(a.out, "w"), indent=1)
    if tp > 1:
        dist.barrier()
    sys.stdout.flush()
    os._exit(0)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", default="64,256,1024,4096,16384")
    ap.add_argument("--cols", type=int, default=8192)
    ap.add_argument("--inner", type=int, default=28672)
    ap.add_argument("--inner-ag", type=int, default=8192, help="K of the all-gather GEMM (activation width)")
    ap.add_argument("--cols-ag", type=int, default=28672, help="N of the all-gather GEMM before sharding")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp8"],
                    help="fp8: e4m3 operands with 1x128 activation and 128x128 weight scales (block-scaled), bf16 out")
    ap.add_argument("--out", default=None)
    ap.add_argument("--peak-tflops", type=float, default=None, help="measured bf16 GEMM rate of this machine (roofline denominator)")
    ap.add_argument("--hbm-gbs", type=float, default=None, help="measured HBM copy rate of this machine")
    ap.add_argument("--nvlink-gbs", type=float, default=None, help="per-direction NVLink bandwidth; default: measure it here with the peer load/store probe")
    ap.add_argument("--probe-only", action="store_true", help="print the link probe table and exit")
    ap.add_argument("--no-literal-ag", action="store_true", help="skip the all-gather GEMM rows with the reduce-scatter operands (K = --inner, N = --cols)")
    a = ap.parse_args()
    global NVLINK_GBS
    info = init_distributed("cuda")
    tp, rank, dev = info.world_size, info.rank, info.device
    ms = [int(x) for x in a.sizes.split(",")]
    k_local = a.inner // tp
    probe = None
    if a.nvlink_gbs is not None:
        NVLINK_GBS, a.nvlink_source = a.nvlink_gbs, "given"
    elif tp > 1:
        probe = probe_nvlink(info)
        NVLINK_GBS, a.nvlink_source = probe["per_direction_gbs"], "measured by the peer load/store probe of this run"
        if rank == 0:
            print(json.dumps({"nvlink_probe": probe}), flush=True)
    else:
        NVLINK_GBS, a.nvlink_source = 900.0, "nominal (one rank: no link is used)"
    if a.probe_only:
        if tp > 1:
            dist.barrier()
        sys.stdout.flush()
        os._exit(0)
    peak = a.peak_tflops if a.peak_tflops is not None else FALLBACK_TFLOPS
    peak_source = "given" if a.peak_tflops is not None else "fallback"
    hbm_gbs = a.hbm_gbs if a.hbm_gbs is not None else FALLBACK_HBM_GBS
    ag_shapes = [("ag_gemm", a.inner_ag, a.cols_ag)] + ([] if a.no_literal_ag else [("ag_gemm_rs_operands", a.inner, a.cols)])
    comm = FusedTPComm(info, max_tokens=max(ms), hidden=a.cols, max_k=max(k for _, k, _ in ag_shapes), timeout_s=3.0)
    rows = []
    if a.dtype == "fp8":
        fp8_sweep(a, info, comm, ms, peak)
        return
    for M in ms:
        Mp = (M + tp - 1) // tp * tp
        x = torch.randn(Mp, k_local, device=dev).bfloat16()
        w = (torch.randn(a.cols, k_local, device=dev) * 0.02).bfloat16()
        y_full = torch.empty(Mp, a.cols, device=dev, dtype=torch.bfloat16)
        y_shard = torch.empty(Mp // tp, a.cols, device=dev, dtype=torch.bfloat16)

        def base_rs():
            torch.matmul(x, w.t(), out=y_full)
            if tp > 1:
                dist.reduce_scatter_tensor(y_shard, y_full)

        def base_ar():
            torch.matmul(x, w.t(), out=y_full)
            if tp > 1:
                dist.all_reduce(y_full)

        t_base_rs = timed(base_rs, a.iters, 3, info)
        t_base_ar = timed(base_ar, a.iters, 3, info)
        t_rs = timed(lambda: comm.linear_reduce_scatter(x, w), a.iters, 3, info)
        t_ar = timed(lambda: comm.linear_all_reduce(x, w), a.iters, 3, info)
        t_gemm = timed(lambda: ops.linear(x, w, out=y_full), a.iters, 3, info)
        flops = 2.0 * Mp * a.cols * k_local
        t_compute = flops / (peak * 1e6)
        rs_bytes = (tp - 1) / tp * Mp * a.cols * 2
        roof_rs = max(t_compute, rs_bytes / (NVLINK_GBS * 1e3))
        roof_ar = max(t_compute, 2 * rs_bytes / (NVLINK_GBS * 1e3))
        hbm = hbm_gbs * 1e3
        roof_rs_hbm = max(roof_rs, (a.cols * k_local + Mp * k_local + Mp * a.cols) * 2 / hbm)
        row = {
            "M": M, "tp": tp, "N": a.cols, "K_local": k_local,
            "gemm_only_us": round(t_gemm, 1),
            "pct_roofline_with_hbm": {"gemm_rs": round(100 * roof_rs_hbm / t_rs, 1)},
            "gemm_rs": {"fused_us": round(t_rs, 1), "matmul_nccl_us": round(t_base_rs, 1), "roofline_us": round(roof_rs, 1),
                        "pct_roofline": round(100 * roof_rs / t_rs, 1)},
            "gemm_ar": {"fused_us": round(t_ar, 1), "matmul_nccl_us": round(t_base_ar, 1), "roofline_us": round(roof_ar, 1),
                        "pct_roofline": round(100 * roof_ar / t_ar, 1)},
        }
        # all-gather GEMM: X_r [M/tp, k_ag] gathered, W shard [n_ag/tp, k_ag]
        for label, k_ag, n_ag in ag_shapes:
            n_loc = n_ag // tp
            xs = torch.randn(Mp, k_ag, device=dev).bfloat16()
            wa = (torch.randn(n_loc, k_ag, device=dev) * 0.02).bfloat16()
            r = Mp // tp
            x_r = xs[rank * r:(rank + 1) * r].contiguous()
            x_all = torch.empty(Mp, k_ag, device=dev, dtype=torch.bfloat16)
            y_ag = torch.empty(Mp, n_loc, device=dev, dtype=torch.bfloat16)

            def base_ag():
                if tp > 1:
                    dist.all_gather_into_tensor(x_all, x_r)
                else:
                    x_all.copy_(x_r)
                torch.matmul(x_all, wa.t(), out=y_ag)

            def fused_ag():
                comm.gather_input(Mp, k_ag).copy_(x_r)
                comm.all_gather_linear(wa, Mp, out=y_ag)

            t_base_ag = timed(base_ag, a.iters, 3, info)
            t_ag = timed(fused_ag, a.iters, 3, info)
            flops_ag = 2.0 * Mp * n_loc * k_ag
            ag_bytes = (tp - 1) / tp * Mp * k_ag * 2
            roof_ag = max(flops_ag / (peak * 1e6), ag_bytes / (NVLINK_GBS * 1e3))
            roof_ag_hbm = max(roof_ag, (n_loc * k_ag + Mp * k_ag + Mp * n_loc) * 2 / hbm)
            row[label] = {"fused_us": round(t_ag, 1), "all_gather_matmul_us": round(t_base_ag, 1), "roofline_us": round(roof_ag, 1),
                          "pct_roofline": round(100 * roof_ag / t_ag, 1), "N_local": n_loc, "K": k_ag}
            row["pct_roofline_with_hbm"][label] = round(100 * roof_ag_hbm / t_ag, 1)
            del xs, wa, x_all, y_ag
        torch.cuda.synchronize()
        ops.check_status(dev)
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
    if rank == 0 and a.out:
        json.dump({"peak_tflops": peak, "peak_source": peak_source, "hbm_gbs": hbm_gbs, "nvlink_gbs": NVLINK_GBS, "nvlink_source": a.nvlink_source,
                   "nvlink_probe": probe, "rows": rows}, open(a.out, "w"), indent=1)
    if tp > 1:
        dist.barrier()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
