"""Run one hot kernel a handful of times on representative shapes: `python -m mojo_b200.utils.kernel_driver <case>`.

Small, self-terminating workloads (inputs larger than the 126 MB L2, a few GB at most) meant to be wrapped by a
profiler capture of one kernel; with `--time` the case is timed with CUDA events instead and one JSON line is printed.
Cases: gemm_large, gemm_pair (the same product on CTA pairs), gemm_prefill, gemm_decode, gemm_swiglu, gemm_fp8,
gemm_fp8_decode, gemm_fp8_decode_nosplit (a narrow tensor-parallel shard at 256 tokens, with and without split-K),
attn_decode, attn_prefill, mla_decode, mla_prefill, rmsnorm, sampling (arg-max), sample_topk_topp, gemm_gguf_q4k,
gemm_gguf_q6k, rope_kvwrite, all_reduce_norm_single.
"""
from __future__ import annotations

import argparse
import json
import math

import torch

from .. import ops
from ..ops import reference as ref

DEV = "cuda"


def _case(name: str):
    g = torch.Generator(device=DEV).manual_seed(0)

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, generator=g, device=DEV) * scale).bfloat16()

    if name in ("gemm_large", "gemm_pair", "gemm_prefill", "gemm_decode", "gemm_swiglu"):
        M, N, K = {"gemm_large": (8192, 8192, 8192), "gemm_pair": (8192, 8192, 8192), "gemm_prefill": (4096, 6144, 4096), "gemm_decode": (64, 28672, 4096),
                   "gemm_swiglu": (2048, 28672, 4096)}[name]
        x, w = rnd(M, K), rnd(N, K, scale=0.02)
        if name == "gemm_swiglu":
            y = torch.empty(M, N // 2, device=DEV, dtype=torch.bfloat16)
            return (lambda: ops.linear_swiglu(x, w, out=y)), 2.0 * M * N * K, (M * K + N * K + M * N // 2) * 2
        y = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
        cfg = ops.PAIR_CONFIG if name == "gemm_pair" else 0
        return (lambda: ops.linear(x, w, out=y, config=cfg)), 2.0 * M * N * K, (M * K + N * K + M * N) * 2
    if name == "gemm_fp8":
        M, N, K = 4096, 8192, 8192
        xq, xs = ops.quant_e4m3(rnd(M, K))
        wq, ws = ref.quant_e4m3_128x128(rnd(N, K, scale=0.02).float().cpu())
        wq, ws = wq.to(DEV), ws.to(DEV)
        y = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
        return (lambda: ops.linear_fp8((xq, xs), wq, ws, out=y)), 2.0 * M * N * K, M * K + N * K + M * N * 2
    if name in ("gemm_fp8_decode", "gemm_fp8_decode_nosplit"):
        # one rank's QKV projection of a 70B model at TP = 8 with 256 decode tokens: 20 output tiles for 148 SMs unless K
        # is split. Sixteen weight copies (168 MB) rotate so that every launch streams its weights from HBM.
        M, N, K = 256, 1280, 8192
        xq, xs = ops.quant_e4m3(rnd(M, K))
        copies = []
        for _ in range(16):
            wq, ws = ref.quant_e4m3_128x128(rnd(N, K, scale=0.02).float().cpu())
            copies.append((wq.to(DEV), ws.to(DEV)))
        y = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
        cfg = ops.gemm_config(False, 128, 1) if name.endswith("nosplit") else 0
        turn = [0]

        def run():
            wq, ws = copies[turn[0] % len(copies)]
            turn[0] += 1
            ops.linear_fp8((xq, xs), wq, ws, out=y, config=cfg)

        return run, 2.0 * M * N * K, M * K + N * K + M * N * 2
    if name in ("attn_decode", "attn_prefill"):
        n_q, n_kv, D, page = 32, 8, 128, 128
        if name == "attn_decode":
            q_lens, ctx = [1] * 256, [1400] * 256
        else:
            q_lens, ctx = [2048, 1024, 1024], [2048, 1024, 1024]
        B, T = len(q_lens), sum(q_lens)
        pages_per = [(c + page - 1) // page for c in ctx]
        bt = torch.zeros(B, max(pages_per), dtype=torch.int32)
        o = 0
        for b, n in enumerate(pages_per):
            bt[b, :n] = torch.arange(o, o + n, dtype=torch.int32)
            o += n
        kc, vc = rnd(o + 1, n_kv, page, D), rnd(o + 1, n_kv, page, D)
        q = rnd(T, n_q * D)
        cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
        cl = torch.tensor(ctx, dtype=torch.int32, device=DEV)
        nd = B if name == "attn_decode" else 0
        meta = ops.AttnMeta(cu, cl, bt.to(DEV), nd, max(q_lens), max(ctx))
        kv_bytes = sum(ctx) * n_kv * D * 2 * 2
        flops = sum(4.0 * ql * c * D * n_q * (0.5 if ql > 1 else 1.0) for ql, c in zip(q_lens, ctx))
        return (lambda: ops.paged_attention(q, kc, vc, meta, 1 / math.sqrt(D), D)), flops, kv_bytes + 2 * T * n_q * D * 2
    if name == "mla_decode":
        B, H, ctx, page = 64, 16, 768, 128
        pages = (ctx + page - 1) // page
        bt = torch.arange(B * pages, dtype=torch.int32).view(B, pages).to(DEV)
        cache = rnd(B * pages + 1, page, 576, scale=0.5)
        ql, qr = rnd(B, H, 512, scale=0.3), rnd(B, H, 64, scale=0.3)
        cl = torch.full((B,), ctx, dtype=torch.int32, device=DEV)
        return (lambda: ops.mla_decode(ql, qr, cache, cl, bt, 1 / math.sqrt(192), ctx)), 2.0 * B * H * ctx * (576 + 512), B * ctx * 576 * 2
    if name == "mla_prefill":
        # one engine step of DeepSeek-V2-Lite prefill: eight 512-token prompts, every token a row group of the latent
        # attention kernel; the query parts are column slices of the fused projection output, as in the model
        S, L, H, page = 8, 512, 16, 128
        pages = L // page
        bt = torch.arange(S * pages, dtype=torch.int32).view(S, pages).to(DEV)
        cache = rnd(S * pages + 1, page, 576, scale=0.5)
        qa = rnd(S * L, H * 576 + 576, scale=0.3)
        ql, qr = qa[:, :H * 512].unflatten(1, (H, 512)), qa[:, H * 512:H * 576].unflatten(1, (H, 64))
        cu = torch.arange(0, (S + 1) * L, L, dtype=torch.int32, device=DEV)
        meta = ops.AttnMeta(cu, torch.full((S,), L, dtype=torch.int32, device=DEV), bt, 0, L, L)
        flops = 2.0 * S * H * (576 + 512) * L * (L + 1) / 2
        return (lambda: ops.mla_attend(ql, qr, cache, meta, 1 / math.sqrt(192))), flops, S * L * 576 * 2 + 2 * S * L * H * 576 * 2
    if name in ("tp_gemm_rs_single", "tp_ag_gemm_single"):
        # The fused tensor-parallel kernels on ONE rank (a world of one: the only peer is this GPU's own region), so that
        # their tensor-core / epilogue / staging behaviour can be captured under a profiler, which never runs on a
        # multi-rank job. Shapes: one rank's share of the 8-GPU op sweep (K or N = 28672 / 8) at 4096 tokens.
        from ..parallel.dist import DistInfo
        from ..parallel.fused import FusedTPComm

        info = DistInfo(0, 1, 0, torch.device(DEV), None, None)
        M, big, shard = 4096, 8192, 3584
        comm = FusedTPComm(info, max_tokens=M, hidden=big, max_k=big, timeout_s=2.0)
        C, turn = comm.C, [0]
        if name == "tp_gemm_rs_single":
            x, w = rnd(M, shard), rnd(big, shard, scale=0.02)
            out = torch.empty(M, big, device=DEV, dtype=torch.bfloat16)

            def run():
                C.tp_gemm_rs(x, w, 0, comm.peers, comm.layout, out, None, 0, turn[0] & 1, comm.timeout_ns, 0, comm.status)
                turn[0] += 1

            want = ops.linear(x, w)
            flops, nbytes = 2.0 * M * big * shard, (M * shard + big * shard + 2 * M * big) * 2
        else:
            w = rnd(shard, big, scale=0.02)
            out = torch.empty(M, shard, device=DEV, dtype=torch.bfloat16)
            x = rnd(M, big)

            def run():
                slot = turn[0] & 1
                full = comm.region.view(comm.layout.off_xall + slot * comm.layout.xall_half_bytes, (M, big), torch.bfloat16)
                full.copy_(x)
                C.tp_ag_gemm(w, 0, comm.peers, comm.layout, out, M, slot, comm.timeout_ns, 0, 0, comm.status)
                turn[0] += 1

            want = ops.linear(x, w)
            flops, nbytes = 2.0 * M * big * shard, (M * big + big * shard + M * shard) * 2
        run()
        torch.cuda.synchronize()
        ops.check_status()
        err = (out.float() - want.float()).abs().max().item()
        if not err <= 0.05 * want.float().abs().max().item() + 0.05:
            raise SystemExit(f"{name}: single-rank result differs from the plain GEMM by {err}")
        return run, flops, nbytes
    if name == "moe_ep_single":
        # One DeepSeek-V2-Lite MoE layer on a world of one (all 64 experts local): router + dispatch, the two grouped
        # tcgen05 GEMMs, combine. The expert-parallel kernels as they run on every rank, without link traffic.
        from ..parallel.dist import DistInfo
        from ..parallel.ep import EPComm

        T, E, k, H, F = 4096, 64, 6, 2048, 1408
        ep = EPComm(DistInfo(0, 1, 0, torch.device(DEV), None, None), E, H, F, k, max_tokens=T, timeout_s=2.0)
        x = rnd(T, H)
        logits = rnd(T, E, scale=1.0)
        w_gu = rnd(E, 2 * F, H, scale=0.02)
        w_down = rnd(E, H, F, scale=0.02)
        flops = 2.0 * T * k * (2 * F * H + H * F)
        nbytes = (w_gu.numel() + w_down.numel()) * 2 + 4 * T * k * H * 2
        return (lambda: ep.moe(x, logits, w_gu, w_down)), flops, nbytes
    if name == "rmsnorm":
        rows, h = 65536, 4096
        x, r, w = rnd(rows, h), rnd(rows, h), torch.ones(h, device=DEV, dtype=torch.bfloat16)
        return (lambda: ops.rms_norm(x, w, 1e-5, r)), 0.0, rows * h * 2 * 4
    if name == "sampling":
        lg = rnd(256, 128256)
        return (lambda: ops.argmax(lg)), 0.0, lg.numel() * 2
    if name == "sample_topk_topp":
        # temperature / top-k / top-p sampling of 256 rows over the Llama-3 vocabulary (radix select + Philox)
        lg = rnd(256, 128256, scale=3.0)
        temp = torch.full((256,), 0.8, device=DEV)
        top_k = torch.full((256,), 50, dtype=torch.int32, device=DEV)
        top_p = torch.full((256,), 0.9, device=DEV)
        step = [0]

        def run():
            step[0] += 1
            return ops.sample(lg, temp, top_k, top_p, 1234, step[0])

        return run, 0.0, lg.numel() * 2
    if name in ("gemm_gguf_q4k", "gemm_gguf_q6k"):
        # decode-sized product against GGUF super-blocks (dequantisation fused into the tcgen05 GEMM): 16 tokens against a
        # Llama-3.1-8B gate/up-sized matrix; the packed weights (Q4_K 4.5 bits, Q6_K 6.56 bits per weight) rotate through
        # more copies than fit the L2
        ggml = ops.GGML_Q4_K if name.endswith("q4k") else ops.GGML_Q6_K
        M, N, K = 16, 28672, 4096
        per = 144 if ggml == ops.GGML_Q4_K else 210
        copies = [ref.random_gguf_blocks(N * K // 256, ggml, seed=i).to(DEV) for i in range(3)]
        x = rnd(M, K)
        turn = [0]

        def run():
            turn[0] += 1
            return ops.linear_gguf(x, copies[turn[0] % len(copies)], ggml, N)

        return run, 2.0 * M * N * K, N * K // 256 * per + (M * K + M * N) * 2
    if name == "all_reduce_norm_single":
        # all-reduce + residual add + RMSNorm on a world of one (the only "peer" is this GPU's own region): the one-shot
        # kernel's memory behaviour without link traffic. The in-switch form needs a multicast mapping, which a single
        # rank does not have; its multi-GPU timings are in the tuning tables of the serving benchmark.
        from ..parallel.coll import SymmCollectives
        from ..parallel.dist import DistInfo

        rows, h = 32768, 4096
        coll = SymmCollectives(DistInfo(0, 1, 0, torch.device(DEV), None, None), max_bytes=rows * h * 2, timeout_s=2.0)
        part, res, w = rnd(rows, h), rnd(rows, h), torch.ones(h, device=DEV, dtype=torch.bfloat16)

        def run():
            coll.staging_view((rows, h)).copy_(part)
            return coll.all_reduce_rmsnorm_staged((rows, h), w, 1e-5, res, form="one_shot")

        return run, 0.0, rows * h * 2 * 4
    if name == "rope_kvwrite":
        T, n_q, n_kv, D, page = 16384, 32, 8, 128, 128
        qkv = rnd(T, (n_q + 2 * n_kv) * D)
        pages = T // page
        kc, vc = torch.zeros(pages, n_kv, page, D, device=DEV, dtype=torch.bfloat16), torch.zeros(pages, n_kv, page, D, device=DEV, dtype=torch.bfloat16)
        cos_sin = ref.rope_table(T, D, 500000.0, None).to(DEV)
        pos = torch.arange(T, dtype=torch.int32, device=DEV)
        slots = torch.arange(T, dtype=torch.int64, device=DEV)
        q, k, v = qkv[:, :n_q * D], qkv[:, n_q * D:(n_q + n_kv) * D], qkv[:, (n_q + n_kv) * D:]
        return (lambda: ops.rope_kvwrite(q, k, v, cos_sin, pos, slots, kc, vc, D)), 0.0, (2 * T * (n_q + n_kv) * D + 3 * T * n_kv * D) * 2
    raise SystemExit(f"unknown case {name!r}")


CASES = ("gemm_large", "gemm_pair", "gemm_prefill", "gemm_decode", "gemm_swiglu", "gemm_fp8", "gemm_fp8_decode", "gemm_fp8_decode_nosplit",
         "attn_decode", "attn_prefill", "mla_decode", "mla_prefill", "rmsnorm", "sampling", "sample_topk_topp", "gemm_gguf_q4k", "gemm_gguf_q6k",
         "rope_kvwrite", "all_reduce_norm_single")
# single-rank forms of the fused tensor-parallel and expert-parallel kernels (profiling only): tp_gemm_rs_single,
# tp_ag_gemm_single, moe_ep_single


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("case")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--time", action="store_true")
    a = ap.parse_args()
    fn, flops, nbytes = _case(a.case)
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    if a.time:
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(a.iters):
            fn()
        e.record()
        torch.cuda.synchronize()
        us = s.elapsed_time(e) * 1e3 / a.iters
        print(json.dumps({"case": a.case, "us": round(us, 2), "tflops": round(flops / us / 1e6, 1), "gbs": round(nbytes / us / 1e3, 1)}))
    else:
        for _ in range(a.iters):
            fn()
        torch.cuda.synchronize()
    ops.check_status()


if __name__ == "__main__":
    main()
