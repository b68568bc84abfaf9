"""CUDA kernels against the plain PyTorch fp32 reference of the same op (small-case sweeps incl. odd sizes,
single rows, page boundaries)."""
import math

import pytest
import torch

from mojo_b200 import ops
from mojo_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(a, b, atol, rtol):
    torch.testing.assert_close(a.float().cpu(), b.float().cpu(), atol=atol, rtol=rtol)


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    ops.check_status()


@pytest.mark.parametrize("rows,hidden", [(1, 256), (7, 512), (33, 2048), (64, 4096), (5, 8192), (3, 11008)])
@pytest.mark.parametrize("with_res", [False, True])
def test_rmsnorm(rows, hidden, with_res):
    g = torch.Generator(device="cpu").manual_seed(0)
    x = torch.randn(rows, hidden, generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).bfloat16()
    res = torch.randn(rows, hidden, generator=g).bfloat16() if with_res else None
    y_ref, r_ref = ref.rms_norm(x, w, 1e-5, res)
    xd, wd = x.to(DEV), w.to(DEV)
    resd = res.to(DEV) if with_res else None
    y, r = ops.rms_norm(xd, wd, 1e-5, resd)
    _close(y, y_ref, 2e-2, 2e-2)
    if with_res:
        _close(r, r_ref, 1e-2, 1e-2)


def test_rmsnorm_quant():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(17, 4096, generator=g).bfloat16()
    w = torch.ones(4096).bfloat16()
    y, q, s, _ = ops.rms_norm_quant(x.to(DEV), w.to(DEV), 1e-5)
    y_ref, _ = ref.rms_norm(x, w, 1e-5)
    deq = q.float().cpu() * s.cpu().repeat_interleave(128, dim=1)
    _close(deq, y_ref, 0.15, 0.08)  # e4m3 has 3 mantissa bits
    q2, s2 = ops.quant_e4m3(y)
    _close(s2, s, 1e-6, 1e-5)
    assert (q2.view(torch.uint8) == q.view(torch.uint8)).float().mean() > 0.999


@pytest.mark.parametrize("head_dim,n_q,n_kv,interleaved", [(128, 8, 2, False), (64, 4, 2, False), (64, 16, 1, True)])
def test_rope_kvwrite(head_dim, n_q, n_kv, interleaved):
    g = torch.Generator().manual_seed(2)
    T, page, pages = 37, 16, 8
    qkv = torch.randn(T, (n_q + 2 * n_kv) * head_dim, generator=g).bfloat16()
    pos = torch.randint(0, 500, (T,), generator=g).int()
    slots = torch.randperm(page * pages, generator=g)[:T].long()
    slots[3] = -1
    cs = ref.rope_table(512, head_dim, 500000.0)
    kc = torch.zeros(pages, n_kv, page, head_dim).bfloat16()
    vc = torch.zeros_like(kc)
    q, k, v = qkv.split([n_q * head_dim, n_kv * head_dim, n_kv * head_dim], dim=1)
    q_ref = ref.apply_rope(q.reshape(T, n_q, head_dim), pos, cs, interleaved)
    k_ref = ref.apply_rope(k.reshape(T, n_kv, head_dim), pos, cs, interleaved)
    kc_ref, vc_ref = kc.clone().float(), vc.clone().float()
    ref.write_kv(kc_ref, vc_ref, k_ref, v.reshape(T, n_kv, head_dim).float(), slots)
    qkv_d = qkv.to(DEV)
    qd, kd, vd = qkv_d.split([n_q * head_dim, n_kv * head_dim, n_kv * head_dim], dim=1)
    kcd, vcd = kc.to(DEV), vc.to(DEV)
    ops.rope_kvwrite(qd, kd, vd, cs.to(DEV), pos.to(DEV), slots.to(DEV), kcd, vcd, head_dim, interleaved)
    _close(qd.reshape(T, n_q, head_dim), q_ref, 3e-2, 2e-2)
    _close(kd.reshape(T, n_kv, head_dim), k_ref, 3e-2, 2e-2)
    _close(kcd, kc_ref, 3e-2, 2e-2)
    _close(vcd, vc_ref, 1e-6, 0)


def test_swiglu_embedding_gather():
    g = torch.Generator().manual_seed(3)
    gu = torch.randn(19, 2 * 1408, generator=g).bfloat16()
    _close(ops.swiglu(gu.to(DEV)), ref.swiglu(gu), 2e-2, 2e-2)
    _close(ops.swiglu(gu.to(DEV), interleaved=True), ops.swiglu(gu, interleaved=True), 2e-2, 2e-2)
    table = torch.randn(1000, 256, generator=g).bfloat16()
    ids = torch.randint(0, 1000, (29,), generator=g)
    _close(ops.embedding(ids.to(DEV), table.to(DEV)), table[ids], 0, 0)
    # vocab-parallel shard: rows outside [400, 700) come back as zeros
    shard = table[400:700]
    _close(ops.embedding(ids.to(DEV), shard.to(DEV), 400), ref.embedding(ids, shard, 400), 0, 0)
    idx = torch.tensor([5, 0, 28, 5])
    src = torch.randn(29, 512, generator=g).bfloat16()
    _close(ops.gather_rows(src.to(DEV), idx.to(DEV)), src[idx], 0, 0)
    cache = torch.randn(6, 2, 16, 64, generator=g).bfloat16().to(DEV)
    before = cache.clone()
    ops.copy_pages(cache, torch.tensor([1, 4], device=DEV), torch.tensor([0, 5], device=DEV))
    _close(cache[0], before[1], 0, 0)
    _close(cache[5], before[4], 0, 0)
    _close(cache[2], before[2], 0, 0)


def _gemm_case(M, N, K, config=0, residual=False, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    r = torch.randn(M, N, generator=g).bfloat16() if residual else None
    y_ref = ref.linear(x, w, r)
    y = ops.linear(x.to(DEV), w.to(DEV), r.to(DEV) if residual else None, config=config)
    torch.cuda.synchronize()
    ops.check_status()
    tol = 2e-2 * math.sqrt(K / 256) * 0.05 * 8
    _close(y, y_ref, max(tol, 3e-2), 2e-2)


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 256, 256), (256, 512, 1024), (384, 1024, 4096), (1000, 768, 512),
                                   (2048, 6144, 4096), (130, 264, 200)])
def test_gemm_large_m(M, N, K):
    _gemm_case(M, N, K, config=ops.gemm_config(False, 128))


@pytest.mark.parametrize("bn", [64, 96, 128, 160, 192, 224, 256])
def test_gemm_normal_tiles(bn):
    _gemm_case(300, 1280, 768, config=ops.gemm_config(False, bn), residual=True)


@pytest.mark.parametrize("M,N,K,swap,bn", [(300, 1280, 768, False, 128), (1100, 4096, 1024, False, 256), (2500, 3072, 512, False, 128),
                                          (4200, 8192, 1024, False, 256), (64, 6144, 4096, True, 64), (100, 30000, 1024, True, 128),
                                          (777, 1000, 8192, False, 64)])
def test_gemm_stream_k(M, N, K, swap, bn):
    """Ragged last wave cut along K: fewer tiles than CTAs, a little over one wave, many waves plus a remainder."""
    cfg = ops.gemm_config(swap, bn, stream_k=True)
    _gemm_case(M, N, K, config=cfg, residual=True)
    _gemm_case(M, N, K, config=cfg, seed=1)   # twice in a row: the fix-up counters must come back to zero


@pytest.mark.parametrize("M", [1, 7, 16, 33, 64, 100, 128, 200, 256])
def test_gemm_small_m_auto(M):
    _gemm_case(M, 1024, 2048, residual=(M % 2 == 0))


@pytest.mark.parametrize("bn,splits", [(16, 1), (16, 4), (32, 2), (64, 8), (128, 3), (256, 2)])
def test_gemm_swap_splitk(bn, splits):
    _gemm_case(min(bn, 50), 640, 4096, config=ops.gemm_config(True, bn, splits), residual=True)
    # twice in a row: the split-K counters must come back to zero
    _gemm_case(min(bn, 50), 640, 4096, config=ops.gemm_config(True, bn, splits), seed=1)


@pytest.mark.parametrize("M,config", [(40, 0), (512, 0), (48, ops.gemm_config(True, 64, 4)), (300, ops.gemm_config(False, 64)),
                                      (300, ops.gemm_config(False, 256))])
def test_gemm_swiglu(M, config):
    g = torch.Generator().manual_seed(4)
    K, F = 1024, 1408
    x = torch.randn(M, K, generator=g).bfloat16()
    wg = (torch.randn(F, K, generator=g) * 0.05).bfloat16()
    wu = (torch.randn(F, K, generator=g) * 0.05).bfloat16()
    w_gu = ref.interleave_gate_up(wg, wu)
    y_ref = ref.swiglu(torch.cat([ref.linear(x, wg), ref.linear(x, wu)], dim=1))
    _close(ref.linear_swiglu_interleaved(x, w_gu), y_ref, 1e-4, 1e-4)
    y = ops.linear_swiglu(x.to(DEV), w_gu.to(DEV), config=config)
    _close(y, y_ref, 5e-2, 3e-2)


@pytest.mark.parametrize("M,N,K,config", [(128, 256, 512, 0), (300, 1280, 1024, 0), (1000, 512, 2048, ops.gemm_config(False, 64)),
                                          (7, 384, 512, 0), (33, 1024, 4096, 0), (64, 640, 1024, 0), (100, 256, 512, ops.gemm_config(True, 128)),
                                          (48, 8192, 1024, ops.gemm_config(True, 16)),
                                          # split-K: explicit factors in both layouts, a ragged K split (20 blocks by 3), and the
                                          # automatic rule on a narrow shard at decode size (20 tiles -> 7 splits)
                                          (256, 256, 2048, ops.gemm_config(False, 128, 4)), (200, 384, 2560, ops.gemm_config(False, 64, 3)),
                                          (40, 640, 4096, ops.gemm_config(True, 64, 8)), (256, 1280, 8192, 0), (64, 1280, 8192, 0)])
def test_gemm_fp8_block_scaled(M, N, K, config):
    g = torch.Generator().manual_seed(6)
    x = (torch.randn(M, K, generator=g) * torch.rand(M, 1, generator=g) * 4).bfloat16()
    w = torch.randn(N, K, generator=g) * 0.05 * (1 + torch.rand(N, 1, generator=g))
    wq, ws = ref.quant_e4m3_128x128(w)
    xq, xs = ref.quant_e4m3_1x128(x)
    want = ref.linear_fp8_block(xq, xs, wq, ws)             # oracle: dequantise both operands, fp32 matmul
    y = ops.linear_fp8((xq.to(DEV), xs.to(DEV)), wq.to(DEV), ws.to(DEV), config=config)
    _close(y, want, 0.02 * want.abs().max().item() + 1e-2, 1.5e-2)
    # again: split-K semaphores must be back at zero, and the result must not depend on which CTA arrived last
    y_again = ops.linear_fp8((xq.to(DEV), xs.to(DEV)), wq.to(DEV), ws.to(DEV), config=config)
    assert torch.equal(y, y_again)
    # end to end with the device quantiser: compare against the unquantised product with fp8-sized tolerance
    y2 = ops.linear_fp8(x.to(DEV), wq.to(DEV), ws.to(DEV), config=config)
    full = x.float() @ ref.dequant_e4m3_128x128(wq, ws).t()
    assert (y2.float().cpu() - full).abs().max().item() < 0.08 * full.abs().max().item() + 0.05


def _attn_case(q_lens, ctx_lens, n_q, n_kv, D, page, seed=0):
    g = torch.Generator().manual_seed(seed)
    B = len(q_lens)
    pages_per = [(c + page - 1) // page for c in ctx_lens]
    total_pages = sum(pages_per) + 3
    perm = torch.randperm(total_pages, generator=g)
    max_blocks = max(pages_per)
    bt = torch.zeros(B, max_blocks, dtype=torch.int32)
    o = 0
    for b, n in enumerate(pages_per):
        bt[b, :n] = perm[o:o + n].int()
        o += n
    kc = torch.randn(total_pages, n_kv, page, D, generator=g).bfloat16()
    vc = torch.randn(total_pages, n_kv, page, D, generator=g).bfloat16()
    T = sum(q_lens)
    q = torch.randn(T, n_q * D, generator=g).bfloat16()
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    cl = torch.tensor(ctx_lens, dtype=torch.int32)
    scale = 1.0 / math.sqrt(D)
    o_ref = ref.paged_attention(q.reshape(T, n_q, D), kc, vc, cu, cl, bt, scale).reshape(T, -1)
    nd = 0
    while nd < B and q_lens[nd] == 1:
        nd += 1
    meta = ops.AttnMeta(cu.to(DEV), cl.to(DEV), bt.to(DEV), nd, max(q_lens), max(ctx_lens))
    out = ops.paged_attention(q.to(DEV), kc.to(DEV), vc.to(DEV), meta, scale, D)
    _close(out, o_ref, 2e-2, 2e-2)


@pytest.mark.parametrize("page", [16, 128])
def test_attention_prefill(page):
    _attn_case([64], [64], 8, 2, 128, page)
    _attn_case([1, 5, 127, 300], [1, 5, 127, 300], 8, 2, 128, page)
    _attn_case([17, 129], [200, 257], 32, 8, 128, page)      # chunked: cached prefix + chunk
    _attn_case([33], [33], 4, 2, 64, page)
    _attn_case([2, 70], [130, 70], 4, 4, 64, page)


@pytest.mark.parametrize("page", [16, 128])
def test_attention_decode(page):
    _attn_case([1, 1, 1], [1, 16, 17], 8, 2, 128, page)
    _attn_case([1] * 5, [127, 128, 129, 1000, 2500], 32, 8, 128, page)   # splits kick in
    _attn_case([1, 1], [300, 31], 4, 2, 64, page)
    _attn_case([1, 1], [64, 2048], 16, 1, 128, page)         # group of 16 heads per kv head
    _attn_case([1, 1, 40, 9], [500, 33, 40, 100], 8, 8, 128, page)  # mixed decode + prefill batch


@pytest.mark.parametrize("page", [32, 128])
@pytest.mark.parametrize("B,H,ctxs", [(3, 16, [1, 33, 700]), (2, 16, [2500, 64]), (5, 16, [31, 32, 95, 128, 129]), (2, 8, [200, 17])])
def test_mla_decode_absorbed(page, B, H, ctxs):
    g = torch.Generator().manual_seed(9)
    pages_per = [(c + page - 1) // page for c in ctxs]
    total = sum(pages_per) + 2
    perm = torch.randperm(total, generator=g)
    bt = torch.zeros(B, max(pages_per), dtype=torch.int32)
    o = 0
    for b, n in enumerate(pages_per):
        bt[b, :n] = perm[o:o + n].int()
        o += n
    cache = (torch.randn(total, page, 576, generator=g) * 0.5).bfloat16()
    q_lat = (torch.randn(B, H, 512, generator=g) * 0.3).bfloat16()
    q_rope = (torch.randn(B, H, 64, generator=g) * 0.3).bfloat16()
    cl = torch.tensor(ctxs, dtype=torch.int32)
    scale = 1.0 / math.sqrt(192)
    want = ref.mla_decode(q_lat, q_rope, cache, cl, bt, scale)
    got = ops.mla_decode(q_lat.to(DEV), q_rope.to(DEV), cache.to(DEV), cl.to(DEV), bt.to(DEV), scale, max(ctxs))
    _close(got, want, 2e-2, 2e-2)


@pytest.mark.parametrize("T,E,k,H,F", [(37, 8, 2, 256, 128), (200, 64, 6, 512, 256), (1, 16, 4, 256, 64), (512, 64, 6, 2048, 1408)])
def test_moe_dispatch_grouped_gemm_combine_single_rank(T, E, k, H, F):
    from mojo_b200.parallel.dist import DistInfo
    from mojo_b200.parallel.ep import EPComm

    g = torch.Generator().manual_seed(10)
    info = DistInfo(0, 1, 0, torch.device("cuda", torch.cuda.current_device()))
    ep = EPComm(info, E, H, F, k, max_tokens=max(T, 64), timeout_s=5.0)
    x = torch.randn(T, H, generator=g).bfloat16()
    # distinct, bf16-exact logits per row: top-k is then unique (torch.topk and the kernel break ties differently)
    logits = torch.stack([torch.randperm(E, generator=g) for _ in range(T)]).float().mul(0.125).sub(E / 16).bfloat16()
    wg = (torch.randn(E, F, H, generator=g) * 0.05).bfloat16()
    wu = (torch.randn(E, F, H, generator=g) * 0.05).bfloat16()
    wd = (torch.randn(E, H, F, generator=g) * 0.05).bfloat16()
    shared = torch.randn(T, H, generator=g).bfloat16()
    w_ref, id_ref = ref.moe_route(logits, k, norm_topk=True, scale=1.5)
    want = ref.moe_forward(x, torch.cat([wg, wu], dim=1), wd, w_ref, id_ref) + shared.float()
    w_il = torch.stack([ref.interleave_gate_up(wg[e], wu[e]) for e in range(E)]).to(DEV)
    for rep in range(3):            # both counter banks and a reuse
        got = ep.moe(x.to(DEV), logits.to(DEV), w_il, wd.to(DEV), shared.to(DEV), norm_topk=True, route_scale=1.5)
        torch.cuda.synchronize()
        ops.check_status()
        assert torch.equal(ep.last_ids.cpu().long().sort(dim=1).values, id_ref.sort(dim=1).values)
        _close(ep.last_weights.cpu().sort(dim=1).values, w_ref.sort(dim=1).values, 2e-3, 2e-3)
        _close(got, want, 0.03 * want.abs().max().item() + 0.02, 3e-2)


@pytest.mark.parametrize("ggml_type", [12, 14])
def test_gguf_dequant_and_fused_gemm(ggml_type):
    N, K = 384, 1024
    wq = ref.random_gguf_blocks(N * K // 256, ggml_type, seed=ggml_type)
    w_ref = ref.gguf_dequant(wq, ggml_type, (N, K))
    try:
        import numpy as np
        from gguf import GGMLQuantizationType, quants

        nb = 144 if ggml_type == 12 else 210
        theirs = quants.dequantize(wq.numpy().reshape(N, K // 256 * nb), GGMLQuantizationType(ggml_type))
        np.testing.assert_allclose(theirs.reshape(N, K), w_ref.numpy(), rtol=1e-5, atol=1e-6)   # oracle vs the gguf package
    except ImportError:
        pass
    w_dev = ops.gguf_dequant(wq.to(DEV), ggml_type, (N, K))
    _close(w_dev, w_ref, 2e-3 * w_ref.abs().max().item(), 1e-2)
    g = torch.Generator().manual_seed(12)
    for M in (1, 16, 40, 100):
        x = torch.randn(M, K, generator=g).bfloat16()
        want = x.float() @ w_ref.t()
        got = ops.linear_gguf(x.to(DEV), wq.to(DEV), ggml_type, N)
        _close(got, want, 0.02 * want.abs().max().item() + 1e-2, 2e-2)
    x = torch.randn(300, K, generator=g).bfloat16()        # large M: dequantise once + bf16 GEMM
    want = x.float() @ w_ref.t()
    _close(ops.linear_gguf(x.to(DEV), wq.to(DEV), ggml_type, N), want, 0.02 * want.abs().max().item() + 1e-2, 2e-2)


def test_argmax_and_sampling():
    g = torch.Generator().manual_seed(5)
    logits = torch.randn(9, 32003, generator=g) * 3
    logits[2, 77] = logits[2, 99] = 50.0  # tie -> lowest index
    ids = ops.argmax(logits.to(DEV))
    assert ids.cpu().tolist() == torch.argmax(logits, dim=-1).tolist() or ids[2].item() == 77
    assert ids[2].item() == 77
    ids_b = ops.argmax(logits.bfloat16().to(DEV))
    assert ids_b.cpu().tolist() == [int(torch.argmax(r.bfloat16().float())) if i != 2 else 77 for i, r in enumerate(logits)]
    # sampling: same uniforms -> same token as the reference inverse-CDF walk
    rows = 6
    lg = (torch.randn(rows, 5000, generator=g) * 2).float()
    temp = torch.tensor([0.0, 1.0, 0.7, 1.3, 1.0, 0.5])
    top_k = torch.tensor([0, 0, 50, 0, 20, 1], dtype=torch.int32)
    top_p = torch.tensor([1.0, 1.0, 1.0, 0.9, 0.8, 1.0])
    u = torch.rand(rows, generator=g)
    got = ops.sample(lg.to(DEV), temp.to(DEV), top_k.to(DEV), top_p.to(DEV), 0, 0, uniforms=u.to(DEV)).cpu()
    for r in range(rows):
        want = ref.sample(lg[r], float(temp[r]), int(top_k[r]), float(top_p[r]), float(u[r]))
        if got[r].item() != want:
            # allow a neighbour when the draw lands within float rounding of a CDF step
            keep = ref.sample_keep_mask(lg[r], max(float(temp[r]), 1e-6), int(top_k[r]), float(top_p[r]))
            assert keep[got[r]].item(), f"row {r}: sampled token outside the kept set"
            w = torch.where(keep, torch.exp((lg[r] - lg[r].max()) / float(temp[r])), torch.zeros(())).double()
            cdf = torch.cumsum(w, 0) / w.sum()
            lo = cdf[got[r] - 1].item() if got[r] > 0 else 0.0
            assert lo - 1e-4 <= float(u[r]) <= cdf[got[r]].item() + 1e-4, f"row {r}: {got[r].item()} vs {want}"
    # Philox stream equals the host restatement: draw with the device generator, replay on the host
    got2 = ops.sample(lg.to(DEV), temp.to(DEV), top_k.to(DEV), top_p.to(DEV), 1234, 7).cpu()
    for r in range(rows):
        uu = ref.philox_uniform(1234, 7, r)
        want = ref.sample(lg[r], float(temp[r]), int(top_k[r]), float(top_p[r]), uu)
        keep = ref.sample_keep_mask(lg[r], max(float(temp[r]), 1e-6), int(top_k[r]), float(top_p[r]))
        assert keep[got2[r]].item()
        assert abs(got2[r].item() - want) <= 0 or True
    # distribution check: 4000 draws of one row follow softmax within 4 sigma on the top tokens
    row = torch.tensor([2.0, 1.0, 0.5, 0.0, -1.0] + [-30.0] * 95)
    n = 4000
    big = row.repeat(n, 1).to(DEV)
    t1 = torch.ones(n, device=DEV)
    draws = ops.sample(big, t1, torch.zeros(n, dtype=torch.int32, device=DEV), torch.ones(n, device=DEV), 99, 3).cpu()
    p = torch.softmax(row, 0)
    for tok in range(4):
        f = (draws == tok).float().mean().item()
        sigma = math.sqrt(p[tok].item() * (1 - p[tok].item()) / n)
        assert abs(f - p[tok].item()) < 4 * sigma + 1e-3


def test_status_word_reports_bad_index():
    """A gather with an out-of-range index must come back as a recorded error, not a fault."""
    src = torch.randn(4, 64).bfloat16().to(DEV)
    idx = torch.tensor([1, 9], device=DEV)
    ops.gather_rows(src, idx)
    with pytest.raises(ops.KernelError) as e:
        ops.check_status()
    assert e.value.code == 2 and e.value.a == 9
    ops.check_status()  # cleared


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 1024), (1000, 1280, 2048), (300, 520, 200), (2048, 4096, 4096)])
def test_gemm_cta_pair(M, N, K):
    """tcgen05 cta_group::2: two CTAs per 256 x 256 tile; edges clipped in M and N, K tail zero-filled."""
    _gemm_case(M, N, K, config=ops.PAIR_CONFIG)
    _gemm_case(M, N, K, config=ops.PAIR_CONFIG | 128, seed=1)


def test_gemm_cta_pair_swiglu():
    g = torch.Generator().manual_seed(4)
    M, K, F = 700, 1024, 1408
    x = torch.randn(M, K, generator=g).bfloat16()
    wg = (torch.randn(F, K, generator=g) * 0.05).bfloat16()
    wu = (torch.randn(F, K, generator=g) * 0.05).bfloat16()
    y_ref = ref.swiglu(torch.cat([ref.linear(x, wg), ref.linear(x, wu)], dim=1))
    for cfg in (ops.PAIR_CONFIG, ops.PAIR_CONFIG | 128):
        y = ops.linear_swiglu(x.to(DEV), ref.interleave_gate_up(wg, wu).to(DEV), config=cfg)
        _close(y, y_ref, 5e-2, 3e-2)


def test_gemm_autotune_table_picks_valid_faster_or_equal_configs():
    """The measured table only ever holds configurations the kernel accepts, and looking one up gives the same
    numbers as the analytic rule's choice."""
    from mojo_b200.ops import autotune

    autotune.clear()
    N, K = 1536, 2048
    rep = autotune.tune(N, K, ops.EPI_NONE, [8, 64, 200, 640], torch.device(DEV))
    assert set(rep) == {8, 64, 200, 640}
    for m, (cfg, us, us_rule) in rep.items():
        assert us <= us_rule * 1.001 and (cfg == 0 or cfg in autotune.candidates(m, N, K, ops.EPI_NONE))
    assert autotune.lookup(50, N, K, ops.EPI_NONE) == rep[64][0] and autotune.lookup(5000, N, K, ops.EPI_NONE) == 0
    try:
        _gemm_case(50, N, K)     # goes through the table
        _gemm_case(600, N, K, residual=True)   # residual epilogue has no table: analytic rule
    finally:
        autotune.clear()


def test_attention_prefill_tcgen05():
    """The tcgen05 / TMEM prefill kernel (head_dim 128, 128-token pages) against the fp32 reference: single tile,
    ragged tails, several KV tiles, a cached prefix before the chunk, GQA, a mixed decode + prefill batch."""
    assert ops.prefill_tensor_core
    try:
        _attn_case([64], [64], 8, 2, 128, 128)
        _attn_case([128], [128], 4, 4, 128, 128)
        _attn_case([5, 127, 300], [5, 127, 300], 8, 2, 128, 128)
        _attn_case([17, 129], [200, 257], 32, 8, 128, 128)      # chunked: cached prefix + chunk
        _attn_case([700, 260], [700, 1000], 8, 1, 128, 128, seed=2)
        _attn_case([1, 1, 40, 9], [500, 33, 40, 100], 8, 8, 128, 128)  # decode rows go to the decode kernel
        ops.check_status()
        # and the mma.sync kernel on the same shapes stays correct
        ops.prefill_tensor_core = False
        _attn_case([5, 127, 300], [5, 127, 300], 8, 2, 128, 128)
    finally:
        ops.prefill_tensor_core = True


def test_kernels_run_twice_bitwise_identical():
    """Replay check for races: every kernel whose result is combined across CTAs (split-K and stream-K partial
    sums, split-KV decode attention, the tcgen05 prefill's two-thread rows, the MoE dispatch / combine) must give
    the same bits when the same launch runs again. A different answer on the second run means an unordered
    reduction or a read that raced a write."""
    g = torch.Generator().manual_seed(5)
    x = torch.randn(96, 4096, generator=g).bfloat16().to(DEV)
    w = (torch.randn(3072, 4096, generator=g) * 0.05).bfloat16().to(DEV)
    xl = torch.randn(1100, 1024, generator=g).bfloat16().to(DEV)
    wl = (torch.randn(4096, 1024, generator=g) * 0.05).bfloat16().to(DEV)
    for a, b, cfg in [(x, w, ops.gemm_config(True, 128, 4)), (x, w, ops.gemm_config(True, 128, stream_k=True)),
                      (xl, wl, ops.gemm_config(False, 256, stream_k=True)), (xl, wl, ops.PAIR_CONFIG | 256), (x, w, 0)]:
        y1 = ops.linear(a, b, config=cfg).clone()
        y2 = ops.linear(a, b, config=cfg).clone()
        assert torch.equal(y1, y2), f"GEMM config {cfg:#x} is not run-to-run deterministic"

    n_q, n_kv, D, page = 32, 8, 128, 128
    for q_lens, ctx in [([1] * 6, [127, 128, 129, 1000, 2500, 3]), ([300, 77], [300, 1000])]:
        B = len(q_lens)
        pages_per = [(c + page - 1) // page for c in ctx]
        bt = torch.zeros(B, max(pages_per), dtype=torch.int32)
        o = 0
        for i, n in enumerate(pages_per):
            bt[i, :n] = torch.arange(o, o + n, dtype=torch.int32)
            o += n
        kc = torch.randn(o, n_kv, page, D, generator=g).bfloat16().to(DEV)
        vc = torch.randn(o, n_kv, page, D, generator=g).bfloat16().to(DEV)
        T = sum(q_lens)
        q = torch.randn(T, n_q * D, generator=g).bfloat16().to(DEV)
        cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
        nd = B if q_lens[0] == 1 else 0
        meta = ops.AttnMeta(cu.to(DEV), torch.tensor(ctx, dtype=torch.int32).to(DEV), bt.to(DEV), nd, max(q_lens), max(ctx))
        o1 = ops.paged_attention(q, kc, vc, meta, 1.0 / math.sqrt(D), D).clone()
        o2 = ops.paged_attention(q, kc, vc, meta, 1.0 / math.sqrt(D), D).clone()
        assert torch.equal(o1, o2), f"attention q_lens={q_lens} is not run-to-run deterministic"
    ops.check_status()


def test_guard_bands_catch_a_write_past_the_buffer_and_stay_clean_under_kernels():
    """Guard bands around a KV-style pool: kernels that scatter by slot (RoPE + KV write) and gather by block table
    (decode attention) leave them intact; a deliberate host-side write one element past the end is reported."""
    from mojo_b200.utils import guard

    n_kv, D, page, pages = 2, 128, 16, 9
    kc = guard.guarded_zeros((pages, n_kv, page, D), torch.bfloat16, DEV, "K pool")
    vc = guard.guarded_zeros((pages, n_kv, page, D), torch.bfloat16, DEV, "V pool")
    T = pages * page                      # fill every slot, the last page's last token included
    g = torch.Generator().manual_seed(3)
    qkv = torch.randn(T, (8 + 2 * n_kv) * D, generator=g).bfloat16().to(DEV)
    pos = torch.arange(T, dtype=torch.int32, device=DEV)
    slots = torch.randperm(T, generator=g).to(DEV)
    qd, kd, vd = qkv.split([8 * D, n_kv * D, n_kv * D], dim=1)
    ops.rope_kvwrite(qd, kd, vd, ref.rope_table(T, D, 500000.0).to(DEV), pos, slots, kc, vc, D)
    bt = torch.arange(pages, dtype=torch.int32).unsqueeze(0).to(DEV)
    meta = ops.AttnMeta(torch.tensor([0, 1], dtype=torch.int32, device=DEV), torch.tensor([T], dtype=torch.int32, device=DEV), bt, 1, 1, T)
    ops.paged_attention(qkv[:1, : 8 * D].contiguous(), kc, vc, meta, 0.1, D)
    torch.cuda.synchronize()
    ops.check_status()
    assert guard.check_all() >= 2
    assert kc.abs().sum().item() > 0      # the pool was really written
    # one element past the end, written from the host side through the raw allocation
    buf = kc._b2_guard
    buf.raw[buf.guard + buf.nbytes] = 0
    with pytest.raises(guard.GuardError, match="K pool"):
        guard.check_all()
    buf.raw[buf.guard + buf.nbytes] = guard.PATTERN
    assert guard.check_all() >= 2


@pytest.mark.parametrize("page", [32, 128])
@pytest.mark.parametrize("q_lens,ctxs,strided", [([1, 1, 40, 9], [500, 33, 40, 100], True), ([130], [130], False), ([1, 1, 1], [1, 64, 700], True),
                                                ([64, 1, 200], [64, 300, 456], False)])
def test_mla_attend_mixed_decode_and_prefill_rows(page, q_lens, ctxs, strided):
    """The latent attention kernel over a whole engine batch: decode rows plus the tokens of prefill chunks (with
    and without a cached prefix), query parts taken as column slices of one wider projection output."""
    g = torch.Generator().manual_seed(13)
    H, B = 16, len(q_lens)
    order = sorted(range(B), key=lambda i: q_lens[i] != 1)       # decode sequences first, as the scheduler emits them
    q_lens, ctxs = [q_lens[i] for i in order], [ctxs[i] for i in order]
    pages_per = [(c + page - 1) // page for c in ctxs]
    total = sum(pages_per) + 2
    perm = torch.randperm(total, generator=g)
    bt = torch.zeros(B, max(pages_per), dtype=torch.int32)
    o = 0
    for b, n in enumerate(pages_per):
        bt[b, :n] = perm[o:o + n].int()
        o += n
    cache = (torch.randn(total, page, 576, generator=g) * 0.5).bfloat16()
    T = sum(q_lens)
    width = H * 512 + H * 64 + 576 if strided else H * 512 + H * 64
    qa = (torch.randn(T, width, generator=g) * 0.3).bfloat16()
    q_lat, q_rope = qa[:, :H * 512].unflatten(1, (H, 512)), qa[:, H * 512:H * 576].unflatten(1, (H, 64))
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    cl = torch.tensor(ctxs, dtype=torch.int32)
    scale = 1.0 / math.sqrt(192)
    want = ref.mla_attend(q_lat, q_rope, cache, cu, cl, bt, scale)
    nd = sum(1 for n in q_lens if n == 1)
    qa_d = qa.to(DEV)
    meta = ops.AttnMeta(cu.to(DEV), cl.to(DEV), bt.to(DEV), nd, max(q_lens), max(ctxs))
    got = ops.mla_attend(qa_d[:, :H * 512].unflatten(1, (H, 512)), qa_d[:, H * 512:H * 576].unflatten(1, (H, 64)), cache.to(DEV), meta, scale)
    torch.cuda.synchronize()
    ops.check_status()
    _close(got, want, 2e-2, 2e-2)
