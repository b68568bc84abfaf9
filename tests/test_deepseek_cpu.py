"""DeepSeek-V2 architecture (MLA + MoE) on CPU: the engine's paged, absorbed-decode path must reproduce a dense,
non-absorbed forward pass token for token."""
import torch

from mojo_b200.engine import EngineConfig, LLMEngine, SamplingParams
from mojo_b200.models.config import tiny_deepseek
from mojo_b200.ops import reference as ref


def dense_logits(model, ids):
    cfg = model.cfg
    T, H = len(ids), cfg.num_heads
    nope, rope, vdim, lora = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank
    h = model.embed[torch.tensor(ids)].float()
    pos = torch.arange(T)
    for lw in model.layers:
        x, _ = ref.rms_norm(h, lw.attn_norm, cfg.rms_norm_eps)
        q = (x @ lw.wq.float().t()).view(T, H, nope + rope)
        kv = x @ lw.w_kv_a.float().t()
        c, _ = ref.rms_norm(kv[:, :lora], lw.kv_a_norm, cfg.rms_norm_eps)
        k_r = ref.apply_rope(kv[:, lora:].view(T, 1, rope), pos, model.cos_sin, interleaved=True)
        q_r = ref.apply_rope(q[:, :, nope:], pos, model.cos_sin, interleaved=True)
        k = torch.cat([torch.einsum("tc,hdc->thd", c, lw.w_uk.float()), k_r.expand(T, H, rope)], dim=2)
        v = torch.einsum("tc,hvc->thv", c, lw.w_uv.float())
        qq = torch.cat([q[:, :, :nope], q_r], dim=2)
        s = torch.einsum("qhd,khd->hqk", qq, k) / (nope + rope) ** 0.5
        s = s.masked_fill(~torch.tril(torch.ones(T, T, dtype=torch.bool)), float("-inf"))
        a = torch.einsum("hqk,khv->qhv", torch.softmax(s, -1), v).reshape(T, -1)
        h = h + a @ lw.wo.float().t()
        x, _ = ref.rms_norm(h, lw.mlp_norm, cfg.rms_norm_eps)
        if lw.w_gu is not None:
            y = ref.linear_swiglu_interleaved(x, lw.w_gu) @ lw.w_down.float().t()
        else:
            w, idx = ref.moe_route(x @ lw.w_router.float().t(), cfg.num_experts_per_tok, cfg.norm_topk_prob, cfg.routed_scaling_factor)
            y = ref.moe_forward(x, lw.w_exp_gu, lw.w_exp_down, w, idx)
            y = y + ref.linear_swiglu_interleaved(x, lw.w_shared_gu) @ lw.w_shared_down.float().t()
        h = h + y
    x, _ = ref.rms_norm(h, model.final_norm, cfg.rms_norm_eps)
    return x[-1] @ model.lm_head.float().t()


def test_tiny_deepseek_engine_matches_dense_forward():
    cfg = EngineConfig(model=tiny_deepseek(), device="cpu", dtype=torch.float32, page_size=16, num_pages=32, max_num_seqs=4,
                       max_num_batched_tokens=24, max_model_len=256, seed=0)
    eng = LLMEngine(cfg)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (40, 9)]
    outs = eng.generate(prompts, SamplingParams(max_tokens=10))     # budget 24 forces chunked MLA prefill
    for p, o in zip(prompts, outs):
        ids = list(p)
        for t in range(10):
            nxt = int(torch.argmax(dense_logits(eng.model, ids)))
            assert nxt == o[t], f"token {t}: engine {o[t]} vs dense {nxt}"
            ids.append(nxt)
    assert eng.kv.check_invariants() == ""


def test_absorbed_attention_path_matches_factored_path():
    """The CUDA formulation (up-projections folded into the query and output weights, one latent-attention call over
    decode rows and prefill chunks) run through the CPU fallbacks of the same ops must equal the factored formulation."""
    import copy

    from mojo_b200 import ops
    from mojo_b200.models import build_model

    cfg = tiny_deepseek()
    model = build_model(cfg, "cpu", torch.float32).init_random(0, std=0.05)
    page, g = 16, torch.Generator().manual_seed(4)
    q_lens, ctxs = [1, 1, 20, 7], [30, 1, 20, 25]      # two decode rows, a fresh prompt, a chunk after an 18-token prefix
    T = sum(q_lens)
    n_pages = [(c + page - 1) // page for c in ctxs]
    bt = torch.zeros(len(q_lens), max(n_pages), dtype=torch.int32)
    o = 1
    for b, n in enumerate(n_pages):
        bt[b, :n] = torch.arange(o, o + n, dtype=torch.int32)
        o += n
    cache = torch.randn(o + 1, page, cfg.kv_lora_rank + cfg.qk_rope_head_dim, generator=g) * 0.3   # cached prefixes: random latents
    positions, slots = [], []
    for b, (ql, c) in enumerate(zip(q_lens, ctxs)):
        for i in range(c - ql, c):
            positions.append(i)
            slots.append(int(bt[b, i // page]) * page + i % page)
    positions = torch.tensor(positions, dtype=torch.int32)
    slots = torch.tensor(slots, dtype=torch.int64)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    meta = ops.AttnMeta(cu, torch.tensor(ctxs, dtype=torch.int32), bt, 2, max(q_lens), max(ctxs))
    x = torch.randn(T, cfg.hidden_size, generator=g)
    lw = model.layers[1]
    cache_a, cache_b = cache.clone(), cache.clone()
    want = ops.linear(model._attention(lw, x, positions, slots, meta, cache_a), lw.wo)
    lw2 = copy.deepcopy(lw)
    got = model._attention_absorbed(lw2, x, positions, slots, meta, cache_b)
    assert lw2.wq is None and lw2.w_qa.shape == (cfg.num_heads * 576 + 576, cfg.hidden_size)
    assert torch.equal(cache_a, cache_b)               # both wrote the same latents
    assert torch.allclose(got, want, atol=2e-5, rtol=1e-4), (got - want).abs().max()
