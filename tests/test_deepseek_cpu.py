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


def _write_tiny_deepseek_checkpoint(tmp_path, model):
    from mojo_b200.loaders.safetensors_loader import deepseek_v2_state_dict, save_llama_safetensors

    cfg = model.cfg
    hf_cfg = {"architectures": ["DeepseekV2ForCausalLM"], "hidden_size": cfg.hidden_size, "num_hidden_layers": cfg.num_layers,
              "num_attention_heads": cfg.num_heads, "num_key_value_heads": cfg.num_heads, "intermediate_size": cfg.intermediate_size,
              "vocab_size": cfg.vocab_size, "rms_norm_eps": cfg.rms_norm_eps, "rope_theta": cfg.rope_theta,
              "max_position_embeddings": cfg.max_position_embeddings, "kv_lora_rank": cfg.kv_lora_rank, "q_lora_rank": None,
              "qk_rope_head_dim": cfg.qk_rope_head_dim, "qk_nope_head_dim": cfg.qk_nope_head_dim, "v_head_dim": cfg.v_head_dim,
              "n_routed_experts": cfg.n_routed_experts, "n_shared_experts": cfg.n_shared_experts,
              "num_experts_per_tok": cfg.num_experts_per_tok, "moe_intermediate_size": cfg.moe_intermediate_size,
              "first_k_dense_replace": cfg.first_k_dense_replace, "routed_scaling_factor": cfg.routed_scaling_factor,
              "norm_topk_prob": cfg.norm_topk_prob}
    save_llama_safetensors(deepseek_v2_state_dict(model), tmp_path, hf_cfg)


def test_deepseek_hf_checkpoint_roundtrip_and_expert_slicing(tmp_path):
    """A checkpoint in the Hugging Face DeepseekV2ForCausalLM layout (kv_b_proj fused, one tensor per expert
    projection) loads into the same model; an expert-parallel rank reads only its own experts."""
    from mojo_b200.loaders import load_safetensors_into
    from mojo_b200.models import build_model
    from mojo_b200.pipelines import LLM, PipelineConfig

    src = build_model(tiny_deepseek(), "cpu", torch.float32).init_random(3, std=0.05)
    _write_tiny_deepseek_checkpoint(tmp_path, src)
    llm = LLM(PipelineConfig(model=str(tmp_path), device="cpu", dtype="float32", page_size=16, num_pages=32, max_num_seqs=4,
                             max_num_batched_tokens=64, max_model_len=128))
    got = llm.engine.model
    assert got.cfg.architecture == "deepseek_v2" and len(got.layers) == len(src.layers)
    for a, b in zip(src.layers, got.layers):
        for name in ("wq", "w_kv_a", "kv_a_norm", "w_uk", "w_uv", "wo", "w_gu", "w_down", "w_router", "w_shared_gu", "w_shared_down",
                     "w_exp_gu", "w_exp_down"):
            x, y = getattr(a, name), getattr(b, name)
            assert (x is None) == (y is None), name
            if x is not None:
                assert torch.equal(x, y), name
    prompt = torch.randint(0, 1024, (12,), generator=torch.Generator().manual_seed(5)).tolist()
    out = llm.generate([prompt], SamplingParams(max_tokens=5))[0]
    ids = list(prompt)
    for t in range(5):
        nxt = int(torch.argmax(dense_logits(src, ids)))
        assert nxt == out.token_ids[t]
        ids.append(nxt)

    class _Ep:          # stands in for the expert-parallel communicator: only its geometry matters at load time
        world_size, rank = 2, 1

    part = build_model(tiny_deepseek(), "cpu", torch.float32, ep=_Ep())
    load_safetensors_into(part, tmp_path)
    moe = [lw for lw in part.layers if lw.w_router is not None]
    ref_moe = [lw for lw in src.layers if lw.w_router is not None]
    half = tiny_deepseek().n_routed_experts // 2
    for a, b in zip(ref_moe, moe):
        assert b.w_exp_gu is None and b.w_exp_gu_il.shape[0] == half
        assert torch.equal(b.w_exp_down, a.w_exp_down[half:])
        f = a.w_exp_gu.shape[1] // 2
        assert torch.equal(b.w_exp_gu_il[0], ref.interleave_gate_up(a.w_exp_gu[half, :f], a.w_exp_gu[half, f:]))
