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
