"""DeepSeek-V2(-Lite) decoder: multi-head latent attention (MLA) + mixture of experts with shared experts.

Cache: one row per token per layer, [c_kv (kv_lora_rank) | k_rope (qk_rope_head_dim)], shared by all heads.

On CUDA attention runs entirely in the absorbed form, for decode tokens and prefill chunks alike. The per-head
up-projections are folded into the neighbouring projection weights once, when the model first runs:
    W_qa[h] = W_UK[h]^T W_q,nope[h]   (query straight into latent space, [H * 512, hidden])
    W_oa[:, h] = W_o[:, h] W_UV[h]     (latent-space output straight to hidden, [hidden, H * 512])
so a layer's attention is one GEMM producing [q_lat | q_rope | c_kv | k_rope], RMSNorm + RoPE + the cache scatter,
one launch of the latent attention kernel over every token of the batch (`ops.mla_attend`), and one GEMM back to
hidden. That costs about 1 % more GEMM FLOPs per token than the factored form and removes every per-head small
matrix product, every K/V expansion and every per-sequence loop. The CPU path keeps the factored weights and the
textbook formulation (per-head K/V expansion for prefill): it is the oracle.

MoE: softmax router over all routed experts, top-k, optional renormalisation; routed experts run through the
expert-parallel path (`parallel.ep`: dispatch, grouped GEMM, combine) and the shared experts as one fused MLP.
Under expert parallelism attention is data-parallel: every rank runs all heads on its own requests.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .. import ops
from ..ops import reference
from .config import ModelConfig


@dataclass
class DsLayer:
    attn_norm: torch.Tensor
    wq: torch.Tensor          # [H * (nope + rope), hidden]
    w_kv_a: torch.Tensor      # [kv_lora + rope, hidden]
    kv_a_norm: torch.Tensor   # [kv_lora]
    w_uk: torch.Tensor        # [H, nope, kv_lora]
    w_uv: torch.Tensor        # [H, v_dim, kv_lora]
    wo: torch.Tensor          # [hidden, H * v_dim]
    mlp_norm: torch.Tensor
    # dense FFN layers
    w_gu: torch.Tensor | None = None      # [2F, hidden] interleaved gate/up
    w_down: torch.Tensor | None = None
    # MoE layers
    w_router: torch.Tensor | None = None  # [E, hidden]
    w_shared_gu: torch.Tensor | None = None
    w_shared_down: torch.Tensor | None = None
    w_exp_gu: torch.Tensor | None = None  # [E_local, 2F_moe, hidden] (gate rows then up rows per expert)
    w_exp_down: torch.Tensor | None = None  # [E_local, hidden, F_moe]
    w_exp_gu_il: torch.Tensor | None = None  # [E_local, 2F_moe, hidden] gate/up interleaved in blocks of 16 (EP kernels)
    # absorbed attention weights (CUDA path, built by `DeepseekV2Model._absorb`)
    w_qa: torch.Tensor | None = None      # [H * kv_lora + H * rope + kv_lora + rope, hidden]: q_lat | q_rope | c_kv | k_rope
    w_oa: torch.Tensor | None = None      # [hidden, H * kv_lora]


class DeepseekV2Model:
    def __init__(self, cfg: ModelConfig, device="cpu", dtype=torch.float32, comm=None, ep=None):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.comm = comm
        self.ep = ep                      # expert-parallel communicator (None: all experts local)
        self.ep_size = ep.world_size if ep is not None else 1
        self.ep_rank = ep.rank if ep is not None else 0
        assert cfg.n_routed_experts % self.ep_size == 0
        self.e_local = cfg.n_routed_experts // self.ep_size
        self.H = cfg.num_heads
        self.nope, self.rope, self.vdim, self.lora = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank
        self.scale = 1.0 / math.sqrt(self.nope + self.rope)
        self.layers: list[DsLayer] = []
        self.embed = self.final_norm = self.lm_head = None
        self.cos_sin = reference.rope_table(cfg.max_position_embeddings, self.rope, cfg.rope_theta, None).to(self.device)

    # ------------------------------------------------------------------------------------------------
    def _put(self, t):
        return t.to(device=self.device, dtype=self.dtype).contiguous()

    def init_random(self, seed: int = 0, std: float = 0.02) -> "DeepseekV2Model":
        cfg = self.cfg
        # small models draw on the CPU so that CPU and GPU instances of one seed hold the same weights
        big = cfg.hidden_size * cfg.vocab_size > (1 << 27)
        gen_dev = self.device if (big and self.device.type == "cuda") else torch.device("cpu")
        g = torch.Generator(device=gen_dev).manual_seed(seed)

        def rnd(*shape):
            return torch.randn(*shape, generator=g, device=gen_dev, dtype=torch.float32) * std

        h = cfg.hidden_size
        self.embed = self._put(rnd(cfg.vocab_size, h))
        for i in range(cfg.num_layers):
            lw = DsLayer(
                attn_norm=self._put(torch.ones(h)), wq=self._put(rnd(self.H * (self.nope + self.rope), h)),
                w_kv_a=self._put(rnd(self.lora + self.rope, h)), kv_a_norm=self._put(torch.ones(self.lora)),
                w_uk=self._put(rnd(self.H, self.nope, self.lora)), w_uv=self._put(rnd(self.H, self.vdim, self.lora)),
                wo=self._put(rnd(h, self.H * self.vdim)), mlp_norm=self._put(torch.ones(h)))
            if i < cfg.first_k_dense_replace:
                f = cfg.intermediate_size
                lw.w_gu = self._put(reference.interleave_gate_up(rnd(f, h), rnd(f, h)))
                lw.w_down = self._put(rnd(h, f))
            else:
                fm, fs = cfg.moe_intermediate_size, cfg.moe_intermediate_size * cfg.n_shared_experts
                lw.w_router = self._put(rnd(cfg.n_routed_experts, h))
                if fs > 0:
                    lw.w_shared_gu = self._put(reference.interleave_gate_up(rnd(fs, h), rnd(fs, h)))
                    lw.w_shared_down = self._put(rnd(h, fs))
                # every rank draws all experts (same stream on every rank) and keeps its slice
                e0 = self.ep_rank * self.e_local
                gu = rnd(cfg.n_routed_experts, 2 * fm, h)
                dn = rnd(cfg.n_routed_experts, h, fm)
                lw.w_exp_gu = self._put(gu[e0:e0 + self.e_local])
                lw.w_exp_down = self._put(dn[e0:e0 + self.e_local])
                if self.ep is not None:
                    lw.w_exp_gu_il = torch.stack([reference.interleave_gate_up(w[:fm], w[fm:]) for w in lw.w_exp_gu])
                    lw.w_exp_gu = None
                del gu, dn
            self.layers.append(lw)
        self.final_norm = self._put(torch.ones(h))
        self.lm_head = self._put(rnd(cfg.vocab_size, h))
        return self.finalize()

    def finalize(self) -> "DeepseekV2Model":
        """Call once after the weights are in place: on CUDA, folds the MLA up-projections into their neighbours."""
        if self.device.type == "cuda" and self.lora == 512 and self.rope == 64:
            for lw in self.layers:
                if lw.w_qa is None:
                    self._absorb(lw)
        return self

    def weight_bytes(self) -> int:
        n = 0
        for lw in self.layers:
            for t in vars(lw).values():
                if t is not None:
                    n += t.numel() * t.element_size()
        return n + sum(t.numel() * t.element_size() for t in (self.embed, self.final_norm, self.lm_head))

    # ------------------------------------------------------------------------------------------------
    def allocate_kv_cache(self, num_pages: int, page_size: int):
        from ..utils import guard

        return [guard.zeros((num_pages, page_size, self.lora + self.rope), self.dtype, self.device, f"latent cache, layer {i}")
                for i in range(self.cfg.num_layers)]

    def kv_bytes_per_page(self, page_size: int) -> int:
        return self.cfg.num_layers * page_size * (self.lora + self.rope) * torch.empty((), dtype=self.dtype).element_size()

    # ------------------------------------------------------------------------------------------------
    def _absorb(self, lw: DsLayer) -> None:
        """Fold W_UK into the query projection and W_UV into the output projection (fp32 products, rounded once)."""
        H, hid = self.H, self.cfg.hidden_size
        wq = lw.wq.float().view(H, self.nope + self.rope, hid)
        w_q_lat = torch.einsum("hdc,hdk->hck", lw.w_uk.float(), wq[:, :self.nope]).reshape(H * self.lora, hid)
        w_q_rope = wq[:, self.nope:].reshape(H * self.rope, hid)
        lw.w_qa = torch.cat([w_q_lat, w_q_rope, lw.w_kv_a.float()], dim=0).to(self.dtype).contiguous()
        wo = lw.wo.float().view(hid, H, self.vdim)
        lw.w_oa = torch.einsum("ohv,hvc->ohc", wo, lw.w_uv.float()).reshape(hid, H * self.lora).to(self.dtype).contiguous()
        # the factored weights are not used again on this device
        lw.wq = lw.w_uk = lw.w_uv = lw.wo = lw.w_kv_a = None

    def _attention_absorbed(self, lw: DsLayer, x: torch.Tensor, positions, slots, meta: ops.AttnMeta, cache: torch.Tensor) -> torch.Tensor:
        """CUDA path: returns the attention block's output in hidden space (output projection included)."""
        if lw.w_qa is None:
            self._absorb(lw)
        T, H = x.shape[0], self.H
        n_lat, n_rope = H * self.lora, H * self.rope
        qa = ops.linear(x, lw.w_qa)                                   # [T, q_lat | q_rope | c_kv | k_rope]
        q_rope = qa[:, n_lat:n_lat + n_rope]
        kv_a = qa[:, n_lat + n_rope:]
        c_kv, _ = ops.rms_norm(kv_a[:, :self.lora].contiguous(), lw.kv_a_norm, self.cfg.rms_norm_eps)
        k_rope = kv_a[:, self.lora:].contiguous()
        ops.rope_kvwrite(q_rope, k_rope, None, self.cos_sin, positions, None, None, None, self.rope, interleaved=self.cfg.rope_interleaved)
        # latent cache row = [c_kv | k_rope]; slots < 0 (graph padding) are skipped by the scatter
        ops.scatter_rows(torch.cat([c_kv, k_rope], dim=1), slots, cache.view(-1, cache.shape[2]))
        o_lat = ops.mla_attend(qa[:, :n_lat].unflatten(1, (H, self.lora)), q_rope.unflatten(1, (H, self.rope)), cache, meta, self.scale)
        return ops.linear(o_lat.view(T, n_lat), lw.w_oa)

    def _attention(self, lw: DsLayer, x: torch.Tensor, positions, slots, meta: ops.AttnMeta, cache: torch.Tensor) -> torch.Tensor:
        T, H = x.shape[0], self.H
        q = ops.linear(x, lw.wq).view(T, H, self.nope + self.rope)
        kv_a = ops.linear(x, lw.w_kv_a)
        c_kv, _ = ops.rms_norm(kv_a[:, :self.lora].contiguous(), lw.kv_a_norm, self.cfg.rms_norm_eps)
        k_rope = kv_a[:, self.lora:].contiguous()
        q_rope = q[:, :, self.nope:].reshape(T, H * self.rope).contiguous()
        ops.rope_kvwrite(q_rope, k_rope, None, self.cos_sin, positions, None, None, None, self.rope, interleaved=self.cfg.rope_interleaved)
        # latent cache row = [c_kv | k_rope]; slots < 0 (graph padding) are skipped by the scatter
        ops.scatter_rows(torch.cat([c_kv, k_rope], dim=1), slots, cache.view(-1, cache.shape[2]))
        q_nope = q[:, :, :self.nope]
        q_rope = q_rope.view(T, H, self.rope)
        out = torch.empty(T, H * self.vdim, dtype=x.dtype, device=x.device)
        nd = meta.num_decode
        if nd > 0:
            # absorbed decode: q_lat[h] = q_nope[h] W_UK[h]; o[h] = o_lat[h] W_UV[h]^T
            q_lat = torch.einsum("thd,hdc->thc", q_nope[:nd].float(), lw.w_uk.float()).to(x.dtype).contiguous()
            o_lat = ops.mla_decode(q_lat, q_rope[:nd].contiguous(), cache, meta.ctx_lens[:nd], meta.block_tables[:nd], self.scale,
                                   meta.max_ctx)
            o = torch.einsum("thc,hvc->thv", o_lat.float(), lw.w_uv.float()).to(x.dtype)
            out[:nd] = o.reshape(nd, H * self.vdim)
        if meta.num_seqs > nd:
            out[nd:] = self._prefill_rows(lw, q_nope, q_rope, meta, cache, nd)
        return out

    def _prefill_rows(self, lw, q_nope, q_rope, meta, cache, nd) -> torch.Tensor:
        """Non-absorbed causal attention for the prefill chunks: expand each sequence's latents to per-head K/V."""
        H, dq = self.H, self.nope + self.rope
        cu = meta.cu_q.tolist() if not isinstance(meta.cu_q, list) else meta.cu_q
        ctx = meta.ctx_lens.tolist()
        outs = []
        page_size = cache.shape[1]
        for b in range(nd, meta.num_seqs):
            s, e, c = cu[b], cu[b + 1], ctx[b]
            n_pages = (c + page_size - 1) // page_size
            lat = cache[meta.block_tables[b, :n_pages].long()].reshape(n_pages * page_size, -1)[:c]
            c_kv, k_r = lat[:, :self.lora], lat[:, self.lora:]
            k_nope = torch.einsum("tc,hdc->thd", c_kv.float(), lw.w_uk.float())
            v = torch.einsum("tc,hvc->thv", c_kv.float(), lw.w_uv.float())
            k = torch.cat([k_nope, k_r.float().unsqueeze(1).expand(c, H, self.rope)], dim=2)
            qq = torch.cat([q_nope[s:e].float(), q_rope[s:e].float()], dim=2)
            sc = torch.einsum("qhd,khd->hqk", qq, k) * self.scale
            qpos = torch.arange(c - (e - s), c, device=lat.device).unsqueeze(1)
            kpos = torch.arange(c, device=lat.device).unsqueeze(0)
            sc = sc.masked_fill(~(kpos <= qpos).unsqueeze(0), float("-inf"))
            o = torch.einsum("hqk,khv->qhv", torch.softmax(sc, dim=-1), v)
            outs.append(o.reshape(e - s, H * self.vdim).to(q_nope.dtype))
        return torch.cat(outs, dim=0)

    def _moe(self, lw: DsLayer, x: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        logits = ops.linear(x, lw.w_router)
        shared = None
        if lw.w_shared_gu is not None:
            shared = ops.linear(ops.linear_swiglu(x, lw.w_shared_gu), lw.w_shared_down)
        if self.ep is not None:
            # fused path: router + dispatch, grouped GEMMs, combine (+ shared) in the expert-parallel kernels
            return self.ep.moe(x, logits, lw.w_exp_gu_il, lw.w_exp_down, shared, cfg.norm_topk_prob, cfg.routed_scaling_factor)
        weights, ids = reference.moe_route(logits, cfg.num_experts_per_tok, cfg.norm_topk_prob, cfg.routed_scaling_factor)
        if x.is_cuda:
            from ..parallel.ep import local_moe

            routed = local_moe(x, weights, ids, lw.w_exp_gu, lw.w_exp_down)
        else:
            routed = reference.moe_forward(x, lw.w_exp_gu, lw.w_exp_down, weights, ids).to(x.dtype)
        return routed + shared if shared is not None else routed

    def forward_idle(self) -> None:
        """A step without tokens on this rank. With data-parallel attention and expert-parallel MoE every rank must
        still take part in each MoE layer's dispatch / combine, so that peers' tokens routed to this rank's experts
        are computed and returned."""
        if self.ep is None or self.ep_size == 1:
            return
        cfg = self.cfg
        x = torch.empty(0, cfg.hidden_size, dtype=self.dtype, device=self.device)
        logits = torch.empty(0, cfg.n_routed_experts, dtype=self.dtype, device=self.device)
        for lw in self.layers:
            if lw.w_gu is None:
                self.ep.moe(x, logits, lw.w_exp_gu_il, lw.w_exp_down, None, cfg.norm_topk_prob, cfg.routed_scaling_factor)

    def forward(self, token_ids, positions, slots, meta: ops.AttnMeta, kv_caches, sample_rows, greedy: bool = False):
        cfg = self.cfg
        h = ops.embedding(token_ids, self.embed)
        residual = None
        for li, lw in enumerate(self.layers):
            x, residual = ops.rms_norm(h, lw.attn_norm, cfg.rms_norm_eps, residual)
            if x.is_cuda and self.lora == 512 and self.rope == 64:
                h = self._attention_absorbed(lw, x, positions, slots, meta, kv_caches[li])
            else:
                h = ops.linear(self._attention(lw, x, positions, slots, meta, kv_caches[li]), lw.wo)
            x, residual = ops.rms_norm(h, lw.mlp_norm, cfg.rms_norm_eps, residual)
            if lw.w_gu is not None:
                h = ops.linear(ops.linear_swiglu(x, lw.w_gu), lw.w_down)
            else:
                h = self._moe(lw, x)
        x, _ = ops.rms_norm(h, self.final_norm, cfg.rms_norm_eps, residual)
        if sample_rows is not None:
            x = ops.gather_rows(x, sample_rows)
        return ops.linear(x, self.lm_head)
