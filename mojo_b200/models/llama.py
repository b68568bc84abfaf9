"""Llama-3 family decoder (GQA, RoPE, RMSNorm, SwiGLU) on the mojo_b200 op library.

One forward pass processes a ragged batch: decode sequences (one token each) followed by prefill chunks, all
flattened to [T, H]. Keys/values go straight into the paged cache; attention reads them back through block
tables. The same code runs on CPU tensors (fp32 reference ops) and on CUDA tensors (sm_100a kernels).

Weight layout per layer (row-major [out, in], like `nn.Linear.weight`):
  wqkv   [(n_q + 2 n_kv) * D / tp, H]   q heads, then k heads, then v heads of this rank
  wo     [H, n_q * D / tp]
  w_gu   [2 F / tp, H]                  gate/up rows interleaved in blocks of 16 (SwiGLU GEMM epilogue)
  w_down [H, F / tp]
Tensor parallelism is Megatron-style: column-parallel qkv / gate-up, row-parallel o / down followed by a
reduction supplied by the `comm` object (identity at tp = 1).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .. import ops
from ..ops import reference
from .config import ModelConfig


@dataclass
class LayerWeights:
    attn_norm: torch.Tensor
    wqkv: torch.Tensor
    wo: torch.Tensor
    mlp_norm: torch.Tensor
    w_gu: torch.Tensor
    w_down: torch.Tensor
    # fp8 block-scaled checkpoints: the four matrices above are float8_e4m3fn and these hold their f32 scales
    # ([ceil(N/128), ceil(K/128)]); w_gu is then stacked gate-then-up (no interleave: scale blocks stay intact)
    s_qkv: torch.Tensor | None = None
    s_o: torch.Tensor | None = None
    s_gu: torch.Tensor | None = None
    s_down: torch.Tensor | None = None


class NoComm:
    """tp = 1: nothing to reduce."""

    world_size = 1
    rank = 0

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        return x

    def linear_all_reduce(self, x, w, residual=None):
        return ops.linear(x, w, residual)

    def linear_fp8_all_reduce(self, x, w_q, w_scale, residual=None):
        y = ops.linear_fp8(x, w_q, w_scale)
        return y if residual is None else y + residual

    def all_gather_vocab(self, logits: torch.Tensor) -> torch.Tensor:
        return logits


class LlamaModel:
    def __init__(self, cfg: ModelConfig, device: torch.device | str = "cpu", dtype: torch.dtype = torch.float32, comm=None):
        self.cfg = cfg
        self.device = torch.device(device)
        self.dtype = dtype
        self.comm = comm or NoComm()
        self.tp = self.comm.world_size
        if cfg.num_heads % self.tp != 0:
            raise ValueError(f"{cfg.num_heads} query heads do not divide by tensor-parallel degree {self.tp}")
        if cfg.intermediate_size % (16 * self.tp) != 0:
            # the SwiGLU GEMM epilogue pairs gate and up rows in blocks of 16 within each rank's shard
            raise ValueError(f"FFN width {cfg.intermediate_size} must be a multiple of 16 x tensor-parallel degree {self.tp}")
        self.n_q = cfg.num_heads // self.tp
        # kv heads are replicated when tp exceeds their number
        self.n_kv = max(1, cfg.num_kv_heads // self.tp)
        self.kv_replicas = max(1, self.tp // cfg.num_kv_heads)
        self.head_dim = cfg.head_dim
        self.ffn_local = cfg.intermediate_size // self.tp
        self.vocab_local = (cfg.vocab_size + self.tp - 1) // self.tp
        self.vocab_start = self.comm.rank * self.vocab_local
        self.scale = 1.0 / math.sqrt(cfg.head_dim)
        self.layers: list[LayerWeights] = []
        self.embed: torch.Tensor | None = None       # [V, H] (replicated)
        self.final_norm: torch.Tensor | None = None
        self.lm_head: torch.Tensor | None = None     # [V / tp, H]
        self.cos_sin = reference.rope_table(cfg.max_position_embeddings, cfg.head_dim, cfg.rope_theta, cfg.rope_scaling).to(self.device)
        # Sequence-parallel dataflow between the tensor-parallel regions (activations sharded by token): needs a
        # communicator with the fused all-gather -> GEMM and GEMM -> reduce-scatter kernels. Off by default.
        self.sequence_parallel = False

    # ------------------------------------------------------------------------------------------------
    # weights
    # ------------------------------------------------------------------------------------------------
    def init_random(self, seed: int = 0, std: float = 0.02) -> "LlamaModel":
        """Random-init N(0, std) weights of the full architecture, generated layer by layer from `seed`, then
        sharded for this rank. Every rank draws the same full tensors, so tp ranks hold consistent shards."""
        cfg = self.cfg
        g = torch.Generator(device="cpu").manual_seed(seed)
        big = cfg.hidden_size * cfg.vocab_size > (1 << 28)
        gen_dev = self.device if (big and self.device.type == "cuda") else torch.device("cpu")
        if gen_dev.type == "cuda":
            g = torch.Generator(device=gen_dev).manual_seed(seed)

        def rnd(*shape):
            return torch.randn(*shape, generator=g, device=gen_dev, dtype=torch.float32) * std

        full = {"embed": rnd(cfg.vocab_size, cfg.hidden_size)}
        self.load_tensor("embed", full["embed"])
        for i in range(cfg.num_layers):
            d, h = cfg.head_dim, cfg.hidden_size
            self.load_layer(i, dict(
                attn_norm=torch.ones(h), mlp_norm=torch.ones(h),
                wq=rnd(cfg.num_heads * d, h), wk=rnd(cfg.num_kv_heads * d, h), wv=rnd(cfg.num_kv_heads * d, h),
                wo=rnd(h, cfg.num_heads * d), w_gate=rnd(cfg.intermediate_size, h), w_up=rnd(cfg.intermediate_size, h),
                w_down=rnd(h, cfg.intermediate_size)))
        self.load_tensor("final_norm", torch.ones(cfg.hidden_size))
        if cfg.tie_word_embeddings:
            self.load_tensor("lm_head", full["embed"])
        else:
            self.load_tensor("lm_head", rnd(cfg.vocab_size, cfg.hidden_size))
        return self

    def _put(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(device=self.device, dtype=self.dtype).contiguous()

    def load_tensor(self, name: str, t: torch.Tensor) -> None:
        if name == "embed":
            self.embed = self._put(t)
        elif name == "final_norm":
            self.final_norm = self._put(t)
        elif name == "lm_head":
            v0 = self.vocab_start
            shard = t[v0:v0 + self.vocab_local]
            if shard.shape[0] < self.vocab_local:  # pad the last rank's shard
                shard = torch.cat([shard, torch.zeros(self.vocab_local - shard.shape[0], t.shape[1], dtype=t.dtype, device=t.device)])
            self.lm_head = self._put(shard)
        else:
            raise KeyError(name)

    def load_layer(self, idx: int, w: dict) -> None:
        """`w` holds the full (unsharded) HF-layout tensors of one layer; keeps this rank's shard."""
        cfg, r, tp, d = self.cfg, self.comm.rank, self.tp, self.cfg.head_dim
        q = w["wq"][r * self.n_q * d:(r + 1) * self.n_q * d]
        kv_rank = r // self.kv_replicas
        k = w["wk"][kv_rank * self.n_kv * d:(kv_rank + 1) * self.n_kv * d]
        v = w["wv"][kv_rank * self.n_kv * d:(kv_rank + 1) * self.n_kv * d]
        f = self.ffn_local
        if cfg.quantization == "fp8_block":
            self._load_layer_fp8(idx, w, q, k, v)
            return
        lw = LayerWeights(
            attn_norm=self._put(w["attn_norm"]),
            wqkv=self._put(torch.cat([q, k, v], dim=0)),
            wo=self._put(w["wo"][:, r * self.n_q * d:(r + 1) * self.n_q * d]),
            mlp_norm=self._put(w["mlp_norm"]),
            w_gu=self._put(reference.interleave_gate_up(w["w_gate"][r * f:(r + 1) * f], w["w_up"][r * f:(r + 1) * f])),
            w_down=self._put(w["w_down"][:, r * f:(r + 1) * f]),
        )
        assert idx == len(self.layers)
        self.layers.append(lw)

    def _load_layer_fp8(self, idx: int, w: dict, q, k, v) -> None:
        """Keep the four linear weights in e4m3 with one f32 scale per 128x128 block. Checkpoint scales
        (`w["scales"]`) are sliced with the weights; bf16 / random weights are quantised here."""
        r, d, f = self.comm.rank, self.cfg.head_dim, self.ffn_local
        sc = w.get("scales")

        def quant(t):
            qt, st = reference.quant_e4m3_128x128(t.to(self.device).float())
            return qt.contiguous(), st.contiguous()

        def put8(t):
            return t.to(self.device).contiguous()

        if sc is None:
            wqkv, s_qkv = quant(torch.cat([q, k, v], dim=0))
            wo, s_o = quant(w["wo"][:, r * self.n_q * d:(r + 1) * self.n_q * d])
            wgu, s_gu = quant(torch.cat([w["w_gate"][r * f:(r + 1) * f], w["w_up"][r * f:(r + 1) * f]], dim=0))
            wdn, s_dn = quant(w["w_down"][:, r * f:(r + 1) * f])
        else:
            def rows(name, lo, hi):
                return w[name][lo:hi], sc[name][lo // 128:(hi + 127) // 128]

            def cols(name, lo, hi):
                return w[name][:, lo:hi], sc[name][:, lo // 128:(hi + 127) // 128]

            kv_rank = r // self.kv_replicas
            parts = [rows("wq", r * self.n_q * d, (r + 1) * self.n_q * d), rows("wk", kv_rank * self.n_kv * d, (kv_rank + 1) * self.n_kv * d),
                     rows("wv", kv_rank * self.n_kv * d, (kv_rank + 1) * self.n_kv * d)]
            wqkv, s_qkv = put8(torch.cat([p[0] for p in parts])), put8(torch.cat([p[1] for p in parts]).float())
            wo, s_o = (put8(t) for t in cols("wo", r * self.n_q * d, (r + 1) * self.n_q * d))
            g, u = rows("w_gate", r * f, (r + 1) * f), rows("w_up", r * f, (r + 1) * f)
            wgu, s_gu = put8(torch.cat([g[0], u[0]])), put8(torch.cat([g[1], u[1]]).float())
            wdn, s_dn = (put8(t) for t in cols("w_down", r * f, (r + 1) * f))
        lw = LayerWeights(attn_norm=self._put(w["attn_norm"]), wqkv=wqkv, wo=wo, mlp_norm=self._put(w["mlp_norm"]), w_gu=wgu, w_down=wdn,
                          s_qkv=s_qkv.float(), s_o=s_o.float(), s_gu=s_gu.float(), s_down=s_dn.float())
        assert idx == len(self.layers)
        self.layers.append(lw)

    def weight_bytes(self) -> int:
        n = sum(t.numel() * t.element_size() for lw in self.layers for t in vars(lw).values() if t is not None)
        for t in (self.embed, self.final_norm, self.lm_head):
            if t is not None:
                n += t.numel() * t.element_size()
        return n

    # ------------------------------------------------------------------------------------------------
    # KV cache
    # ------------------------------------------------------------------------------------------------
    def allocate_kv_cache(self, num_pages: int, page_size: int):
        from ..utils import guard

        shape = (num_pages, self.n_kv, page_size, self.head_dim)
        return [(guard.zeros(shape, self.dtype, self.device, f"K cache, layer {i}"), guard.zeros(shape, self.dtype, self.device, f"V cache, layer {i}"))
                for i in range(self.cfg.num_layers)]

    def kv_bytes_per_page(self, page_size: int) -> int:
        esz = torch.empty((), dtype=self.dtype).element_size()
        return self.cfg.num_layers * 2 * self.n_kv * page_size * self.head_dim * esz

    # ------------------------------------------------------------------------------------------------
    # forward
    # ------------------------------------------------------------------------------------------------
    def forward(self, token_ids: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, meta: ops.AttnMeta,
                kv_caches, sample_rows: torch.Tensor | None, greedy: bool = False) -> torch.Tensor:
        """Returns logits [len(sample_rows), vocab] (fp32 on CPU, bf16 on CUDA). With sample_rows None, logits
        for every token are returned. `greedy=True` on a model whose `greedy_in_forward` is set returns int64
        token ids instead (arg-max merged across the vocabulary shards without gathering the logits)."""
        cfg, d = self.cfg, self.head_dim
        q_cols, kv_cols = self.n_q * d, self.n_kv * d
        if self.sequence_parallel and self.tp > 1 and hasattr(self.comm, "all_gather_linear"):
            return self._forward_sp(token_ids, positions, slots, meta, kv_caches, sample_rows, greedy)
        h = ops.embedding(token_ids, self.embed)
        residual = None
        if cfg.quantization == "fp8_block":
            return self._forward_fp8(h, positions, slots, meta, kv_caches, sample_rows, greedy)
        fuse_norm = hasattr(self.comm, "linear_all_reduce_norm") and self.tp > 1
        x = None   # normed input of the next block when the previous all-reduce kernel already produced it
        for li, lw in enumerate(self.layers):
            if x is None:
                x, residual = ops.rms_norm(h, lw.attn_norm, cfg.rms_norm_eps, residual)
            qkv = ops.linear(x, lw.wqkv)
            q, k, v = qkv[:, :q_cols], qkv[:, q_cols:q_cols + kv_cols], qkv[:, q_cols + kv_cols:]
            kc, vc = kv_caches[li]
            ops.rope_kvwrite(q, k, v, self.cos_sin, positions, slots, kc, vc, d)
            attn = ops.paged_attention(q, kc, vc, meta, self.scale, d)
            if fuse_norm:
                # all-reduce + residual add + the MLP norm in one kernel after the GEMM (decode-sized token counts)
                x, residual = self.comm.linear_all_reduce_norm(attn, lw.wo, lw.mlp_norm, cfg.rms_norm_eps, residual)
            else:
                h = self.comm.linear_all_reduce(attn, lw.wo)
                x, residual = ops.rms_norm(h, lw.mlp_norm, cfg.rms_norm_eps, residual)
            act = ops.linear_swiglu(x, lw.w_gu)
            if fuse_norm:
                next_norm = self.layers[li + 1].attn_norm if li + 1 < len(self.layers) else self.final_norm
                x, residual = self.comm.linear_all_reduce_norm(act, lw.w_down, next_norm, cfg.rms_norm_eps, residual)
            else:
                h = self.comm.linear_all_reduce(act, lw.w_down)
                x = None
        if fuse_norm and self.layers:
            return self._head(None, residual, sample_rows, greedy, normed=x)
        return self._head(h, residual, sample_rows, greedy)

    def _forward_sp(self, token_ids, positions, slots, meta, kv_caches, sample_rows, greedy=False):
        """Sequence-parallel layer structure: the residual stream and the norms live on T / tp token rows per rank;
        every column-parallel GEMM is `all-gather -> GEMM` in one kernel and every row-parallel GEMM is
        `GEMM -> reduce-scatter` in one kernel, in bf16 or block-scaled fp8. Tokens are padded to a multiple of tp
        (padding rows carry slot -1 and feed nothing that is read)."""
        cfg, d, comm = self.cfg, self.head_dim, self.comm
        tp, rank, H = self.tp, comm.rank, cfg.hidden_size
        q_cols, kv_cols = self.n_q * d, self.n_kv * d
        fp8 = cfg.quantization == "fp8_block"
        T = token_ids.shape[0]
        Tp = (T + tp - 1) // tp * tp
        r = Tp // tp
        if Tp != T:
            pad = Tp - T
            token_ids = torch.nn.functional.pad(token_ids, (0, pad))
            positions = torch.nn.functional.pad(positions, (0, pad))
            slots = torch.nn.functional.pad(slots, (0, pad), value=-1)
        h = ops.embedding(token_ids[rank * r:(rank + 1) * r], self.embed)
        residual = None

        def norm_gather_linear(h, residual, norm_w, w, w_scale):
            if fp8:
                qv, sv = comm.gather_input_fp8(Tp, H)
                _, _, _, residual = ops.rms_norm_quant(h, norm_w, cfg.rms_norm_eps, residual, out_q=qv, out_s=sv)
                return comm.all_gather_linear_fp8(w, w_scale, Tp), residual
            _, residual = ops.rms_norm(h, norm_w, cfg.rms_norm_eps, residual, out=comm.gather_input(Tp, H))
            return comm.all_gather_linear(w, Tp), residual

        for li, lw in enumerate(self.layers):
            qkv, residual = norm_gather_linear(h, residual, lw.attn_norm, lw.wqkv, getattr(lw, "s_qkv", None))
            q, k, v = qkv[:, :q_cols], qkv[:, q_cols:q_cols + kv_cols], qkv[:, q_cols + kv_cols:]
            kc, vc = kv_caches[li]
            ops.rope_kvwrite(q, k, v, self.cos_sin, positions, slots, kc, vc, d)
            attn = ops.paged_attention(q[:T], kc, vc, meta, self.scale, d)
            if Tp != T:
                attn = torch.nn.functional.pad(attn, (0, 0, 0, Tp - T))
            h = comm.linear_fp8_reduce_scatter(attn, lw.wo, lw.s_o) if fp8 else comm.linear_reduce_scatter(attn, lw.wo)
            gu, residual = norm_gather_linear(h, residual, lw.mlp_norm, lw.w_gu, getattr(lw, "s_gu", None))
            act = ops.swiglu(gu, interleaved=not fp8)   # bf16 gate/up weights are stacked for the SwiGLU GEMM epilogue
            h = comm.linear_fp8_reduce_scatter(act, lw.w_down, lw.s_down) if fp8 else comm.linear_reduce_scatter(act, lw.w_down)
        if sample_rows is not None and sample_rows.numel() == 0:
            return self._no_rows(greedy)
        # final norm on the local rows, then gather the hidden states for the LM head
        ops.rms_norm(h, self.final_norm, cfg.rms_norm_eps, residual, out=comm.gather_input(Tp, H))
        x = comm.all_gather_rows(Tp, H)[:T]
        if sample_rows is not None:
            x = ops.gather_rows(x, sample_rows)
        logits = ops.linear(x, self.lm_head)
        if greedy and self.greedy_in_forward:
            valid = max(1, min(self.vocab_local, cfg.vocab_size - self.vocab_start))
            return comm.vocab_argmax(logits[:, :valid], self.vocab_local)
        return comm.all_gather_vocab(logits)[:, :cfg.vocab_size]

    def gemm_shapes(self) -> list[tuple[int, int, int, int]]:
        """(N, K, epilogue, max tokens or 0) of every weight that goes through `ops.linear` / `ops.linear_swiglu` on
        this rank, for the measured GEMM configuration tables (the row-parallel weights too: under tensor
        parallelism they run either in the fused GEMM+all-reduce kernel or as plain GEMM -> all-reduce kernel)."""
        if self.cfg.quantization == "fp8_block" or not self.layers:
            return []
        lw = self.layers[0]
        shapes = [(lw.wqkv.shape[0], lw.wqkv.shape[1], ops.EPI_NONE, 0), (lw.w_gu.shape[0], lw.w_gu.shape[1], ops.EPI_SWIGLU, 0),
                  (self.lm_head.shape[0], self.lm_head.shape[1], ops.EPI_NONE, 256),
                  (lw.wo.shape[0], lw.wo.shape[1], ops.EPI_NONE, 0), (lw.w_down.shape[0], lw.w_down.shape[1], ops.EPI_NONE, 0)]
        return shapes

    def row_parallel_shapes(self) -> list[tuple[int, int]]:
        """(N, K per rank) of the row-parallel bf16 linears (attention output, FFN down) under tensor parallelism."""
        if self.tp == 1 or self.cfg.quantization == "fp8_block" or not self.layers:
            return []
        lw = self.layers[0]
        return [(lw.wo.shape[0], lw.wo.shape[1]), (lw.w_down.shape[0], lw.w_down.shape[1])]

    def _head(self, h, residual, sample_rows, greedy: bool, normed: torch.Tensor | None = None):
        """Final norm (unless `normed` already holds it), row gather and the vocabulary-parallel LM head. `greedy`
        on a tensor-parallel communicator that can merge arg-maxes returns int64 token ids instead of gathered logits."""
        cfg = self.cfg
        if sample_rows is not None and sample_rows.numel() == 0:
            return self._no_rows(greedy)
        x = normed if normed is not None else ops.rms_norm(h, self.final_norm, cfg.rms_norm_eps, residual)[0]
        if sample_rows is not None:
            x = ops.gather_rows(x, sample_rows)
        logits = ops.linear(x, self.lm_head)
        if greedy and self.greedy_in_forward:
            valid = max(1, min(self.vocab_local, cfg.vocab_size - self.vocab_start))
            return self.comm.vocab_argmax(logits[:, :valid], self.vocab_local)
        return self.comm.all_gather_vocab(logits)[:, :cfg.vocab_size]

    def supports_static_attention(self, page_size: int) -> bool:
        """Whether a whole step of this model (decode rows and prefill chunks together) can run with fixed launch
        shapes, i.e. inside a CUDA graph: needs the prefill kernel that takes a device-side work list (head dim 128,
        128-token pages) and the token-replicated dataflow (the sequence-parallel one pads and slices per step)."""
        return (self.device.type == "cuda" and not self.sequence_parallel and ops.prefill_on_tensor_core(self.head_dim, page_size))

    def _no_rows(self, greedy: bool) -> torch.Tensor:
        """Result of a step that samples nothing (only chunks from the middle of prompts): the layers ran for their
        KV writes, the LM head and its collective are skipped."""
        if greedy and self.greedy_in_forward:
            return torch.empty(0, dtype=torch.int64, device=self.device)
        return torch.empty(0, self.cfg.vocab_size, dtype=self.dtype, device=self.device)

    @property
    def greedy_in_forward(self) -> bool:
        return self.tp > 1 and hasattr(self.comm, "vocab_argmax")

    def _forward_fp8(self, h, positions, slots, meta, kv_caches, sample_rows, greedy=False):
        """Same layer structure with block-scaled fp8 linears: RMSNorm emits the e4m3 row + per-128 scales for the
        column-parallel GEMMs; attention output and the SwiGLU activation are quantised by a small kernel."""
        cfg, d = self.cfg, self.head_dim
        q_cols, kv_cols = self.n_q * d, self.n_kv * d
        residual = None
        for li, lw in enumerate(self.layers):
            _, xq, xs, residual = ops.rms_norm_quant(h, lw.attn_norm, cfg.rms_norm_eps, residual)
            qkv = ops.linear_fp8((xq, xs), lw.wqkv, lw.s_qkv)
            q, k, v = qkv[:, :q_cols], qkv[:, q_cols:q_cols + kv_cols], qkv[:, q_cols + kv_cols:]
            kc, vc = kv_caches[li]
            ops.rope_kvwrite(q, k, v, self.cos_sin, positions, slots, kc, vc, d)
            attn = ops.paged_attention(q, kc, vc, meta, self.scale, d)
            h = self.comm.linear_fp8_all_reduce(attn, lw.wo, lw.s_o)
            _, xq, xs, residual = ops.rms_norm_quant(h, lw.mlp_norm, cfg.rms_norm_eps, residual)
            act = ops.swiglu(ops.linear_fp8((xq, xs), lw.w_gu, lw.s_gu))
            h = self.comm.linear_fp8_all_reduce(act, lw.w_down, lw.s_down)
        return self._head(h, residual, sample_rows, greedy)
