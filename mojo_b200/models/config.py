"""Architecture descriptions. Field names follow the Hugging Face `config.json` keys so a checkpoint directory
can be read directly; named presets cover the architectures the engine is benchmarked on."""
from __future__ import annotations

import json
from dataclasses import dataclass, field, asdict
from pathlib import Path


@dataclass
class ModelConfig:
    architecture: str = "llama"            # "llama" | "deepseek_v2"
    hidden_size: int = 4096
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 14336
    vocab_size: int = 128256
    rms_norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    rope_scaling: dict | None = None
    max_position_embeddings: int = 8192
    tie_word_embeddings: bool = False
    # quantisation of the linear weights: None | "fp8_block" (128x128 e4m3 + f32 scales) | "gguf"
    quantization: str | None = None
    # DeepSeek-V2 (MLA + MoE)
    kv_lora_rank: int = 0
    q_lora_rank: int = 0
    qk_rope_head_dim: int = 0
    qk_nope_head_dim: int = 0
    v_head_dim: int = 0
    n_routed_experts: int = 0
    n_shared_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    first_k_dense_replace: int = 0
    routed_scaling_factor: float = 1.0
    norm_topk_prob: bool = False
    rope_interleaved: bool = False
    extra: dict = field(default_factory=dict)

    def to_dict(self) -> dict:
        return asdict(self)

    @property
    def is_mla(self) -> bool:
        return self.kv_lora_rank > 0

    @property
    def is_moe(self) -> bool:
        return self.n_routed_experts > 0

    def kv_bytes_per_token(self, dtype_bytes: int = 2, tp: int = 1) -> int:
        if self.is_mla:
            return self.num_layers * (self.kv_lora_rank + self.qk_rope_head_dim) * dtype_bytes
        return self.num_layers * 2 * max(1, self.num_kv_heads // tp) * self.head_dim * dtype_bytes

    def num_params(self) -> int:
        h = self.hidden_size
        emb = self.vocab_size * h * (1 if self.tie_word_embeddings else 2)
        if self.architecture == "llama":
            attn = h * (self.num_heads + 2 * self.num_kv_heads) * self.head_dim + self.num_heads * self.head_dim * h
            mlp = 3 * h * self.intermediate_size
            return emb + self.num_layers * (attn + mlp + 2 * h) + h
        attn = h * self.num_heads * (self.qk_nope_head_dim + self.qk_rope_head_dim) + h * (self.kv_lora_rank + self.qk_rope_head_dim) \
            + self.kv_lora_rank * self.num_heads * (self.qk_nope_head_dim + self.v_head_dim) + self.num_heads * self.v_head_dim * h
        dense = 3 * h * self.intermediate_size
        moe = 3 * h * self.moe_intermediate_size * (self.n_routed_experts + self.n_shared_experts) + h * self.n_routed_experts
        nd = self.first_k_dense_replace
        return emb + self.num_layers * attn + nd * dense + (self.num_layers - nd) * moe

    @staticmethod
    def from_hf(path: str | Path) -> "ModelConfig":
        cfg = json.loads((Path(path) / "config.json").read_text())
        arch = (cfg.get("architectures") or ["LlamaForCausalLM"])[0]
        n_heads = cfg["num_attention_heads"]
        c = ModelConfig(
            architecture="deepseek_v2" if "Deepseek" in arch else "llama",
            hidden_size=cfg["hidden_size"], num_layers=cfg["num_hidden_layers"], num_heads=n_heads,
            num_kv_heads=cfg.get("num_key_value_heads", n_heads),
            head_dim=cfg.get("head_dim") or cfg["hidden_size"] // n_heads,
            intermediate_size=cfg["intermediate_size"], vocab_size=cfg["vocab_size"],
            rms_norm_eps=cfg.get("rms_norm_eps", 1e-5), rope_theta=cfg.get("rope_theta", 10000.0),
            rope_scaling=cfg.get("rope_scaling"), max_position_embeddings=cfg.get("max_position_embeddings", 8192),
            tie_word_embeddings=cfg.get("tie_word_embeddings", False),
        )
        q = cfg.get("quantization_config") or {}
        if q.get("quant_method") == "fp8" and q.get("weight_block_size"):
            c.quantization = "fp8_block"
        if c.architecture == "deepseek_v2":
            c.kv_lora_rank = cfg["kv_lora_rank"]; c.q_lora_rank = cfg.get("q_lora_rank") or 0
            c.qk_rope_head_dim = cfg["qk_rope_head_dim"]; c.qk_nope_head_dim = cfg["qk_nope_head_dim"]
            c.v_head_dim = cfg["v_head_dim"]; c.n_routed_experts = cfg["n_routed_experts"]
            c.n_shared_experts = cfg.get("n_shared_experts") or 0; c.num_experts_per_tok = cfg["num_experts_per_tok"]
            c.moe_intermediate_size = cfg["moe_intermediate_size"]; c.first_k_dense_replace = cfg.get("first_k_dense_replace", 0)
            c.routed_scaling_factor = cfg.get("routed_scaling_factor", 1.0); c.norm_topk_prob = cfg.get("norm_topk_prob", False)
            c.rope_interleaved = True
        return c


def tiny_llama() -> ModelConfig:
    """The CPU plumbing/numerics configuration: 2 layers, hidden 256, 4 q / 2 kv heads of 64, FFN 688,
    vocab 32000, tied embeddings."""
    return ModelConfig(hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64, intermediate_size=688,
                       vocab_size=32000, rms_norm_eps=1e-5, rope_theta=500000.0, tie_word_embeddings=True,
                       max_position_embeddings=2048)


def llama31_8b() -> ModelConfig:
    return ModelConfig(hidden_size=4096, num_layers=32, num_heads=32, num_kv_heads=8, head_dim=128, intermediate_size=14336,
                       vocab_size=128256, rope_theta=500000.0, max_position_embeddings=8192,
                       rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                     "original_max_position_embeddings": 8192})


def llama33_70b_fp8() -> ModelConfig:
    return ModelConfig(hidden_size=8192, num_layers=80, num_heads=64, num_kv_heads=8, head_dim=128, intermediate_size=28672,
                       vocab_size=128256, rope_theta=500000.0, max_position_embeddings=8192, quantization="fp8_block",
                       rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                     "original_max_position_embeddings": 8192})


def deepseek_v2_lite() -> ModelConfig:
    return ModelConfig(architecture="deepseek_v2", hidden_size=2048, num_layers=27, num_heads=16, num_kv_heads=16, head_dim=192,
                       intermediate_size=10944, vocab_size=102400, rms_norm_eps=1e-6, rope_theta=10000.0,
                       max_position_embeddings=4096, kv_lora_rank=512, qk_rope_head_dim=64, qk_nope_head_dim=128,
                       v_head_dim=128, n_routed_experts=64, n_shared_experts=2, num_experts_per_tok=6,
                       moe_intermediate_size=1408, first_k_dense_replace=1, routed_scaling_factor=1.0, norm_topk_prob=False,
                       rope_interleaved=True)


def tiny_deepseek() -> ModelConfig:
    """Small MLA + MoE model with the DeepSeek-V2-Lite head geometry, for tests."""
    return ModelConfig(architecture="deepseek_v2", hidden_size=256, num_layers=3, num_heads=16, num_kv_heads=16, head_dim=192,
                       intermediate_size=512, vocab_size=1024, rms_norm_eps=1e-6, rope_theta=10000.0,
                       max_position_embeddings=1024, kv_lora_rank=512, qk_rope_head_dim=64, qk_nope_head_dim=128,
                       v_head_dim=128, n_routed_experts=8, n_shared_experts=2, num_experts_per_tok=2,
                       moe_intermediate_size=128, first_k_dense_replace=1, rope_interleaved=True)


PRESETS = {
    "tiny-llama": tiny_llama,
    "llama-3.1-8b": llama31_8b,
    "llama-3.3-70b-fp8": llama33_70b_fp8,
    "deepseek-v2-lite": deepseek_v2_lite,
    "tiny-deepseek": tiny_deepseek,
}


def get_config(name_or_path: str) -> ModelConfig:
    key = name_or_path.lower()
    if key in PRESETS:
        return PRESETS[key]()
    p = Path(name_or_path)
    if (p / "config.json").exists():
        return ModelConfig.from_hf(p)
    raise ValueError(f"unknown model {name_or_path!r}; presets: {sorted(PRESETS)}")
