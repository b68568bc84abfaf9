"""Hugging Face safetensors checkpoints -> model shards.

Files are memory-mapped (`safetensors.safe_open`), tensors are read one layer at a time, sliced for this rank's
tensor-parallel shard and copied to the device; nothing bigger than one layer is ever held on the host. This is the
product's counterpart of the reference's buffered file layer (stdlib/src/builtin/file.mojo:71-498).

fp8 checkpoints in the 128x128 block-scaled format carry `<name>.weight` as float8_e4m3fn and
`<name>.weight_scale_inv` as fp32 [ceil(N/128), ceil(K/128)]; both are kept as they are for the fp8 GEMM.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch


def read_safetensors_index(path: str | Path) -> dict[str, Path]:
    """tensor name -> file, for a checkpoint directory (sharded or single-file)."""
    path = Path(path)
    idx = path / "model.safetensors.index.json"
    if idx.exists():
        wm = json.loads(idx.read_text())["weight_map"]
        return {k: path / v for k, v in wm.items()}
    from safetensors import safe_open

    out = {}
    for f in sorted(path.glob("*.safetensors")):
        with safe_open(str(f), framework="pt") as sf:
            for k in sf.keys():
                out[k] = f
    if not out:
        raise FileNotFoundError(f"no safetensors files under {path}")
    return out


class _Reader:
    def __init__(self, index: dict[str, Path]):
        self.index = index
        self._open: dict[Path, object] = {}

    def get(self, name: str) -> torch.Tensor:
        from safetensors import safe_open

        f = self.index[name]
        h = self._open.get(f)
        if h is None:
            h = safe_open(str(f), framework="pt")
            self._open[f] = h
        return h.get_tensor(name)

    def has(self, name: str) -> bool:
        return name in self.index


def load_safetensors_into(model, path: str | Path) -> None:
    """Fill a `LlamaModel` from a Hugging Face Llama-family checkpoint directory."""
    rd = _Reader(read_safetensors_index(path))
    cfg = model.cfg
    model.layers.clear()
    model.load_tensor("embed", rd.get("model.embed_tokens.weight"))
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        w = dict(
            attn_norm=rd.get(p + "input_layernorm.weight"), mlp_norm=rd.get(p + "post_attention_layernorm.weight"),
            wq=rd.get(p + "self_attn.q_proj.weight"), wk=rd.get(p + "self_attn.k_proj.weight"),
            wv=rd.get(p + "self_attn.v_proj.weight"), wo=rd.get(p + "self_attn.o_proj.weight"),
            w_gate=rd.get(p + "mlp.gate_proj.weight"), w_up=rd.get(p + "mlp.up_proj.weight"),
            w_down=rd.get(p + "mlp.down_proj.weight"))
        scales = {}
        for short, hf in (("wq", "self_attn.q_proj"), ("wk", "self_attn.k_proj"), ("wv", "self_attn.v_proj"), ("wo", "self_attn.o_proj"),
                          ("w_gate", "mlp.gate_proj"), ("w_up", "mlp.up_proj"), ("w_down", "mlp.down_proj")):
            if rd.has(p + hf + ".weight_scale_inv"):
                scales[short] = rd.get(p + hf + ".weight_scale_inv")
        if scales:
            w["scales"] = scales
        model.load_layer(i, w)
    model.load_tensor("final_norm", rd.get("model.norm.weight"))
    head = "lm_head.weight" if rd.has("lm_head.weight") else "model.embed_tokens.weight"
    model.load_tensor("lm_head", rd.get(head))


def save_llama_safetensors(model_full: dict, path: str | Path, config: dict) -> None:
    """Write a tiny HF-layout checkpoint (used by tests and examples)."""
    from safetensors.torch import save_file

    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    save_file({k: v.contiguous() for k, v in model_full.items()}, str(path / "model.safetensors"))
    (path / "config.json").write_text(json.dumps(config))
