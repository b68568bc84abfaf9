"""Hugging Face safetensors checkpoints -> model shards.

Files are memory-mapped by the C++ runtime (`SafetensorsFile`: header parser, read-only mapping, tensors handed out
as views of the mapping with no copy; whole-tensor reads go through the worker pool, to device memory through
pinned staging buffers). Tensors are read one layer at a time, sliced for this rank's tensor-parallel shard and
copied to the device; nothing bigger than one layer is ever held on the host. This is the product's counterpart of
the reference's buffered file layer (stdlib/src/builtin/file.mojo:71-498).

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
    from .. import _ext

    C = _ext.require()
    out = {}
    for f in sorted(path.glob("*.safetensors")):
        for k in C.SafetensorsFile(str(f)).keys():
            out[k] = f
    if not out:
        raise FileNotFoundError(f"no safetensors files under {path}")
    return out


class _Reader:
    def __init__(self, index: dict[str, Path]):
        self.index = index
        self._open: dict[Path, object] = {}

    def _file(self, name: str):
        from .. import _ext

        f = self.index[name]
        h = self._open.get(f)
        if h is None:
            h = _ext.require().SafetensorsFile(str(f))
            self._open[f] = h
        return h

    def get(self, name: str) -> torch.Tensor:
        """The tensor as a read-only view of the file mapping (no copy): slice it, then move the slice."""
        return self._file(name).get(name)

    def read_into(self, name: str, dst: torch.Tensor) -> None:
        """Whole tensor straight into `dst` (host: parallel copy; device: through pinned staging)."""
        self._file(name).read_into(name, dst)

    def has(self, name: str) -> bool:
        return name in self.index


def load_safetensors_into(model, path: str | Path) -> None:
    """Fill a model from a Hugging Face checkpoint directory: Llama family, or DeepSeek-V2(-Lite) (MLA + MoE)."""
    rd = _Reader(read_safetensors_index(path))
    cfg = model.cfg
    if getattr(cfg, "architecture", "llama") == "deepseek_v2":
        _load_deepseek_v2(model, rd)
        return
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


def _load_deepseek_v2(model, rd: _Reader) -> None:
    """HF `DeepseekV2ForCausalLM` names -> `DeepseekV2Model` layers. Each rank reads only its slice of the routed
    experts (expert parallelism shards at load); `kv_b_proj` [H * (nope + v), kv_lora] is split into the per-head
    up-projections W_UK and W_UV that the model folds into its query / output weights on CUDA."""
    from ..models.deepseek_v2 import DsLayer
    from ..ops import reference

    cfg = model.cfg
    if rd.has("model.layers.0.self_attn.q_a_proj.weight"):
        raise NotImplementedError("DeepSeek-V2 checkpoints with a low-rank query projection (q_lora_rank) are not supported; V2-Lite is")
    put = model._put
    H, nope, vdim = model.H, model.nope, model.vdim
    model.layers.clear()
    model.embed = put(rd.get("model.embed_tokens.weight"))
    e0 = model.ep_rank * model.e_local
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        kv_b = rd.get(p + "self_attn.kv_b_proj.weight").view(H, nope + vdim, model.lora)
        lw = DsLayer(
            attn_norm=put(rd.get(p + "input_layernorm.weight")), wq=put(rd.get(p + "self_attn.q_proj.weight")),
            w_kv_a=put(rd.get(p + "self_attn.kv_a_proj_with_mqa.weight")), kv_a_norm=put(rd.get(p + "self_attn.kv_a_layernorm.weight")),
            w_uk=put(kv_b[:, :nope]), w_uv=put(kv_b[:, nope:]), wo=put(rd.get(p + "self_attn.o_proj.weight")),
            mlp_norm=put(rd.get(p + "post_attention_layernorm.weight")))
        if rd.has(p + "mlp.gate_proj.weight"):
            lw.w_gu = put(reference.interleave_gate_up(rd.get(p + "mlp.gate_proj.weight"), rd.get(p + "mlp.up_proj.weight")))
            lw.w_down = put(rd.get(p + "mlp.down_proj.weight"))
        else:
            lw.w_router = put(rd.get(p + "mlp.gate.weight"))
            if rd.has(p + "mlp.shared_experts.gate_proj.weight"):
                lw.w_shared_gu = put(reference.interleave_gate_up(rd.get(p + "mlp.shared_experts.gate_proj.weight"),
                                                                  rd.get(p + "mlp.shared_experts.up_proj.weight")))
                lw.w_shared_down = put(rd.get(p + "mlp.shared_experts.down_proj.weight"))
            gates, ups, downs = [], [], []
            for e in range(e0, e0 + model.e_local):
                q = f"{p}mlp.experts.{e}."
                gates.append(rd.get(q + "gate_proj.weight"))
                ups.append(rd.get(q + "up_proj.weight"))
                downs.append(rd.get(q + "down_proj.weight"))
            lw.w_exp_down = put(torch.stack(downs))
            if model.ep is not None:
                lw.w_exp_gu_il = put(torch.stack([reference.interleave_gate_up(g, u) for g, u in zip(gates, ups)]))
            else:
                lw.w_exp_gu = put(torch.stack([torch.cat([g, u], dim=0) for g, u in zip(gates, ups)]))
        model.layers.append(lw)
    model.final_norm = put(rd.get("model.norm.weight"))
    model.lm_head = put(rd.get("lm_head.weight" if rd.has("lm_head.weight") else "model.embed_tokens.weight"))
    model.finalize()


def deepseek_v2_state_dict(model) -> dict:
    """HF-named tensors of a `DeepseekV2Model` that still holds its factored weights (a CPU model, all experts local):
    the inverse of the loader, used to write test checkpoints."""
    from ..ops import reference

    out = {"model.embed_tokens.weight": model.embed, "model.norm.weight": model.final_norm, "lm_head.weight": model.lm_head}
    for i, lw in enumerate(model.layers):
        p = f"model.layers.{i}."
        out[p + "input_layernorm.weight"] = lw.attn_norm
        out[p + "post_attention_layernorm.weight"] = lw.mlp_norm
        out[p + "self_attn.q_proj.weight"] = lw.wq
        out[p + "self_attn.kv_a_proj_with_mqa.weight"] = lw.w_kv_a
        out[p + "self_attn.kv_a_layernorm.weight"] = lw.kv_a_norm
        out[p + "self_attn.kv_b_proj.weight"] = torch.cat([lw.w_uk, lw.w_uv], dim=1).reshape(-1, lw.w_uk.shape[2])
        out[p + "self_attn.o_proj.weight"] = lw.wo
        if lw.w_gu is not None:
            g, u = reference.deinterleave_gate_up(lw.w_gu)
            out[p + "mlp.gate_proj.weight"], out[p + "mlp.up_proj.weight"], out[p + "mlp.down_proj.weight"] = g, u, lw.w_down
        else:
            out[p + "mlp.gate.weight"] = lw.w_router
            if lw.w_shared_gu is not None:
                g, u = reference.deinterleave_gate_up(lw.w_shared_gu)
                out[p + "mlp.shared_experts.gate_proj.weight"], out[p + "mlp.shared_experts.up_proj.weight"] = g, u
                out[p + "mlp.shared_experts.down_proj.weight"] = lw.w_shared_down
            f = lw.w_exp_gu.shape[1] // 2
            for e in range(lw.w_exp_gu.shape[0]):
                q = f"{p}mlp.experts.{e}."
                out[q + "gate_proj.weight"], out[q + "up_proj.weight"] = lw.w_exp_gu[e, :f], lw.w_exp_gu[e, f:]
                out[q + "down_proj.weight"] = lw.w_exp_down[e]
    return out


def save_llama_safetensors(model_full: dict, path: str | Path, config: dict) -> None:
    """Write a tiny HF-layout checkpoint (used by tests and examples)."""
    from safetensors.torch import save_file

    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    save_file({k: v.contiguous() for k, v in model_full.items()}, str(path / "model.safetensors"))
    (path / "config.json").write_text(json.dumps(config))
