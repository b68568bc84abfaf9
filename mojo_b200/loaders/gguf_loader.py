"""GGUF checkpoints. Metadata and tensor directory are parsed with the `gguf` package; tensor payloads stay
memory-mapped. Q4_K / Q6_K tensors are uploaded as raw super-blocks and consumed by the dequant-fused GEMM
(`ops.linear_gguf`); F32 / F16 / BF16 tensors are converted to the model dtype."""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

from .. import ops

_LLAMA_MAP = {
    "token_embd.weight": "embed", "output_norm.weight": "final_norm", "output.weight": "lm_head",
}
_LAYER_MAP = {
    "attn_norm.weight": "attn_norm", "ffn_norm.weight": "mlp_norm", "attn_q.weight": "wq", "attn_k.weight": "wk",
    "attn_v.weight": "wv", "attn_output.weight": "wo", "ffn_gate.weight": "w_gate", "ffn_up.weight": "w_up",
    "ffn_down.weight": "w_down",
}


class GGUFFile:
    def __init__(self, path: str | Path):
        from gguf import GGUFReader

        self.reader = GGUFReader(str(path))
        self.tensors = {t.name: t for t in self.reader.tensors}

    def metadata(self) -> dict:
        out = {}
        for k, f in self.reader.fields.items():
            try:
                out[k] = f.contents()
            except Exception:  # noqa: BLE001
                pass
        return out

    def tensor(self, name: str):
        """Returns (kind, payload, shape): kind 'q' -> (ggml_type, uint8 tensor of raw blocks); kind 'f' -> float tensor."""
        t = self.tensors[name]
        shape = tuple(int(x) for x in reversed(t.shape))  # gguf stores dims innermost-first
        ty = int(t.tensor_type)
        if ty in (ops.GGML_Q4_K, ops.GGML_Q6_K):
            return "q", (ty, torch.from_numpy(np.ascontiguousarray(t.data).reshape(-1).view(np.uint8))), shape
        arr = np.asarray(t.data)
        if arr.dtype == np.uint16:  # bf16 payload
            return "f", torch.from_numpy(arr.astype(np.int32) << 16).view(torch.float32).reshape(shape), shape
        return "f", torch.from_numpy(np.ascontiguousarray(arr, dtype=np.float32)).reshape(shape), shape


def load_gguf_into(model, path: str | Path, dequantize: bool = True) -> None:
    """Fill a Llama-family model from a GGUF file. With `dequantize`, k-quant tensors are expanded to the model dtype
    at load time (on the device when it is a GPU); otherwise they are kept packed in `model.gguf_weights`."""
    gf = GGUFFile(path)
    cfg = model.cfg
    model.layers.clear()
    model.gguf_weights = {}

    def get(name: str) -> torch.Tensor:
        kind, payload, shape = gf.tensor(name)
        if kind == "f":
            return payload
        ty, raw = payload
        if not dequantize:
            model.gguf_weights[name] = (ty, raw.to(model.device), shape)
        return ops.gguf_dequant(raw.to(model.device) if model.device.type == "cuda" else raw, ty, shape).float().cpu()

    model.load_tensor("embed", get("token_embd.weight"))
    for i in range(cfg.num_layers):
        w = {short: get(f"blk.{i}.{g}") for g, short in _LAYER_MAP.items()}
        model.load_layer(i, w)
    model.load_tensor("final_norm", get("output_norm.weight"))
    model.load_tensor("lm_head", get("output.weight" if "output.weight" in gf.tensors else "token_embd.weight"))
