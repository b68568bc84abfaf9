"""Model zoo: architecture configs and the decoder implementations built on `mojo_b200.ops`."""
from __future__ import annotations

import torch

from .config import ModelConfig, get_config, PRESETS  # noqa: F401


def build_model(cfg: ModelConfig, device="cpu", dtype=torch.float32, comm=None, ep=None):
    if cfg.architecture == "llama":
        from .llama import LlamaModel

        return LlamaModel(cfg, device, dtype, comm=comm)
    if cfg.architecture == "deepseek_v2":
        from .deepseek_v2 import DeepseekV2Model

        return DeepseekV2Model(cfg, device, dtype, comm=comm, ep=ep)
    raise ValueError(f"unsupported architecture {cfg.architecture!r}")
