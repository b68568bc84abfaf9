"""PipelineConfig: one dataclass that round-trips through CLI flags and JSON, echoed into every benchmark result.
(Three-tier configuration like the reference's: compile-time `-D` macros in `csrc/include/b2/config.h`, `B2_*`
environment variables for assert / trace / timeout knobs, and this run-time object.)"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, fields


@dataclass
class PipelineConfig:
    model: str = "tiny-llama"             # preset name, HF checkpoint directory, or .gguf file
    random_init: bool = False             # random N(0, 0.02) weights of the named architecture
    dtype: str = "bfloat16"               # compute dtype on CUDA; CPU always runs fp32
    quantization: str | None = None       # None | "fp8_block" | "gguf"
    device: str | None = None             # default: cuda if available
    tensor_parallel: int = 1
    expert_parallel: int = 1
    data_parallel: int = 1                # independent replicas, one per rank, behind one endpoint (`cli serve`)
    page_size: int = 128
    max_num_seqs: int = 256
    max_num_batched_tokens: int = 4096
    max_model_len: int = 4096
    gpu_memory_utilization: float = 0.9
    num_pages: int | None = None
    enable_prefix_cache: bool = False
    enable_chunked_prefill: bool = True
    use_cuda_graphs: bool = True
    seed: int = 0
    tokenizer: str | None = None          # HF tokenizer directory; None -> token-id passthrough
    eos_token_id: int | None = None

    def to_json(self) -> str:
        return json.dumps(asdict(self), indent=1)

    @staticmethod
    def from_json(s: str) -> "PipelineConfig":
        return PipelineConfig(**json.loads(s))

    @staticmethod
    def add_cli_args(ap) -> None:
        for f in fields(PipelineConfig):
            name = "--" + f.name.replace("_", "-")
            if f.type in ("bool", bool):
                ap.add_argument(name, action="store_true" if not f.default else "store_false", dest=f.name, default=f.default)
            elif f.name in ("tensor_parallel", "expert_parallel", "data_parallel", "page_size", "max_num_seqs", "max_num_batched_tokens", "max_model_len", "seed"):
                ap.add_argument(name, type=int, default=f.default, dest=f.name)
            elif f.name in ("num_pages", "eos_token_id"):
                ap.add_argument(name, type=int, default=None, dest=f.name)
            elif f.name == "gpu_memory_utilization":
                ap.add_argument(name, type=float, default=f.default, dest=f.name)
            else:
                ap.add_argument(name, default=f.default, dest=f.name)

    @staticmethod
    def from_args(ns) -> "PipelineConfig":
        return PipelineConfig(**{f.name: getattr(ns, f.name) for f in fields(PipelineConfig) if hasattr(ns, f.name)})
