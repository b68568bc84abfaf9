"""mojo_b200: a Blackwell-native (sm_100a) LLM inference engine.

Layers, bottom up: `csrc/` (CUDA kernels + C++ engine runtime), `ops` (Python entry points with a CPU fp32
reference for every op), `parallel` (tensor/expert parallel groups and symmetric memory), `models`
(Llama-3, DeepSeek-V2-Lite), `loaders` (safetensors, fp8 block-scaled, GGUF), `engine` (paged KV cache,
continuous-batching scheduler, model runner), `pipelines` (`PipelineConfig`, `LLM`), `serve`
(OpenAI-compatible HTTP server) and `cli`.
"""
__version__ = "0.1.0"

from . import _ext  # noqa: F401
