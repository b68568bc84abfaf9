"""Serving engine: scheduler + KV cache (C++), model runner, sampling."""
from .llm_engine import EngineConfig, LLMEngine, RequestOutput, SamplingParams  # noqa: F401
