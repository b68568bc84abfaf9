"""`max.pipelines`-style entry points: `PipelineConfig` describes what to run, `LLM` runs it.

    from mojo_b200.pipelines import LLM, PipelineConfig, SamplingParams
    llm = LLM(PipelineConfig(model="llama-3.1-8b", random_init=True))
    outs = llm.generate([[1, 2, 3, 4]], SamplingParams(max_tokens=16))
"""
from .config import PipelineConfig  # noqa: F401
from .llm import LLM, TextGenerationPipeline, GenerationOutput  # noqa: F401
from ..engine import SamplingParams  # noqa: F401
