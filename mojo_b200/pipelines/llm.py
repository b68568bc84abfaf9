"""`LLM`: build the model (random-init, safetensors or GGUF), wrap it in the engine, generate."""
from __future__ import annotations

import os
from dataclasses import dataclass
from pathlib import Path
from typing import Iterator

import torch

from ..engine import EngineConfig, LLMEngine, SamplingParams
from ..models import build_model, get_config
from .config import PipelineConfig


@dataclass
class GenerationOutput:
    request_id: int
    prompt_token_ids: list
    token_ids: list
    text: str | None
    finish_reason: str | None
    logprobs: list | None = None      # per token (logprob, [(token id, logprob), ...]) when SamplingParams.logprobs was set


class _Tokenizer:
    """Thin glue over a Hugging Face tokenizer; absent one, prompts must already be token ids."""

    def __init__(self, path: str | None):
        self.tok = None
        if path:
            from transformers import AutoTokenizer

            self.tok = AutoTokenizer.from_pretrained(path)

    def encode(self, prompt) -> list[int]:
        if isinstance(prompt, str):
            if self.tok is None:
                raise ValueError("a text prompt needs PipelineConfig.tokenizer; pass token ids otherwise")
            return self.tok.encode(prompt)
        return list(prompt)

    def decode(self, ids) -> str | None:
        return self.tok.decode(ids) if self.tok is not None else None

    def apply_chat_template(self, messages) -> list[int]:
        if self.tok is not None and getattr(self.tok, "chat_template", None):
            return self.tok.apply_chat_template(messages, add_generation_prompt=True)
        text = "".join(f"<|{m['role']}|>\n{m['content']}\n" for m in messages) + "<|assistant|>\n"
        if self.tok is not None:
            return self.tok.encode(text)
        return list(text.encode("utf-8"))  # byte-level fallback for token-id passthrough servers


class LLM:
    """`LLM(config).generate(...)`. With `tensor_parallel` or `expert_parallel` above 1 the process must be one of
    that many ranks started by `python -m torch.distributed.run --nproc-per-node N ...` (one rank per GPU): the
    constructor joins the process group and builds the communicator itself (fused GEMM+collective kernels over
    symmetric memory on CUDA, `torch.distributed` collectives on CPU); every rank then makes the same `generate`
    calls (tensor parallelism) or serves its own prompts in lock-step (expert parallelism with data-parallel
    attention). A ready-made communicator can be passed instead (`comm` for tensor, `ep` for expert parallelism)."""

    def __init__(self, config: PipelineConfig, comm=None, ep=None):
        self.config = config
        device = config.device or ("cuda" if torch.cuda.is_available() else "cpu")
        dtype = getattr(torch, config.dtype) if device.startswith("cuda") else torch.float32
        src = config.model
        is_gguf = src.endswith(".gguf") and os.path.exists(src)
        if is_gguf:
            from ..loaders.gguf_loader import GGUFFile

            md = GGUFFile(src).metadata()
            arch = md.get("general.architecture", "llama")
            mcfg = get_config("tiny-llama")
            mcfg.hidden_size = int(md[f"{arch}.embedding_length"]); mcfg.num_layers = int(md[f"{arch}.block_count"])
            mcfg.num_heads = int(md[f"{arch}.attention.head_count"]); mcfg.num_kv_heads = int(md.get(f"{arch}.attention.head_count_kv", mcfg.num_heads))
            mcfg.head_dim = mcfg.hidden_size // mcfg.num_heads; mcfg.intermediate_size = int(md[f"{arch}.feed_forward_length"])
            mcfg.rms_norm_eps = float(md.get(f"{arch}.attention.layer_norm_rms_epsilon", 1e-5)); mcfg.rope_theta = float(md.get(f"{arch}.rope.freq_base", 10000.0))
            mcfg.vocab_size = int(md.get(f"{arch}.vocab_size", 0)) or None
            mcfg.tie_word_embeddings = False
        else:
            mcfg = get_config(src)
        if config.quantization:
            mcfg.quantization = config.quantization
        self.model_config = mcfg
        degree = max(config.tensor_parallel, config.expert_parallel)
        self.dist_info = None
        if config.data_parallel > 1:
            if degree > 1:
                raise ValueError("data_parallel replicas are whole models: combine it with neither tensor_parallel nor expert_parallel")
            self.dist_info = self._join_replicas(device, config.data_parallel)
            device = str(self.dist_info.device)
        if degree > 1 and comm is None and ep is None:
            comm, ep, device = self._join_ranks(mcfg, device, degree)
        model = build_model(mcfg, device, dtype, comm=comm, ep=ep)
        if config.random_init or (not is_gguf and not (Path(src) / "config.json").exists()):
            model.init_random(config.seed)
        elif is_gguf:
            from ..loaders import load_gguf_into

            if mcfg.vocab_size is None:
                from ..loaders.gguf_loader import GGUFFile

                mcfg.vocab_size = GGUFFile(src).tensor("token_embd.weight")[2][0]
            load_gguf_into(model, src)
        else:
            from ..loaders import load_safetensors_into

            load_safetensors_into(model, src)
        ecfg = EngineConfig(model=mcfg, device=device, dtype=dtype, page_size=config.page_size, num_pages=config.num_pages,
                            gpu_memory_utilization=config.gpu_memory_utilization, max_num_seqs=config.max_num_seqs,
                            max_num_batched_tokens=config.max_num_batched_tokens, max_model_len=config.max_model_len,
                            enable_prefix_cache=config.enable_prefix_cache, enable_chunked_prefill=config.enable_chunked_prefill,
                            eos_token_id=config.eos_token_id, seed=config.seed, use_cuda_graphs=config.use_cuda_graphs,
                            tp_size=config.tensor_parallel, ep_size=config.expert_parallel,
                            lockstep=ep is not None and getattr(ep, "world_size", 1) > 1)
        self.engine = LLMEngine(ecfg, model=model, comm=comm)
        self.comm, self.ep = comm, ep
        self.tokenizer = _Tokenizer(config.tokenizer)

    @staticmethod
    def _join_replicas(device: str, degree: int):
        """Data parallelism: every rank holds the whole model on its own device; the process group only carries the
        serving front end's control messages."""
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if world != degree:
            raise RuntimeError(f"data_parallel={degree} needs {degree} ranks (WORLD_SIZE={world}): start the program with "
                               f"`python -m torch.distributed.run --nproc-per-node {degree} --master-addr 127.0.0.1 ...`")
        from ..parallel import init_distributed

        return init_distributed("cuda" if device.startswith("cuda") else "cpu")

    def _join_ranks(self, mcfg, device: str, degree: int):
        """Join the process group of a `torch.distributed.run` launch and build this rank's communicator."""
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if world != degree:
            raise RuntimeError(f"parallel degree {degree} needs {degree} ranks (WORLD_SIZE={world}): start the program with "
                               f"`python -m torch.distributed.run --nproc-per-node {degree} --master-addr 127.0.0.1 ...`")
        from ..parallel import init_distributed

        info = init_distributed("cuda" if device.startswith("cuda") else "cpu")
        cfg = self.config
        if cfg.expert_parallel > 1:
            if mcfg.architecture != "deepseek_v2":
                raise ValueError("expert_parallel applies to mixture-of-experts models")
            if info.device.type != "cuda":
                raise RuntimeError("expert parallelism runs on CUDA devices")
            from ..parallel.ep import EPComm

            ep = EPComm(info, mcfg.n_routed_experts, mcfg.hidden_size, mcfg.moe_intermediate_size, mcfg.num_experts_per_tok,
                        max_tokens=cfg.max_num_batched_tokens)
            return None, ep, str(info.device)
        if info.device.type == "cuda":
            from ..parallel.fused import FusedTPComm

            comm = FusedTPComm(info, max_tokens=cfg.max_num_batched_tokens, hidden=mcfg.hidden_size, max_k=mcfg.hidden_size)
        else:
            from ..parallel.tp import NcclTPComm

            comm = NcclTPComm(info)
        return comm, None, str(info.device)

    def generate(self, prompts, sampling_params: SamplingParams | list | None = None) -> list[GenerationOutput]:
        ids = [self.tokenizer.encode(p) for p in prompts]
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params or SamplingParams()] * len(ids)
        rids = [self.engine.add_request(p, sp) for p, sp in zip(ids, sampling_params)]
        self.engine.run_until_done()
        outs = []
        for rid, p in zip(rids, ids):
            st = self.engine.requests[rid]
            outs.append(GenerationOutput(rid, p, list(st.output_ids), self.tokenizer.decode(st.output_ids), st.finish_reason,
                                         list(st.logprobs) if st.params.logprobs is not None else None))
            self.engine.forget(rid)
        return outs

    def stream(self, prompt, sampling_params: SamplingParams | None = None) -> Iterator[int]:
        """Yield the tokens of one request as they are produced (other requests may run concurrently)."""
        rid = self.engine.add_request(self.tokenizer.encode(prompt), sampling_params or SamplingParams())
        done = False
        while not done:
            for o in self.engine.step():
                if o.request_id == rid:
                    yield from o.new_token_ids
                    done = done or o.finished


TextGenerationPipeline = LLM
