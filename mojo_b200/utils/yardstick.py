"""A same-box yardstick for the headline workload: vLLM (a library in the image, not part of this engine) serving the
same architecture with random weights, the same 512-request trace, the same limits (256 running sequences, 4096
batched tokens, chunked prefill, greedy, fixed output lengths).

    python bench.py --impl vllm-yardstick --gpus N        (one process; vLLM starts its own workers for N > 1)

It exists to give the numbers in the performance notes something outside this repository to stand against; it is not
the reference arm (`--impl reference`), and nothing of this engine runs on its path. The whole trace is handed over
at t = 0 and run to completion, so its figure is output tokens / wall time of the complete run; the product's matching
figure is `bench.py --whole-batch`. If vLLM cannot be imported or started, one line says why and the exit code is 0.
"""
from __future__ import annotations

import json
import os
import tempfile
import time


def _write_config(model_name: str, path: str) -> None:
    """A Hugging Face style config.json of the named architecture (no weights, no tokenizer: vLLM gets
    `load_format="dummy"` and token-id prompts)."""
    from ..models import get_config

    c = get_config(model_name)
    cfg = {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": c.hidden_size, "intermediate_size": c.intermediate_size,
        "num_hidden_layers": c.num_layers, "num_attention_heads": c.num_heads, "num_key_value_heads": c.num_kv_heads, "head_dim": c.head_dim,
        "vocab_size": c.vocab_size, "max_position_embeddings": 8192, "rms_norm_eps": c.rms_norm_eps, "rope_theta": c.rope_theta,
        "hidden_act": "silu", "tie_word_embeddings": bool(c.tie_word_embeddings), "torch_dtype": "bfloat16", "bos_token_id": 1, "eos_token_id": 2,
        "attention_bias": False, "mlp_bias": False,
    }
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)


def main(args) -> None:
    out = {"impl": "vllm-yardstick", "n_gpus": args.gpus, "config": {"model": args.model, "requests": args.requests, "max_num_seqs": args.max_num_seqs,
                                                                      "max_num_batched_tokens": args.max_batched_tokens, "timed_region": "whole trace, all requests present at t = 0"}}
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    os.environ.setdefault("TRANSFORMERS_OFFLINE", "1")
    os.environ.setdefault("VLLM_NO_USAGE_STATS", "1")
    try:
        import vllm
        from vllm import LLM, SamplingParams

        from .workload import poisson_trace

        out["vllm_version"] = getattr(vllm, "__version__", "?")
        d = tempfile.mkdtemp(prefix="b2_yardstick_")
        _write_config(args.model, d)
        from ..models import get_config

        vocab = get_config(args.model).vocab_size
        trace = poisson_trace(args.requests, args.rate, (128, 2048), (64, 512), vocab, seed=1)
        llm = LLM(model=d, load_format="dummy", skip_tokenizer_init=True, dtype="bfloat16", tensor_parallel_size=args.gpus,
                  max_num_seqs=args.max_num_seqs, max_num_batched_tokens=args.max_batched_tokens, enable_chunked_prefill=True,
                  max_model_len=2048 + 512 + 128, gpu_memory_utilization=0.9, seed=0, enable_prefix_caching=False)
        prompts = [{"prompt_token_ids": [int(t) for t in r.prompt]} for r in trace]
        params = [SamplingParams(temperature=0.0, max_tokens=int(r.max_tokens), ignore_eos=True, detokenize=False) for r in trace]
        llm.generate(prompts[:8], params[:8], use_tqdm=False)      # warm-up: graphs captured, kernels loaded
        t0 = time.perf_counter()
        res = llm.generate(prompts, params, use_tqdm=False)
        dt = time.perf_counter() - t0
        tokens = sum(len(r.outputs[0].token_ids) for r in res)
        out.update({"metric": "output tok/s/box, whole trace", "value": round(tokens / dt, 2), "unit": "tok/s", "output_tokens": tokens,
                    "wall_s": round(dt, 3), "higher_is_better": True})
    except Exception as e:  # noqa: BLE001 - the yardstick is optional: say why it is missing
        out["unavailable"] = f"{type(e).__name__}: {str(e)[:300]}"
    print(json.dumps(out), flush=True)
