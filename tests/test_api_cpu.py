"""Pipelines API, loaders and the OpenAI-compatible server on CPU (tiny model, token-id passthrough)."""
import json

import numpy as np
import pytest
import torch

from mojo_b200.pipelines import LLM, PipelineConfig, SamplingParams


def tiny_llm(**kw):
    return LLM(PipelineConfig(model="tiny-llama", random_init=True, device="cpu", page_size=16, num_pages=64, max_num_seqs=8,
                              max_num_batched_tokens=128, max_model_len=256, **kw))


def test_llm_generate_and_stream_agree():
    llm = tiny_llm()
    prompt = list(range(100, 130))
    out = llm.generate([prompt], SamplingParams(max_tokens=8))[0]
    assert len(out.token_ids) == 8 and out.finish_reason == "length"
    assert list(tiny_llm().stream(prompt, SamplingParams(max_tokens=8))) == out.token_ids
    cfg = PipelineConfig.from_json(llm.config.to_json())
    assert cfg == llm.config


def test_safetensors_roundtrip_matches_random_init(tmp_path):
    from mojo_b200.loaders.safetensors_loader import save_llama_safetensors
    from mojo_b200.models.config import tiny_llama

    cfg = tiny_llama()
    g = torch.Generator().manual_seed(0)
    full = {"model.embed_tokens.weight": torch.randn(cfg.vocab_size, cfg.hidden_size, generator=g) * 0.02,
            "model.norm.weight": torch.ones(cfg.hidden_size)}
    d = cfg.head_dim
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        full[p + "input_layernorm.weight"] = torch.ones(cfg.hidden_size)
        full[p + "post_attention_layernorm.weight"] = torch.ones(cfg.hidden_size)
        for name, shape in (("self_attn.q_proj", (cfg.num_heads * d, cfg.hidden_size)), ("self_attn.k_proj", (cfg.num_kv_heads * d, cfg.hidden_size)),
                            ("self_attn.v_proj", (cfg.num_kv_heads * d, cfg.hidden_size)), ("self_attn.o_proj", (cfg.hidden_size, cfg.num_heads * d)),
                            ("mlp.gate_proj", (cfg.intermediate_size, cfg.hidden_size)), ("mlp.up_proj", (cfg.intermediate_size, cfg.hidden_size)),
                            ("mlp.down_proj", (cfg.hidden_size, cfg.intermediate_size))):
            full[p + name + ".weight"] = torch.randn(*shape, generator=g) * 0.02
    hf_cfg = {"architectures": ["LlamaForCausalLM"], "hidden_size": cfg.hidden_size, "num_hidden_layers": cfg.num_layers,
              "num_attention_heads": cfg.num_heads, "num_key_value_heads": cfg.num_kv_heads, "intermediate_size": cfg.intermediate_size,
              "vocab_size": cfg.vocab_size, "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "max_position_embeddings": 2048,
              "tie_word_embeddings": True}
    save_llama_safetensors(full, tmp_path, hf_cfg)
    llm = LLM(PipelineConfig(model=str(tmp_path), device="cpu", page_size=16, num_pages=32, max_num_seqs=4, max_num_batched_tokens=64, max_model_len=128))
    assert torch.equal(llm.engine.model.layers[1].wo, full["model.layers.1.self_attn.o_proj.weight"])
    out = llm.generate([[5, 6, 7, 8, 9]], SamplingParams(max_tokens=4))[0]
    assert len(out.token_ids) == 4


def test_gguf_file_roundtrip(tmp_path):
    gguf = pytest.importorskip("gguf")
    from mojo_b200.loaders.gguf_loader import GGUFFile
    from mojo_b200.ops import reference as ref

    path = tmp_path / "t.gguf"
    w = gguf.GGUFWriter(str(path), "llama")
    w.add_uint32("llama.block_count", 1)
    raw = ref.random_gguf_blocks(4 * 512 // 256, 12, seed=1).numpy().reshape(4, 512 // 256 * 144)
    w.add_tensor("blk.0.attn_q.weight", raw, raw_dtype=gguf.GGMLQuantizationType.Q4_K)
    w.add_tensor("output_norm.weight", np.ones(8, dtype=np.float32))
    w.write_header_to_file(); w.write_kv_data_to_file(); w.write_tensors_to_file(); w.close()
    gf = GGUFFile(path)
    kind, (ty, blocks), shape = gf.tensor("blk.0.attn_q.weight")
    assert kind == "q" and ty == 12 and shape == (4, 512) and blocks.numel() == raw.size
    assert torch.equal(ref.gguf_dequant(blocks, 12, shape), ref.gguf_dequant(torch.from_numpy(raw.reshape(-1)), 12, shape))
    assert gf.tensor("output_norm.weight")[0] == "f" and gf.metadata()["llama.block_count"] == 1


def test_openai_server_endpoints():
    from fastapi.testclient import TestClient

    from mojo_b200.serve import build_app

    llm = tiny_llm()
    want = tiny_llm().generate([[11, 12, 13, 14]], SamplingParams(max_tokens=5))[0].token_ids
    app = build_app(llm, "tiny-llama")
    with TestClient(app) as c:
        assert c.get("/health").json()["status"] == "ok"
        assert c.get("/v1/models").json()["data"][0]["id"] == "tiny-llama"
        r = c.post("/v1/completions", json={"prompt": [11, 12, 13, 14], "max_tokens": 5}).json()
        assert r["choices"][0]["token_ids"] == want and r["usage"]["completion_tokens"] == 5
        with c.stream("POST", "/v1/completions", json={"prompt": [11, 12, 13, 14], "max_tokens": 5, "stream": True}) as s:
            lines = [l for l in s.iter_lines() if l.startswith("data: ")]
        assert lines[-1] == "data: [DONE]"
        toks = [t for l in lines[:-1] for t in json.loads(l[6:])["choices"][0]["token_ids"]]
        assert toks == want
        r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 3}).json()
        assert r["object"] == "chat.completion" and r["usage"]["completion_tokens"] == 3
        assert c.post("/v1/completions", json={"max_tokens": 3}).status_code == 400
        # a prompt that leaves no room in the context is refused before it reaches the engine thread
        too_long = c.post("/v1/completions", json={"prompt": [7] * llm.engine.cfg.max_model_len, "max_tokens": 3})
        assert too_long.status_code == 400 and "context limit" in too_long.json()["detail"]
        assert c.post("/v1/completions", json={"prompt": [], "max_tokens": 3}).status_code == 400
        text = c.get("/metrics").text
        assert "b2_output_tokens" in text or "b2_generated_tokens_total" in text
        assert 'b2_ttft_milliseconds_bucket{le="+Inf"} 3' in text          # three requests were served
        assert "b2_itl_milliseconds_count 10" in text                       # 5 + 5 + 3 tokens -> 4 + 4 + 2 gaps
        assert "b2_kv_utilisation" in text and "b2_requests_finished_total 3" in text and "b2_generated_tokens_total 13" in text
        assert llm.engine.requests == {}                                     # finished streams leave no per-request state
    app.state.engine.shutdown()


def _write_tp_checkpoint(tmp_path):
    """A small Llama checkpoint whose FFN width divides by 16 x 2 ranks."""
    from mojo_b200.loaders.safetensors_loader import save_llama_safetensors

    hid, heads, kv, d, ffn, vocab, layers = 256, 4, 2, 64, 704, 1000, 2
    g = torch.Generator().manual_seed(1)
    full = {"model.embed_tokens.weight": torch.randn(vocab, hid, generator=g) * 0.05, "model.norm.weight": torch.ones(hid),
            "lm_head.weight": torch.randn(vocab, hid, generator=g) * 0.05}
    for i in range(layers):
        p = f"model.layers.{i}."
        full[p + "input_layernorm.weight"] = torch.ones(hid)
        full[p + "post_attention_layernorm.weight"] = torch.ones(hid)
        for name, shape in (("self_attn.q_proj", (heads * d, hid)), ("self_attn.k_proj", (kv * d, hid)), ("self_attn.v_proj", (kv * d, hid)),
                            ("self_attn.o_proj", (hid, heads * d)), ("mlp.gate_proj", (ffn, hid)), ("mlp.up_proj", (ffn, hid)),
                            ("mlp.down_proj", (hid, ffn))):
            full[p + name + ".weight"] = torch.randn(*shape, generator=g) * 0.05
    save_llama_safetensors(full, tmp_path, {"architectures": ["LlamaForCausalLM"], "hidden_size": hid, "num_hidden_layers": layers,
                                            "num_attention_heads": heads, "num_key_value_heads": kv, "intermediate_size": ffn,
                                            "vocab_size": vocab, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
                                            "max_position_embeddings": 256, "tie_word_embeddings": False})


def test_llm_tensor_parallel_joins_ranks_itself_on_cpu(tmp_path):
    """`LLM(PipelineConfig(tensor_parallel=2))` under a two-process gloo launch: each rank loads its shard of a
    safetensors checkpoint and produces the same tokens as one process."""
    import os
    import subprocess
    import sys

    _write_tp_checkpoint(tmp_path)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29641", os.path.join(root, "tests", "mp_pipeline_cpu.py")]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", B2_TEST_CHECKPOINT=str(tmp_path))
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env, cwd=root)
    assert "PIPELINE_TP_OK 2" in p.stdout, p.stdout[-2000:] + p.stderr[-3000:]


def test_llm_parallel_degree_without_ranks_is_refused():
    with pytest.raises(RuntimeError, match="torch.distributed.run"):
        LLM(PipelineConfig(model="tiny-llama", random_init=True, device="cpu", tensor_parallel=2))


@pytest.mark.parametrize("fault", ["", "raise_after:rank=1:step=17"])
def test_openai_server_over_two_tensor_parallel_ranks_on_cpu(tmp_path, fault):
    """Rank 0 serves HTTP and broadcasts its commands, rank 1 follows: same completions as one process. With a fault
    injected on rank 1 alone (host side, at the end of the third step of a later request, as a kernel status error would surface) both ranks must drop that request,
    report the error to the client and serve the next request correctly."""
    import os
    import subprocess
    import sys

    _write_tp_checkpoint(tmp_path)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29643" if not fault else "29645", os.path.join(root, "tests", "mp_serve_cpu.py")]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", B2_TEST_CHECKPOINT=str(tmp_path), B2_FAULT=fault)
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env, cwd=root)
    assert "SERVE_TP_OK 2" in p.stdout, p.stdout[-2000:] + p.stderr[-3000:]


def test_openai_server_over_two_data_parallel_ranks_on_cpu():
    """Rank 0 serves HTTP, routes requests to their owner rank and gathers the tokens of every iteration."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29644", os.path.join(root, "tests", "mp_serve_dp_cpu.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""), cwd=root)
    assert "SERVE_DP_OK 2" in p.stdout, p.stdout[-2000:] + p.stderr[-3000:]


def test_text_stream_holds_back_possible_stop_prefixes_and_cuts_at_the_stop():
    from mojo_b200.serve.api_server import _TextStream

    table = {1: "Hel", 2: "lo", 3: " wor", 4: "ld", 5: "!<", 6: "end", 7: ">"}
    ts = _TextStream(lambda ids: "".join(table[i] for i in ids), ["<end>", "ZZ"])
    out = []
    for i, t in enumerate([1, 2, 3, 4, 5]):
        d, stop = ts.push([t], False)
        assert not stop
        out.append(d)
    assert "".join(out) == "Hello wor"                 # len("<end>") - 1 = 4 characters are held back: "ld!<" is not out yet
    d, stop = ts.push([6], False)
    assert not stop and "".join(out + [d]) == "Hello world!"          # "<end" could still become the stop string
    d2, stop = ts.push([7], False)
    assert stop and d2 == ""                           # the stop string itself is never emitted
    # without a stop the tail is flushed when the request finishes
    ts = _TextStream(lambda ids: "".join(table[i] for i in ids), ["<end>"])
    assert ts.push([1, 2], False) == ("H", False)
    assert ts.push([3], True) == ("ello wor", False)
    # no stop strings: nothing is held back
    ts = _TextStream(lambda ids: "".join(table[i] for i in ids), [])
    assert ts.push([1], False) == ("Hel", False)


def test_openai_server_stop_strings():
    from fastapi.testclient import TestClient

    from mojo_b200.serve import build_app

    llm = tiny_llm()
    prompt = [5, 900, 77, 3021, 15000]
    want = tiny_llm().generate([prompt], SamplingParams(max_tokens=8))[0].token_ids
    k = next(i for i, t in enumerate(want) if t != want[0])          # the first token that differs from the repeated one
    stop = f" {want[k]}"                                             # without a tokenizer the text is the ids joined by spaces
    cut_text = " ".join(str(t) for t in want[:k])
    app = build_app(llm, "tiny-llama")
    with TestClient(app) as c:
        r = c.post("/v1/completions", json={"prompt": prompt, "max_tokens": 8, "stop": stop}).json()
        ch = r["choices"][0]
        assert ch["finish_reason"] == "stop" and ch["text"] == cut_text
        assert ch["token_ids"] == want[:k + 1]                        # the token that completed the stop string was generated, not shown
        with c.stream("POST", "/v1/completions", json={"prompt": prompt, "max_tokens": 8, "stream": True, "stop": [stop, "nope"]}) as s:
            lines = [json.loads(l[6:]) for l in s.iter_lines() if l.startswith("data: ") and l != "data: [DONE]"]
        assert "".join(l["choices"][0]["text"] for l in lines) == cut_text
        assert lines[-1]["choices"][0]["finish_reason"] == "stop"
        r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4, "stop": "never-there"}).json()
        assert r["choices"][0]["finish_reason"] == "length"
        assert c.post("/v1/completions", json={"prompt": [1, 2], "stop": 5}).status_code == 400
        # the engine thread is still healthy and serves the next request after the aborts
        r = c.post("/v1/completions", json={"prompt": prompt, "max_tokens": 8}).json()
        assert r["choices"][0]["token_ids"] == want
    app.state.engine.shutdown()


def test_openai_server_logprobs():
    from fastapi.testclient import TestClient

    from mojo_b200.serve import build_app

    llm = tiny_llm()
    prompt = [5, 900, 77, 3021, 15000]
    ref = tiny_llm().generate([prompt], SamplingParams(max_tokens=4, logprobs=2))[0]
    assert len(ref.logprobs) == 4 and all(len(top) == 2 for _, top in ref.logprobs)
    app = build_app(llm, "tiny-llama")
    with TestClient(app) as c:
        r = c.post("/v1/completions", json={"prompt": prompt, "max_tokens": 4, "logprobs": 2}).json()["choices"][0]
        assert r["token_ids"] == ref.token_ids
        assert r["logprobs"]["token_logprobs"] == pytest.approx([lp for lp, _ in ref.logprobs], abs=1e-5)
        assert [len(m) for m in r["logprobs"]["top_logprobs"]] == [2, 2, 2, 2] and all(v <= 0 for m in r["logprobs"]["top_logprobs"] for v in m.values())
        assert c.post("/v1/completions", json={"prompt": prompt, "max_tokens": 2}).json()["choices"][0]["logprobs"] is None
        r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 3, "logprobs": True,
                                                 "top_logprobs": 1}).json()["choices"][0]
        assert len(r["logprobs"]["content"]) == 3 and len(r["logprobs"]["content"][0]["top_logprobs"]) == 1
        with c.stream("POST", "/v1/completions", json={"prompt": prompt, "max_tokens": 4, "stream": True, "logprobs": 0}) as s:
            lines = [json.loads(l[6:]) for l in s.iter_lines() if l.startswith("data: ") and l != "data: [DONE]"]
        got = [v for l in lines for v in l["choices"][0]["logprobs"]["token_logprobs"]]
        assert got == pytest.approx([lp for lp, _ in ref.logprobs], abs=1e-5)
        assert c.post("/v1/completions", json={"prompt": prompt, "logprobs": 99}).status_code == 400
    app.state.engine.shutdown()


def test_openai_server_refuses_what_it_does_not_implement():
    """Fields that would change the answer but are not implemented get HTTP 400 (never silently dropped); values that mean
    "default" pass; sampling parameters are range-checked before anything is queued."""
    from fastapi.testclient import TestClient

    from mojo_b200.serve import build_app

    app = build_app(tiny_llm(), "tiny-llama")
    base = {"prompt": [5, 900, 77], "max_tokens": 2}
    with TestClient(app) as c:
        for extra in ({"n": 2}, {"best_of": 3}, {"presence_penalty": 0.5}, {"frequency_penalty": -1}, {"repetition_penalty": 1.2},
                      {"logit_bias": {"50": 10}}, {"echo": True}, {"suffix": "x"}, {"temperature": -0.5}, {"top_p": 0.0}, {"top_p": 1.5},
                      {"top_k": -1}, {"max_tokens": -3}, {"temperature": "hot"}):
            r = c.post("/v1/completions", json={**base, **extra})
            assert r.status_code == 400, (extra, r.status_code)
        chat = {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 2}
        assert c.post("/v1/chat/completions", json={**chat, "tools": [{"type": "function"}]}).status_code == 400
        assert c.post("/v1/chat/completions", json={**chat, "response_format": {"type": "json_object"}}).status_code == 400
        assert c.post("/v1/chat/completions", json={**chat, "n": 2}).status_code == 400
        # the spellings of "default" are accepted
        ok = c.post("/v1/completions", json={**base, "n": 1, "best_of": 1, "presence_penalty": 0, "frequency_penalty": 0.0, "logit_bias": {},
                                             "echo": False, "temperature": 0, "top_p": 1})
        assert ok.status_code == 200 and len(ok.json()["choices"][0]["token_ids"]) == 2
        ok = c.post("/v1/chat/completions", json={**{k: v for k, v in chat.items() if k != "max_tokens"}, "max_completion_tokens": 3,
                                                  "response_format": {"type": "text"}})
        assert ok.status_code == 200 and ok.json()["usage"]["completion_tokens"] == 3
    app.state.engine.shutdown()
