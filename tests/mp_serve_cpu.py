"""CPU worker (two gloo ranks): the OpenAI-compatible server over a tensor-parallel engine. Rank 0 serves HTTP
(through FastAPI's in-process test client) and broadcasts its commands; rank 1 runs the follower loop. Completions
must equal the single-process model's, streaming included, and a refused request must not desynchronise the ranks.
Prints `SERVE_TP_OK <world>` on rank 0."""
import json
import os
import sys

import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mojo_b200.pipelines import LLM, PipelineConfig, SamplingParams  # noqa: E402
from mojo_b200.serve.api_server import RankSync, build_app, follower_loop  # noqa: E402


def main():
    world = int(os.environ["WORLD_SIZE"])
    common = dict(model=os.environ["B2_TEST_CHECKPOINT"], device="cpu", page_size=16, num_pages=64, max_num_seqs=4,
                  max_num_batched_tokens=48, max_model_len=128, seed=0)
    llm = LLM(PipelineConfig(tensor_parallel=world, **common))
    sync = RankSync(llm.comm.info)
    if not sync.leader:
        follower_loop(llm, sync)
        dist.destroy_process_group()
        return
    from fastapi.testclient import TestClient

    p1, p2 = [11, 12, 13, 14, 15], list(range(20, 60))
    ref = LLM(PipelineConfig(**common))
    want1 = ref.generate([p1], SamplingParams(max_tokens=6))[0].token_ids
    want2 = ref.generate([p2], SamplingParams(max_tokens=9))[0].token_ids
    app = build_app(llm, "tp-model", sync=sync)
    with TestClient(app) as c:
        r = c.post("/v1/completions", json={"prompt": p1, "max_tokens": 6}).json()
        assert r["choices"][0]["token_ids"] == want1, (r, want1)
        too_long = c.post("/v1/completions", json={"prompt": [1] * 500, "max_tokens": 2})
        assert too_long.status_code == 400
        with c.stream("POST", "/v1/completions", json={"prompt": p2, "max_tokens": 9, "stream": True}) as s:
            lines = [l for l in s.iter_lines() if l.startswith("data: ")]
        toks = [t for l in lines[:-1] for t in json.loads(l[6:])["choices"][0]["token_ids"]]
        assert lines[-1] == "data: [DONE]" and toks == want2, (toks, want2)
        assert c.get("/health").json()["status"] == "ok"
        if os.environ.get("B2_FAULT"):
            # A step fails on rank 1 only (host-side injection). Both ranks must agree to drop the in-flight request:
            # the client gets an error, and the next request is served by engines that are still in step.
            bad = c.post("/v1/completions", json={"prompt": p1, "max_tokens": 6})
            assert bad.status_code == 500 and "another rank" in bad.json()["detail"], bad.text
            r = c.post("/v1/completions", json={"prompt": p1, "max_tokens": 6}).json()
            assert r["choices"][0]["token_ids"] == want1, (r, want1)
    app.state.engine.shutdown()          # the stop command reaches the follower through the next broadcast
    print(f"SERVE_TP_OK {world}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
