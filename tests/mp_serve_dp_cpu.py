"""CPU worker (two gloo ranks): data-parallel serving. Each rank holds a full replica; rank 0 serves HTTP, routes
every request to its owner rank (request id modulo ranks) and gathers the tokens. Requests land on both ranks; the
completions must equal the single-process model's. Prints `SERVE_DP_OK <world>` on rank 0."""
import json
import os
import sys
import threading

import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mojo_b200.pipelines import LLM, PipelineConfig, SamplingParams  # noqa: E402
from mojo_b200.serve.api_server import RankSync, build_app, follower_loop  # noqa: E402


def main():
    world = int(os.environ["WORLD_SIZE"])
    llm = LLM(PipelineConfig(model="tiny-llama", random_init=True, device="cpu", page_size=16, num_pages=64, max_num_seqs=4,
                             max_num_batched_tokens=48, max_model_len=128, seed=0, data_parallel=world))   # joins the ranks itself
    info = llm.dist_info
    assert info is not None and info.world_size == world
    sync = RankSync(info, data_parallel=True)
    if not sync.leader:
        follower_loop(llm, sync)
        dist.destroy_process_group()
        return
    from fastapi.testclient import TestClient

    prompts = [[11, 12, 13, 14, 15], list(range(20, 60)), [7, 8, 9], list(range(100, 117))]
    ref = LLM(PipelineConfig(model="tiny-llama", random_init=True, device="cpu", page_size=16, num_pages=64, max_num_seqs=4,
                             max_num_batched_tokens=48, max_model_len=128, seed=0))
    want = [o.token_ids for o in ref.generate(prompts, SamplingParams(max_tokens=7))]
    app = build_app(llm, "dp-model", sync=sync)
    got = [None] * len(prompts)
    with TestClient(app) as c:
        def ask(i):
            got[i] = c.post("/v1/completions", json={"prompt": prompts[i], "max_tokens": 7}).json()["choices"][0]["token_ids"]

        threads = [threading.Thread(target=ask, args=(i,)) for i in range(len(prompts))]   # in flight together, on both ranks
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        assert got == want, (got, want)
        assert c.post("/v1/completions", json={"prompt": [1] * 500, "max_tokens": 2}).status_code == 400
        with c.stream("POST", "/v1/completions", json={"prompt": prompts[1], "max_tokens": 7, "stream": True}) as s:
            lines = [l for l in s.iter_lines() if l.startswith("data: ")]
        toks = [t for l in lines[:-1] for t in json.loads(l[6:])["choices"][0]["token_ids"]]
        assert toks == want[1]
    app.state.engine.shutdown()
    print(f"SERVE_DP_OK {info.world_size}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
