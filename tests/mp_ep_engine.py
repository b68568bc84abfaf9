"""Multi-GPU worker: the DeepSeek-architecture engine with data-parallel attention and expert-parallel MoE.
Every rank serves its own requests (different counts and lengths, so ranks finish at different steps and idle
steps are exercised) while all ranks move through the MoE layers in lock-step. The run is done twice, with eager
steps only and with decode graphs captured at start-up: both must produce the same tokens bit for bit.
Prints `EP_ENGINE_OK <world>` on rank 0."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mojo_b200 import ops  # noqa: E402
from mojo_b200.engine import EngineConfig, LLMEngine, SamplingParams  # noqa: E402
from mojo_b200.models import build_model  # noqa: E402
from mojo_b200.models.config import tiny_deepseek  # noqa: E402
from mojo_b200.parallel import init_distributed  # noqa: E402
from mojo_b200.parallel.ep import EPComm  # noqa: E402


def main():
    info = init_distributed("cuda")
    rank, world, dev = info.rank, info.world_size, info.device
    mcfg = tiny_deepseek()
    ep = EPComm(info, mcfg.n_routed_experts, mcfg.hidden_size, mcfg.moe_intermediate_size, mcfg.num_experts_per_tok,
                max_tokens=256, timeout_s=10.0)
    g = torch.Generator().manual_seed(50 + rank)
    lens = [40 + 13 * rank, 9, 130][: 2 + rank % 2]
    prompts = [torch.randint(0, mcfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    params = [SamplingParams(max_tokens=6 + 5 * rank + i) for i in range(len(prompts))]

    def run(graphs: bool):
        ecfg = EngineConfig(model=mcfg, device=str(dev), dtype=torch.bfloat16, page_size=32, num_pages=48, max_num_seqs=4,
                            max_num_batched_tokens=96, max_model_len=256, seed=0, use_cuda_graphs=graphs, ep_size=world, lockstep=True)
        model = build_model(mcfg, dev, torch.bfloat16, ep=ep).init_random(0, std=0.08)
        eng = LLMEngine(ecfg, model=model)
        outs = eng.generate(prompts, params)
        torch.cuda.synchronize()
        ops.check_status(dev)
        replays = eng.runner.graph_launches
        steps = eng.step_count
        del eng, model
        return outs, replays, steps

    eager, r0, steps_a = run(False)
    graphed, r1, steps_b = run(True)
    assert r0 == 0 and r1 > 0, f"rank {rank}: graph replays eager={r0} graphed={r1}"
    assert all(len(o) == p.max_tokens for o, p in zip(eager, params))
    assert eager == graphed, f"rank {rank}: tokens differ between eager and graph decode\n{eager}\n{graphed}"
    # every rank took the same number of steps (idle ones included)
    t = torch.tensor([steps_a, steps_b], dtype=torch.int64)
    lo, hi = t.clone(), t.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=info.host_group)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=info.host_group)
    assert torch.equal(lo, hi), f"step counts differ across ranks: {lo.tolist()} .. {hi.tolist()}"
    torch.cuda.synchronize()
    dist.barrier()
    assert ep.region.check_guard() == 0
    dist.barrier()
    if rank == 0:
        print(f"EP_ENGINE_OK {world}", flush=True)
    from mojo_b200.parallel.dist import shutdown

    shutdown()


if __name__ == "__main__":
    main()
