"""CPU worker (launched by torch.distributed.run with the gloo backend): the public `LLM` entry point with
`tensor_parallel` equal to the world size joins the process group itself, shards the model and must produce, on
every rank, the tokens of the single-process model of the same seed. Prints `PIPELINE_TP_OK <world>` on rank 0."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mojo_b200.pipelines import LLM, PipelineConfig, SamplingParams  # noqa: E402


def main():
    world = int(os.environ["WORLD_SIZE"])
    # a small Llama checkpoint written by the launching test (FFN width divisible by 16 * world)
    common = dict(model=os.environ["B2_TEST_CHECKPOINT"], device="cpu", page_size=16, num_pages=64, max_num_seqs=4,
                  max_num_batched_tokens=48, max_model_len=128, seed=0)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (19, 60, 7)]
    sp = SamplingParams(max_tokens=8)
    want = [o.token_ids for o in LLM(PipelineConfig(**common)).generate(prompts, sp)]
    llm = LLM(PipelineConfig(tensor_parallel=world, **common))
    assert llm.comm is not None and llm.comm.world_size == world
    assert llm.engine.model.tp == world
    got = [o.token_ids for o in llm.generate(prompts, sp)]
    assert got == want, f"rank {dist.get_rank()}: {got} vs {want}"
    dist.barrier()
    if dist.get_rank() == 0:
        print(f"PIPELINE_TP_OK {world}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
