"""CPU worker (gloo ranks): the descriptor exchange of the symmetric heap's rendezvous. Every rank opens a temporary file
that holds its rank number and hands the descriptor to every peer over the AF_UNIX / SCM_RIGHTS channel; each rank
then reads its peers' numbers through the descriptors it received. A second round has a single sender (the form the
multicast object takes). Prints `FD_EXCHANGE_OK <world>` on rank 0."""
import os
import sys
import tempfile

import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mojo_b200.parallel import init_distributed  # noqa: E402
from mojo_b200.parallel.symm import _all_ok, _exchange_fds  # noqa: E402


def main():
    info = init_distributed("cpu")
    rank, world = info.rank, info.world_size
    with tempfile.TemporaryFile() as f:
        f.write(f"rank {rank}".encode())
        f.flush()
        got = _exchange_fds(info, f"test{os.environ.get('MASTER_PORT', '0')}a", f.fileno(), list(range(world)))
        assert sorted(got) == [r for r in range(world) if r != rank], got
        for peer, fd in got.items():
            assert fd != f.fileno()
            assert os.pread(fd, 64, 0) == f"rank {peer}".encode()
            os.close(fd)
        # one sender: only rank 0's descriptor travels
        got = _exchange_fds(info, f"test{os.environ.get('MASTER_PORT', '0')}m", f.fileno() if rank == 0 else None, [0])
        if rank == 0:
            assert got == {}
        else:
            assert list(got) == [0] and os.pread(got[0], 64, 0) == b"rank 0"
            os.close(got[0])
    assert _all_ok(info, True) and not _all_ok(info, rank != world - 1)     # one rank's failure is everybody's
    dist.barrier()
    if rank == 0:
        print(f"FD_EXCHANGE_OK {world}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
