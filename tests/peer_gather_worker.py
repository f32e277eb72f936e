"""Worker of tests/test_peer_gather_gpu.py: one process per GPU (torchrun), compares PeerGatherer with
RootGatherer over several gathers (more than `depth`, so that buffers are reused under flow control)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from raptor_t_b200 import parallel  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lens = [256, 1024, 64, 512, 2048, 128, 320, 1536, 192, 704, 64, 896, 448, 1280, 640, 384][: 4 * world]
    assignment = [[i for i in range(len(lens)) if i % world == r] for r in range(world)]
    hidden = 768
    ref = parallel.RootGatherer(assignment, lens, hidden, torch.float16, "cuda", depth=3)
    peer = parallel.make_root_gatherer(assignment, lens, hidden, torch.float16, "cuda", depth=3, kind="peer")
    host = torch.empty(sum(lens), hidden, dtype=torch.float16).pin_memory() if rank == 0 else None
    ok = True
    for it in range(8):
        g = torch.Generator(device="cuda").manual_seed(100 * it + rank)
        mine = torch.randn(sum(lens[i] for i in assignment[rank]), hidden, device="cuda", generator=g).half()
        a = ref.finish(ref.start(mine))
        b = peer.finish(peer.start(mine, host_out=host))
        torch.cuda.synchronize()
        if rank == 0:
            ok = ok and bool((a == b).all()) and bool((host.cuda() == a).all())
    dist.barrier()
    if rank == 0:
        print("PEER GATHER OK" if ok else "PEER GATHER MISMATCH", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
