"""Worker of the 2-GPU column-parallel test (launched by torch.distributed.run, one rank per GPU):
the N-split layer, all-gathered over NCCL, must equal the unsplit layer bit for bit."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from tailquant_kernel_b200 import SplitLinear  # noqa: E402
from tailquant_kernel_b200.shard import ColumnParallelSplitLinear  # noqa: E402


def main() -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    g = torch.Generator().manual_seed(11)
    M, K, N = 200, 1024, 7 * 64
    W = (torch.randn((N, K), generator=g) * 0.02).to(torch.bfloat16).cuda()
    bias = torch.randn(N, generator=g).cuda()
    x = torch.randn((M, K), generator=g).to(torch.bfloat16).cuda()
    full = SplitLinear(W, bias=bias, ratio=0.05)(x).clone()
    part = ColumnParallelSplitLinear(W, rank, world, bias=bias, ratio=0.05)
    got = part(x)
    torch.cuda.synchronize()
    assert got.shape == full.shape and torch.equal(got, full), f"rank {rank}: gathered output differs"
    dist.barrier()
    dist.destroy_process_group()
    print("ok", rank)


if __name__ == "__main__":
    main()
