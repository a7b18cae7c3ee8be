"""One rank of the sharded-bmm tests (launched by tests/test_sharded.py through torch.distributed.run)."""
import argparse
import os

import torch
import torch.distributed as dist

from torchvulkan_b200.sharded import ShardedBmm, shard_range


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", required=True)
    ap.add_argument("--batch", type=int, required=True)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    gpu = args.backend == "nccl"
    if gpu:
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group(args.backend)
    dev = torch.device("cuda", torch.cuda.current_device()) if gpu else torch.device("cpu")
    dtype = torch.bfloat16 if gpu else torch.float32
    m, k, n = (256, 192, 320) if gpu else (6, 5, 7)
    g = torch.Generator().manual_seed(17)
    a = torch.randint(-2, 3, (args.batch, m, k), generator=g).to(dtype)   # small integers: every product and sum is exact
    b = torch.randint(-2, 3, (args.batch, k, n), generator=g).to(dtype)
    want = torch.bmm(a.float(), b.float())
    lo, hi = shard_range(args.batch, rank, world)
    a_mine, b_mine = a[lo:hi].to(dev), b[lo:hi].to(dev)
    compute = None if gpu else (lambda x, y, out: torch.bmm(x, y, out=out))
    modes = ("push", "copy", "pipelined", "allgather") if gpu else ("pipelined", "allgather")
    for mode in modes:
        if mode == "push" and args.batch % world:
            continue
        for chunks in ((1, 3) if mode in ("pipelined", "copy") else (1,)):
            out = torch.full((args.batch, m, n), float("nan"), dtype=dtype, device=dev)
            op = ShardedBmm(out, mode=mode, chunks=chunks, compute=compute)
            # two steps with different operands and a reader of the first result in between: the second step must
            # not disturb what the reader sees, and must itself be complete on every rank
            op.run(a_mine, b_mine)
            seen = out.float().sum(dim=(1, 2))                       # consumer of step 1, same stream
            op.run(a_mine, -b_mine)
            if gpu:
                torch.cuda.synchronize()
            assert torch.equal(seen.cpu(), want.sum(dim=(1, 2))), (mode, chunks, rank, "first result")
            assert torch.equal(out.float().cpu(), -want), (mode, chunks, rank)
            op.close()
    if gpu:
        from torchvulkan_b200 import cuda_ops
        cuda_ops.check_device_status(torch.cuda.current_device())
    dist.barrier()
    if rank == 0:
        print("sharded ok", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
