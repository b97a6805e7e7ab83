"""Launched under torchrun by tests/test_gpu_sharded.py: the sharded operator over NCCL on
2+ GPUs against the unsharded fused operator run on each rank's GPU (product-key scores,
float32 and bfloat16 banks), then both routing modes against the CPU oracle through the same
checked epoch the benchmark records (bench.parity_check)."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def main():
    from gl_sdm_b200.operator import SharedBankOperator
    from gl_sdm_b200.sharded import ShardedBankOperator
    from test_gpu_sharded import _inputs
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    for dtype in (torch.float32, torch.bfloat16):
        bank, x, K, T = _inputs(world, dtype, half=64, D=128, K=16, H=1, T=64)
        dx = {k: v.to(dev) for k, v in x.items()}
        single = SharedBankOperator(bank.to(dev).clone(), K, K, chunk_size=T)
        want = [single.epoch(dx["q"], dx["k"], dx["target"], dx["beta"], dx["log_decay"]).clone() for _ in range(2)]
        op = ShardedBankOperator(bank.to(dev).clone(), K, K, dist, chunk_size=T)
        per = x["q"].shape[0] // world
        mine = slice(rank * per, (rank + 1) * per)
        tol = dict(rtol=1e-5, atol=1e-6) if dtype == torch.float32 else dict(rtol=2e-2, atol=1e-4)
        for e in range(2):
            got = op.epoch(dx["q"][mine].contiguous(), dx["k"][mine].contiguous(), dx["target"][mine].contiguous(),
                           dx["beta"][mine].contiguous(), dx["log_decay"][mine].contiguous())
            torch.testing.assert_close(got, want[e][mine], **tol)
        torch.testing.assert_close(op.gather_bank().float(), single.values.float(), **tol)
    import bench
    for routing in ("pk", "dense"):
        parity = bench.parity_check(routing, rank, world, dist, dev)
        if rank == 0:
            print("parity", routing, parity)
            assert parity["ok"] and parity["wrong"] == 0 and parity["ranks_agree_on_routes"], parity
            if routing == "pk":
                assert parity["near_tie_exempt"] == 0
    dist.barrier()
    if rank == 0:
        print("sharded-nccl-ok")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
