"""The multi-GPU exchange logic of ShardedBankOperator on two gloo ranks (CPU): routes
all-gather, partial-read reduce-scatter, write-operand all-gather, owner-side expansion and
local commit reproduce the unsharded oracle. The kernels are replaced by CPU stand-ins
(tests/cpu_kernels.py); the GPU variant of this test is tests/test_gpu_sharded.py."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import sdm_oracle as oracle


def _inputs(world):
    g = torch.Generator().manual_seed(17)
    H, half, D, K, seqs, T = 2, 8, 8, 4, 2 * world, 6
    bank = torch.randn(1, H, half * half, D, generator=g)
    x = dict(q=torch.randn(seqs, T, H, 2 * half, generator=g), k=torch.randn(seqs, T, H, 2 * half, generator=g).round(),
             target=torch.randn(seqs, T, H, D, generator=g), beta=torch.rand(seqs, T, H, generator=g),
             log_decay=-torch.rand(seqs, T, H, generator=g))
    return bank, x, (H, half, D, K, seqs, T)


def _rank(rank, world, port, result):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import cpu_kernels
    from gl_sdm_b200.sharded import ShardedBankOperator
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        bank, x, (H, half, D, K, seqs, T) = _inputs(world)
        op = ShardedBankOperator(bank.clone(), K, K, dist, chunk_size=T, kernels=cpu_kernels)
        per = seqs // world
        mine = slice(rank * per, (rank + 1) * per)
        out = []
        for epoch in range(2):   # the second epoch reads what the first committed
            out.append(op.epoch(x["q"][mine], x["k"][mine], x["target"][mine], x["beta"][mine], x["log_decay"][mine]))
        full = op.gather_bank()
        if rank == 0:
            result["bank"] = full.numpy()
        result[f"read{rank}"] = torch.stack(out).numpy()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_sharded_epochs_match_unsharded_oracle(world):
    bank, x, (H, half, D, K, seqs, T) = _inputs(world)
    manager = mp.Manager()
    result = manager.dict()
    mp.spawn(_rank, args=(world, 29533, result), nprocs=world, join=True)
    memory = bank.numpy()
    reads = []
    for epoch in range(2):
        r, _, _ = oracle.routed_read(memory, x["q"].numpy(), K)
        reads.append(r)
        a, d, k = oracle.propose(memory, x["k"].numpy(), K, x["target"].numpy(), x["beta"].numpy(),
                                 x["log_decay"].numpy(), None, 0, 0, T, 1)
        memory = oracle.commit(memory, a, d, k)
    np.testing.assert_allclose(result["bank"], memory, rtol=1e-5, atol=1e-6)
    per = seqs // world
    for rank in range(world):
        got = result[f"read{rank}"]
        for epoch in range(2):
            np.testing.assert_allclose(got[epoch], reads[epoch][rank * per:(rank + 1) * per], rtol=1e-5, atol=1e-6)


def test_shard_range_partitions_the_slots():
    from gl_sdm_b200.sharded import shard_range
    assert [shard_range(64, r, 4) for r in range(4)] == [(0, 16), (16, 32), (32, 48), (48, 64)]
    with pytest.raises(ValueError):
        shard_range(10, 0, 4)
