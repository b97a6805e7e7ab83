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


@pytest.mark.parametrize("world", [2, 4])
def test_dense_routing_shares_bounds_between_ranks(world):
    """Host side of the routing bounds (ShardedBankOperator._score_all_rows) with stand-in
    kernels, the ranks as threads of one process: every rank scores a rotated copy of the rows,
    tells its peers the K-th best scores through their inboxes (two halves used alternately)
    and drops what cannot enter the top-k any more; routes, readings and banks are those of a
    single rank, epoch after epoch."""
    import cpu_kernels
    from thread_dist import ThreadWorld
    from gl_sdm_b200.sharded import ShardedBankOperator
    g = torch.Generator().manual_seed(3)
    slots, dk, D, K, T, seqs = 512, 16, 8, 4, 128, 2 * world
    bank = torch.randn(1, 1, slots, D, generator=g)
    keys = torch.nn.functional.normalize(torch.randn(slots, dk, generator=g), dim=-1).bfloat16()
    x = dict(q=torch.randn(seqs, T, dk, generator=g).bfloat16(), kq=torch.randn(seqs, T, dk, generator=g).bfloat16(),
             target=torch.randn(seqs, T, 1, D, generator=g), beta=torch.rand(seqs, T, 1, generator=g),
             log_decay=-torch.rand(seqs, T, 1, generator=g) * 0.2)
    per = seqs // world

    def epochs(op, mine):
        out = []
        for _ in range(3):
            reads = op.epoch_dense(*[x[k][mine].contiguous() for k in ("q", "kq", "target", "beta", "log_decay")]).clone()
            out.append((reads, [t.clone() for t in op.last_routes()]))
        return out

    # The stand-in reads its bounds when it starts and stores its own when it ends; the ranks
    # take turns inside it, so that every rank but the first finds what the earlier ones reached.
    import threading
    import types
    turn, order = [0], threading.Condition()

    def in_turn(rank):
        def score_topk(*args, **kwargs):
            with order:
                order.wait_for(lambda: turn[0] % world == rank, timeout=60)
                result = cpu_kernels.score_topk(*args, **kwargs)
                turn[0] += 1
                order.notify_all()
            return result
        return types.SimpleNamespace(**{**vars(cpu_kernels), "score_topk": score_topk})

    def body(rank, dist):
        op = ShardedBankOperator(bank.clone(), K, K, dist, chunk_size=T, keys=keys, kernels=in_turn(rank))
        out = epochs(op, slice(rank * per, (rank + 1) * per))
        rows = world * 2 * per * T
        assert op._floor_state[1] is not None and op._floor_calls == 3
        assert (rows // world // 128) * 128 * rank == (128 * 2 * per * T // 128) * rank      # the rotation is in use
        padded = int((op._buf["cand"][rows * K:2 * rows * K] < 0).sum())
        return out, op.gather_bank(), padded

    shared = ThreadWorld(world).run(body)
    alone = ShardedBankOperator(bank.clone(), K, K, None, chunk_size=T, keys=keys, kernels=cpu_kernels)
    want = epochs(alone, slice(None))
    assert sum(padded for _, _, padded in shared) > 0
    for e in range(3):
        for rank, (out, _, _) in enumerate(shared):
            for got, expected in zip(out[e][1], want[e][1]):
                assert torch.equal(got, expected)
            torch.testing.assert_close(out[e][0], want[e][0][rank * per:(rank + 1) * per], atol=1e-6, rtol=1e-5)
    for _, after, _ in shared:
        torch.testing.assert_close(after, alone.gather_bank(), atol=1e-6, rtol=1e-5)
