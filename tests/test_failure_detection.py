"""Failure detection, without faulting anything.

On the host (gloo ranks on CPU, kernels replaced by the stand-ins of tests/cpu_kernels.py): a
rank that never joins an epoch makes the others raise through the process group's timeout
instead of waiting for ever; a rank at another bank version, or one that brings truncated
candidate lists, is rejected before the exchange. On the GPU: a wait that nobody answers
runs out after a bounded number of polls, the kernel returns, the status word says so, and
the context is still usable."""
import datetime
import os
import socket
import time

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        return probe.getsockname()[1]


def _operator(world):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import cpu_kernels
    from gl_sdm_b200.sharded import ShardedBankOperator
    from test_sharded_cpu import _inputs
    bank, x, (H, half, D, K, seqs, T) = _inputs(world)
    return ShardedBankOperator(bank.clone(), K, K, dist, chunk_size=T, kernels=cpu_kernels), x, seqs // world


def _absent_rank(rank, world, port, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    op, x, per = _operator(world)
    if rank == 1:
        time.sleep(8)            # never joins the epoch; leaves only after the others have given up
        result["absent"] = True
        os._exit(0)
    mine = slice(rank * per, (rank + 1) * per)
    began = time.time()
    try:
        op.epoch(x["q"][mine], x["k"][mine], x["target"][mine], x["beta"][mine], x["log_decay"][mine])
        result["outcome"] = "returned"
    except Exception as exc:   # noqa: BLE001 - the backend's own exception type
        result["outcome"] = "raised " + type(exc).__name__
    result["seconds"] = time.time() - began
    os._exit(0)


def test_a_rank_that_never_joins_times_the_others_out():
    manager = mp.Manager()
    result = manager.dict()
    mp.spawn(_absent_rank, args=(2, _free_port(), result), nprocs=2, join=True)
    assert result["outcome"].startswith("raised"), dict(result)
    assert result["seconds"] < 30


def _mismatched_rank(rank, world, port, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        op, x, per = _operator(world)
        rows = per * x["q"].shape[1] * x["q"].shape[2]
        op.validate_peers(rows)                                   # everyone agrees: passes
        if rank == 1:
            op.version += 1                                       # one shard missed a commit
        try:
            op.validate_peers(rows)
            result[f"stale{rank}"] = "passed"
        except ValueError as exc:
            result[f"stale{rank}"] = str(exc)
        if rank == 1:
            op.version -= 1
        try:
            op.validate_peers(rows - (3 if rank == 1 else 0))     # one rank brings a truncated list
            result[f"short{rank}"] = "passed"
        except ValueError as exc:
            result[f"short{rank}"] = str(exc)
    finally:
        dist.destroy_process_group()


def test_stale_version_and_truncated_candidates_are_rejected_on_every_rank():
    manager = mp.Manager()
    result = manager.dict()
    mp.spawn(_mismatched_rank, args=(2, _free_port(), result), nprocs=2, join=True)
    for rank in range(2):
        assert result[f"stale{rank}"].startswith("stale memory transaction"), dict(result)
        assert "candidate lists" in result[f"short{rank}"], dict(result)


@pytest.mark.gpu
def test_a_wait_nobody_answers_ends_with_a_status(native):
    dev = "cuda:0"
    native.raise_on_device_status(dev)
    prefix = lambda count: np.array([(2 << 62) | (1 << 56) | count], dtype=np.uint64).view(np.int64)[0]   # noqa: E731
    aggregate = lambda count: np.array([(1 << 62) | (1 << 56) | count], dtype=np.uint64).view(np.int64)[0]  # noqa: E731
    # answered: prefix 5, then aggregates 2 and 4 -> 11 entries before position 3
    words = torch.tensor([prefix(5), aggregate(2), aggregate(4)], dtype=torch.int64, device=dev)
    assert int(native.wait_probe(words, 3).item()) == 11
    native.raise_on_device_status(dev)
    # position 1 never published: the walk from position 3 meets it, polls, and gives up
    words = torch.tensor([prefix(5), 0, aggregate(4)], dtype=torch.int64, device=dev)
    began = time.time()
    reached = native.wait_probe(words, 3)
    torch.cuda.synchronize()
    assert time.time() - began < 20
    assert int(reached.item()) == 4
    with pytest.raises(RuntimeError, match="bounded wait expired"):
        native.raise_on_device_status(dev)
    native.raise_on_device_status(dev)                            # the word was cleared
    # the context is intact: an ordinary kernel still runs and is right
    scores = torch.zeros(1, 5, 2, 8, device=dev)
    index, weights = native.pk_select(scores, 4)
    assert index[0, 0, 0].tolist() == [12, 13, 14, 15]
