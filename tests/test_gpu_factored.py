"""The factored commit (delta rows rebuilt inside the reducer, never written to memory) must
leave exactly the bank that the proposal + commit pair with materialised deltas leaves — the
pair that is pinned to the reference (projects/gl-sdm/src/gl_sdm/runtime/dense.py:11-14,
layers/global_layer.py:44-54, memory/transactions.py:90-96) in test_gpu_parity.py."""
import pytest
import torch

from thread_dist import ThreadWorld

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _inputs(seqs, T, H, half, D, dtype, seed, hot=False):
    g = torch.Generator().manual_seed(seed)
    bank = (torch.randn(1, H, half * half, D, generator=g) * 0.05).to(dtype)
    x = dict(q=torch.randn(seqs, T, H, 2 * half, generator=g), k=torch.randn(seqs, T, H, 2 * half, generator=g),
             target=(torch.randn(seqs, T, H, D, generator=g) * 0.05).to(dtype), beta=torch.rand(seqs, T, H, generator=g),
             log_decay=-torch.rand(seqs, T, H, generator=g) * 0.2)
    x["k"][:, :, :, :half] = x["k"][:, :, :, :half].round()          # ties: many rows share slots
    if hot:
        x["k"][..., 0] += 6.0                                          # every row writes slot row 0 ...
        x["k"][..., half] += 6.0                                       # ... column 0: one very long segment
    return bank, {k: v.to(DEV) for k, v in x.items()}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(4, 16, 2, 32, 64, 8, False), (2, 24, 1, 16, 128, 4, False),
                                   (2, 16, 1, 16, 256, 16, False), (3, 8, 2, 8, 40, 4, False),
                                   (4, 160, 1, 4, 32, 2, True)])
def test_unsharded_epochs_are_bit_identical(native, dtype, shape):
    from gl_sdm_b200.operator import SharedBankOperator
    seqs, T, H, half, D, K, hot = shape
    bank, x = _inputs(seqs, T, H, half, D, dtype, 7, hot)
    a = SharedBankOperator(bank.to(DEV).clone(), K, K, chunk_size=T, factored=True)
    b = SharedBankOperator(bank.to(DEV).clone(), K, K, chunk_size=T, factored=False)
    for epoch in range(3):
        ra = a.epoch(x["q"], x["k"], x["target"], x["beta"], x["log_decay"], offset=epoch * T)
        rb = b.epoch(x["q"], x["k"], x["target"], x["beta"], x["log_decay"], offset=epoch * T)
        assert torch.equal(ra, rb)
        assert torch.equal(a.values, b.values), f"epoch {epoch}"
    assert not torch.equal(a.values, bank.to(DEV))
    native.raise_on_device_status(DEV)


@pytest.mark.parametrize("world", [1, 2, 4])
def test_sharded_epochs_are_bit_identical(native, world):
    from gl_sdm_b200.sharded import ShardedBankOperator
    seqs, T, H, half, D, K = 2 * world, 16, 2, 32, 64, 8
    bank, x = _inputs(seqs, T, H, half, D, torch.bfloat16, 11)
    per = seqs // world
    banks = {}
    for factored in (True, False):
        tw = ThreadWorld(world)

        def body(rank, dist):
            torch.cuda.set_device(0)
            op = ShardedBankOperator(bank.to(DEV).clone(), K, K, dist, chunk_size=T, factored=factored)
            mine = slice(rank * per, (rank + 1) * per)
            for _ in range(2):
                op.epoch(*(x[n][mine].contiguous() for n in ("q", "k", "target", "beta", "log_decay")))
            return op.gather_bank()

        banks[factored] = tw.run(body)[0]
    assert torch.equal(banks[True], banks[False])
    native.raise_on_device_status(DEV)
