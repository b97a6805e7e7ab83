"""The factored commit (delta rows rebuilt inside the reducer, never written to memory) must
leave exactly the bank that the proposal + commit pair with materialised deltas leaves — the
pair that is pinned to the reference (projects/gl-sdm/src/gl_sdm/runtime/dense.py:11-14,
layers/global_layer.py:44-54, memory/transactions.py:90-96) in test_gpu_parity.py."""
import pytest
import torch

from thread_dist import ThreadWorld

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(params=[1, 0], ids=["single-writer rows unsorted", "all entries sorted"])
def commit_mode(request, native):
    """Both ways the factored commit can treat rows with one writer (the default picks by size,
    which would leave test-sized commits on one of them)."""
    lib = native.library()
    before = lib.glsdm_commit_factored_mode(request.param)
    yield request.param
    lib.glsdm_commit_factored_mode(before)


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
                                   (4, 160, 1, 4, 32, 2, True),
                                   # more bank rows than bits in the commit's address map: distinct rows share a bit
                                   (2, 16, 1, 512, 32, 4, False), (3, 40, 2, 256, 64, 32, False)])
def test_unsharded_epochs_are_bit_identical(native, commit_mode, dtype, shape):
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


def test_slot_outside_the_bank_is_reported_and_dropped(native, commit_mode):
    """Dense numbering (every route an entry): a route whose slot is not in the bank changes
    nothing and raises the device status; the other routes of the epoch still commit."""
    from gl_sdm_b200.operator import SharedBankOperator
    bank, x = _inputs(2, 16, 1, 16, 64, torch.float32, 5)
    a = SharedBankOperator(bank.to(DEV).clone(), 4, 4, chunk_size=16, factored=True)
    b = SharedBankOperator(bank.to(DEV).clone(), 4, 4, chunk_size=16, factored=True)
    index, weights, packed = a.write_operands(x["k"], x["target"], x["beta"], x["log_decay"])
    a.commit_operands(index, weights, packed)
    native.raise_on_device_status(DEV)
    index_b, weights_b, packed_b = b.write_operands(x["k"], x["target"], x["beta"], x["log_decay"])
    assert torch.equal(index, index_b)
    bad = index_b.clone()
    bad.view(-1)[5] = 16 * 16 + 3
    zeroed = weights_b.clone()
    b.commit_operands(bad, zeroed, packed_b)
    with pytest.raises(RuntimeError, match="address out of range"):
        native.raise_on_device_status(DEV)
    # every row but the one the dropped route pointed at is the same as in the clean commit
    lost = int(index.view(-1)[5])
    same = torch.ones(16 * 16, dtype=torch.bool, device=DEV)
    same[lost] = False
    assert torch.equal(a.values[0, 0][same], b.values[0, 0][same])


def test_large_sparse_commit_defaults_to_the_single_writer_path(native):
    """1,048,576 entries on 4,194,304 slots: large and sparse enough for the default to leave
    single-writer rows unsorted. Same bank, bit for bit, as with every entry sorted."""
    from gl_sdm_b200.operator import SharedBankOperator
    lib = native.library()
    seqs, T, half, D, K = 64, 512, 2048, 32, 32
    g = torch.Generator(device=DEV).manual_seed(3)
    bank = (torch.randn(1, 1, half * half, D, generator=g, device=DEV) * 0.05).to(torch.bfloat16)
    k = torch.randn(seqs, T, 1, 2 * half, generator=g, device=DEV)
    target = (torch.randn(seqs, T, 1, D, generator=g, device=DEV) * 0.05).to(torch.bfloat16)
    beta = torch.rand(seqs, T, 1, generator=g, device=DEV)
    log_decay = -torch.rand(seqs, T, 1, generator=g, device=DEV) * 0.2
    banks = []
    for mode in (-1, 0):
        before = lib.glsdm_commit_factored_mode(mode)
        try:
            op = SharedBankOperator(bank.clone(), K, K, chunk_size=T, factored=True)
            launches = lib.glsdm_kernel_launches()
            op.commit_operands(*op.write_operands(k, target, beta, log_decay))
            torch.cuda.synchronize()
            banks.append((op.values, lib.glsdm_kernel_launches() - launches))
        finally:
            lib.glsdm_commit_factored_mode(before)
    assert torch.equal(banks[0][0], banks[1][0]) and not torch.equal(banks[0][0], bank)
    assert banks[0][1] != banks[1][1]      # the default really took the other path
    native.raise_on_device_status(DEV)
