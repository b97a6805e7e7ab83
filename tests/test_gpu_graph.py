"""A captured epoch replays to exactly the banks and readings of eagerly issued epochs."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_graphed_epochs_match_eager_epochs(native):
    from gl_sdm_b200.operator import GraphedEpoch, SharedBankOperator
    g = torch.Generator().manual_seed(3)
    seqs, T, H, half, D, K = 3, 32, 2, 32, 64, 8
    bank = (torch.randn(1, H, half * half, D, generator=g) * 0.05).bfloat16()
    epochs = [[t.to(DEV) for t in (torch.randn(seqs, T, H, 2 * half, generator=g), torch.randn(seqs, T, H, 2 * half, generator=g),
                                    (torch.randn(seqs, T, H, D, generator=g) * 0.05).bfloat16(),
                                    torch.rand(seqs, T, H, generator=g), -torch.rand(seqs, T, H, generator=g) * 0.2)]
              for _ in range(3)]
    eager = SharedBankOperator(bank.to(DEV).clone(), K, K, chunk_size=T)
    want = [eager.epoch(*x).clone() for x in epochs]
    graphed_op = SharedBankOperator(bank.to(DEV).clone(), K, K, chunk_size=T)
    replay = GraphedEpoch(graphed_op.epoch, graphed_op.values, epochs[0])
    assert torch.equal(graphed_op.values, bank.to(DEV))         # construction leaves the bank alone
    for x, w in zip(epochs, want):
        assert torch.equal(replay(*x), w)
    assert torch.equal(graphed_op.values, eager.values)
    native.raise_on_device_status(DEV)
