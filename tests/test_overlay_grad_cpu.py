"""Gradients through copy-free commits: the autograd plumbing, on stand-in kernels."""
import pytest
import torch

import cpu_kernels
import overlay_grad_checks as checks
from gl_sdm_b200 import _native
from gl_sdm_b200.memory import routing, transactions
from gl_sdm_b200.memory.state import MemoryBank, WriteProposal


@pytest.fixture
def standins(monkeypatch):
    for name, fn in cpu_kernels.memory_api_standins().items():
        monkeypatch.setattr(_native, name, fn)


def test_copy_free_step_matches_copying_step(standins):
    checks.assert_same_step("cpu")


def test_bf16_request_banks(standins):
    checks.assert_same_step("cpu", storage=torch.bfloat16)


def test_chain_longer_than_one_call_takes(standins, monkeypatch):
    monkeypatch.setattr(_native, "MAX_UNDO_LOGS", 2)
    checks.assert_same_step("cpu", commits=5)


def _one_commit(view, scores, width, donate):
    prediction, index, weights = routing.torch_routed_read(view.values, scores, width)
    addresses = routing.absolute_addresses(view.values, index)
    delta = weights.unsqueeze(-1) * prediction.unsqueeze(-2)
    proposal = WriteProposal(view.version, addresses.flatten(), delta.flatten(0, 3), view.lineage)
    return prediction, transactions.commit(view, transactions.merge(view, [proposal]), donate=donate)


def test_unlogged_change_of_the_bank_is_refused(standins):
    bank = MemoryBank(2, 16, 8)
    view = bank.snapshot(1)
    scores = torch.randn(1, 4, 2, 8, requires_grad=True)
    prediction, newer = _one_commit(view, scores, 2, donate="overlay")
    newer.values.detach().add_(1.0)            # not a commit: nothing recorded the old rows
    with pytest.raises(RuntimeError, match="modified in place"):
        prediction.sum().backward()


def test_stale_view_is_not_rebuilt_differentiably(standins):
    bank = MemoryBank(2, 16, 8)
    view = bank.snapshot(1)
    scores = torch.randn(1, 4, 2, 8, requires_grad=True)
    _, newer = _one_commit(view, scores, 2, donate="overlay")
    assert view.stale and not newer.stale
    with pytest.raises(RuntimeError, match="cannot be rebuilt differentiably"):
        view.values
    with torch.no_grad():
        assert torch.equal(view.values, bank.memory.detach().unsqueeze(0))


def test_logs_are_freed_with_their_readers(standins):
    import gc
    import weakref
    bank = MemoryBank(2, 16, 8)
    view = bank.snapshot(1)
    scores = torch.randn(1, 4, 2, 8)
    with torch.no_grad():
        _, view1 = _one_commit(view, scores, 2, donate="overlay")
        first = weakref.ref(view._undo)
        _, view2 = _one_commit(view1, scores, 2, donate="overlay")
    assert first() is not None and first().next is view1._undo
    del view, view1
    gc.collect()
    assert first() is None                       # only the newest node stays with the tensor
    assert view2.values._glsdm_tail.next is None
