"""Host-side logic of the gl_sdm.memory mirror: value objects, validation, error text,
no CPU fallback, and the module shim - the CPU-checkable parts of the reference's tests
(projects/gl-sdm/tests/test_global_memory.py:27-54,57-66; test_native_memory.py:141-144)."""
import dataclasses
import sys

import pytest
import torch

from gl_sdm_b200.memory import (MemoryBank, MemoryCache, MemoryView, WriteBuffer, WriteProposal, commit, merge,
                                read, propose_write, routing)
from gl_sdm_b200.memory import oracle_hook


def test_view_validation():
    MemoryView(torch.zeros(1, 1, 4, 2))
    MemoryView(torch.zeros(1, 1, 4, 2, dtype=torch.bfloat16))  # extension: bf16 storage
    for bad in (torch.zeros(4, 2), torch.zeros(1, 1, 0, 2), torch.zeros(1, 1, 4, 2, dtype=torch.float64)):
        with pytest.raises(ValueError, match="memory views require"):
            MemoryView(bad)
    with pytest.raises(ValueError, match="nonnegative version"):
        MemoryView(torch.zeros(1, 1, 4, 2), version=-1)
    a, b = MemoryView(torch.zeros(1, 1, 4, 2)), MemoryView(torch.zeros(1, 1, 4, 2))
    assert a.lineage is not b.lineage and a.version == 0


def test_merge_and_commit_reject_stale_or_foreign_transactions():
    view = MemoryView(torch.zeros(1, 1, 4, 1))
    p = WriteProposal(0, torch.tensor([3]), torch.tensor([[1.0]]), view.lineage)
    assert isinstance(merge(view, [p]), WriteBuffer)
    with pytest.raises(ValueError, match="snapshot"):
        merge(view, [])
    newer = MemoryView(view.values, 1, view.lineage)
    with pytest.raises(ValueError, match="snapshot"):
        merge(newer, [p])
    with pytest.raises(ValueError, match="snapshot"):
        merge(MemoryView(view.values), [p])
    buffer = merge(view, [p])
    with pytest.raises(ValueError, match="stale"):
        commit(newer, buffer)
    with pytest.raises(ValueError, match="stale"):
        commit(MemoryView(view.values), buffer)
    keyed = WriteProposal(0, torch.tensor([3]), torch.tensor([[1.0]]), view.lineage, torch.tensor([7]))
    with pytest.raises(ValueError, match="cannot mix keyed and unkeyed"):
        commit(view, merge(view, [p, keyed]))
    with pytest.raises(ValueError, match="memory backend must be torch or urm"):
        commit(view, buffer, backend="triton")
    with pytest.raises(ValueError, match="memory backend must be torch or urm"):
        read(view, torch.tensor([0]), torch.zeros(1, 1, 1, dtype=torch.long), torch.ones(1, 1, 1), backend="x")


def test_no_cpu_fallback():
    """Every compute entry raises on CPU tensors (reference test_native_memory.py:141-144)."""
    view = MemoryView(torch.zeros(1, 1, 4, 2))
    p = WriteProposal(0, torch.tensor([3]), torch.tensor([[1.0, 1.0]]), view.lineage)
    with pytest.raises(ValueError, match="CUDA"):
        commit(view, merge(view, [p]))
    with pytest.raises(ValueError, match="CUDA"):
        routing.torch_routed_read(view.values, torch.zeros(1, 3, 1, 4), 2)
    with pytest.raises(ValueError, match="CUDA"):
        routing.gather_rows(view.values, torch.zeros(1, 3, 1, 2, dtype=torch.long))
    with pytest.raises(ValueError, match="CUDA"):
        read(view, torch.tensor([0]), torch.zeros(1, 1, 1, dtype=torch.long), torch.ones(1, 1, 1))
    with pytest.raises(ValueError, match="CUDA"):
        propose_write(view, torch.tensor([0]), torch.zeros(1, 1, 1, dtype=torch.long), torch.ones(1, 1, 1),
                      torch.zeros(1, 1, 2), torch.ones(1, 1, 1), torch.zeros(1, 1, 1), torch.ones(1))


def test_reference_switch_needs_a_registered_oracle():
    oracle_hook.clear()
    view = MemoryView(torch.zeros(1, 1, 4, 2))
    p = WriteProposal(0, torch.tensor([3]), torch.tensor([[1.0, 1.0]]), view.lineage)
    with pytest.raises(RuntimeError, match="oracle"):
        commit(view, merge(view, [p]), reference=True)
    calls = []
    oracle_hook.register(commit=lambda v, b: calls.append(1) or MemoryView(v.values + 1, v.version + 1, v.lineage))
    try:
        assert commit(view, merge(view, [p]), reference=True).version == 1 and calls == [1]
    finally:
        oracle_hook.clear()


def test_bank_stays_fp32_and_owns_its_caches():
    bank = MemoryBank(2, 16, 8)
    assert bank.memory.shape == (2, 16, 8) and bank.memory._sdm_memory_bank
    before = bank.memory.detach().clone()
    bank = bank.to(torch.bfloat16)
    assert bank.memory.dtype == torch.float32 and torch.equal(bank.memory, before)
    cache = bank.new_cache(3)
    assert isinstance(cache, MemoryCache) and cache.view.values.shape == (3, 2, 16, 8) and cache.tokens == 0
    bank.validate_cache(cache, 3)
    with pytest.raises(ValueError, match="another model"):
        bank.validate_cache(cache, 2)
    with pytest.raises(ValueError, match="another model"):
        MemoryBank(2, 16, 8).validate_cache(cache, 3)
    assert [n for n, _ in bank.named_parameters()] == ["memory"]


def test_absolute_addresses_and_token_addresses():
    from gl_sdm_b200.memory.transactions import addresses
    memory = torch.zeros(2, 3, 5, 1)
    index = torch.tensor([0, 4]).expand(2, 1, 3, 2)
    out = routing.absolute_addresses(memory, index)
    assert out[1, 0, 2].tolist() == [(1 * 3 + 2) * 5, (1 * 3 + 2) * 5 + 4]
    view = MemoryView(memory)
    token = addresses(view, torch.tensor([1]), torch.tensor([[[0], [1], [2]]]))
    assert token.flatten().tolist() == [15, 21, 27]


def test_install_shim_binds_reference_module_names():
    from gl_sdm_b200 import install, memory
    previous = install.install()
    try:
        import importlib
        assert importlib.import_module("gl_sdm.memory") is memory
        assert importlib.import_module("gl_sdm.memory.routing") is memory.routing
        from gl_sdm.memory.backends import commit as native_commit, urm
        assert callable(native_commit.commit) and callable(urm.routed_snapshot_read) and callable(urm.verify_dependency)
    finally:
        install.uninstall(previous)
    assert sys.modules.get("gl_sdm.memory") is not memory


def test_overlay_commit_bookkeeping(monkeypatch):
    """Host side of the copy-free commit (kernels replaced by torch stand-ins): versions,
    lineage, which views go stale, how logs chain, and when a snapshot is declared lost."""
    from gl_sdm_b200 import _native
    from gl_sdm_b200.memory import overlay

    def commit_undo(values, addresses, deltas, keys=None, key_bits=0):
        flat = values.view(-1, values.shape[-1])
        order = torch.sort(addresses if keys is None else keys, stable=True).indices
        ordered = addresses[order]
        old = flat[ordered].clone()
        rows, counts = torch.unique_consecutive(ordered, return_counts=True)
        flat[rows] = flat[rows] + torch.segment_reduce(deltas[order], "sum", lengths=counts)
        return ordered, old

    def undo_apply(values, addresses, rows):
        flat = values.view(-1, values.shape[-1])
        head = torch.ones_like(addresses, dtype=torch.bool)
        head[1:] = addresses[1:] != addresses[:-1]
        flat[addresses[head]] = rows[head]
        return values

    def commit_rows(values, addresses, deltas, keys=None, out=None, key_bits=0):
        out = values.clone() if out is None else out
        commit_undo(out, addresses, deltas, keys)
        return out

    for name, fn in (("commit_undo", commit_undo), ("undo_apply", undo_apply), ("commit_rows", commit_rows),
                     ("require_cuda", lambda *a: None)):
        monkeypatch.setattr(_native, name, fn)

    def proposal(view, seed):
        g = torch.Generator().manual_seed(seed)
        a = torch.randint(0, 16, (10,), generator=g)
        return WriteProposal(view.version, a, torch.randn(10, 4, generator=g), view.lineage, a * 100 + torch.arange(10))

    bank = torch.randn(1, 1, 16, 4)
    v0 = MemoryView(bank.clone())
    v1 = commit(v0, merge(v0, [proposal(v0, 1)]), donate="overlay")
    assert (v1.version, v1.lineage is v0.lineage, v0.stale, v1.stale) == (1, True, True, False)
    state1 = v1.values.clone()
    v2 = commit(v1, merge(v1, [proposal(v1, 2)]), donate="overlay")
    assert len(overlay.logs_of(v0)) == 2 and len(overlay.logs_of(v1)) == 1 and overlay.logs_of(v2) == []
    with pytest.raises(ValueError, match="newest view"):
        commit(v0, merge(v0, [proposal(v0, 3)]), donate=True)
    assert torch.equal(v1.values, state1) and not v1.stale          # rebuilt into storage of its own
    assert torch.equal(v0.values, bank)
    with pytest.raises(dataclasses.FrozenInstanceError):
        v2.version = 9
    # a donated commit of the newest view leaves no log: snapshots that still hang on it are lost
    w0 = MemoryView(bank.clone())
    w1 = commit(w0, merge(w0, [proposal(w0, 4)]), donate="overlay")
    commit(w1, merge(w1, [proposal(w1, 5)]), donate=True)
    with pytest.raises(RuntimeError, match="invalidated"):
        w0.values


def test_token_clock_backward_wiring_against_reference_gradients(monkeypatch):
    """The host side of the differentiable token-clock read / write proposal (what is saved,
    which cotangent goes where) checked on the CPU: the three kernel entry points it calls are
    replaced by tensor expressions of what they compute, the gradients must then be the
    reference's autograd (tests/golden/token_gradients.npz). The kernels themselves are
    checked against the same file in tests/test_gpu_backward.py."""
    import numpy as np
    import golden_inputs as gi
    from conftest import load_golden
    from gl_sdm_b200 import _native

    def snapshot_read(values, index, weights, rows_per_bank, requests=None, **_):
        heads, slots = values.shape[1:3]
        flat = (requests.view(-1, 1, 1) * heads + torch.arange(heads).view(1, heads, 1)) * slots + index
        return (values.flatten(0, 2)[flat].float() * weights.unsqueeze(-1)).sum(-2)

    def commit_rows(values, idx, delta, keys, out=None, key_bits=0):
        return out.index_add_(0, idx, delta)

    monkeypatch.setattr(_native, "require_cuda", lambda *a: None)
    monkeypatch.setattr(_native, "snapshot_read", snapshot_read)
    monkeypatch.setattr(_native, "gather_rows", lambda flat, addresses: flat[addresses])
    monkeypatch.setattr(_native, "commit_rows", commit_rows)
    gold = load_golden("token_gradients")
    t = gi.token_case()
    names = ("memory", "weights", "targets", "beta", "log_decay", "mass")
    leaves = {k: t[k].clone().requires_grad_() for k in names}
    view = MemoryView(leaves["memory"])
    retrieved = read(view, t["requests"], t["indices"], leaves["weights"])
    p = propose_write(view, t["requests"], t["indices"], leaves["weights"], leaves["targets"], leaves["beta"],
                      leaves["log_decay"], leaves["mass"])
    cot_read, cot_delta = gi.cotangents("token", retrieved.shape, p.deltas.shape)
    grads = torch.autograd.grad((retrieved * cot_read).sum(), (leaves["memory"], leaves["weights"]))
    np.testing.assert_allclose(grads[0].numpy(), gold["read_grad_memory"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(grads[1].numpy(), gold["read_grad_weights"], rtol=1e-5, atol=1e-5)
    grads = torch.autograd.grad((p.deltas * cot_delta).sum(), [leaves[k] for k in names])
    for k, g in zip(names, grads):
        np.testing.assert_allclose(g.numpy(), gold[f"propose_grad_{k}"], rtol=1e-4, atol=1e-5, err_msg=k)


def test_concatenation_of_side_by_side_proposals_copies_nothing():
    """Proposals written into consecutive pieces of one buffer (gl_sdm_b200.layers) reach the
    commit as one tensor over the same memory; anything else is concatenated as before."""
    from gl_sdm_b200.memory import transactions
    buffer = torch.arange(24.0).view(12, 2)
    pieces = [buffer[0:3], buffer[3:8], buffer[8:12]]
    joined = transactions._concat(pieces)
    assert joined.data_ptr() == buffer.data_ptr() and torch.equal(joined, buffer)
    inner = transactions._concat([buffer[3:8], buffer[8:12]])
    assert inner.data_ptr() == buffer[3:].data_ptr() and torch.equal(inner, buffer[3:])
    for other in ([buffer[0:3], buffer[4:8]],                 # a gap
                  [buffer[3:8], buffer[0:3]],                 # out of order
                  [buffer[0:3], buffer[3:8].clone()],         # another allocation
                  [buffer[0:3], buffer[3:8].double()]):       # another type
        assert not transactions._adjacent(other)
    assert torch.equal(transactions._concat([buffer[3:8], buffer[0:3]]), torch.cat([buffer[3:8], buffer[0:3]]))
    leaf = torch.arange(24.0).view(12, 2).requires_grad_()
    tracked = [leaf[0:3], leaf[3:12]]
    assert not transactions._adjacent(tracked)                # their graphs must survive
    transactions._concat(tracked).sum().backward()
    assert torch.equal(leaf.grad, torch.ones(12, 2))
    with torch.no_grad():
        assert transactions._adjacent(tracked)
