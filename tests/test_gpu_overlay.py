"""Copy-free versioned commits: the new view equals the reference's functional commit, and
every older view stays readable bit-for-bit (reference semantics: a commit never changes its
input view, gl_sdm/memory/transactions.py:96-97; the overlay representation is the reference's
own plan, OPTIMIZATION_PLAN.md "Represent commits as compact overlays")."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def native():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from gl_sdm_b200 import _native
    _native.library()
    return _native


def proposal(view, entries, seed, hot=None):
    from gl_sdm_b200.memory import WriteProposal
    g = torch.Generator().manual_seed(seed)
    B, H, S, D = view._storage.shape
    addresses = torch.randint(0, B * H * S, (entries,), generator=g)
    if hot is not None:
        addresses[: hot[1]] = hot[0]
    deltas = torch.randn(entries, D, generator=g) * 0.1
    keys = addresses * entries + torch.randperm(entries, generator=g)
    return WriteProposal(view.version, addresses.to(DEV), deltas.to(DEV), view.lineage, keys.to(DEV))


@pytest.mark.parametrize("dtype,shape", [(torch.float32, (2, 2, 64, 16)), (torch.bfloat16, (1, 1, 4096, 128)),
                                         (torch.bfloat16, (1, 2, 512, 256)), (torch.float32, (1, 3, 50, 7))])
def test_overlay_commit_matches_functional_commit_and_keeps_old_views(native, dtype, shape):
    from gl_sdm_b200.memory import MemoryView, commit, merge, overlay
    g = torch.Generator().manual_seed(5)
    bank = torch.randn(shape, generator=g).to(dtype).to(DEV)
    B, H, S, D = shape
    K, T = 4, 9
    index = torch.randint(0, S, (B, T, H, K), generator=g).sort(-1).values.to(DEV)
    weights = torch.randn(B, T, H, K, generator=g).softmax(-1).to(DEV)

    functional = MemoryView(bank.clone())
    live = MemoryView(bank.clone())
    held, copies = [live], [functional]
    for step in range(3):
        p = proposal(live, 300, 10 + step, hot=(7, 40))
        q = type(p)(functional.version, p.addresses, p.deltas, functional.lineage, p.sort_keys)
        functional = commit(functional, merge(functional, [q]))
        newer = commit(live, merge(live, [p]), donate="overlay")
        assert newer.version == live.version + 1 and newer.lineage is live.lineage
        assert live.stale and not newer.stale
        assert newer.values.data_ptr() == held[0]._storage.data_ptr()      # no bank copy was made
        assert torch.equal(newer.values, functional.values)                 # bit-exact new version
        live = newer
        held.append(live)
        copies.append(functional)
    # every held version reads exactly like its functional twin, without being rebuilt
    for view, twin in zip(held, copies):
        want = native.snapshot_read(twin.values, index, weights, rows_per_bank=T * H)
        got = overlay.read(view, index, weights)
        assert torch.equal(got, want), f"version {view.version}"
    assert held[0].stale and len(overlay.logs_of(held[0])) == 3 and len(overlay.logs_of(held[2])) == 1
    # ... and rebuilds to exactly the old bank on demand
    for view, twin in zip(held, copies):
        assert torch.equal(view.values, twin.values)
    assert not held[0].stale and held[0].values.data_ptr() != live.values.data_ptr()
    native.raise_on_device_status(DEV)


def test_long_segment_rows_are_logged(native):
    from gl_sdm_b200.memory import MemoryView, commit, merge
    bank = torch.randn(1, 1, 128, 64, generator=torch.Generator().manual_seed(2)).to(DEV)
    view = MemoryView(bank.clone())
    p = proposal(view, 2000, 3, hot=(5, 900))       # 900 entries on one address: block-per-segment path
    newer = commit(view, merge(view, [p]), donate="overlay")
    twin = commit(MemoryView(bank.clone(), 0, view.lineage), merge(view, [p]))
    assert torch.equal(newer.values, twin.values)
    assert torch.equal(view.values, bank)


def test_routed_read_of_a_stale_view(native):
    from gl_sdm_b200.memory import MemoryView, commit, merge, overlay, routing
    g = torch.Generator().manual_seed(8)
    bank = (torch.randn(2, 2, 256, 32, generator=g) * 0.1).to(DEV)
    scores = torch.randn(2, 11, 2, 32, generator=g).to(DEV)
    view = MemoryView(bank.clone())
    before = routing.torch_routed_read(view.values, scores, 4)
    newer = commit(view, merge(view, [proposal(view, 500, 4)]), donate="overlay")
    after = overlay.routed_read(view, scores, 4)
    for a, b in zip(before, after):
        assert torch.equal(a, b)
    changed = overlay.routed_read(newer, scores, 4)[0]
    assert not torch.equal(changed, before[0])


def test_invalidated_and_misused_views(native):
    from gl_sdm_b200.memory import MemoryView, commit, merge, overlay
    bank = torch.zeros(1, 1, 16, 4, device=DEV)
    v0 = MemoryView(bank)
    v1 = commit(v0, merge(v0, [proposal(v0, 8, 1)]), donate="overlay")
    with pytest.raises(ValueError, match="newest view"):
        commit(v0, merge(v0, [proposal(v0, 8, 2)]), donate="overlay")
    with pytest.raises(ValueError, match="donate must be"):
        commit(v1, merge(v1, [proposal(v1, 8, 2)]), donate="yes")
    commit(v1, merge(v1, [proposal(v1, 8, 2)]), donate=True)             # no log: v0 cannot be rebuilt any more
    with pytest.raises(RuntimeError, match="invalidated"):
        v0.values
    with pytest.raises(RuntimeError, match="invalidated"):
        overlay.read(v0, torch.zeros(1, 1, 1, 2, dtype=torch.long, device=DEV), torch.ones(1, 1, 1, 2, device=DEV))


def test_views_far_behind_are_rebuilt_once(native):
    from gl_sdm_b200.memory import MemoryView, commit, merge, overlay
    g = torch.Generator().manual_seed(12)
    bank = torch.randn(1, 1, 64, 8, generator=g).to(DEV)
    first = MemoryView(bank.clone())
    live = first
    for step in range(native.MAX_UNDO_LOGS + 2):
        live = commit(live, merge(live, [proposal(live, 20, 30 + step)]), donate="overlay")
    index = torch.arange(64, device=DEV).view(1, 16, 1, 4)
    weights = torch.ones(1, 16, 1, 4, device=DEV)
    got = overlay.read(first, index, weights)
    assert not first.stale                                                 # rebuilt, not chained
    assert torch.equal(got, native.snapshot_read(bank, index, weights, rows_per_bank=16))
    np.testing.assert_array_equal(first.values.cpu().numpy(), bank.cpu().numpy())


def test_keys_that_group_but_do_not_ascend_are_flagged(native):
    """Keys only have to group equal addresses for the commit itself, but the overlay read
    bisects the undo log: keys that order the addresses downwards must set the status bit (and
    the rebuild through glsdm_undo_apply stays right whatever the order)."""
    g = torch.Generator().manual_seed(3)
    bank = torch.randn(1, 1, 64, 16, generator=g).to(DEV)
    before = bank.clone()
    addresses = torch.tensor([5, 9, 5, 40, 9], device=DEV)
    deltas = torch.randn(5, 16, generator=g).to(DEV)
    keys = (63 - addresses) * 8 + torch.arange(5, device=DEV)        # groups, but descending in the address
    log_addresses, log_rows = native.commit_undo(bank, addresses, deltas, keys)
    assert log_addresses.tolist() == [40, 9, 9, 5, 5]
    with pytest.raises(RuntimeError, match="not ascending"):
        native.raise_on_device_status(DEV)
    native.undo_apply(bank, log_addresses, log_rows)
    assert torch.equal(bank, before)
    # ascending keys leave the status clear
    native.commit_undo(bank, addresses, deltas, addresses * 8 + torch.arange(5, device=DEV))
    native.raise_on_device_status(DEV)
