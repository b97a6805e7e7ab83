"""Parity of the CUDA path (through the C ABI) with the reference's golden vectors and with
the numpy oracle. Integer outputs (routes, addresses, sort keys) must be bit-exact; float
outputs within the reference's own test tolerances (atol 1e-6, rtol 1e-5 in fp32; 2e-2 for
bf16 banks)."""
import numpy as np
import pytest
import torch

import golden_inputs as gi
from conftest import load_golden
from oracle import sdm_oracle as oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def cpu(t):
    return t.detach().cpu().numpy()


@pytest.fixture(autouse=True)
def _device_status_is_clean(native):
    yield
    native.raise_on_device_status(DEV)


# ---- routed read -----------------------------------------------------------------------------

@pytest.mark.parametrize("name", gi.ROUTED_CASES)
def test_routed_read_matches_reference_golden(native, name):
    from gl_sdm_b200.memory import routing
    gold = load_golden(f"routed_{name}")
    memory, scores, width = gi.routed_case(name)
    np.testing.assert_allclose(gold["checksum"], [gi.checksum(memory), gi.checksum(scores)], rtol=1e-12)
    values, s = memory.to(DEV), scores.to(DEV)
    readings, index, weights = routing.torch_routed_read(values, s, width)
    assert index.dtype == torch.int64
    np.testing.assert_array_equal(cpu(index), gold["index"].astype(np.int64))
    np.testing.assert_allclose(cpu(weights), gold["weights"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(cpu(readings), gold["readings"], rtol=1e-5, atol=1e-6)
    # the unfused pieces give the same answer: select alone, then read with supplied routes
    i32, w = native.pk_select(s, width, index_dtype=torch.int32)
    np.testing.assert_array_equal(cpu(i32), gold["index"])
    same = lambda a, b: torch.equal(torch.nan_to_num(a, nan=7.0), torch.nan_to_num(b, nan=7.0))  # noqa: E731
    assert same(w, weights)
    B, T, H, _ = scores.shape
    again = native.snapshot_read(values, i32, w, rows_per_bank=T * H)
    assert same(again, readings)
    # gather_rows / absolute_addresses
    rows = routing.gather_rows(values, index)
    np.testing.assert_array_equal(cpu(rows), oracle.gather_rows(memory.numpy(), gold["index"].astype(np.int64)))
    # reading only (no routes written) gives the same readings
    only, none_i, none_w = native.pk_select_read(values, s, width, rows_per_bank=T * H, want_routes=False)
    assert none_i is None and none_w is None and same(only, readings)


@pytest.mark.parametrize("half,width,dim,dtype", [
    (128, 16, 64, torch.float32), (1024, 32, 128, torch.bfloat16), (256, 32, 256, torch.bfloat16),
    (64, 8, 64, torch.bfloat16), (32, 5, 24, torch.float32), (512, 16, 128, torch.bfloat16),
    (16, 4, 512, torch.float32)])
def test_routed_read_matches_oracle_on_seeded_inputs(native, half, width, dim, dtype):
    """One shared bank (banks=1) and per-head partitions, bf16 and fp32 storage."""
    g = torch.Generator().manual_seed(half * 131 + width)
    H, N = (1 if half >= 1024 else 2), 96
    bank = (torch.randn(1, H, half * half, dim, generator=g) * 0.02).to(dtype)
    scores = torch.randn(3, N // 3, H, 2 * half, generator=g)
    scores[0, :4] = scores[0, :4].bfloat16().float().round()  # heavy ties
    readings, index, weights = native.pk_select_read(bank.to(DEV), scores.to(DEV), width, rows_per_bank=(N // 3) * H)
    o_read, o_index, o_weights = oracle.routed_read(bank.float().numpy(), scores.numpy(), width)
    np.testing.assert_array_equal(cpu(index), o_index)
    np.testing.assert_allclose(cpu(weights), o_weights, rtol=1e-5, atol=1e-6)
    tol = dict(rtol=1e-5, atol=1e-6) if dtype == torch.float32 else dict(rtol=2e-2, atol=1e-5)
    np.testing.assert_allclose(cpu(readings), o_read, **tol)


def test_routes_are_canonical_and_reads_are_linear(native):
    """Size-independent properties at a large shape: slots ascending and distinct, weights
    sum to one, and doubling the bank doubles the reading exactly."""
    g = torch.Generator().manual_seed(4)
    half, width, dim, rows = 1024, 32, 128, 4096
    bank = (torch.randn(1, 1, half * half, dim, generator=g) * 0.02).bfloat16().to(DEV)
    scores = torch.randn(1, rows, 1, 2 * half, generator=g).to(DEV)
    readings, index, weights = native.pk_select_read(bank, scores, width, rows_per_bank=rows)
    assert bool((index[..., 1:] > index[..., :-1]).all())
    assert int(index.min()) >= 0 and int(index.max()) < half * half
    torch.testing.assert_close(weights.sum(-1), torch.ones_like(weights[..., 0]), rtol=1e-5, atol=1e-5)
    doubled, _, _ = native.pk_select_read(bank * 2, scores, width, rows_per_bank=rows)
    assert torch.equal(doubled, readings * 2)
    again, index2, _ = native.pk_select_read(bank, scores, width, rows_per_bank=rows)
    assert torch.equal(again, readings) and torch.equal(index, index2)


def test_partial_reads_of_slot_shards_sum_to_the_full_read(native):
    g = torch.Generator().manual_seed(12)
    half, width, dim, rows, parts = 64, 8, 64, 300, 4
    bank = torch.randn(1, 2, half * half, dim, generator=g).to(DEV)
    scores = torch.randn(1, rows, 2, 2 * half, generator=g).to(DEV)
    full, index, weights = native.pk_select_read(bank, scores, width, rows_per_bank=rows * 2)
    total = torch.zeros_like(full)
    per = half * half // parts
    for r in range(parts):
        shard = bank[:, :, r * per:(r + 1) * per].contiguous()
        total += native.snapshot_read(shard, index, weights, rows_per_bank=rows * 2, slot_lo=r * per, slots=half * half)
    torch.testing.assert_close(total, full, rtol=1e-5, atol=1e-6)


def test_out_of_range_route_sets_the_device_status(native):
    bank = torch.zeros(1, 1, 16, 8, device=DEV)
    index = torch.tensor([[[[3, 16]]]], device=DEV)
    weights = torch.full((1, 1, 1, 2), 0.5, device=DEV)
    native.snapshot_read(bank, index, weights, rows_per_bank=1)
    with pytest.raises(RuntimeError, match="address out of range"):
        native.raise_on_device_status(DEV)


# ---- write proposal and commit ----------------------------------------------------------------

@pytest.mark.parametrize("name", gi.PROPOSE_CASES)
def test_propose_and_commit_match_reference_golden(native, name):
    from gl_sdm_b200.memory import MemoryView, WriteProposal, commit, merge
    gold = load_golden(f"propose_{name}")
    case = gi.propose_case(name)
    view = MemoryView(case["memory"].to(DEV))
    B, T, H, _ = case["scores"].shape
    proposals, reference_proposals = [], []
    for j, layer in enumerate(case["layers"]):
        scores = case["scores"] if j == 0 else case["extra_scores"][j - 1]
        addresses, deltas, keys = native.pk_propose(
            view.values, scores.to(DEV), case["target"].to(DEV), case["beta"].to(DEV), case["log_decay"].to(DEV),
            None, T, case["width"], case["offset"], case["chunk_size"], case["num_layers"], layer)
        np.testing.assert_array_equal(cpu(addresses), gold[f"addresses{j}"])
        np.testing.assert_array_equal(cpu(keys), gold[f"keys{j}"])
        np.testing.assert_allclose(cpu(deltas), gold[f"deltas{j}"], rtol=1e-5, atol=1e-7)
        proposals.append(WriteProposal(0, addresses, deltas, view.lineage, keys))
        reference_proposals.append(WriteProposal(0, addresses, torch.from_numpy(gold[f"deltas{j}"]).to(DEV),
                                                 view.lineage, keys))
    before = view.values.clone()
    after = commit(view, merge(view, proposals))
    assert after.version == 1 and after.lineage is view.lineage
    assert torch.equal(view.values, before), "commit must not modify its input view"
    flat = cpu(after.values).reshape(-1, before.shape[-1])
    np.testing.assert_allclose(flat[gold["touched"]], gold["touched_rows"], rtol=1e-5, atol=1e-7)
    untouched = np.ones(flat.shape[0], bool)
    untouched[gold["touched"]] = False
    np.testing.assert_array_equal(flat[untouched], cpu(before).reshape(flat.shape)[untouched])
    # With the reference's own deltas the ordered fp32 sums are reproduced bit for bit while
    # every address receives at most 256 entries (hot_slots exceeds that: blocked sums).
    exact = cpu(commit(view, merge(view, reference_proposals)).values).reshape(flat.shape)
    if name == "hot_slots":
        np.testing.assert_allclose(exact[gold["touched"]], gold["touched_rows"], rtol=1e-5, atol=1e-7)
    else:
        np.testing.assert_array_equal(exact[gold["touched"]], gold["touched_rows"])
    # arrival order of keyed proposals does not matter; repeats are bit-identical
    shuffled = commit(view, merge(view, list(reversed(proposals))))
    assert torch.equal(shuffled.values, after.values)
    for _ in range(3):
        assert torch.equal(commit(view, merge(view, proposals)).values, after.values)


def test_commit_known_answers_and_immutability(native):
    """projects/gl-sdm/tests/test_global_memory.py:27-54,69-73, test_native_memory.py:95-106,
    test_chunk_memory.py:43-51."""
    from gl_sdm_b200.memory import MemoryView, WriteProposal, commit, merge
    gold = load_golden("commit_cases")
    for name, (shape, idx, delta, keys) in gi.commit_cases().items():
        bank = gi.commit_random_bank(shape) if name == "random_duplicates" else torch.zeros(shape)
        view = MemoryView(bank.to(DEV))
        p = WriteProposal(0, idx.to(DEV), delta.to(DEV), view.lineage, None if keys is None else keys.to(DEV))
        result = commit(view, merge(view, [p]))
        np.testing.assert_array_equal(cpu(result.values), gold[f"{name}_out"])
        assert torch.equal(view.values.cpu(), bank)
        with pytest.raises(ValueError, match="stale"):
            commit(result, merge(view, [p]))
    view = MemoryView(torch.zeros(1, 1, 4, 1, device=DEV))
    p = WriteProposal(0, torch.tensor([0, 3, 0, 0, 3], device=DEV),
                      torch.tensor([[1e8], [0.125], [-1e8], [1.0], [0.25]], device=DEV), view.lineage)
    assert commit(view, merge(view, [p])).values.flatten().tolist() == [1.0, 0.0, 0.0, 0.375]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim", [64, 128, 256, 32, 48])
def test_commit_matches_oracle_with_random_keys(native, dim, dtype):
    """Random signed 64-bit keys exercise every radix digit; duplicates exercise stability."""
    g = torch.Generator().manual_seed(dim)
    rows, entries = 5000, 60000
    bank = torch.randn(rows, dim, generator=g).to(dtype)
    addresses = torch.randint(0, rows, (entries,), generator=g)
    minor = torch.randint(0, 64, (entries,), generator=g)
    keys = addresses * 64 + minor                      # groups addresses; repeated keys inside
    deltas = torch.randn(entries, dim, generator=g)
    out = native.commit_rows(bank.to(DEV), addresses.to(DEV), deltas.to(DEV), keys.to(DEV))
    want = oracle.commit(bank.float().numpy(), addresses.numpy(), deltas.numpy(), keys.numpy())
    if dtype == torch.float32:
        np.testing.assert_array_equal(cpu(out), want)
    else:
        np.testing.assert_array_equal(cpu(out.float()), torch.from_numpy(want).bfloat16().float().numpy())
    # the same entries with a key_bits hint, in place
    donated = bank.to(DEV).clone()
    same = native.commit_rows(donated, addresses.to(DEV), deltas.to(DEV), keys.to(DEV), out=donated, key_bits=20)
    assert same.data_ptr() == donated.data_ptr() and torch.equal(same, out)
    # unkeyed: arrival order inside an address
    unkeyed = native.commit_rows(bank.to(DEV), addresses.to(DEV), deltas.to(DEV), None)
    want = oracle.commit(bank.float().numpy(), addresses.numpy(), deltas.numpy(), None)
    got = cpu(unkeyed.float())
    np.testing.assert_array_equal(got, want if dtype == torch.float32 else torch.from_numpy(want).bfloat16().float().numpy())


def test_commit_sorts_full_width_signed_keys(native):
    """Keys spanning the signed 64-bit range, one entry per address: pure sort + scatter."""
    g = torch.Generator().manual_seed(99)
    rows = 4096
    addresses = torch.randperm(rows, generator=g)
    keys = torch.randint(-(1 << 62), 1 << 62, (rows,), generator=g)
    deltas = torch.randn(rows, 16, generator=g)
    bank = torch.zeros(rows, 16)
    out = native.commit_rows(bank.to(DEV), addresses.to(DEV), deltas.to(DEV), keys.to(DEV))
    np.testing.assert_array_equal(cpu(out), oracle.commit(bank.numpy(), addresses.numpy(), deltas.numpy(), keys.numpy()))


def test_commit_hot_slot_long_segments_are_deterministic(native):
    """Thousands of entries on a few addresses: blocked sums, repeatable bit for bit, close
    to the sequential oracle, and the bank total moves by the total of the deltas."""
    g = torch.Generator().manual_seed(5)
    rows, entries, dim = 64, 50000, 128
    hot = torch.tensor([3, 17, 40])
    addresses = torch.where(torch.rand(entries, generator=g) < 0.9, hot[torch.randint(0, 3, (entries,), generator=g)],
                            torch.randint(0, rows, (entries,), generator=g))
    keys = addresses * entries + torch.randperm(entries, generator=g)
    deltas = torch.randn(entries, dim, generator=g) * 0.01
    bank = torch.randn(rows, dim, generator=g)
    out = native.commit_rows(bank.to(DEV), addresses.to(DEV), deltas.to(DEV), keys.to(DEV))
    for _ in range(2):
        assert torch.equal(native.commit_rows(bank.to(DEV), addresses.to(DEV), deltas.to(DEV), keys.to(DEV)), out)
    want = oracle.commit(bank.numpy(), addresses.numpy(), deltas.numpy(), keys.numpy())
    np.testing.assert_allclose(cpu(out), want, rtol=1e-4, atol=5e-5)
    moved = cpu(out).astype(np.float64).sum() - bank.numpy().astype(np.float64).sum()
    np.testing.assert_allclose(moved, deltas.numpy().astype(np.float64).sum(), rtol=0, atol=1e-2)


def test_empty_and_single_entry_commits(native):
    bank = torch.randn(8, 4, device=DEV)
    none = native.commit_rows(bank, torch.empty(0, dtype=torch.long, device=DEV), torch.empty(0, 4, device=DEV))
    assert torch.equal(none, bank) and none.data_ptr() != bank.data_ptr()
    one = native.commit_rows(bank, torch.tensor([5], device=DEV), torch.ones(1, 4, device=DEV))
    assert torch.equal(one[5], bank[5] + 1) and torch.equal(one[:5], bank[:5])
    native.commit_rows(bank, torch.tensor([8], device=DEV), torch.ones(1, 4, device=DEV))
    with pytest.raises(RuntimeError, match="address out of range"):
        native.raise_on_device_status(DEV)


# ---- token-clock API ----------------------------------------------------------------------------

def test_token_api_matches_reference_golden(native):
    """projects/gl-sdm/tests/test_native_memory.py:52-92, forward part."""
    from gl_sdm_b200.memory import MemoryView, commit, merge, propose_write, read
    gold = load_golden("token_api")
    t = {k: v.to(DEV) for k, v in gi.token_case().items()}
    view = MemoryView(t["memory"])
    retrieved = read(view, t["requests"], t["indices"], t["weights"], backend="urm")
    np.testing.assert_allclose(cpu(retrieved), gold["read"], rtol=2e-6, atol=5e-7)
    p = propose_write(view, t["requests"], t["indices"], t["weights"], t["targets"], t["beta"], t["log_decay"], t["mass"])
    p2 = propose_write(view, t["requests"], t["indices"], t["weights"], t["targets"] * 2, t["beta"], t["log_decay"],
                       1 - t["mass"], backend="urm")
    np.testing.assert_array_equal(cpu(p.addresses), gold["addresses"])
    np.testing.assert_allclose(cpu(p.deltas), gold["deltas"], rtol=2e-6, atol=5e-7)
    np.testing.assert_allclose(cpu(p2.deltas), gold["deltas2"], rtol=2e-6, atol=5e-7)
    updated = commit(view, merge(view, [p, p2]), backend="urm")
    np.testing.assert_allclose(cpu(updated.values), gold["updated"], rtol=2e-6, atol=1e-6)
    for _ in range(4):
        assert torch.equal(commit(view, merge(view, [p, p2])).values, updated.values)


# ---- shard merge -----------------------------------------------------------------------------------

def test_topk_merge_matches_oracle(native):
    g = torch.Generator().manual_seed(8)
    parts, rows, width = 4, 500, 16
    score = (torch.randn(parts, rows, width, generator=g) * 2).round() / 2     # ties across shards
    slot = torch.stack([torch.stack([torch.randperm(1000, generator=g)[:width] + 1000 * p for _ in range(rows)])
                        for p in range(parts)]).int()
    slot[3, :, -2:] = -1                                                        # short shard lists
    index, weights = native.topk_merge(score.to(DEV), slot.to(DEV))
    want_slot, want_w = oracle.merge_candidates(slot.numpy(), score.numpy(), width)
    np.testing.assert_array_equal(cpu(index), want_slot)
    np.testing.assert_allclose(cpu(weights), want_w, rtol=1e-5, atol=1e-6)


# ---- edge cases -----------------------------------------------------------------------------------

def test_empty_and_minimal_shapes(native):
    """Zero rows launch nothing; one slot, one route and width > slots behave as the reference
    (projects/gl-sdm/src/gl_sdm/memory/routing.py slices what exists)."""
    bank = torch.randn(1, 1, 1, 4, device=DEV)
    out, index, weights = native.pk_select_read(bank, torch.zeros(1, 3, 1, 2, device=DEV), 1, rows_per_bank=3)
    assert index.flatten().tolist() == [0, 0, 0] and weights.flatten().tolist() == [1.0, 1.0, 1.0]
    assert torch.equal(out, bank.expand(1, 3, 1, 4))
    empty_scores = torch.zeros(1, 0, 1, 2, device=DEV)
    out, index, weights = native.pk_select_read(bank, empty_scores, 1, rows_per_bank=1)
    assert out.shape == (1, 0, 1, 4) and index.numel() == 0
    # width larger than the slots of a 2 x 2 product: all four slots, ascending
    bank4 = torch.randn(1, 1, 4, 8, device=DEV)
    scores = torch.tensor([[[[0.5, -1.0, 2.0, 0.25]]]], device=DEV)
    out, index, weights = native.pk_select_read(bank4, scores, 7, rows_per_bank=1)
    want_read, want_index, want_w = oracle.routed_read(bank4.cpu().numpy(), scores.cpu().numpy(), 7)
    np.testing.assert_array_equal(cpu(index), want_index)
    np.testing.assert_allclose(cpu(weights), want_w, rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(cpu(out), want_read, rtol=1e-5, atol=1e-6)


def test_unsupported_shapes_are_refused_not_approximated(native):
    bank = torch.zeros(1, 1, 64 * 64, 8, device=DEV)
    with pytest.raises(ValueError, match="not supported"):
        native.pk_select(torch.zeros(2, 128, device=DEV), 33)          # more than 32 routes
    with pytest.raises(ValueError, match="invalid argument"):
        native.pk_select_read(bank, torch.zeros(1, 2, 1, 64, device=DEV), 4, rows_per_bank=2)  # half^2 != slots
    with pytest.raises(ValueError, match="float32"):
        native.pk_select(torch.zeros(2, 128, device=DEV, dtype=torch.bfloat16), 4)
    with pytest.raises(ValueError, match="contiguous CUDA"):
        native.pk_select(torch.zeros(2, 256, device=DEV)[:, ::2], 4)


def test_nan_and_infinite_scores_follow_the_sort_order_of_the_reference(native):
    """torch sorts NaN above +inf; -inf stays last; the selection must agree on the slots."""
    g = torch.Generator().manual_seed(2)
    scores = torch.randn(1, 16, 1, 32, generator=g)
    scores[0, 0, 0, 3] = float("inf")
    scores[0, 1, 0, 5] = float("-inf")
    scores[0, 2, 0, :16] = float("-inf")
    scores[0, 3, 0, 20] = float("inf")
    scores[0, 3, 0, 2] = float("inf")
    index, _ = native.pk_select(scores.to(DEV), 4)
    want, _ = oracle.select_routes(scores.numpy(), 4)
    np.testing.assert_array_equal(cpu(index), want)


@pytest.mark.parametrize("half,width", [(256, 8), (512, 32), (1024, 32), (4096, 32), (2048, 16), (4096, 1), (260, 7)])
def test_long_factor_selection_is_exact_on_awkward_rows(native, half, width):
    """Long factors take a two-pass selection (group maxima bound, then one sort) that hands a
    row back to the streaming selector when too many elements reach the bound. Whatever path
    a row takes, the routes are the reference's (gl_sdm/memory/routing.py:10-26), bit-exact:
    plain and bf16-rounded normals, integer grids (ties everywhere), constants, monotone
    rows, all winners on one lane, NaN and infinities, signed zeros."""
    g = torch.Generator().manual_seed(half + width)
    rows = []
    rows.append(torch.randn(6, 2 * half, generator=g))
    rows.append(torch.randn(6, 2 * half, generator=g).bfloat16().float())
    rows.append(torch.randint(-3, 4, (4, 2 * half), generator=g).float())
    rows.append(torch.zeros(1, 2 * half))
    rows.append(torch.arange(2 * half, dtype=torch.float32).view(1, -1))
    rows.append(-torch.arange(2 * half, dtype=torch.float32).view(1, -1))
    lane_heavy = torch.randn(2, 2 * half, generator=g)
    lane_heavy[:, 0:half:128] += 8.0            # every winner of the left factor sits on lane 0
    lane_heavy[:, half + 5::128] += 8.0
    rows.append(lane_heavy)
    special = torch.randn(5, 2 * half, generator=g)
    special[0, 7] = float("nan")
    special[0, half + 9] = float("nan")
    special[1, :40] = float("inf")
    special[2, half:half + 200] = float("-inf")
    special[3, ::3] = -0.0
    special[3, 1::3] = 0.0
    special[4, :half] = float("nan")
    rows.append(special)
    scores = torch.cat(rows).view(1, -1, 1, 2 * half).contiguous()
    index, weights = native.pk_select(scores.to(DEV), width)
    want_index, want_weights = oracle.select_routes(scores.numpy(), width)
    np.testing.assert_array_equal(cpu(index), want_index)
    finite = np.isfinite(want_weights).all(axis=-1)
    np.testing.assert_allclose(cpu(weights)[finite], want_weights[finite], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("name", gi.STEP_CASES)
def test_c1_step_through_the_memory_api_matches_the_reference(native, name):
    """The per-request-bank benchmark configurations (all of c1: two commit epochs; one request
    and chunk of c2: eight layers writing into one commit), one whole step through
    gl_sdm_b200.memory with the call sequence bench.py times, against the same step driven
    through the reference's gl_sdm.memory (tests/golden/c1_step.npz, c2_chunk_step.npz)."""
    import bench
    import gl_sdm_b200.memory as memory
    gold = load_golden(name)
    w, values, inputs = gi.c1_step_case(name)
    moved = [[{k: v.to(DEV) for k, v in x.items()} for x in layers] for layers in inputs]
    before = values.clone()
    on_device = values.to(DEV)
    readings, view = bench.api_step(w, on_device, moved, memory)
    assert view.version == w.epochs
    assert torch.equal(on_device.cpu(), before)        # functional commits: the input bank is untouched
    gi.assert_c1_step(view.values, readings, gold, rtol=1e-5)
    native.raise_on_device_status(DEV)
