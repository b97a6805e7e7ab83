"""Dense-key routing on the tensor cores (glsdm_score_topk) against the CPU oracle.

The scoring stage q @ keys^T has no counterpart in the reference (parity unpinned): the
oracle computes it in float32 on the CPU, the kernel with bf16 tensor-core products (exact in
float32) accumulated in float32 in a different order. What is checked:
  * every reported score lies within the forward error bound of a d_k-term float32 sum,
    2 * d_k * 2^-24 * sum_i |q_i * k_i| (twice the round-to-nearest bound: the accumulator of
    the tensor cores may truncate), and the largest discrepancy actually seen is kept;
  * the selected slots are identical to the oracle's, except on rows where a slot only one of
    the two took lies within FOUR times that largest discrepancy of the oracle's k-th score
    ("documented exact-score ties"): EVERY differing row is audited, and they are counted;
  * the selection rule itself (score descending, larger slot first among equals) is pinned
    by rows with bit-equal scores (duplicated keys);
  * NaN scores are never candidates (the documented behaviour of glsdm_score_topk)."""
import numpy as np
import pytest
import torch

from oracle import sdm_oracle as oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
UNIT = 2.0 ** -24


def error_bound(q, keys, slots):
    """Forward bound of the float32 sum for the given (row, slot) pairs: [rows, width]."""
    magnitude = np.abs(q.float().numpy()) @ np.abs(keys.float().numpy()).T
    return 2 * q.shape[1] * UNIT * np.take_along_axis(magnitude, slots, 1)


def audit_rows(scores, got_slot, want_slot, want_score, window, col_base=0):
    """Every row whose slots differ from the oracle's must differ only through slots within
    `window` of the oracle's k-th score. Returns how many rows that is."""
    exempt = 0
    for r in np.flatnonzero((np.sort(got_slot, 1) != np.sort(want_slot, 1)).any(1)):
        boundary = want_score[r].min()
        for s in set(got_slot[r].tolist()) ^ set(want_slot[r].tolist()):
            gap = abs(scores[r, s - col_base] - boundary)
            assert gap <= window, f"row {r}: slot {s} is {gap} from the k-th score, window {window}"
        exempt += 1
    return exempt


def _case(rows, slots, dk, seed, duplicate=0):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(rows, dk, generator=g).bfloat16()
    keys = torch.randn(slots, dk, generator=g)
    keys = (keys / keys.norm(dim=1, keepdim=True)).bfloat16()
    if duplicate:
        keys[slots - duplicate:] = keys[:duplicate]          # bit-equal scores at two slots
    return q, keys


def _check(q, keys, width, got_score, got_slot, col_base=0):
    scores = oracle.flat_scores(q.float().numpy(), keys.float().numpy())
    want_slot, want_score = oracle.top_routes(scores, width, slot_base=col_base)
    got_slot, got_score = got_slot.cpu().numpy().astype(np.int64), got_score.cpu().numpy()
    assert (got_slot >= col_base).all() and (got_slot < col_base + keys.shape[0]).all()
    # scores reported for the chosen slots are the oracle's scores of those slots, to the bound
    off = np.abs(got_score - np.take_along_axis(scores, got_slot - col_base, 1))
    assert (off <= error_bound(q, keys, got_slot - col_base)).all()
    seen = float(off.max())
    # best first, and slots distinct
    assert (np.diff(got_score, axis=1) <= 0).all()
    assert all(len(set(r)) == width for r in got_slot)
    window = max(4 * seen, 1e-7)
    exempt = audit_rows(scores, got_slot, want_slot, want_score, window, col_base)
    # rows with the oracle's slots in another order: their scores must tie within the window too
    for r in np.flatnonzero((got_slot != want_slot).any(1)):
        if set(got_slot[r].tolist()) == set(want_slot[r].tolist()):
            np.testing.assert_allclose(np.sort(got_score[r]), np.sort(want_score[r]), rtol=0, atol=window)
    print(f"score_topk {q.shape[0]}x{keys.shape[0]}: largest score discrepancy {seen:.2e}, "
          f"{exempt} documented near-tie rows")
    assert exempt <= max(2, q.shape[0] // 100), f"{exempt} rows differ from the oracle"
    return exempt


@pytest.fixture(params=[0, 2], ids=["one-cta", "wide-tile"])
def variant(native, request):
    """Run a test under both kernels behind glsdm_score_topk: 128x128x16 MMAs over 256 rows and
    128x256x16 MMAs over 128 rows (the default)."""
    lib = native.library()
    before = lib.glsdm_score_topk_variant(request.param)
    yield request.param
    lib.glsdm_score_topk_variant(before)


@pytest.mark.parametrize("rows,slots,dk,width", [(300, 5000, 128, 32), (256, 4096, 64, 16), (1000, 70000, 128, 32),
                                                 (40, 1000, 128, 8), (513, 16384, 64, 32)])
def test_score_topk_matches_oracle(native, variant, rows, slots, dk, width):
    q, keys = _case(rows, slots, dk, seed=rows + slots)
    score, slot = native.score_topk(q.to(DEV), keys.to(DEV), width)
    native.raise_on_device_status(DEV)
    _check(q, keys, width, score, slot)


def test_score_topk_tie_rule_and_shard_offset(native, variant):
    """Duplicated keys give bit-equal scores at slot s and s + slots - 500: the larger slot
    must come first; col_base shifts the reported slots of a shard."""
    q, keys = _case(200, 3000, 128, seed=5, duplicate=500)
    score, slot = native.score_topk(q.to(DEV), keys.to(DEV), 16, col_base=7000)
    native.raise_on_device_status(DEV)
    _check(q, keys, 16, score, slot, col_base=7000)
    got_slot, got_score = slot.cpu().numpy() - 7000, score.cpu().numpy()
    pairs = 0
    for r in range(200):
        where = {int(s): i for i, s in enumerate(got_slot[r])}
        for s, i in where.items():
            twin = s + 2500
            if s < 500 and twin in where:
                assert got_score[r, i] == got_score[r, where[twin]] and where[twin] < i
                pairs += 1
    assert pairs > 50


def test_score_topk_feeds_the_merge_and_read(native):
    """Two key shards -> candidates -> glsdm_topk_merge -> canonical routes, against the oracle's
    flat routes; then a snapshot read with those routes."""
    q, keys = _case(128, 4096, 128, seed=9)
    halves = [native.score_topk(q.to(DEV), keys[i * 2048:(i + 1) * 2048].contiguous().to(DEV), 8, col_base=i * 2048)
              for i in range(2)]
    cand_score = torch.stack([h[0] for h in halves])
    cand_slot = torch.stack([h[1] for h in halves])
    index, weights = native.topk_merge(cand_score, cand_slot)
    scores = oracle.flat_scores(q.float().numpy(), keys.float().numpy())
    want_slot, want_w = oracle.canonical_routes(*oracle.top_routes(scores, 8))
    same = (index.cpu().numpy() == want_slot).all(1)
    top_slot, top_score = oracle.top_routes(scores, 8)
    assert audit_rows(scores, index.cpu().numpy(), top_slot, top_score, 2e-6) == int((~same).sum()) <= 2
    np.testing.assert_allclose(weights.cpu().numpy()[same], want_w[same], rtol=1e-4, atol=1e-5)
    bank = torch.randn(1, 1, 4096, 64, generator=torch.Generator().manual_seed(1)).to(DEV)
    out = native.snapshot_read(bank, index.view(1, 128, 1, 8), weights.view(1, 128, 1, 8), rows_per_bank=128)
    want = oracle.weighted_read(bank.cpu().numpy(), index.cpu().numpy().reshape(1, 128, 1, 8),
                                weights.cpu().numpy().reshape(1, 128, 1, 8))
    np.testing.assert_allclose(out.cpu().numpy(), want, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("rows,half,width", [(300, 256, 8), (1024, 1024, 32), (130, 64, 16)])
def test_pk_gemm_select_matches_the_product_key_oracle(native, rows, half, width):
    """Product-key routing straight from queries and sub-key codebooks (factor scores never
    materialised): routes equal the oracle's except on rows with a near-tie at a boundary."""
    g = torch.Generator().manual_seed(rows + half)
    q = torch.randn(rows, 128, generator=g).bfloat16()
    books = torch.randn(2, half, 64, generator=g)
    books = (books / books.norm(dim=-1, keepdim=True)).bfloat16()
    index, weights = native.pk_gemm_select(q.to(DEV), books.to(DEV), width)
    native.raise_on_device_status(DEV)
    scores = oracle.pk_gemm_scores(q.float().numpy(), books.float().numpy())
    want_index, want_weights = oracle.select_routes(scores.reshape(1, rows, 1, -1), width)
    want_index, want_weights = want_index.reshape(rows, -1), want_weights.reshape(rows, -1)
    got = index.cpu().numpy()
    assert (np.diff(got, axis=1) > 0).all() and got.min() >= 0 and got.max() < half * half
    same = (got == want_index).all(1)
    np.testing.assert_allclose(weights.cpu().numpy()[same], want_weights[same], rtol=1e-4, atol=1e-5)
    # every row that differs must differ only through candidates whose sums (two 64-term
    # float32 sums each) tie within 4e-5
    left, right = scores[:, :half], scores[:, half:]
    window = 4e-5
    for r in np.flatnonzero(~same):
        boundary = np.sort((left[r][:, None] + right[r][None, :]).ravel())[-width]
        for s in set(got[r]) ^ set(want_index[r]):
            assert abs(left[r, s // half] + right[r, s % half] - boundary) <= window
    print(f"pk_gemm {rows}x{half}^2: {(~same).sum()} documented near-tie rows, window {window:.1e}")
    assert (~same).sum() <= max(2, rows // 50), f"{(~same).sum()} of {rows} rows differ"


def test_nan_scores_are_never_candidates(native, variant):
    """glsdm_score_topk keeps the `width` largest scores that are not NaN: a slot whose key holds
    a NaN is never selected, and a row whose query holds a NaN has no candidates at all - its
    list is padding (score -inf, slot -1), which glsdm_topk_merge ranks below every real
    candidate. (The product-key kernels follow the reference's sort order, NaN first; a dense
    score can only be NaN when the operands already are.)"""
    q, keys = _case(300, 5000, 128, seed=21)
    keys[7] = float("nan")
    keys[4000] = float("nan")
    q[5] = float("nan")
    score, slot = native.score_topk(q.to(DEV), keys.to(DEV), 16)
    native.raise_on_device_status(DEV)
    got_slot, got_score = slot.cpu().numpy().astype(np.int64), score.cpu().numpy()
    assert (got_slot[5] == -1).all() and np.isneginf(got_score[5]).all()
    rest = np.r_[0:5, 6:300]
    assert not np.isin(got_slot[rest], [7, 4000]).any() and np.isfinite(got_score[rest]).all()
    clean = keys.clone()
    clean[7] = 0
    clean[4000] = 0
    scores = oracle.flat_scores(q.float().numpy()[rest], clean.float().numpy())
    scores[:, [7, 4000]] = -np.inf
    want_slot, want_score = oracle.top_routes(scores, 16)
    assert audit_rows(scores, got_slot[rest], want_slot, want_score, 2e-6) <= 3


def test_tail_split_units_agree_with_the_uniform_plan(native):
    """More row blocks than SMs and a long slot range: the wide-tile kernel keeps one split for
    the blocks that fill whole waves and cuts only the last wave's blocks in parts. Its routes
    must be those of the 128x128 kernel (pinned to the oracle above), row for row."""
    lib = native.library()
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    rows, slots, width = (sms + 20) * 128 - 37, 1 << 20, 32
    g = torch.Generator(device=DEV).manual_seed(77)
    q = torch.randn(rows, 128, generator=g, device=DEV).bfloat16()
    k = torch.randn(slots, 128, generator=g, device=DEV)
    k = (k / k.norm(dim=1, keepdim=True)).bfloat16()
    before = lib.glsdm_score_topk_variant(0)
    try:
        want_score, want_slot = native.score_topk(q, k, width, col_base=5)
        lib.glsdm_score_topk_variant(2)
        got_score, got_slot = native.score_topk(q, k, width, col_base=5)
    finally:
        lib.glsdm_score_topk_variant(before)
    native.raise_on_device_status(DEV)
    order_w, order_g = torch.sort(want_slot, dim=-1), torch.sort(got_slot, dim=-1)
    assert torch.equal(order_w.values, order_g.values)
    assert torch.equal(torch.gather(want_score, -1, order_w.indices), torch.gather(got_score, -1, order_g.indices))


@pytest.mark.parametrize("rows,slots,width", [(300, 4096, 8), (5000, 1 << 18, 32), ((148 + 20) * 128 - 37, 1 << 19, 32)])
def test_bounded_routing_keeps_exactly_what_reaches_the_bound(native, rows, slots, width):
    """glsdm_score_topk_bounded on one shard with the K-th best score of ANOTHER shard as the
    row bound: every list is the unbounded list cut at the bound (scores equal to the bound
    stay), padded with (-inf, slot -1); merged with the other shard's list the routes are
    those of the unbounded pair. A bound above every score empties the row."""
    g = torch.Generator(device=DEV).manual_seed(rows + width)
    q = torch.randn(rows, 128, generator=g, device=DEV).bfloat16()
    k = torch.randn(2 * slots, 128, generator=g, device=DEV)
    k = (k / k.norm(dim=1, keepdim=True)).bfloat16()
    k[slots:slots + 64] = k[:64]                                       # bit-equal scores across the shards
    here, there = k[:slots].contiguous(), k[slots:].contiguous()
    free_score, free_slot = native.score_topk(q, here, width, col_base=0)
    peer_score, peer_slot = native.score_topk(q, there, width, col_base=slots)
    bound = peer_score[:, width - 1].contiguous()
    bound[::7] = float("inf")                                          # rows this shard cannot contribute to
    bound[3::7] = float("-inf")                                        # rows without any knowledge
    got_score, got_slot = native.score_topk(q, here, width, col_base=0, row_floor=bound)
    native.raise_on_device_status(DEV)
    keep = free_score >= bound.unsqueeze(1)
    assert torch.equal(got_slot >= 0, keep)
    assert torch.equal(got_slot[keep], free_slot[keep]) and torch.equal(got_score[keep], free_score[keep])
    assert (got_score[~keep] == float("-inf")).all() and (got_slot[~keep] == -1).all()
    assert not keep[::7].any() and keep[3::7].all()
    usable = torch.ones(rows, dtype=torch.bool, device=DEV)
    usable[::7] = False                                                # their bound was not a true one
    want = native.topk_merge(torch.stack([free_score, peer_score]), torch.stack([free_slot, peer_slot]))
    got = native.topk_merge(torch.stack([got_score, peer_score]), torch.stack([got_slot, peer_slot]))
    assert torch.equal(got[0][usable], want[0][usable]) and torch.equal(got[1][usable], want[1][usable])


def test_bounds_pushed_by_one_shard_are_read_by_the_next(native):
    """glsdm_score_topk_shared, two shards of one bank on one GPU, one after the other: the
    first stores the K-th best score of every row in the second's floor_in; the second, which
    walks a rotated copy of the rows, keeps exactly the candidates that reach those bounds, and
    the merged routes are those of two unbounded shards."""
    rows, slots, width, shift = 5000, 1 << 18, 32, 128 * 17
    g = torch.Generator(device=DEV).manual_seed(5)
    q = torch.randn(rows, 128, generator=g, device=DEV).bfloat16()
    k = torch.randn(2 * slots, 128, generator=g, device=DEV)
    k = (k / k.norm(dim=1, keepdim=True)).bfloat16()
    first, second = k[:slots].contiguous(), k[slots:].contiguous()
    inbox = torch.full((1, rows), float("-inf"), device=DEV)
    a_score, a_slot = native.score_topk(q, first, width, col_base=0, floor_out=[inbox[0].data_ptr()])
    # 40 row blocks on 148 SMs: the slot range is cut in parts, and a part's K-th best is what gets stored
    assert (inbox[0] <= a_score[:, width - 1]).all() and (inbox[0] > float("-inf")).all()
    free_score, free_slot = native.score_topk(q, second, width, col_base=slots)
    turned = torch.roll(q, -shift, 0).contiguous()             # logical row l is row (l + shift) % rows
    outbox = torch.full((rows,), float("-inf"), device=DEV)
    b_score, b_slot = native.score_topk(turned, second, width, col_base=slots, floor_in=inbox,
                                        floor_out=[outbox.data_ptr()], row_shift=shift)
    b_score, b_slot = torch.roll(b_score, shift, 0), torch.roll(b_slot, shift, 0)
    native.raise_on_device_status(DEV)
    keep = free_score >= inbox[0].unsqueeze(1)
    assert torch.equal(b_slot >= 0, keep) and torch.equal(b_slot[keep], free_slot[keep])
    assert (outbox <= free_score[:, width - 1]).all()
    assert (outbox[~keep[:, width - 1]] == float("-inf")).all()   # fewer than K reached the bound: nothing to tell
    want = native.topk_merge(torch.stack([a_score, free_score]), torch.stack([a_slot, free_slot]))
    got = native.topk_merge(torch.stack([a_score, b_score]), torch.stack([a_slot, b_slot]))
    assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])
    assert 0.02 < keep.float().mean().item() < 0.99            # the bounds did prune
