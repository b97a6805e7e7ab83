"""Checks that run the UNMODIFIED reference stack (oracle/_ref) over this package.

Shared by the CPU dry run (kernels replaced by stand-ins, tests/test_ref_stack_cpu.py) and
the GPU tests proper (tests/test_gpu_ref_stack.py). The oracle is the same reference source
bound to its own memory package (torch path). Bounds are the reference's own gate
(gl_sdm/experiments/verify.py:98-165): fp32 logits atol 5e-4 / rtol 3e-3, fp32 gradients
atol 1e-5 / rtol 5e-3, continuation and causality atol 1e-4 / rtol 3e-3.
"""
import types
from unittest.mock import patch

import torch

import ref_package


def seeded_pair(cfg, device, kind="shim", redraw=None, seed=1234):
    """(reference binding, its model, other binding, its model) with identical parameters."""
    reference, other = ref_package.load("reference"), ref_package.load(kind)
    torch.manual_seed(seed)
    ref_cfg = {**cfg, "gl_memory_backend": "torch"}
    expected = reference.create_model(ref_cfg)
    if redraw is not None:
        gen = torch.Generator().manual_seed(seed)
        with torch.no_grad():
            for name, p in expected.named_parameters():
                if p.ndim >= 2 and name != "bank.memory":
                    p.copy_((torch.randn(p.shape, generator=gen) * redraw).to(p.dtype))
    actual = other.create_model(cfg)
    missing = actual.load_state_dict(expected.state_dict())
    assert not missing.missing_keys and not missing.unexpected_keys
    assert [n for n, _ in actual.named_parameters()] == [n for n, _ in expected.named_parameters()]
    assert actual.bank.memory.dtype == torch.float32
    return reference, expected.to(device), other, actual.to(device)


def tokens(cfg, batch, length, device, seed=99):
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(cfg["vocab_size"], (batch, length), generator=gen).to(device)


def close(actual, expected, label, atol, rtol):
    assert torch.isfinite(actual).all() and torch.isfinite(expected).all(), f"{label}: non-finite"
    torch.testing.assert_close(actual.float(), expected.float(), atol=atol, rtol=rtol,
                               msg=lambda detail: f"{label}\n{detail}")
    return (actual.float() - expected.float()).abs().max().item()


def relative_l2(actual, expected):
    return ((actual.float() - expected.float()).norm() / expected.float().norm().clamp_min(1e-12)).item()


def prefill_matches(cfg, device, batch, length, kind="shim", redraw=None, atol=5e-4, rtol=3e-3):
    """Prefill logits and the committed banks of the request caches (verify.py:90-101)."""
    reference, expected, other, actual = seeded_pair(cfg, device, kind, redraw)
    x = tokens(cfg, batch, length, device)
    expected.eval(), actual.eval()
    with reference:
        want, want_cache = expected.prefill(x)
    with other:
        got, got_cache = actual.prefill(x)
    worst = close(got, want, "prefill logits", atol, rtol)
    a, b = got_cache[0], want_cache[0]
    assert a.tokens == b.tokens == length and a.view.version == b.view.version
    assert len(a.pending) == len(b.pending)
    close(a.view.values, b.view.values, "bank after the prefill", 1e-6, 1e-5)
    return {"logits_max_abs": worst, "logits_relative_l2": relative_l2(got, want), "commits": a.view.version}


def gradients_match(cfg, device, batch, length, kind="shim"):
    """Loss and every parameter gradient of a training-mode forward (verify.py:102-112)."""
    reference, expected, other, actual = seeded_pair(cfg, device, kind)
    x, targets = tokens(cfg, batch, length, device), tokens(cfg, batch, length, device, seed=7)

    def loss_of(binding, model):
        with binding:
            hidden, _, _ = model.hidden(x)
            logits = model.head(hidden)
            loss = torch.nn.functional.cross_entropy(logits.reshape(-1, cfg["vocab_size"]), targets.flatten())
            loss.backward()
        return logits.detach()

    want, got = loss_of(reference, expected), loss_of(other, actual)
    close(got, want, "training-mode logits", 5e-4, 3e-3)
    worst = 0.0
    for (name, p), (_, r) in zip(actual.named_parameters(), expected.named_parameters(), strict=True):
        assert p.grad is not None and r.grad is not None, f"missing gradient for {name}"
        worst = max(worst, close(p.grad, r.grad, f"gradient {name}", 1e-5, 5e-3))
    assert actual.bank.memory.grad.abs().sum() > 0, "no gradient reached the bank"
    return {"gradient_max_abs": worst}


def continuation_reset_causality(cfg, device, batch=2, length=65, kind="shim", against_reference=True):
    """Forward parts of verify.py:113-165 on the model bound to this package: split prefill
    + decode equals one pass, a new request starts from the learned bank, the past does not
    depend on the future, inference leaves the parameters alone."""
    reference, expected, other, actual = seeded_pair(cfg, device, kind)
    x = tokens(cfg, batch, length, device)
    actual.eval(), expected.eval()
    before = {n: p.detach().clone() for n, p in actual.named_parameters()}
    with torch.inference_mode():
        with reference:
            want = expected.head(expected.hidden(x)[0])
        with other:
            full = actual.head(actual.hidden(x)[0])
            cache = actual.new_cache(batch)
            first, cache = actual.prefill(x[:, :17], cache)
            second, cache = actual.prefill(x[:, 17:-2], cache)
            third, cache = actual.decode(x[:, -2:-1], cache)
            fourth, cache = actual.decode(x[:, -1:], cache)
            fresh, _ = actual.prefill(x)
            changed = x.clone()
            changed[:, length // 2:] = tokens(cfg, batch, length - length // 2, device, seed=5)
            causal = actual.head(actual.hidden(changed)[0])
    out = {"reference_relative_l2": relative_l2(full, want)}
    if against_reference:
        out["reference_max_abs"] = close(full, want, "one-pass logits against the reference", 5e-4, 3e-3)
    continued = torch.cat((first, second, third, fourth), 1)
    out["continuation_max_abs"] = close(continued, full, "prefill/decode continuation", 1e-4, 3e-3)
    close(fresh, full, "request reset", 1e-4, 3e-3)
    close(causal[:, :length // 2], full[:, :length // 2], "causality", 1e-4, 2e-3)
    chunk = cfg["gl_chunk_size"]
    assert cache[0].tokens == length and cache[0].view.version == length // chunk
    globals_ = sum(k == "global" for k in layer_kinds(cfg))
    pending = len(cache[0].pending)           # one proposal per global layer and call inside the open chunk
    assert pending % globals_ == 0 and (pending > 0) == (length % chunk != 0)
    for n, p in actual.named_parameters():
        assert torch.equal(p, before[n]), f"inference changed {n}"
    return out


def layer_kinds(cfg):
    pattern = cfg["gl_layer_pattern"]
    return [pattern[i % len(pattern)] for i in range(cfg["num_hidden_layers"])]


def teacher_forced_replay(cfg, device, batch, length, redraw=None, read_tol=(1e-6, 1e-5)):
    """Every routed_read and commit the reference stack makes (its own torch path) is replayed
    on the spot through this package with the same inputs - the method of the reference's
    scripts/check_chunk_precision.py:46-63 - so one flipped route cannot hide later ones:
    routes bit-exact, weights / readings / committed banks to tolerance. Returns counts."""
    from gl_sdm_b200.memory import MemoryView, WriteProposal, commit as our_commit, merge as our_merge, routing as ours
    reference = ref_package.load("reference")
    torch.manual_seed(1234)
    model = reference.create_model(cfg)
    if redraw is not None:
        gen = torch.Generator().manual_seed(1234)
        with torch.no_grad():
            for name, p in model.named_parameters():
                if p.ndim >= 2 and name != "bank.memory":
                    p.copy_((torch.randn(p.shape, generator=gen) * redraw).to(p.dtype))
    model = model.to(device).eval()
    x = tokens(cfg, batch, length, device)
    routing = reference.module("gl_sdm.memory.routing")
    stack = reference.module("gl_sdm.layers.stack")
    inner_read, inner_commit = routing.routed_read, stack.commit
    stub = types.SimpleNamespace(attn=types.SimpleNamespace(reference=False, backend="urm"))
    seen = {"reads": 0, "commits": 0, "rows": 0, "tie_rows": 0, "entries": 0, "banks_bit_exact": 0,
            "read_max_abs": 0.0, "bank_max_abs": 0.0}
    atol, rtol = read_tol

    def spy_read(block, memory, scores, width, physical=None):
        want = inner_read(block, memory, scores, width, physical)
        got = ours.routed_read(stub, memory, scores, width, physical)
        assert torch.equal(got[1], want[1]), f"routed_read call {seen['reads']}: routes differ"
        torch.testing.assert_close(got[2], want[2], atol=atol, rtol=rtol)
        torch.testing.assert_close(got[0], want[0], atol=atol, rtol=rtol)
        half = scores.shape[-1] // 2
        ranked = scores.reshape(-1, 2, half).sort(-1).values
        seen["tie_rows"] += int((ranked[..., -width] == ranked[..., -width - 1]).any(-1).sum())
        seen["rows"] += scores.numel() // scores.shape[-1]
        seen["reads"] += 1
        seen["read_max_abs"] = max(seen["read_max_abs"], (got[0] - want[0]).abs().max().item())
        return want

    def spy_commit(view, buffer, reference=False, backend="torch"):
        want = inner_commit(view, buffer, reference=reference, backend=backend)
        mine = MemoryView(view.values, view.version)
        proposals = [WriteProposal(p.base_version, p.addresses, p.deltas, mine.lineage, p.sort_keys)
                     for p in buffer.proposals]
        got = our_commit(mine, our_merge(mine, proposals), backend="urm")
        assert got.version == want.version
        torch.testing.assert_close(got.values, want.values, atol=1e-6, rtol=1e-5)
        seen["banks_bit_exact"] += int(torch.equal(got.values, want.values))
        seen["bank_max_abs"] = max(seen["bank_max_abs"], (got.values - want.values).abs().max().item())
        seen["entries"] += sum(p.addresses.numel() for p in buffer.proposals)
        seen["commits"] += 1
        return want

    with reference, patch.object(routing, "routed_read", spy_read), patch.object(stack, "commit", spy_commit):
        logits, cache = model.prefill(x)
    globals_ = sum(k == "global" for k in layer_kinds(cfg))
    chunk = cfg["gl_chunk_size"]
    chunks = -(-length // chunk)
    assert seen["reads"] == 2 * globals_ * chunks and seen["commits"] == length // chunk
    seen["logits"] = logits
    return seen


def one_ulp_control(cfg, device, batch, length, redraw=None):
    """How far the REFERENCE drifts from itself when every reading is moved by one float32
    ulp in half of its elements (the size of the difference between two correct summation
    orders): relative L2 of the logits. The yardstick for any free-running comparison."""
    reference = ref_package.load("reference")
    torch.manual_seed(1234)
    model = reference.create_model({**cfg, "gl_memory_backend": "torch"})
    if redraw is not None:
        gen = torch.Generator().manual_seed(1234)
        with torch.no_grad():
            for name, p in model.named_parameters():
                if p.ndim >= 2 and name != "bank.memory":
                    p.copy_((torch.randn(p.shape, generator=gen) * redraw).to(p.dtype))
    model = model.to(device).eval()
    x = tokens(cfg, batch, length, device)
    routing = reference.module("gl_sdm.memory.routing")
    inner = routing.routed_read

    def nudged(block, memory, scores, width, physical=None):
        readings, index, weights = inner(block, memory, scores, width, physical)
        up = torch.nextafter(readings, torch.full_like(readings, float("inf")))
        readings = torch.where(torch.arange(readings.shape[-1], device=readings.device) % 2 == 0, up, readings)
        return readings, index, weights

    with reference:
        plain, _ = model.prefill(x)
        with patch.object(routing, "routed_read", nudged):
            moved, _ = model.prefill(x)
    return relative_l2(moved, plain)


def audited_free_run(cfg, device, batch, length, redraw=None, noise_tol=1e-4):
    """A free-running prefill of the stack on this package, audited call by call.

    Routes are discrete: a last-bit difference between two correct implementations of the read
    moves a later score by a last bit, and where that score sits on a selection boundary the
    route changes and the two runs part ways (the reference documents this for its own two
    backends, results/loop_results.md:99-111). So a long free run is judged in three parts:
      1. every routed_read and commit THIS run makes is compared, on its own inputs, with the
         reference's torch_routed_read / commit: routes bit-exact, the rest to tolerance;
      2. up to the first call whose routes differ from the reference run, the two runs'
         scores agree to rounding noise, and every row that differs in that call is a near
         tie: the reference's own margin between the routes only one run took is within the
         noise of its scores;
      3. the drift of the logits is reported (fraction of positions outside the strict fp32
         bounds, relative L2).
    """
    import gl_sdm_b200.memory as ours
    reference, expected, shim, actual = seeded_pair(cfg, device, "shim", redraw)
    ref_routing = reference.module("gl_sdm.memory.routing")
    ref_memory = reference.module("gl_sdm.memory")
    ref_stack, shim_stack = reference.module("gl_sdm.layers.stack"), shim.module("gl_sdm.layers.stack")
    assert shim_stack.commit is ours.commit
    x = tokens(cfg, batch, length, device)
    expected.eval(), actual.eval()
    theirs, mine = [], []
    inner_ref = ref_routing.routed_read

    def record_reference(block, memory, scores, width, physical=None):
        out = inner_ref(block, memory, scores, width, physical)
        theirs.append((scores.clone(), out[1].clone()))
        return out

    with reference, patch.object(ref_routing, "routed_read", record_reference):
        want, _ = expected.prefill(x)

    inner_ours, inner_commit = ours.routing.routed_read, ours.commit
    audited = {"reads": 0, "commits": 0}

    def audit_read(block, memory, scores, width, physical=None):
        got = inner_ours(block, memory, scores, width, physical)
        with reference:
            check = ref_routing.torch_routed_read(memory, scores, width)
        assert torch.equal(got[1], check[1]), f"routed_read call {audited['reads']}: routes differ on identical inputs"
        torch.testing.assert_close(got[2], check[2], atol=1e-6, rtol=1e-5)
        torch.testing.assert_close(got[0], check[0], atol=1e-6, rtol=1e-5)
        mine.append((scores.clone(), got[1].clone()))
        audited["reads"] += 1
        return got

    def audit_commit(view, buffer, reference_flag=False, backend="torch", **kw):
        got = inner_commit(view, buffer, reference_flag, backend, **kw)
        with reference:
            theirs_view = ref_memory.MemoryView(view.values, view.version)
            proposals = [ref_memory.WriteProposal(p.base_version, p.addresses, p.deltas, theirs_view.lineage, p.sort_keys)
                         for p in buffer.proposals]
            check = ref_memory.commit(theirs_view, ref_memory.merge(theirs_view, proposals), backend="torch")
        torch.testing.assert_close(got.values, check.values, atol=1e-6, rtol=1e-5)
        audited["commits"] += 1
        return got

    with shim, patch.object(ours.routing, "routed_read", audit_read), patch.object(shim_stack, "commit", audit_commit):
        got, _ = actual.prefill(x)
    assert audited["reads"] == len(theirs) == len(mine) and audited["commits"] == length // cfg["gl_chunk_size"]

    report = {"reads": audited["reads"], "commits": audited["commits"], "first_split_call": None,
              "rows_split_there": 0, "score_noise": 0.0, "worst_margin": 0.0}
    for call, ((s_ref, i_ref), (s_our, i_our)) in enumerate(zip(theirs, mine)):
        noise = (s_ref - s_our).abs().max().item()
        scale = s_ref.abs().max().item()
        rows = (i_ref != i_our).any(-1)
        if not rows.any():
            assert noise <= noise_tol * scale, f"call {call}: same routes but scores {noise} apart"
            report["score_noise"] = max(report["score_noise"], noise)
            continue
        # the first call that splits: its inputs still agree to rounding noise ...
        assert noise <= noise_tol * scale, f"call {call}: scores differ by {noise} before any route did"
        half, width = s_ref.shape[-1] // 2, i_ref.shape[-1]
        s, a, b = s_ref[rows], i_ref[rows], i_our[rows]
        sums_a = s[..., :half].gather(-1, a // half) + s[..., half:].gather(-1, a % half)
        sums_b = s[..., :half].gather(-1, b // half) + s[..., half:].gather(-1, b % half)
        only_a = (a.unsqueeze(-1) != b.unsqueeze(-2)).all(-1)
        only_b = (b.unsqueeze(-1) != a.unsqueeze(-2)).all(-1)
        # every route only the reference took ranks (for the reference) above every route only this
        # run took, and the other way round for this run's scores: all of them lie within the noise
        best_kept = torch.where(only_a, sums_a, torch.full_like(sums_a, float("-inf"))).max(-1).values
        worst_taken = torch.where(only_b, sums_b, torch.full_like(sums_b, float("inf"))).min(-1).values
        margin = (best_kept - worst_taken).max().item()
        # ... and each split row is a near tie: the margin is within the noise of two scores of each run
        assert margin <= 4 * noise + 1e-7 * scale, f"call {call}: a route changed across a margin of {margin} (noise {noise})"
        report.update(first_split_call=call, rows_split_there=int(rows.sum()), worst_margin=margin)
        report["score_noise"] = max(report["score_noise"], noise)
        break
    bad = ((got - want).abs() > 5e-4 + 3e-3 * want.abs()).any(-1)
    report["positions_outside_strict_bounds"] = bad.float().mean().item()
    report["logits_relative_l2"] = relative_l2(got, want)
    report["logits_max_abs"] = (got - want).abs().max().item()
    if report["first_split_call"] is None:
        close(got, want, "prefill logits", 5e-4, 3e-3)
    return report


def copy_free_training_matches(cfg, device, batch, length, strict=False, kind="shim"):
    """The same training-mode forward + backward of the stack bound to this package, once with
    the reference's per-commit bank copy (gl_sdm/memory/transactions.py:96) and once with
    copy-free commits: logits and every gradient agree (``strict``: bit for bit, for runs whose
    dense surround is deterministic; otherwise to 1e-6 / 1e-5, the embedding and attention
    backwards of the library use atomics)."""
    _, _, other, model = seeded_pair(cfg, device, kind)
    x, targets = tokens(cfg, batch, length, device), tokens(cfg, batch, length, device, seed=7)
    with other:
        transactions = other.module("gl_sdm.memory.transactions")

    def run(copy_free):
        model.zero_grad(set_to_none=True)
        if device != "cpu":
            torch.cuda.reset_peak_memory_stats()
        previous = transactions.copy_free_commits(copy_free)
        try:
            with other:
                hidden, _, _ = model.hidden(x)
                logits = model.head(hidden)
                loss = torch.nn.functional.cross_entropy(logits.reshape(-1, cfg["vocab_size"]), targets.flatten())
                loss.backward()
        finally:
            transactions.copy_free_commits(previous)
        peak = torch.cuda.max_memory_allocated() if device != "cpu" else 0
        return logits.detach(), {n: p.grad.clone() for n, p in model.named_parameters()}, peak

    want, want_grads, copied_peak = run(False)
    got, got_grads, free_peak = run(True)
    exact = 0
    if strict:
        assert torch.equal(got, want)
    else:
        close(got, want, "logits with copy-free commits", 1e-6, 1e-5)
    for name, expected in want_grads.items():
        if strict:
            assert torch.equal(got_grads[name], expected), name
        else:
            close(got_grads[name], expected, f"gradient {name} with copy-free commits", 1e-6, 1e-5)
        exact += int(torch.equal(got_grads[name], expected))
    assert want_grads["bank.memory"].abs().sum() > 0
    return {"bit_equal_gradients": exact, "gradients": len(want_grads), "peak_bytes_copying": copied_peak,
            "peak_bytes_copy_free": free_peak}
