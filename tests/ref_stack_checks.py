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


def continuation_reset_causality(cfg, device, batch=2, length=65, kind="shim"):
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
    out = {"reference_max_abs": close(full, want, "one-pass logits against the reference", 5e-4, 3e-3)}
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
