"""The unmodified reference stack over the package shim, on CPU.

The kernels are replaced by the stand-ins of tests/cpu_kernels.py (built from the CPU port),
so what runs here is the HOST side of gl_sdm_b200.memory under the reference's own
layers/stack.py: views and caches, pending proposals across calls, the absolute commit
clock, the autograd wiring. The GPU tests (tests/test_gpu_ref_stack.py) run the same checks
on the real kernels. Skipped when the reference is not staged under oracle/_ref.
"""
import pytest
import torch

import cpu_kernels
import ref_package
import ref_stack_checks as checks

SMALL = dict(hidden_size=64, head_dim=16, num_hidden_layers=4, intermediate_size=128, vocab_size=257,
             gl_slots=256, gl_reads=4, gl_writes=4, gl_chunk_size=16, gl_local_window=8)


@pytest.fixture
def standins(monkeypatch):
    ref_package.require()
    from gl_sdm_b200 import _native
    for name, fn in cpu_kernels.memory_api_standins().items():
        monkeypatch.setattr(_native, name, fn)


def test_bindings_resolve_to_the_right_packages():
    ref_package.require()
    shim, reference = ref_package.load("shim"), ref_package.load("reference")
    import gl_sdm_b200.memory as ours
    assert shim.module("gl_sdm.layers.stack").commit is ours.commit
    assert shim.module("gl_sdm.layers.global_layer").routing is ours.routing
    assert reference.module("gl_sdm.layers.stack").commit is not ours.commit
    assert shim.module("gl_sdm.layers.stack").__file__ == reference.module("gl_sdm.layers.stack").__file__
    seam = ref_package.load("seam")
    from gl_sdm_b200.memory.backends import urm
    assert seam.module("gl_sdm.memory.backends.urm") is urm
    assert seam.module("gl_sdm.memory").commit is not ours.commit


def test_prefill_logits_and_banks(standins):
    out = checks.prefill_matches(checks.ref_package.stack_config(**SMALL), "cpu", batch=2, length=40)
    assert out["commits"] == 2


def test_gradients(standins):
    checks.gradients_match(checks.ref_package.stack_config(**SMALL), "cpu", batch=2, length=40)


def test_continuation_reset_causality(standins):
    checks.continuation_reset_causality(checks.ref_package.stack_config(**SMALL), "cpu", batch=2, length=37)


def test_teacher_forced_replay(standins):
    seen = checks.teacher_forced_replay(checks.ref_package.stack_config(**SMALL), "cpu", batch=2, length=40)
    assert seen["reads"] == 2 * 2 * 3 and seen["commits"] == 2


def test_audited_free_run(standins):
    out = checks.audited_free_run(checks.ref_package.stack_config(**SMALL), "cpu", batch=2, length=40)
    assert out["reads"] == 12 and out["commits"] == 2 and out["first_split_call"] is None


def test_backend_seam_runs_the_stack(standins):
    """Config "urm": the reference's own memory package calls backends.urm / backends.commit."""
    from gl_sdm_b200.memory.backends import commit, urm
    from unittest.mock import patch
    cfg = checks.ref_package.stack_config(**SMALL, gl_memory_backend="urm")
    with patch.object(urm, "routed_snapshot_read", wraps=urm.routed_snapshot_read) as reads, \
            patch.object(commit, "commit", wraps=commit.commit) as commits:
        checks.prefill_matches(cfg, "cpu", batch=2, length=40, kind="seam")
        assert reads.call_count == 2 * 2 * 3 and commits.call_count == 2
        checks.gradients_match(cfg, "cpu", batch=2, length=40, kind="seam")


def test_copy_free_commits_train_the_stack_identically(standins):
    out = checks.copy_free_training_matches(checks.ref_package.stack_config(**SMALL), "cpu", batch=2, length=40,
                                            strict=True)
    assert out["bit_equal_gradients"] == out["gradients"]


def test_fused_proposals_serve_the_stack(standins, monkeypatch):
    from gl_sdm_b200 import _native
    calls = []
    fused = _native.pk_propose
    monkeypatch.setattr(_native, "pk_propose", lambda *a, **k: calls.append(k["layer_index"]) or fused(*a, **k))
    cfg = checks.ref_package.stack_config(**SMALL)
    out = checks.prefill_matches(cfg, "cpu", batch=2, length=40, kind="fused")
    assert out["commits"] == 2
    assert calls == [1, 3] * 3               # both global layers, three chunk pieces (16 + 16 + 8 tokens)
    calls.clear()
    # from the second stack call on, the proposals of one call sit side by side in one buffer
    # and the commit concatenates without a copy
    from gl_sdm_b200.memory import transactions
    copies = []
    joined = transactions._concat
    monkeypatch.setattr(transactions, "_concat", lambda ts: copies.append(transactions._adjacent(ts)) or joined(ts))
    checks.prefill_matches(cfg, "cpu", batch=2, length=32, kind="fused")
    assert copies and all(copies)
    calls.clear()
    checks.continuation_reset_causality(cfg, "cpu", batch=2, length=37, kind="fused")
    calls.clear()
    checks.gradients_match(cfg, "cpu", batch=2, length=40, kind="fused")   # forward and backward on the fused pair
    assert calls == [1, 3] * 2               # the last piece of a training forward needs no proposals
