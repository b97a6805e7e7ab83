"""The UNMODIFIED reference stack (gl_sdm/layers/stack.py and everything above it, staged
under oracle/_ref) running on the CUDA kernels, against the same source on the reference's
own torch path - both on the GPU, same parameters, same tokens.

Two bindings are exercised: the package seam (gl_sdm_b200.install replaces gl_sdm.memory) and
the backend seam (the reference's own memory package with gl_memory_backend="urm" calling
gl_sdm_b200.memory.backends.urm / .commit). Bounds are the reference's own gate
(gl_sdm/experiments/verify.py:98-165). Skipped when oracle/_ref is not staged.
"""
import types
from unittest.mock import patch

import pytest
import torch

import ref_package
import ref_stack_checks as checks

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
# widths of benchmark configuration 2; the clocked tests shorten the chunk so that a short
# sequence crosses several commits
FAST_CLOCK = dict(num_hidden_layers=4, gl_chunk_size=16, gl_local_window=16, vocab_size=4096)


@pytest.fixture(autouse=True)
def _staged(native):
    ref_package.require()
    yield
    native.raise_on_device_status(DEV)


def test_prefill_at_c2_widths_fp32_one_chunk_strict():
    """16 layers, 8 heads, 16,384 slots, 16 routes: 2 x 512 tokens (one chunk, one commit)
    agree with the reference run at its own fp32 bounds."""
    out = checks.prefill_matches(ref_package.stack_config(), DEV, batch=2, length=512, redraw=0.02)
    assert out["commits"] == 1
    print("c2-width fp32 prefill, one chunk:", out)


def test_free_run_at_c2_widths_fp32_is_exact_call_by_call():
    """2 x 1024 tokens, 512-token chunks, 32 routed reads of 65,536 rows each and 2 commits of
    1,048,576 entries: every call exact on its own inputs; where the run parts from the
    reference run it does so at a near tie."""
    cfg = ref_package.stack_config()
    out = checks.audited_free_run(cfg, DEV, batch=2, length=1024, redraw=0.02)
    assert out["reads"] == 32 and out["commits"] == 2
    control = checks.one_ulp_control(cfg, DEV, batch=2, length=1024, redraw=0.02)
    print("c2-width fp32 free run:", out, "| reference against itself, readings moved by one ulp:", control)
    assert out["logits_relative_l2"] <= max(1e-5, 3 * control)


def test_gradients_fp32():
    out = checks.gradients_match(ref_package.stack_config(**FAST_CLOCK), DEV, batch=2, length=65)
    print("fp32 gradients:", out)


def test_continuation_reset_causality_fast_clock():
    out = checks.continuation_reset_causality(ref_package.stack_config(**FAST_CLOCK), DEV, batch=2, length=65)
    print("continuation (16-token chunks):", out)


def test_continuation_across_512_token_commits():
    """17 + 1081 + 1 + 1 tokens: pending proposals carried between calls, commits at the
    absolute positions 512 and 1024 (layers/stack.py:41-68). The dense surround runs in
    float64 here, so that GEMMs of different batch shapes (17 rows, 1081 rows, 1 row) produce
    the same float32 scores and a split run can be compared with a one-pass run at strict
    bounds over thousands of routing rows; the memory operator itself stays float32."""
    cfg = ref_package.stack_config(dtype="float64", num_hidden_layers=8)
    out = checks.continuation_reset_causality(cfg, DEV, batch=1, length=1100, against_reference=False)
    print("continuation (512-token chunks):", out)


def test_teacher_forced_replay_bf16_at_c2_widths():
    """bf16 weights (scores are bf16 GEMM outputs: exact ties at the selection boundary are
    common): every call's routes bit-exact. The end-to-end drift of a free-running bf16 stack
    is reported separately, bounded like the reference bounds bf16 runs (verify.py:19-28)."""
    cfg = ref_package.stack_config(dtype="bfloat16")
    seen = checks.teacher_forced_replay(cfg, DEV, batch=2, length=1024, redraw=0.02)
    assert seen["reads"] == 32 and seen["commits"] == 2 and seen["entries"] == 2 * 2 * 512 * 8 * 16 * 8
    assert seen["tie_rows"] > 0, "bf16 scores are expected to tie at the selection boundary"
    seen.pop("logits")
    print("bf16 replay:", seen)


def test_free_run_bf16_at_c2_widths_is_exact_call_by_call():
    """The free-running bf16 stack on the kernels: every call exact on its own inputs. How far
    the logits end up from the reference run is reported beside the reference's own
    sensitivity (one ulp on its readings); the reference's own bf16 gate fails at full size
    for the same reason (results/initial_sixteen_layers.md:107-120)."""
    cfg = ref_package.stack_config(dtype="bfloat16")
    out = checks.audited_free_run(cfg, DEV, batch=2, length=1024, noise_tol=2e-2)
    control = checks.one_ulp_control(cfg, DEV, batch=2, length=1024)
    print("c2-width bf16 free run:", out, "| reference against itself, readings moved by one ulp:", control)
    assert out["reads"] == 32 and out["commits"] == 2
    assert out["logits_relative_l2"] <= max(0.05, 3 * control)


def test_backend_seam_prefill_and_gradients():
    """verify.py:32-42: with gl_memory_backend="urm" the reference's memory package must reach
    backends.urm.routed_snapshot_read and backends.commit.commit; both are ours here. Under
    grad mode the stack hands the zero-padded 128-wide physical bank (stack.py:50-51)."""
    from gl_sdm_b200.memory.backends import commit, urm
    cfg = ref_package.stack_config(**FAST_CLOCK, gl_memory_backend="urm")
    widths = []
    inner = urm.routed_snapshot_read

    def spy(values, scores, width, allow_large_route=False):
        widths.append(values.shape[-1])
        out = inner(values, scores, width, allow_large_route=allow_large_route)
        assert out[1].dtype == torch.int32
        return out

    with patch.object(urm, "routed_snapshot_read", spy), patch.object(commit, "commit", wraps=commit.commit) as commits:
        checks.prefill_matches(cfg, DEV, batch=2, length=65, kind="seam")
        assert len(widths) == 2 * 2 * 5 and set(widths) == {64} and commits.call_count == 4
        widths.clear()
        checks.gradients_match(cfg, DEV, batch=2, length=65, kind="seam")
        assert set(widths) == {128}, "the padded physical bank did not reach the read"
        assert commits.call_count > 4


def test_backend_seam_five_dimensional_scores():
    """memory/routing.py:48-55: [batch, reasoning, token, head, factor] scores are split in
    groups of passes, each flattened for the native read and reshaped back."""
    seam, reference = ref_package.load("seam"), ref_package.load("reference")
    gen = torch.Generator().manual_seed(11)
    memory = (torch.randn(2, 3, 64 * 64, 64, generator=gen) * 0.1).to(DEV)
    scores = torch.randn(2, 3, 700, 3, 128, generator=gen).bfloat16().float().to(DEV)
    block = types.SimpleNamespace(attn=types.SimpleNamespace(reference=False, backend="urm", experimental_large_route=False))
    physical = torch.nn.functional.pad(memory, (0, 64))
    with seam:
        got = seam.module("gl_sdm.memory.routing").routed_read(block, memory, scores, 8, physical)
    with reference:
        flat = reference.module("gl_sdm.memory.routing").torch_routed_read(memory, scores.flatten(1, 2), 8)
    want = tuple(t.reshape(2, 3, 700, 3, -1) for t in flat)
    assert got[0].shape == (2, 3, 700, 3, 64) and got[1].dtype == torch.int32
    assert torch.equal(got[1].long(), want[1])
    torch.testing.assert_close(got[2], want[2], atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(got[0], want[0], atol=1e-6, rtol=1e-5)
    # the package seam takes the same call through its own dispatcher
    from gl_sdm_b200.memory import routing as ours
    mine = ours.routed_read(block, memory, scores, 8, physical)
    assert mine[0].shape == (2, 3, 700, 3, 64) and torch.equal(mine[1], want[1])
    torch.testing.assert_close(mine[0], want[0], atol=1e-6, rtol=1e-5)


def test_fused_proposals_one_chunk_and_fast_clock():
    """GlobalLayer.propose served by the fused write proposal (gl_sdm_b200.layers): one chunk at
    c2 widths against the reference at its fp32 bounds, then the 16-token clock (pending
    proposals across calls, several commits) with continuation, reset and causality."""
    out = checks.prefill_matches(ref_package.stack_config(), DEV, batch=2, length=512, redraw=0.02, kind="fused")
    assert out["commits"] == 1
    clocked = checks.continuation_reset_causality(ref_package.stack_config(**FAST_CLOCK), DEV, batch=2, length=65,
                                                  kind="fused")
    print("fused proposals, one chunk:", out, "| 16-token chunks:", clocked)


def test_fused_proposals_equal_the_layer_method_call_by_call():
    """The same layer, the same inputs: the fused proposal against the reference method bound
    to this package (addresses and keys identical, delta rows to 1e-6 / 1e-5)."""
    _, _, binding, model = checks.seeded_pair(ref_package.stack_config(num_hidden_layers=2), DEV, "fused")
    with binding, torch.inference_mode():
        layer = next(b for b in model.blocks if hasattr(b, "propose"))
        cache = model.bank.new_cache(2)
        x = torch.randn(2, 96, 512, device=DEV)
        got = layer.propose(x, cache.view, 40, 1, 512, 2)
        want = layer._glsdm_reference_propose(x, cache.view, 40, 1, 512, 2)
    assert torch.equal(got.addresses, want.addresses) and torch.equal(got.sort_keys, want.sort_keys)
    torch.testing.assert_close(got.deltas, want.deltas, atol=1e-6, rtol=1e-5)
    assert got.base_version == want.base_version and got.lineage is want.lineage


def test_fused_proposal_gradients_equal_autograd_through_the_layer_method():
    """Training: the fused proposal's backward kernel against autograd through the method it
    replaces, same layer, same inputs, a random gradient arriving at the delta rows - for the
    hidden state, every parameter of the write side and the bank."""
    _, _, binding, model = checks.seeded_pair(ref_package.stack_config(num_hidden_layers=2), DEV, "fused")
    torch.manual_seed(3)
    with binding:
        layer = next(b for b in model.blocks if hasattr(b, "propose"))
        x = torch.randn(2, 96, 512, device=DEV, requires_grad=True)
        incoming = None
        results = []
        for method in (layer.propose, layer._glsdm_reference_propose):
            model.zero_grad(set_to_none=True)
            x.grad = None
            cache = model.bank.new_cache(2)
            proposal = method(x, cache.view, 40, 1, 512, 2)
            if incoming is None:
                incoming = torch.randn_like(proposal.deltas)
            (proposal.deltas * incoming).sum().backward()
            grads = {"x": x.grad.clone(), "bank": model.bank.memory.grad.clone()}
            grads.update({n: p.grad.clone() for n, p in layer.named_parameters() if p.grad is not None})
            results.append((proposal, grads))
    (got, got_grads), (want, want_grads) = results
    assert torch.equal(got.addresses, want.addresses)
    assert set(got_grads) == set(want_grads) and {"attn.k.weight", "attn.v.weight", "attn.beta.weight",
                                                  "attn.decay.weight", "norm1.weight"} <= set(got_grads)
    for name, expected in want_grads.items():
        scale = expected.abs().max().item()
        torch.testing.assert_close(got_grads[name], expected, atol=2e-5 * max(scale, 1e-6), rtol=2e-4,
                                   msg=lambda detail, name=name: f"gradient {name}\n{detail}")


def test_stack_gradients_with_fused_proposals_and_copy_free_commits():
    out = checks.gradients_match(ref_package.stack_config(**FAST_CLOCK), DEV, batch=2, length=65, kind="fused")
    cfg = ref_package.stack_config(num_hidden_layers=4, gl_slots=4096, gl_chunk_size=128, gl_local_window=64,
                                   vocab_size=4096)
    free = checks.copy_free_training_matches(cfg, DEV, batch=2, length=512, kind="fused")
    print("fused proposals, fp32 gradients:", out, "| with copy-free commits:", free)
