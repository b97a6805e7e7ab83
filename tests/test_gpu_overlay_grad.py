"""Gradients through copy-free commits on the CUDA kernels (the reference's plan:
OPTIMIZATION_PLAN.md "Represent commits as compact overlays ... carry gradients back through
updates"; the per-commit bank clone they replace is gl_sdm/memory/transactions.py:96)."""
import pytest
import torch

import overlay_grad_checks as checks
import ref_package
import ref_stack_checks as stack_checks
from gl_sdm_b200 import _native
from gl_sdm_b200.memory import routing

pytestmark = pytest.mark.gpu


def test_copy_free_step_matches_copying_step():
    checks.assert_same_step("cuda", commits=3, batch=2, tokens=64, heads=4, half=32, dim=64, width=8)
    _native.raise_on_device_status("cuda")


def test_bf16_request_banks():
    checks.assert_same_step("cuda", commits=4, batch=2, tokens=64, heads=4, half=32, dim=128, width=8,
                            storage=torch.bfloat16, seed=11)
    _native.raise_on_device_status("cuda")


def test_wide_rows_and_long_chain():
    # more commits than one kernel call takes logs: the oldest reads rebuild their version once
    checks.assert_same_step("cuda", commits=_native.MAX_UNDO_LOGS + 3, batch=1, tokens=32, heads=2, half=16, dim=256,
                            width=16, seed=3)
    _native.raise_on_device_status("cuda")


def test_read_backward_through_logs_equals_the_kept_version():
    """The kernel alone: the backward of a read of version 0 against (a) the kept copy of
    version 0 and (b) the in-place bank two commits later plus the two undo logs."""
    torch.manual_seed(5)
    dev = "cuda"
    B, T, H, half, D, K = 2, 48, 4, 16, 64, 8
    bank = torch.randn(B, H, half * half, D, device=dev)
    kept = bank.clone()
    scores = torch.randn(B, T, H, 2 * half, device=dev)
    _, index, weights = routing.torch_routed_read(bank, scores, K)
    logs = []
    for c in range(2):
        n = 4096
        addresses = torch.randint(B * H * half * half, (n,), device=dev)
        deltas = torch.randn(n, D, device=dev)
        logs.append(_native.commit_undo(bank, addresses, deltas))
    assert not torch.equal(bank, kept)
    g = torch.randn(B, T, H, D, device=dev)
    gw = torch.randn(B, T, H, K, device=dev)
    want = _native.read_backward(kept, g, gw, index, weights, T * H, half)
    got = _native.read_backward(bank, g, gw, index, weights, T * H, half, logs)
    stale = _native.read_backward(bank, g, gw, index, weights, T * H, half)
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    assert not torch.equal(stale[0], want[0])       # the logs matter for these routes
    _native.raise_on_device_status(dev)


def test_reference_stack_trains_identically_without_bank_copies():
    ref_package.require()
    cfg = ref_package.stack_config(num_hidden_layers=4, gl_slots=4096, gl_chunk_size=128, gl_local_window=64,
                                   vocab_size=4096)
    out = stack_checks.copy_free_training_matches(cfg, "cuda", batch=2, length=512)
    print("copy-free training:", out)
    _native.raise_on_device_status("cuda")
