"""Backward of the operator on the CUDA kernels against the reference's autograd
(tests/golden/gradients.npz, generated from the reference's torch path; the reference checks
the same gradients on its native path in projects/gl-sdm/tests/test_chunk_memory.py:86-121).
Tolerances are the reference's: atol 1e-5, rtol 1e-5 (looser only where sums are long)."""
import numpy as np
import pytest
import torch

import golden_inputs as gi
from conftest import load_golden
from oracle import torch_port as port

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("name", gi.GRAD_CASES)
def test_routed_read_gradients_match_reference_autograd(native, name):
    from gl_sdm_b200.memory import routing
    gold = load_golden("gradients")
    memory, scores, width = gi.grad_case(name)
    memory, scores = memory.to(DEV).requires_grad_(), scores.to(DEV).requires_grad_()
    readings, index, weights = routing.torch_routed_read(memory, scores, width)
    assert readings.requires_grad and weights.requires_grad and not index.requires_grad
    cot_r, cot_w = gi.cotangents(name, readings.shape, weights.shape)
    loss = (readings * cot_r.to(DEV)).sum() + (weights * cot_w.to(DEV)).sum()
    g_memory, g_scores = torch.autograd.grad(loss, (memory, scores), retain_graph=True)
    np.testing.assert_allclose(g_scores.cpu().numpy(), gold[f"{name}_grad_scores"], rtol=1e-4, atol=1e-5)
    flat = g_memory.flatten(0, 2).cpu().numpy()
    np.testing.assert_allclose(flat[gold[f"{name}_touched"]], gold[f"{name}_grad_rows"], rtol=1e-4, atol=1e-5)
    untouched = np.ones(flat.shape[0], bool)
    untouched[gold[f"{name}_touched"]] = False
    assert not flat[untouched].any()
    # deterministic: the same backward again is bit-identical
    again = torch.autograd.grad(loss, (memory, scores))
    assert torch.equal(again[0], g_memory) and torch.equal(again[1], g_scores)


def test_write_chain_gradients_match_reference_autograd(native):
    """routed read -> gather_rows -> delta (dense.py:11-14, torch ops) -> commit; gradient of
    the committed bank w.r.t. the old bank, the write scores and the targets."""
    from gl_sdm_b200.memory import MemoryView, WriteProposal, commit, merge, routing
    gold = load_golden("gradients")
    chain = gi.chain_case()
    memory, scores, target = (chain[k].to(DEV).requires_grad_() for k in ("memory", "scores", "target"))
    B, T, H, _ = scores.shape
    prediction, index, weights = routing.torch_routed_read(memory, scores, chain["width"])
    rows = routing.gather_rows(memory, index)
    addresses = routing.absolute_addresses(memory, index)
    delta = port.delta_rows(rows, weights, prediction, target, chain["beta"].to(DEV).unsqueeze(-1),
                            chain["log_decay"].to(DEV).unsqueeze(-1), torch.ones(B, T, device=DEV))
    keys = addresses * (T * 2) + torch.arange(T, device=DEV).view(1, T, 1, 1) * 2 + 1
    view = MemoryView(memory)
    after = commit(view, merge(view, [WriteProposal(0, addresses.flatten(), delta.flatten(0, 3), view.lineage, keys.flatten())]))
    np.testing.assert_allclose(after.values.detach().cpu().numpy(), gold["chain_after"], rtol=1e-5, atol=1e-6)
    grads = torch.autograd.grad((after.values * chain["cotangent"].to(DEV)).sum(), (memory, scores, target))
    for name, g in zip(("memory", "scores", "target"), grads):
        np.testing.assert_allclose(g.cpu().numpy(), gold[f"chain_grad_{name}"], rtol=1e-4, atol=1e-5, err_msg=name)
    with pytest.raises(ValueError, match="donated"):
        commit(view, merge(view, [WriteProposal(0, addresses.flatten(), delta.flatten(0, 3), view.lineage, keys.flatten())]),
               donate=True)


def test_token_clock_gradients_match_reference_autograd(native):
    """Token-clock read and write proposal (gl_sdm/memory/transactions.py:28-59) with every
    operand requiring grad, against the reference's autograd on the same inputs; the forward
    results under grad mode still match the forward-only golden vectors."""
    from gl_sdm_b200.memory import MemoryView, propose_write, read
    gold, forward = load_golden("token_gradients"), load_golden("token_api")
    t = {k: v.to(DEV) for k, v in gi.token_case().items()}
    names = ("memory", "weights", "targets", "beta", "log_decay", "mass")
    leaves = {k: t[k].clone().requires_grad_() for k in names}
    view = MemoryView(leaves["memory"])
    retrieved = read(view, t["requests"], t["indices"], leaves["weights"])
    p = propose_write(view, t["requests"], t["indices"], leaves["weights"], leaves["targets"], leaves["beta"],
                      leaves["log_decay"], leaves["mass"])
    assert retrieved.requires_grad and p.deltas.requires_grad
    np.testing.assert_allclose(retrieved.detach().cpu().numpy(), forward["read"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(p.deltas.detach().cpu().numpy(), forward["deltas"], rtol=1e-5, atol=1e-5)
    assert np.array_equal(p.addresses.cpu().numpy(), forward["addresses"])
    cot_read, cot_delta = gi.cotangents("token", retrieved.shape, p.deltas.shape)
    grads = torch.autograd.grad((retrieved * cot_read.to(DEV)).sum(), (leaves["memory"], leaves["weights"]), retain_graph=True)
    np.testing.assert_allclose(grads[0].cpu().numpy(), gold["read_grad_memory"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(grads[1].cpu().numpy(), gold["read_grad_weights"], rtol=1e-5, atol=1e-5)
    grads = torch.autograd.grad((p.deltas * cot_delta.to(DEV)).sum(), [leaves[k] for k in names])
    for k, g in zip(names, grads):
        np.testing.assert_allclose(g.cpu().numpy(), gold[f"propose_grad_{k}"], rtol=1e-4, atol=1e-5, err_msg=k)
    # only the bank requires grad: the weight gradient (and its saved rows) is skipped
    only_bank = read(view, t["requests"], t["indices"], t["weights"])
    (g,) = torch.autograd.grad((only_bank * cot_read.to(DEV)).sum(), (leaves["memory"],))
    np.testing.assert_allclose(g.cpu().numpy(), gold["read_grad_memory"], rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("half,width,dim,bank_dtype,target_dtype,commits", [
    (32, 8, 64, torch.float32, torch.float32, 0),
    (16, 4, 48, torch.float32, torch.float32, 0),          # rows that do not fill the lanes
    (64, 32, 256, torch.bfloat16, torch.bfloat16, 0),      # widest rows, most routes
    (32, 16, 128, torch.float32, torch.bfloat16, 2),       # the bank has moved on: rows through undo logs
])
def test_fused_proposal_backward_matches_autograd_of_the_expression(native, half, width, dim, bank_dtype,
                                                                    target_dtype, commits):
    """glsdm_pk_propose_backward against float32 autograd through the port's statement of
    gl_sdm/layers/global_layer.py:41-51 + gl_sdm/runtime/dense.py:11-14 on the same routes."""
    from gl_sdm_b200.memory import autograd as ours
    torch.manual_seed(half * 131 + dim)
    B, T, H = 2, 24, 3
    bank = (torch.randn(B, H, half * half, dim, device=DEV) * 0.5).to(bank_dtype)
    kept = bank.clone()
    scores = torch.randn(B, T, H, 2 * half, device=DEV)
    target = torch.randn(B, T, H, dim, device=DEV).to(target_dtype)
    beta = torch.rand(B, T, H, device=DEV) * 0.8 + 0.1
    log_decay = -torch.rand(B, T, H, device=DEV) * 0.3
    leaves = [t.clone().requires_grad_() for t in (bank, scores, target, beta, log_decay)]
    addresses, deltas, keys = ours.FusedProposal.apply(*leaves, (T, width, 5, 64, 3, 1))
    incoming = torch.randn_like(deltas)
    for _ in range(commits):                                  # copy-free commits between forward and backward
        n = 2048
        hit = torch.randint(bank.numel() // dim, (n,), device=DEV)
        log = native.commit_undo(leaves[0].detach(), hit, torch.randn(n, dim, device=DEV))
        from gl_sdm_b200.memory.state import UndoLog, tail_of
        node = UndoLog(*log)
        node.accounted = leaves[0]._version
        tail_of(leaves[0]).next = node
        leaves[0]._glsdm_tail = node
    got = torch.autograd.grad(deltas, leaves, incoming)
    if commits:
        assert not torch.equal(leaves[0].detach(), kept)

    exact = [kept.float().requires_grad_(), scores.clone().requires_grad_(), target.float().requires_grad_(),
             beta.clone().requires_grad_(), log_decay.clone().requires_grad_()]
    want_addresses, want_deltas, want_keys = port.propose(exact[0], exact[1], width, exact[2], exact[3], exact[4], None,
                                                          5, 1, 64, 3)
    assert torch.equal(addresses, want_addresses) and torch.equal(keys, want_keys)
    torch.testing.assert_close(deltas, want_deltas, atol=1e-5, rtol=1e-5 if bank_dtype == torch.float32 else 1e-4)
    want = torch.autograd.grad(want_deltas, exact, incoming)
    for name, g, w in zip(("bank", "scores", "target", "beta", "log_decay"), got, want):
        scale = w.abs().max().item()
        loose = 2e-2 if name in ("bank", "target") and g.dtype == torch.bfloat16 else 1e-4
        torch.testing.assert_close(g.float(), w, atol=loose * scale, rtol=loose,
                                   msg=lambda detail, name=name: f"gradient {name}\n{detail}")
    native.raise_on_device_status(DEV)
