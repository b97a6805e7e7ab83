"""A small training step over several commits, run with copying and with copy-free commits.

Shared by the CPU test (stand-in kernels) and the GPU test (the CUDA kernels): the two runs
have to agree bit for bit in the loss, the final bank and every gradient, because the
copy-free run reads the same rows - through the undo logs - that the copying run keeps alive
as whole bank versions (reference: the per-commit clone at gl_sdm/memory/transactions.py:96
and the plan to replace it, OPTIMIZATION_PLAN.md "Represent commits as compact overlays").
"""
import torch

from gl_sdm_b200.memory import routing, transactions
from gl_sdm_b200.memory.state import MemoryBank, MemoryView, WriteProposal


def training_step(device, copy_free, commits=3, batch=2, tokens=8, heads=2, half=8, dim=32, width=4, seed=0,
                  storage=torch.float32):
    """Returns (loss, final bank, {name: gradient})."""
    gen = torch.Generator().manual_seed(seed)
    bank = MemoryBank(heads, half * half, dim)
    with torch.no_grad():
        bank.memory.copy_(torch.randn(bank.memory.shape, generator=gen))
    bank = bank.to(device)
    project = torch.randn(commits + 1, dim, 2 * half, generator=gen).to(device).requires_grad_()
    targets = torch.randn(commits, batch, tokens, heads, dim, generator=gen).to(device).requires_grad_()
    hidden = torch.randn(batch, tokens, heads, dim, generator=gen).to(device)
    view = bank.snapshot(batch)
    if storage != torch.float32:           # a bf16 request bank derived from the fp32 initialiser
        view = MemoryView(bank.memory.unsqueeze(0).expand(batch, -1, -1, -1).to(storage))
    previous = transactions.copy_free_commits(copy_free)
    try:
        loss = hidden.new_zeros(())
        first_scores = None
        for c in range(commits):
            scores = hidden @ project[c]
            if first_scores is None:
                first_scores = scores
            prediction, index, weights = routing.torch_routed_read(view.values, scores, width)
            rows = routing.gather_rows(view.values, index)
            addresses = routing.absolute_addresses(view.values, index)
            error = targets[c] - prediction
            delta = weights.unsqueeze(-1) * error.unsqueeze(-2) - 0.125 * rows.float()
            positions = torch.arange(tokens, device=device).view(1, tokens, 1, 1)
            keys = addresses * tokens + positions
            proposal = WriteProposal(view.version, addresses.flatten(), delta.flatten(0, 3), view.lineage, keys.flatten())
            view = transactions.commit(view, transactions.merge(view, [proposal]))
            hidden = hidden + 0.5 * prediction
            loss = loss + prediction.square().mean()
        final, _, final_weights = routing.torch_routed_read(view.values, hidden @ project[commits], width)
        loss = loss + final.square().mean() + final_weights.square().sum() * 1e-3
        loss.backward()
    finally:
        transactions.copy_free_commits(previous)
    grads = {"bank": bank.memory.grad, "project": project.grad, "targets": targets.grad}
    return loss.detach(), view.values.detach(), grads


def assert_same_step(device, **kwargs):
    copied = training_step(device, copy_free=False, **kwargs)
    in_place = training_step(device, copy_free=True, **kwargs)
    assert torch.equal(copied[0], in_place[0])
    assert torch.equal(copied[1], in_place[1])
    for name in copied[2]:
        assert copied[2][name] is not None and copied[2][name].abs().sum() > 0, name
        assert torch.equal(copied[2][name], in_place[2][name]), name
