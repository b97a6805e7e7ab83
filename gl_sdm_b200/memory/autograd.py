"""Differentiable wrappers of the CUDA operator (forward AND backward on the kernels).

The reference differentiates its torch path with autograd and its native path with custom
backward kernels that fill a dense, zero-initialised bank gradient per read
(gl_sdm/memory/backends/token.py:134-168, OPTIMIZATION_PLAN.md:45-54). Here the bank gradient
of a read or a row gather stays compact - one (flat address, row) pair per route - and is
folded into the dense tensor autograd expects by the same deterministic sort + segmented sum
the commit uses, so gradients are reproducible bit for bit.
"""
import torch

from .. import _native
from . import state


def _dense_bank_gradient(shape, device, addresses, rows):
    """Scatter-add compact row gradients into a zero fp32 bank of the given shape."""
    zero = torch.zeros(shape, dtype=torch.float32, device=device)
    if addresses.numel() == 0:
        return zero
    flat = zero.view(-1, shape[-1])
    _native.commit_rows(flat, addresses.reshape(-1), rows.reshape(-1, shape[-1]).contiguous(), None, out=flat)
    return zero


def version_operand(bank, node):
    """What a backward reads the rows of an older bank version from: (tensor, undo logs).

    ``node`` is the chain node (state.tail_of) the forward saw. If copy-free commits have
    since updated the tensor in place, their logs lead back to that version; a chain longer
    than one kernel call takes is resolved by rebuilding the version once (kept on the node).
    Any other in-place change of the tensor is an error, as it is for tensors autograd saves."""
    logs, last = node.later()
    if bank._version != last.accounted:
        raise RuntimeError("the memory bank a differentiable read used was modified in place by something other "
                           "than a copy-free commit")
    if len(logs) <= _native.MAX_UNDO_LOGS:
        return bank, [(log.addresses, log.rows) for log in logs]
    if node.rebuilt is None:
        rebuilt = bank.clone()
        for log in reversed(logs):         # newest commit first, so the oldest row wins
            _native.undo_apply(rebuilt, log.addresses, log.rows)
        node.rebuilt = rebuilt
    return node.rebuilt, []


class RoutedRead(torch.autograd.Function):
    """(readings, index, weights) = routed read of factor scores [B, T, H, 2*half].

    The bank is not handed to autograd's saved tensors: a copy-free commit may update it in
    place before the backward runs, and the backward then reads the version the forward saw
    through the undo logs (``version_operand``)."""

    @staticmethod
    def forward(ctx, memory, scores, width):
        B, T, H, L = scores.shape
        scores = scores.detach().float().contiguous()
        readings, index, weights = _native.pk_select_read(memory.detach(), scores, width, rows_per_bank=T * H)
        ctx.save_for_backward(index, weights)
        ctx.bank, ctx.node = memory.detach(), state.tail_of(memory)
        ctx.geometry = (T * H, L // 2)
        ctx.mark_non_differentiable(index)
        return readings, index, weights

    @staticmethod
    def backward(ctx, grad_readings, _grad_index, grad_weights):
        index, weights = ctx.saved_tensors
        memory, logs = version_operand(ctx.bank, ctx.node)
        rows_per_bank, half = ctx.geometry
        if grad_readings is None:
            grad_readings = torch.zeros((*index.shape[:-1], memory.shape[-1]), device=memory.device)
        grad_weights = None if grad_weights is None else grad_weights.float().contiguous()
        grad_scores, addresses, rows = _native.read_backward(memory, grad_readings.float().contiguous(), grad_weights,
                                                             index, weights, rows_per_bank, half, logs)
        grad_memory = (_dense_bank_gradient(memory.shape, memory.device, addresses, rows).to(memory.dtype)
                       if ctx.needs_input_grad[0] else None)
        return grad_memory, grad_scores if ctx.needs_input_grad[1] else None, None


class GatherRows(torch.autograd.Function):
    """rows = flat[addresses]; the backward folds the row gradients back deterministically."""

    @staticmethod
    def forward(ctx, memory, addresses):
        ctx.save_for_backward(addresses)
        ctx.bank = (memory.shape, memory.device, memory.dtype)
        return _native.gather_rows(memory.detach().flatten(0, 2), addresses)

    @staticmethod
    def backward(ctx, grad_rows):
        (addresses,) = ctx.saved_tensors
        shape, device, dtype = ctx.bank
        return _dense_bank_gradient(shape, device, addresses, grad_rows.float()).to(dtype), None


class Commit(torch.autograd.Function):
    """new bank = commit(bank, addresses, deltas, keys) (reference backends/commit.py:36-54)."""

    @staticmethod
    def forward(ctx, values, addresses, deltas, keys, key_bits):
        ctx.save_for_backward(addresses)
        return _native.commit_rows(values.detach(), addresses, deltas.detach(), keys, key_bits=key_bits)

    @staticmethod
    def backward(ctx, incoming):
        (addresses,) = ctx.saved_tensors
        incoming = incoming.contiguous()
        grad_deltas = None
        if ctx.needs_input_grad[2]:
            grad_deltas = _native.gather_rows(incoming.float().view(-1, incoming.shape[-1]), addresses)
        return incoming if ctx.needs_input_grad[0] else None, None, grad_deltas, None, None


class OverlayCommit(torch.autograd.Function):
    """The same commit applied to the bank tensor IN PLACE (no per-commit copy, which the
    reference pays at gl_sdm/memory/transactions.py:96), differentiable like ``Commit``: the
    gradient passes through to the previous version unchanged and every delta receives the
    gradient row of its address. The undo log the kernel writes is appended to ``made``; the
    caller links it into the tensor's chain so that backwards of earlier reads still find the
    rows they read (OPTIMIZATION_PLAN.md, "carry gradients back through updates")."""

    @staticmethod
    def forward(ctx, values, addresses, deltas, keys, key_bits, made):
        ctx.mark_dirty(values)
        ctx.save_for_backward(addresses)
        made.append(_native.commit_undo(values.detach(), addresses, deltas.detach(), keys, key_bits=key_bits))
        return values

    @staticmethod
    def backward(ctx, incoming):
        (addresses,) = ctx.saved_tensors
        incoming = incoming.contiguous()
        grad_deltas = None
        if ctx.needs_input_grad[2]:
            grad_deltas = _native.gather_rows(incoming.float().view(-1, incoming.shape[-1]), addresses)
        return incoming if ctx.needs_input_grad[0] else None, None, grad_deltas, None, None, None


class FusedProposal(torch.autograd.Function):
    """(addresses, deltas, keys) of the fused write proposal, differentiable in the bank, the
    write scores, the target, beta and the log-decay (reference: autograd through
    gl_sdm/layers/global_layer.py:41-51 and gl_sdm/runtime/dense.py:11-14). Forward and backward
    are one kernel each; nothing of size [rows, routes, dim] is kept between them except the
    delta rows themselves. Like ``RoutedRead`` the backward reads the rows of the bank version
    the forward saw through the undo logs of later copy-free commits."""

    @staticmethod
    def forward(ctx, values, scores, target, beta, log_decay, geometry):
        tokens, width, chunk_offset, chunk_size, num_layers, layer_index = geometry
        scores = scores.detach().float().contiguous()
        target = target.detach().contiguous()
        beta, log_decay = beta.detach().float().contiguous(), log_decay.detach().float().contiguous()
        addresses, deltas, keys = _native.pk_propose(values.detach(), scores, target, beta, log_decay, None,
                                                     tokens=tokens, width=width, chunk_offset=chunk_offset,
                                                     chunk_size=chunk_size, num_layers=num_layers, layer_index=layer_index)
        ctx.save_for_backward(scores, target, beta, log_decay, addresses)
        ctx.bank, ctx.node = values.detach(), state.tail_of(values)
        ctx.geometry = (tokens, width)
        ctx.mark_non_differentiable(addresses, keys)
        return addresses, deltas, keys

    @staticmethod
    def backward(ctx, _grad_addresses, grad_deltas, _grad_keys):
        scores, target, beta, log_decay, addresses = ctx.saved_tensors
        memory, logs = version_operand(ctx.bank, ctx.node)
        tokens, width = ctx.geometry
        if grad_deltas is None:
            return None, None, None, None, None, None
        grad_scores, grad_target, grad_beta, grad_log_decay, grad_rows = _native.pk_propose_backward(
            memory, scores, target, beta, log_decay, None, addresses, grad_deltas.float().contiguous(), tokens, width, logs)
        need = ctx.needs_input_grad
        grad_memory = (_dense_bank_gradient(memory.shape, memory.device, addresses, grad_rows).to(memory.dtype)
                       if need[0] else None)
        return (grad_memory, grad_scores if need[1] else None,
                grad_target.view(target.shape).to(target.dtype) if need[2] else None,
                grad_beta.view(beta.shape) if need[3] else None,
                grad_log_decay.view(log_decay.shape) if need[4] else None, None)


class TokenRead(torch.autograd.Function):
    """Token-clock weighted read of supplied routes [A, H, K] -> [A, H, D].

    The forward is the same kernel the forward-only call runs. Like the reference's wrapper
    (gl_sdm/memory/backends/token.py:134-168) it keeps the selected rows, not the bank, for
    the backward; unlike it the bank gradient is scattered deterministically.
    """

    @staticmethod
    def forward(ctx, values, requests, indices, weights, addresses):
        heads = values.shape[1]
        weights = weights.detach().float().contiguous()
        out = _native.snapshot_read(values.detach(), indices, weights, rows_per_bank=heads, requests=requests)
        rows = _native.gather_rows(values.detach().flatten(0, 2), addresses) if ctx.needs_input_grad[3] else None
        ctx.save_for_backward(addresses, weights, rows)
        ctx.bank = (values.shape, values.device, values.dtype)
        return out

    @staticmethod
    def backward(ctx, incoming):
        addresses, weights, rows = ctx.saved_tensors
        shape, device, dtype = ctx.bank
        incoming = incoming.float()
        grad_values = grad_weights = None
        if ctx.needs_input_grad[0]:
            grad_values = _dense_bank_gradient(shape, device, addresses,
                                               weights.unsqueeze(-1) * incoming.unsqueeze(-2)).to(dtype)
        if ctx.needs_input_grad[3]:
            grad_weights = (rows.float() * incoming.unsqueeze(-2)).sum(-1)
        return grad_values, None, None, grad_weights, None


def token_proposal_deltas(values, addresses, weights, targets, beta, log_decay, mass):
    """Differentiable token-clock write proposal: the row gather runs on the kernels (its
    backward is the deterministic scatter), the delta itself is the reference's expression
    (gl_sdm/memory/transactions.py:52-58) in tensor ops so autograd covers every operand."""
    rows = GatherRows.apply(values, addresses).float()
    decay = log_decay.float().exp().unsqueeze(-1)
    decayed = rows * decay
    w = weights.float().unsqueeze(-1)
    retrieved = (decayed * w).sum(-2)
    error = beta.float() * (targets.float() - retrieved)
    delta = decayed - rows + w * error.unsqueeze(-2)
    return delta * mass.float()[:, None, None, None]


def needs_grad(*tensors):
    return torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors)
