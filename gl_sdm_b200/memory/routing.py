"""Chunk-clock product-key routing and snapshot read on the CUDA kernels.

Public names and signatures are the reference's (gl_sdm/memory/routing.py:10-66). Scores
are [batch, token, head, 2*half] (or [batch, reasoning, token, head, 2*half]); equal
scores prefer the larger address; indices come back ascending with softmax weights.
"""
import torch

from .. import _native
from . import autograd, oracle_hook


def torch_routed_read(memory, scores, width, reference=False):
    """Routed read of [B, T, H, 2*half] scores: (readings, index int64, weights).

    Keeps the reference's name (routing.py:10-28); the arithmetic is the fused
    select + read kernel. ``reference=True`` resolves to a registered oracle.
    """
    if reference:
        return oracle_hook.get("routed_read")(memory, scores, width)
    _native.require_cuda(memory)
    _native.require_device(scores)
    B, T, H, _ = scores.shape
    if memory.shape[0] not in (1, B) or memory.shape[1] != H:
        raise ValueError("scores and memory disagree on batch or heads")
    if autograd.needs_grad(memory, scores):
        return autograd.RoutedRead.apply(memory, scores, width)
    return _native.pk_select_read(memory, scores.float().contiguous(), width, rows_per_bank=T * H)


def absolute_addresses(memory, index):
    """Flat bank row (request*heads + head)*slots + slot of index [B, T, H, K]."""
    B, H, S, _ = memory.shape
    partitions = torch.arange(B * H, device=memory.device).view(B, 1, H, 1)
    return partitions * S + index.long()


def gather_rows(memory, index, reference=False):
    """Selected rows [B, T, H, K, D] (reference routing.py:37-42)."""
    if reference:
        return oracle_hook.get("gather_rows")(memory, index)
    _native.require_cuda(memory)
    addresses = absolute_addresses(memory, index).contiguous()
    if autograd.needs_grad(memory):
        return autograd.GatherRows.apply(memory, addresses)
    return _native.gather_rows(memory.flatten(0, 2), addresses)


def routed_read(block, memory, scores, width, physical=None):
    """Dispatcher with the reference's signature (routing.py:45-66).

    ``block.attn.reference`` requests the registered oracle; otherwise the CUDA path runs
    whatever ``block.attn.backend`` says. ``physical`` (a bank padded for the reference's
    external read schedule, layers/stack.py:50-51) is accepted and ignored: the kernels read
    the logical bank directly.
    """
    shape = scores.shape
    flat = scores.reshape(shape[0], -1, *shape[-2:])
    if block.attn.reference:
        out = oracle_hook.get("routed_read")(memory, flat, width)
    else:
        out = torch_routed_read(memory, flat, width)
    if len(shape) == 5:
        out = tuple(t.reshape(*shape[:-1], t.shape[-1]) for t in out)
    return out
