"""Deterministic sparse commit (reference gl_sdm/memory/backends/commit.py:36-58)."""
from ... import _native
from .. import autograd


def commit(memory, indices, deltas, keys=None):
    """memory [B, H, S, D]; returns a new bank, the input is unchanged. Differentiable in the
    bank and the deltas, as the reference's autograd function is."""
    _native.require_cuda(memory)
    indices = indices.long().contiguous()
    deltas = deltas.float().contiguous()
    keys = None if keys is None else keys.long().contiguous()
    if autograd.needs_grad(memory, deltas):
        return autograd.Commit.apply(memory, indices, deltas, keys, 0)
    return _native.commit_rows(memory, indices, deltas, keys)
