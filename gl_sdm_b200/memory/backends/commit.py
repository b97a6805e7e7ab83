"""Deterministic sparse commit (reference gl_sdm/memory/backends/commit.py:57-58)."""
from ... import _native


def commit(memory, indices, deltas, keys=None):
    """memory [B, H, S, D]; returns a new bank, the input is unchanged."""
    return _native.commit_rows(memory, indices.long().contiguous(), deltas.float().contiguous(),
                               None if keys is None else keys.long().contiguous())
