"""Snapshot / proposal / commit API, name-for-name the reference's gl_sdm.memory
(projects/gl-sdm/src/gl_sdm/memory/__init__.py:5-9)."""
from .state import MemoryView, WriteProposal, WriteBuffer, MemoryCache, MemoryBank
from .transactions import read, propose_write, merge, commit
from . import routing  # noqa: F401

__all__ = ["MemoryView", "WriteProposal", "WriteBuffer", "MemoryCache",
           "MemoryBank", "read", "propose_write", "merge", "commit"]
