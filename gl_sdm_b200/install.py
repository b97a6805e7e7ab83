"""Register this package under the reference's module names.

``gl_sdm/layers/stack.py``, ``global_layer.py``, ``router.py`` and ``model.py`` import
``gl_sdm.memory`` lazily (model.py:33-34,58), so installing substitutes in ``sys.modules``
before the model is created makes the unmodified reference stack run on these kernels.
"""
import sys

from . import memory
from .memory import state, transactions, routing, backends
from .memory.backends import urm, commit, primitives

_NAMES = {
    "gl_sdm.memory": memory,
    "gl_sdm.memory.state": state,
    "gl_sdm.memory.transactions": transactions,
    "gl_sdm.memory.routing": routing,
    "gl_sdm.memory.backends": backends,
    "gl_sdm.memory.backends.urm": urm,
    "gl_sdm.memory.backends.commit": commit,
    "gl_sdm.memory.backends.primitives": primitives,
}


def install(copy_free_commits=None, fused_proposals=False):
    """Make ``import gl_sdm.memory`` resolve to gl_sdm_b200.memory. Returns the replaced modules.

    ``fused_proposals`` additionally replaces the reference's ``GlobalLayer.propose``
    (layers/global_layer.py:33-54) by ``gl_sdm_b200.layers.propose``: forward-only calls then
    build their write proposal with one kernel; it imports ``gl_sdm.layers.global_layer``.

    ``copy_free_commits`` (True / False; None leaves the setting alone) chooses whether the
    commits the reference's layers issue (layers/stack.py:65, chunk.py:95, token.py:62,68) copy
    the bank as the reference does or update it in place with undo logs, see
    ``memory.transactions.copy_free_commits``."""
    if copy_free_commits is not None:
        transactions.copy_free_commits(copy_free_commits)
    previous = {name: sys.modules.get(name) for name in _NAMES}
    sys.modules.update(_NAMES)
    parent = sys.modules.get("gl_sdm")
    if parent is not None:
        parent.memory = memory
    if fused_proposals:
        import importlib
        from .layers import install_fused_proposals
        install_fused_proposals(importlib.import_module("gl_sdm.layers.global_layer"))
    return previous


def uninstall(previous):
    for name, module in previous.items():
        if module is None:
            sys.modules.pop(name, None)
        else:
            sys.modules[name] = module
