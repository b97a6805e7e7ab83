"""Reads of a snapshot whose storage has moved on (copy-free commits).

The reference keeps snapshots valid by cloning the bank at every commit
(gl_sdm/memory/transactions.py:96, state.py:61-62) and plans compact overlays instead
(OPTIMIZATION_PLAN.md, "Represent commits as compact overlays ... resolve a snapshot read
from the correct version"). ``commit(view, buffer, donate="overlay")`` updates the bank in
place and records the rows it overwrites; the functions here read the OLD view through those
records without rebuilding it. The newest view needs none of this: it is the plain bank.
These reads are forward-only. Training needs older versions only inside backwards (a read of
the then-newest view whose bank has moved on by the time its backward runs); ``autograd``
resolves those through the same logs.

Growth is bounded by the views themselves: a log lives as long as some older view (or the
chain hanging off it) is alive, and a view more than ``_native.MAX_UNDO_LOGS`` commits behind
is rebuilt once (``view.values``) instead of being read through an ever longer chain.
"""
from .. import _native
from . import autograd, routing


def logs_of(view):
    """(addresses, rows) of every commit applied to the view's storage since its version,
    oldest commit first; empty for the newest view."""
    if not view.stale:
        return []
    return [(log.addresses, log.rows) for log in view._undo.chain()]


def read(view, index, weights):
    """Weighted read of supplied routes [B, T, H, K] against ``view``'s version -> [B, T, H, D]."""
    if view.stale and autograd.needs_grad(view._storage, weights):
        raise ValueError("reads of an older view are forward-only: a differentiable read uses the newest view")
    logs = logs_of(view)
    if len(logs) > _native.MAX_UNDO_LOGS:
        logs = []                      # too far behind: rebuild this version once and read it plainly
    storage = view._storage if logs else view.values
    _, T, H, _ = index.shape
    return _native.overlay_read(storage, index.contiguous(), weights.float().contiguous(), T * H, logs)


def routed_read(view, scores, width):
    """Product-key routed read (gl_sdm/memory/routing.py:10-28) against ``view``'s version:
    (readings, index int64, weights). Routes do not depend on the bank's contents."""
    if not view.stale:
        return routing.torch_routed_read(view.values, scores, width)
    if autograd.needs_grad(view._storage, scores):
        raise ValueError("reads of an older view are forward-only: a differentiable read uses the newest view")
    index, weights = _native.pk_select(scores.float().contiguous(), width)
    return read(view, index, weights), index, weights
