"""Token-clock reads/proposals and the buffered commit, on the CUDA kernels.

Interface, validation order and error text follow the reference
(gl_sdm/memory/transactions.py:13-97). ``backend`` is accepted for call compatibility
("torch" or "urm") but selects nothing: every call runs the sm_100a kernels, and tensors
that are not on a CUDA device raise. ``reference=True`` asks for an oracle that only a test
harness provides (see oracle_hook).
"""
import torch

from .. import _native
from . import autograd, oracle_hook
from .state import MemoryView, UndoLog, WriteProposal, WriteBuffer, tail_of

_BACKENDS = {"torch", "urm"}


def _check_backend(backend):
    if backend not in _BACKENDS:
        raise ValueError("memory backend must be torch or urm")


def addresses(view, requests, indices):
    """Flat bank row of every selected slot: (request*heads + head)*slots + slot."""
    heads, slots = view.values.shape[1:3]
    head = torch.arange(heads, device=indices.device).view(1, heads, 1)
    return (requests.view(-1, 1, 1) * heads + head) * slots + indices


def selected(view, requests, indices, reference=False):
    """Rows [A, H, K, D] of the selected slots (reference transactions.py:19-25)."""
    if reference:
        return oracle_hook.get("selected")(view, requests, indices)
    _native.require_cuda(view.values)
    return _native.gather_rows(view.values.flatten(0, 2), addresses(view, requests, indices).contiguous())


def read(view, requests, indices, weights, reference=False, backend="torch"):
    """Weighted read of supplied routes: [A, H, K] routes -> [A, H, D]."""
    _check_backend(backend)
    if reference:
        return oracle_hook.get("read")(view, requests, indices, weights)
    _native.require_cuda(view.values)
    if autograd.needs_grad(view.values, weights):
        return autograd.TokenRead.apply(view.values, requests.long().contiguous(), indices.contiguous(), weights,
                                        addresses(view, requests, indices).contiguous())
    heads = view.values.shape[1]
    return _native.snapshot_read(view.values, indices.contiguous(), weights.float().contiguous(),
                                 rows_per_bank=heads, requests=requests.long().contiguous())


def propose_write(view, requests, indices, weights, targets, beta, log_decay,
                  mass, reference=False, backend="torch"):
    """One delta update against the immutable snapshot (reference transactions.py:38-59).

    delta_k = mass * (decay*row_k - row_k + w_k * beta * (target - sum_j w_j*decay*row_j)).
    """
    _check_backend(backend)
    if reference:
        return oracle_hook.get("propose_write")(view, requests, indices, weights, targets, beta, log_decay, mass)
    _native.require_cuda(view.values)
    if autograd.needs_grad(view.values, weights, targets, beta, log_decay, mass):
        flat = addresses(view, requests, indices).contiguous()
        deltas = autograd.token_proposal_deltas(view.values, flat, weights, targets, beta, log_decay, mass)
        return WriteProposal(view.version, flat.flatten(), deltas.flatten(0, 2), view.lineage)
    flat_addresses, deltas = _native.token_propose(
        view.values, requests.long().contiguous(), indices.contiguous(), weights.float().contiguous(),
        targets.float().contiguous(), beta.float().contiguous(), log_decay.float().contiguous(),
        mass.float().contiguous())
    return WriteProposal(view.version, flat_addresses, deltas, view.lineage)


def merge(view, proposals):
    proposals = tuple(proposals)
    stale = any(p.base_version != view.version or p.lineage is not view.lineage for p in proposals)
    if not proposals or stale:
        raise ValueError("write buffers must be nonempty and use the same snapshot version")
    return WriteBuffer(view.version, proposals, view.lineage)


def _adjacent(tensors):
    """True when the tensors are consecutive contiguous pieces of one allocation (proposals
    written side by side into one buffer, see gl_sdm_b200.layers): no copy is needed then."""
    first = tensors[0]
    if torch.is_grad_enabled() and any(t.requires_grad for t in tensors):
        return False                      # a view over the pieces would cut their graphs
    at = first.storage_offset()
    base = first.untyped_storage().data_ptr()
    for t in tensors:
        if (t.dtype != first.dtype or t.shape[1:] != first.shape[1:] or not t.is_contiguous()
                or t.untyped_storage().data_ptr() != base or t.storage_offset() != at):
            return False
        at += t.numel()
    return True


def _concat(tensors):
    if len(tensors) == 1:
        return tensors[0]
    if _adjacent(tensors):
        first = tensors[0]
        rows = sum(t.shape[0] for t in tensors)
        return torch.as_strided(first, (rows, *first.shape[1:]), first.stride())
    return torch.cat(tensors)


_default_donate = False


def copy_free_commits(enabled):
    """Choose what ``commit`` does when its caller does not say (``donate=None``, which is what
    the reference's layers pass): False copies the bank per commit as the reference does,
    True commits in place with undo logs (``donate="overlay"``). Returns the previous choice."""
    global _default_donate
    previous = _default_donate == "overlay"
    _default_donate = "overlay" if enabled else False
    return previous


def commit(view, buffer, reference=False, backend="torch", donate=None, key_bits=0):
    """Apply a write buffer: stable sort by key, per-address fp32 sums, one write per row.

    Returns a new view (version + 1, same lineage). ``donate`` chooses what happens to the
    input view's storage (extensions for banks too large to copy per commit):
      False      the bank is copied, the input view's tensor stays bit-for-bit unchanged
                 (the reference's behaviour, gl_sdm/memory/transactions.py:96);
      True       update in place and hand the same storage to the new view; the old view must
                 not be read afterwards (not differentiable);
      "overlay"  update in place AND keep the old view valid: the commit records the rows it
                 overwrites (an undo log of the touched rows only) and the old view reads
                 through it (see ``MemoryView`` and ``memory.overlay``). The sort keys of such
                 a commit must be monotone in the address, as the reference's keys are: the
                 log is searched by bisection (a log that is not sets a device status bit).
                 Differentiable: gradients flow to the deltas and through to the previous
                 version, and backwards of reads made before the commit resolve the rows they
                 read through the logs, so a training step needs no bank copy per commit;
      None       (default) False, or "overlay" after ``copy_free_commits(True)``.
    ``key_bits`` optionally bounds the sort keys.
    """
    _check_backend(backend)
    if buffer.base_version != view.version or buffer.lineage is not view.lineage:
        raise ValueError("stale memory transaction")
    keyed = [p.sort_keys is not None for p in buffer.proposals]
    if any(keyed) and not all(keyed):
        raise ValueError("cannot mix keyed and unkeyed proposals")
    if reference:
        return oracle_hook.get("commit")(view, buffer)
    if donate is None:
        donate = _default_donate
    if donate not in (False, True, "overlay"):
        raise ValueError('donate must be False, True or "overlay"')
    if donate and view.stale:
        raise ValueError("an in-place commit needs the newest view of its storage")
    values = view.values
    _native.require_cuda(values)
    idx = _concat([p.addresses.reshape(-1) for p in buffer.proposals]).long().contiguous()
    delta = _concat([p.deltas for p in buffer.proposals]).float().contiguous()
    keys = _concat([p.sort_keys.reshape(-1) for p in buffer.proposals]).long().contiguous() if all(keyed) else None
    differentiable = autograd.needs_grad(values, delta)
    if donate == "overlay":
        if differentiable:
            made = []
            values = autograd.OverlayCommit.apply(values, idx, delta, keys, key_bits, made)
            log = UndoLog(*made[0])
        else:
            log = UndoLog(*_native.commit_undo(values, idx, delta, keys, key_bits=key_bits))
        log.accounted = values._version
        tail_of(values).next = log         # backwards of earlier differentiable reads continue here
        values._glsdm_tail = log
        object.__setattr__(view, "_undo", log)   # the old view reads through this commit and later ones
        return MemoryView(values, view.version + 1, view.lineage)
    if differentiable:
        if donate:
            raise ValueError("a donated (in-place) commit cannot be differentiated")
        updated = autograd.Commit.apply(values, idx, delta, keys, key_bits)
        return MemoryView(updated, view.version + 1, view.lineage)
    if donate:
        tail_of(values).broken = True      # older snapshots (and reads awaiting a backward) end here
        values._glsdm_tail = None
    updated = _native.commit_rows(values, idx, delta, keys, out=values if donate else None, key_bits=key_bits)
    return MemoryView(updated, view.version + 1, view.lineage)
