"""The write side of the reference's global layer on ONE fused kernel.

``GlobalLayer.propose`` (gl_sdm/layers/global_layer.py:33-54) routes the write scores, reads
the prediction, gathers the selected rows, forms the delta rows with tensor arithmetic
(gl_sdm/runtime/dense.py:11-14) and builds the canonical sort keys: three operator calls and
about a dozen elementwise passes over [batch, token, head, route, dim]. ``propose`` below is a
drop-in for that method: the projections stay the layer's own modules (same parameters, same
checkpoint), everything after them is ``glsdm_pk_propose``, and under autograd its backward
is ``glsdm_pk_propose_backward``: none of the [batch, token, head, route, dim] intermediates
of the tensor-op expression is computed or kept for the backward. A layer that asks for the
reference path gets the method this one replaced.
"""
import torch
import torch.nn.functional as F

from .. import _native
from ..memory import autograd
from ..memory.state import WriteProposal


class _Arena:
    """One allocation for the proposals of all global layers of one stack call against one
    snapshot: the commit then finds them side by side and concatenates nothing (the stack's
    functional commit otherwise copies every delta row once more, gl_sdm/memory/transactions.py:80)."""

    def __init__(self, capacity, dim, device):
        self.addresses = torch.empty(capacity, dtype=torch.int64, device=device)
        self.deltas = torch.empty((capacity, dim), dtype=torch.float32, device=device)
        self.keys = torch.empty(capacity, dtype=torch.int64, device=device)
        self.capacity, self.used, self.last_layer, self.calls = capacity, 0, -1, 0

    def take(self, entries):
        lo, hi = self.used, self.used + entries
        self.used = hi
        return self.addresses[lo:hi], self.deltas[lo:hi], self.keys[lo:hi]


# global layers per stack call of a model with that many blocks: the most seen so far
_layers_per_call = {}


def _buffers(snapshot, entries, dim, device, layer_idx, num_layers):
    """Where this proposal goes: the next piece of the snapshot's arena when the number of
    global layers is known (from an earlier call) and the piece fits, else nothing (the
    kernel wrapper allocates, the commit concatenates)."""
    if not hasattr(snapshot, "_arena"):
        return None
    arena = snapshot._arena
    fresh = arena is None or layer_idx <= arena.last_layer        # a new stack call begins
    if fresh:
        count = _layers_per_call.get(num_layers)
        arena = _Arena(entries * count if count else 0, dim, device)
        object.__setattr__(snapshot, "_arena", arena)
    arena.last_layer = layer_idx
    arena.calls += 1
    if arena.calls > _layers_per_call.get(num_layers, 0):
        _layers_per_call[num_layers] = arena.calls
    if arena.used + entries > arena.capacity:
        return None
    return arena.take(entries)


def _needs_grad(layer, x, snapshot):
    if not torch.is_grad_enabled():
        return False
    return (x.requires_grad or snapshot.values.requires_grad
            or any(p.requires_grad for p in layer.attn.parameters()) or any(p.requires_grad for p in layer.norm1.parameters()))


def propose(self, x, snapshot, offset, layer_idx, chunk_size, num_layers, physical=None):
    """Same arguments and result as the reference method: a ``WriteProposal`` of
    [batch*token*head*writes] addresses, delta rows and (address, position, layer) keys
    against ``snapshot``. ``physical`` (the reference's padded bank) is not needed.
    Differentiable (``autograd.FusedProposal``) for rows of up to 256 values; wider rows under
    autograd, and layers that ask for the reference path, go to the replaced method."""
    router = self.attn
    values = snapshot.values
    training = _needs_grad(self, x, snapshot)
    if router.reference or (training and values.shape[-1] > 256):
        return self._glsdm_reference_propose(x, snapshot, offset, layer_idx, chunk_size, num_layers, physical)
    B, T, _ = x.shape
    z = self.norm1(x)
    scores = router.k(z.to(router.k.weight.dtype)).float().view(B, T, router.heads, -1)
    dense = z.to(router.v.weight.dtype)
    target = router.v(dense)
    if target.dtype not in (torch.float32, torch.bfloat16):
        target = target.float()
    beta = router.beta(dense).float().sigmoid()
    log_decay = -F.softplus(router.decay(dense).float() - 4)
    _native.require_cuda(values)
    geometry = dict(tokens=T, width=router.num_writes, chunk_offset=offset, chunk_size=chunk_size,
                    num_layers=num_layers, layer_index=layer_idx)
    if training:
        addresses, deltas, keys = autograd.FusedProposal.apply(values, scores, target, beta, log_decay,
                                                               tuple(geometry.values()))
    else:
        entries = B * T * router.heads * _native.routes_out(router.num_writes, router.half)
        addresses, deltas, keys = _native.pk_propose(
            values, scores.contiguous(), target.contiguous(), beta.contiguous(), log_decay.contiguous(), None,
            out=_buffers(snapshot, entries, values.shape[-1], values.device, layer_idx, num_layers), **geometry)
    return WriteProposal(snapshot.version, addresses, deltas, snapshot.lineage, keys)


def install_fused_proposals(global_layer_module):
    """Replace ``GlobalLayer.propose`` of the given ``gl_sdm.layers.global_layer`` module (the
    reference's own, unmodified) with the fused one. Returns a function that undoes it."""
    cls = global_layer_module.GlobalLayer
    if getattr(cls, "_glsdm_reference_propose", None) is None:
        cls._glsdm_reference_propose = cls.propose
    cls.propose = propose

    def undo():
        cls.propose = cls._glsdm_reference_propose
    return undo
