"""The write side of the reference's global layer on ONE fused kernel.

``GlobalLayer.propose`` (gl_sdm/layers/global_layer.py:33-54) routes the write scores, reads
the prediction, gathers the selected rows, forms the delta rows with tensor arithmetic
(gl_sdm/runtime/dense.py:11-14) and builds the canonical sort keys: three operator calls and
about a dozen elementwise passes over [batch, token, head, route, dim]. ``propose`` below is a
drop-in for that method: the projections stay the layer's own modules (same parameters, same
checkpoint), everything after them is ``glsdm_pk_propose``. It serves forward-only calls
(prefill, decode, evaluation); when a gradient is needed, or the layer asks for the
reference path, it hands the call to the method it replaced.
"""
import torch
import torch.nn.functional as F

from .. import _native
from ..memory.state import WriteProposal


def _forward_only(layer, x, snapshot):
    if layer.attn.reference:
        return False
    if not torch.is_grad_enabled():
        return True
    return not (x.requires_grad or snapshot.values.requires_grad
                or any(p.requires_grad for p in layer.attn.parameters()))


def propose(self, x, snapshot, offset, layer_idx, chunk_size, num_layers, physical=None):
    """Same arguments and result as the reference method: a ``WriteProposal`` of
    [batch*token*head*writes] addresses, delta rows and (address, position, layer) keys
    against ``snapshot``. ``physical`` (the reference's padded bank) is not needed."""
    if not _forward_only(self, x, snapshot):
        return self._glsdm_reference_propose(x, snapshot, offset, layer_idx, chunk_size, num_layers, physical)
    B, T, _ = x.shape
    router = self.attn
    z = self.norm1(x)
    scores = router.k(z.to(router.k.weight.dtype)).float().view(B, T, router.heads, -1)
    dense = z.to(router.v.weight.dtype)
    target = router.v(dense)
    if target.dtype not in (torch.float32, torch.bfloat16):
        target = target.float()
    beta = router.beta(dense).float().sigmoid()
    log_decay = -F.softplus(router.decay(dense).float() - 4)
    values = snapshot.values
    _native.require_cuda(values)
    addresses, deltas, keys = _native.pk_propose(
        values, scores.contiguous(), target.contiguous(), beta.contiguous(), log_decay.contiguous(), None,
        tokens=T, width=router.num_writes, chunk_offset=offset, chunk_size=chunk_size, num_layers=num_layers,
        layer_index=layer_idx)
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
