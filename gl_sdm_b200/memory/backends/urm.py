"""The three names the reference calls on its external-read backend
(gl_sdm/memory/backends/urm.py:40-46,49-82,109-122), served by the in-tree kernels."""
import torch

from ... import _native
from .. import autograd


def verify_dependency():
    """The reference pins an external package here; this build needs only its own library."""
    lib = _native.library()
    return {"repository": "in-tree", "revision": f"glsdm-abi-{lib.glsdm_abi_version()}"}


def snapshot_read(values, addresses, weights):
    """Supplied-route read; addresses are flat rows of values.view(1, 1, -1, dim)."""
    dim = values.shape[-1]
    flat = values.reshape(1, 1, -1, dim)
    lead = weights.shape[:-1]
    rows = weights.numel() // weights.shape[-1]
    out = _native.snapshot_read(flat, addresses.reshape(rows, -1).contiguous(),
                                weights.reshape(rows, -1).float().contiguous(), rows_per_bank=rows)
    return out.view(*lead, dim)


def routed_snapshot_read(values, scores, width, allow_large_route=False):
    """Fused route + read of scores [B, T, H, 2*half] against values [B, H, S, D] (the logical
    bank or the reference's zero-padded physical one, layers/stack.py:50-51); int32 indices as
    the reference's native path returns them (memory/backends/urm.py:109-122). Differentiable
    in the bank and the scores."""
    _native.require_cuda(values)
    if scores.ndim != 4 or values.ndim != 4:
        raise ValueError("routed_snapshot_read expects values [B, H, S, D] and scores [B, T, H, 2*half]")
    _native.require_device(scores)
    B, T, H, _ = scores.shape
    if values.shape[0] not in (1, B) or values.shape[1] != H:
        raise ValueError("scores and memory disagree on batch or heads")
    if autograd.needs_grad(values, scores):
        readings, index, weights = autograd.RoutedRead.apply(values, scores, width)
        return readings, index.to(torch.int32), weights
    return _native.pk_select_read(values, scores.float().contiguous(), width, rows_per_bank=T * H,
                                  index_dtype=torch.int32)
