"""Value objects of a memory transaction and the learned bank.

Same fields, defaults and error text as the reference (gl_sdm/memory/state.py:7-70). One
extension: a view may hold bfloat16 values (the reference plans bf16 storage with fp32
accumulation, OPTIMIZATION_PLAN.md:99-105); the learned parameter itself stays float32.
"""
from dataclasses import FrozenInstanceError, dataclass, field

import torch
from torch import nn

_VIEW_DTYPES = (torch.float32, torch.bfloat16)


class UndoLog:
    """Rows one copy-free commit overwrote: ``addresses`` [entries] int64 sorted (runs of equal
    addresses), ``rows`` [entries, dim] with the old row at the first position of every run.
    ``next`` is the log of the following copy-free commit on the same storage, ``broken`` is
    set when the next change of the storage was made without a log (a donated commit)."""
    __slots__ = ("addresses", "rows", "next", "broken", "accounted", "rebuilt", "__weakref__")

    def __init__(self, addresses, rows):
        self.addresses, self.rows, self.next, self.broken = addresses, rows, None, False
        self.accounted = None   # the bank tensor's autograd version once this commit was applied
        self.rebuilt = None     # the version this commit produced, materialised for a long chain

    def later(self):
        """Logs of the commits applied after this one, oldest first, and the last of them
        (this one if there is none)."""
        if self.broken:
            raise RuntimeError("this snapshot was invalidated by an in-place (donated) commit of a later version")
        logs = self.next.chain() if self.next is not None else []
        return logs, (logs[-1] if logs else self)

    def chain(self):
        """This log and every later one, oldest commit first."""
        out, log = [], self
        while log is not None:
            if log.broken:
                raise RuntimeError("this snapshot was invalidated by an in-place (donated) commit of a later version")
            out.append(log)
            log = log.next
        return out


def tail_of(values):
    """The newest node of the undo-log chain of a bank tensor, kept on the tensor object
    itself: the log of the last copy-free commit, or a node without rows that marks "no such
    commit yet". A differentiable read holds the node it saw; whatever hangs off it when the
    backward runs are the commits that have since overwritten rows of the version it read.
    Nodes nobody holds any more are freed with their rows."""
    node = getattr(values, "_glsdm_tail", None)
    if node is None:
        node = UndoLog(None, None)
        node.accounted = values._version
        values._glsdm_tail = node
    return node


class MemoryView:
    """An immutable bank version: values [requests, heads, slots, dim].

    Same fields, defaults and validation as the reference's frozen dataclass
    (gl_sdm/memory/state.py:7-15). One addition: after a copy-free commit
    (``commit(..., donate="overlay")``) the storage behind this view holds the NEWER version
    and the view keeps the undo log that leads back to its own; ``values`` then rebuilds this
    version on first use (one bank copy plus the touched rows), while
    ``gl_sdm_b200.memory.overlay.read`` reads it without any copy.
    """
    __slots__ = ("_storage", "version", "lineage", "_undo", "_arena")

    def __init__(self, values, version=0, lineage=None):
        bad_shape = values.ndim != 4 or min(values.shape) < 1
        if bad_shape or values.dtype not in _VIEW_DTYPES or version < 0:
            raise ValueError("memory views require nonempty [batch, heads, slots, dim] FP32 values and a nonnegative version")
        set_ = object.__setattr__
        set_(self, "_storage", values)
        set_(self, "version", version)
        set_(self, "lineage", object() if lineage is None else lineage)
        set_(self, "_undo", None)      # first log between this version and the storage's content
        set_(self, "_arena", None)     # scratch of the proposals being collected against this view

    def __setattr__(self, name, value):
        raise FrozenInstanceError(f"cannot assign to field {name!r}")

    def __delattr__(self, name):
        raise FrozenInstanceError(f"cannot delete field {name!r}")

    def __repr__(self):
        return f"MemoryView(values={tuple(self._storage.shape)}, version={self.version}, stale={self._undo is not None})"

    @property
    def stale(self):
        """True when the storage has moved on and this version lives in undo logs."""
        return self._undo is not None

    @property
    def values(self):
        if self._undo is None:
            return self._storage
        if self._storage.requires_grad and torch.is_grad_enabled():
            raise RuntimeError("a snapshot behind copy-free commits cannot be rebuilt differentiably: "
                               "read the newest view, or rebuild under torch.no_grad()")
        from .. import _native
        rebuilt = self._storage.clone()
        for log in reversed(self._undo.chain()):   # newest commit first, so the oldest row wins
            _native.undo_apply(rebuilt, log.addresses, log.rows)
        object.__setattr__(self, "_storage", rebuilt)
        object.__setattr__(self, "_undo", None)
        return rebuilt


@dataclass(frozen=True)
class WriteProposal:
    """Weighted row deltas computed against one snapshot version."""
    base_version: int
    addresses: torch.Tensor          # [entries] flat (request, head, slot) rows
    deltas: torch.Tensor             # [entries, dim]
    lineage: object
    sort_keys: torch.Tensor | None = None  # [entries] canonical (address, position, layer) order


@dataclass(frozen=True)
class WriteBuffer:
    base_version: int
    proposals: tuple[WriteProposal, ...]
    lineage: object


@dataclass
class MemoryCache:
    """Per-request mutable state: the current view, pending proposals, local KV."""
    view: MemoryView
    owner: object
    tokens: int = 0
    pending: tuple[WriteProposal, ...] = ()
    local: dict = field(default_factory=dict)


class MemoryBank(nn.Module):
    """Learned initial bank [heads, slots, dim]; float32 whatever the model is cast to."""

    def __init__(self, heads, slots, dim):
        super().__init__()
        scale = (heads * dim) ** -0.5
        self.memory = nn.Parameter(torch.randn(heads, slots, dim) * scale)
        self.memory._sdm_memory_bank = True
        self.owner = object()

    def _apply(self, fn, recurse=True):
        # Moving devices is honoured, dtype casts are not: keep the exact fp32 initialiser.
        kept = self.memory.detach()
        kept_grad = self.memory.grad.detach() if self.memory.grad is not None else None
        super()._apply(fn, recurse)
        self.memory.data = kept.to(device=self.memory.device, dtype=torch.float32)
        if kept_grad is not None:
            self.memory.grad.data = kept_grad.to(device=self.memory.device, dtype=torch.float32)
        return self

    def snapshot(self, batch_size):
        per_request = self.memory.unsqueeze(0).expand(batch_size, -1, -1, -1)
        return MemoryView(per_request.clone())

    def new_cache(self, batch_size):
        return MemoryCache(self.snapshot(batch_size), self.owner)

    def validate_cache(self, cache, batch_size):
        values = cache.view.values
        ok = (cache.owner is self.owner and values.shape == (batch_size, *self.memory.shape)
              and values.device == self.memory.device and values.dtype == torch.float32)
        if not ok:
            raise ValueError("memory cache belongs to another model, batch, device or dtype")
