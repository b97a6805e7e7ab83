"""Value objects of a memory transaction and the learned bank.

Same fields, defaults and error text as the reference (gl_sdm/memory/state.py:7-70). One
extension: a view may hold bfloat16 values (the reference plans bf16 storage with fp32
accumulation, OPTIMIZATION_PLAN.md:99-105); the learned parameter itself stays float32.
"""
from dataclasses import dataclass, field

import torch
from torch import nn

_VIEW_DTYPES = (torch.float32, torch.bfloat16)


@dataclass(frozen=True)
class MemoryView:
    """An immutable bank version: values [requests, heads, slots, dim]."""
    values: torch.Tensor
    version: int = 0
    lineage: object = field(default_factory=object)

    def __post_init__(self):
        v = self.values
        bad_shape = v.ndim != 4 or min(v.shape) < 1
        if bad_shape or v.dtype not in _VIEW_DTYPES or self.version < 0:
            raise ValueError("memory views require nonempty [batch, heads, slots, dim] FP32 values and a nonnegative version")


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
