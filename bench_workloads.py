"""The five benchmark configurations as seeded synthetic inputs.

No public dataset is involved: the reference's own operator benchmark draws random tensors
(projects/gl-sdm/scripts/benchmark_memory.py:26-38) and so does this. Shapes, sizes and value
distributions follow the configuration texts: keys / factor scores N(0,1), bank values
N(0, 0.02), write targets N(0, 0.02), beta = sigmoid(N(0,1)), log-decay = -softplus(N(0,1)-4)
(gl_sdm/layers/global_layer.py:48-49). Every configuration is product-key shaped
(slots = half^2, gl_sdm/layers/router.py:18-22).
"""
from dataclasses import dataclass

import torch
import torch.nn.functional as F


@dataclass(frozen=True)
class Workload:
    name: str
    description: str
    heads: int
    half: int
    dim: int
    dk: int
    width: int
    sequences: int
    seq_len: int
    bank_dtype: torch.dtype
    per_request_banks: bool = False
    global_layers: int = 1
    chunk: int = 512
    zipf: float = 0.0

    @property
    def slots(self):
        return self.half * self.half

    @property
    def tokens_per_step(self):
        return self.sequences * self.seq_len

    @property
    def epochs(self):
        return self.seq_len // self.chunk

    @property
    def tokens_per_epoch(self):
        return self.sequences * self.chunk

    def scaled(self, sequences=None, seq_len=None):
        return Workload(**{**self.__dict__, "sequences": sequences or self.sequences, "seq_len": seq_len or self.seq_len})


WORKLOADS = {
    "c1": Workload("c1", "operator alone, fp32, batch 2 x 1024, 4096 slots, d_v 64, top-8", 4, 64, 64, 64, 8, 2, 1024,
                   torch.float32, per_request_banks=True),
    "c2": Workload("c2", "memory op of the 16-layer stack: 8 global layers, fp32 per-request banks of 16384 slots, "
                   "d_v 64, top-16, batch 8 x 4096", 8, 128, 64, 64, 16, 8, 4096, torch.float32,
                   per_request_banks=True, global_layers=8),
    "c3": Workload("c3", "bandwidth sweep: bf16 bank 1,048,576 slots, d_v 128, top-32, 16 x 4096 tokens", 1, 1024, 128,
                   128, 32, 16, 4096, torch.bfloat16),
    "c4": Workload("c4", "slot-sharded large bank: bf16 16,777,216 slots, d_v 256, top-32, 64 x 8192 tokens", 1, 4096,
                   256, 128, 32, 64, 8192, torch.bfloat16),
    "c4s": Workload("c4s", "one quarter of c4's slots (the key shard a GPU holds at 4 GPUs): bf16 4,194,304 slots, d_v 256, "
                    "top-32, 64 x 8192 tokens; for profiler captures that must stay small", 1, 2048, 256, 128, 32, 64, 8192,
                    torch.bfloat16),
    "c5": Workload("c5", "skewed routing: bf16 bank 4,194,304 slots, d_v 128, top-16, 4 x 32768 tokens, Zipf(1.1)", 1,
                   2048, 128, 128, 16, 4, 32768, torch.bfloat16, zipf=1.1),
}


def make_bank(w, device, seed=1234, banks=None):
    """Bank values N(0, 0.02) in the workload's storage dtype, drawn on `device` in slabs."""
    g = torch.Generator(device=device).manual_seed(seed)
    banks = (w.sequences if w.per_request_banks else 1) if banks is None else banks
    out = torch.empty((banks, w.heads, w.slots, w.dim), dtype=w.bank_dtype, device=device)
    flat = out.view(-1, w.dim)
    slab = 1 << 20
    for lo in range(0, flat.shape[0], slab):
        hi = min(lo + slab, flat.shape[0])
        flat[lo:hi] = (torch.randn((hi - lo, w.dim), generator=g, device=device) * 0.02).to(w.bank_dtype)
    return out


def zipf_targets(w, count, generator, device):
    """Slot per token with Zipf(s) popularity over a fixed random permutation of slots."""
    ranks = torch.arange(1, w.slots + 1, dtype=torch.float64, device=device)
    cdf = torch.cumsum(ranks.pow(-w.zipf), 0)
    cdf /= cdf[-1].clone()
    u = torch.rand(count, generator=generator, device=device, dtype=torch.float64)
    rank = torch.searchsorted(cdf, u).clamp_(max=w.slots - 1)
    perm = torch.randperm(w.slots, generator=torch.Generator(device=device).manual_seed(99), device=device)
    return perm[rank]


def make_epoch_inputs(w, device, seed, sequences=None, tokens=None, plant=4.0):
    """Factor scores and write operands of one commit epoch, rows [sequence, token, head].

    With w.zipf > 0 the scores of a planted target slot are raised by `plant` in both
    factors, so the selected slots follow the Zipf popularity (hot-slot commit contention).
    """
    g = torch.Generator(device=device).manual_seed(seed)
    n, t = sequences or w.sequences, tokens or w.chunk
    shape = (n, t, w.heads)
    out = {}
    for name in ("q_scores", "k_scores"):
        s = torch.randn((*shape, 2 * w.half), generator=g, device=device)
        if w.zipf > 0:
            slot = zipf_targets(w, n * t * w.heads, g, device).view(*shape, 1)
            s.scatter_add_(-1, slot // w.half, torch.full_like(slot, plant, dtype=s.dtype))
            s.scatter_add_(-1, w.half + slot % w.half, torch.full_like(slot, plant, dtype=s.dtype))
        out[name] = s
    out["target"] = (torch.randn((*shape, w.dim), generator=g, device=device) * 0.02).to(torch.bfloat16 if w.bank_dtype == torch.bfloat16 else torch.float32)
    out["beta"] = torch.randn(shape, generator=g, device=device).sigmoid()
    out["log_decay"] = -F.softplus(torch.randn(shape, generator=g, device=device) - 4)
    return out


def make_keys(w, device, seed=4321):
    """Slot keys [slots, dk] bf16: N(0,1) rows scaled to unit L2 norm, drawn in slabs."""
    g = torch.Generator(device=device).manual_seed(seed)
    out = torch.empty((w.slots, w.dk), dtype=torch.bfloat16, device=device)
    slab = 1 << 20
    for lo in range(0, w.slots, slab):
        hi = min(lo + slab, w.slots)
        x = torch.randn((hi - lo, w.dk), generator=g, device=device)
        out[lo:hi] = (x / x.norm(dim=1, keepdim=True)).to(torch.bfloat16)
    return out


def make_epoch_inputs_dense(w, device, seed, sequences=None, tokens=None, keys=None, plant=6.0):
    """Queries (read and write side) N(0,1) bf16 and the write operands of one commit epoch.

    With w.zipf > 0 and the slot keys given, every query is pulled toward the key of a target
    slot drawn from the Zipf popularity (q = plant * key[target] + N(0,1)), so routes pile up
    on hot slots."""
    g = torch.Generator(device=device).manual_seed(seed)
    n, t = sequences or w.sequences, tokens or w.chunk

    def queries():
        x = torch.randn((n, t, w.dk), generator=g, device=device)
        if w.zipf > 0 and keys is not None:
            target = zipf_targets(w, n * t, g, device)
            x = x + plant * keys[target].float().view(n, t, w.dk)
        return x.to(torch.bfloat16)

    out = {
        "q": queries(),
        "kq": queries(),
        "target": (torch.randn((n, t, 1, w.dim), generator=g, device=device) * 0.02).to(
            torch.bfloat16 if w.bank_dtype == torch.bfloat16 else torch.float32),
        "beta": torch.randn((n, t, 1), generator=g, device=device).sigmoid(),
        "log_decay": -F.softplus(torch.randn((n, t, 1), generator=g, device=device) - 4),
    }
    return out


def algorithmic_bytes(w, tokens, unique_fraction=1.0, layers=None, factored=False):
    """Bytes each stage must move for `tokens` tokens (per routing row: K routes, D value width, e bank element bytes, u unique-row fraction):
    query read K*D*e + 4*D plus 8*half of factor scores; proposal K*D*e + 8*half + target +
    K*(4*D+16) written; commit K*(4*D+16) read + u*K*2*D*e rows. With the factored commit no
    delta rows exist: the proposal stage ends at the error vector (4*(D+1) written), the commit
    reads 8 bytes of route per entry and the error vector once, and updates u*K rows."""
    e = 2 if w.bank_dtype == torch.bfloat16 else 4
    te = e
    L = layers or w.global_layers
    th = tokens * w.heads * L
    K, D, half = w.width, w.dim, w.half
    if factored:
        return {
            "read": th * (8 * half + K * D * e + 4 * D),
            "propose": th * (8 * half + K * D * e + D * te + 8 + 4 * (D + 1)),
            "commit": th * (K * 8 + 4 * (D + 1) + unique_fraction * K * 2 * D * e),
        }
    return {
        "read": th * (8 * half + K * D * e + 4 * D),
        "propose": th * (8 * half + K * D * e + D * te + 8 + K * (4 * D + 16)),
        "commit": th * (K * (4 * D + 16) + unique_fraction * K * 2 * D * e),
    }
