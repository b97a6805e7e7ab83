"""Slot-sharded shared bank across the GPUs of one node (one process per GPU, NCCL).

The reference is single-GPU (no torch.distributed anywhere); this is the multi-GPU design of
the same operator. Rank r of R owns the contiguous slot block [r*S/R, (r+1)*S/R) of every head
(for product keys: a block of left-factor indices). Tokens are data-parallel: each rank routes
its own tokens, whose factor scores already cover all slots. Per 512-token commit epoch there
are three collectives, none of them inside a kernel:

  1. all-gather of the routes (int32 slot + fp32 weight, query and write side): K candidates
     per token instead of value rows;
  2. every rank forms partial readings of ALL tokens over the rows it owns; a reduce-scatter
     returns each rank the finished readings / write predictions of its own tokens;
  3. at the commit clock the write operands go to the owning shard: an all-gather of the
     per-token error vector beta*(target - decay*prediction) and decay-1. The slot owner
     expands them against its own rows into delta rows (delta_k = (decay-1)*row_k + w_k*err,
     gl_sdm/runtime/dense.py:11-14) and commits locally. Shipping the factored form moves
     dim+1 floats per token instead of K*(dim+1) per token of expanded deltas.

Entry order inside a shard is (global token row, route), so the stable commit sums each
address in the same order as the unsharded operator.
"""
import torch

from . import _native


def shard_range(slots, rank, world):
    if slots % world:
        raise ValueError("slots must divide evenly over the ranks")
    per = slots // world
    return rank * per, (rank + 1) * per


class ShardedBankOperator:
    """Same epoch interface as SharedBankOperator; `values` is the full bank [1, H, S, D]
    (each rank keeps its slice) or, with ``is_shard=True``, already this rank's slice."""

    def __init__(self, values, reads, writes, dist, chunk_size=512, num_layers=1, layer_index=0,
                 group=None, is_shard=False, slots=None, kernels=_native):
        if reads != writes:
            raise ValueError("the sharded operator needs equal read and write widths")
        self.dist, self.group, self.k = dist, group, kernels
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if values.ndim != 4 or values.shape[0] != 1:
            raise ValueError("a shared bank is [1, heads, slots, dim]")
        self.heads, self.dim = values.shape[1], values.shape[3]
        self.slots = slots if is_shard else values.shape[2]
        self.slot_lo, self.slot_hi = shard_range(self.slots, self.rank, self.world)
        self.shard = values if is_shard else values[:, :, self.slot_lo:self.slot_hi].contiguous()
        self.half = int(round(self.slots ** 0.5))
        if self.half * self.half != self.slots:
            raise ValueError("product-key routing needs a square number of slots")
        self.width = kernels.routes_out(reads, self.half)
        self.reads = reads
        self.chunk_size, self.num_layers, self.layer_index = chunk_size, num_layers, layer_index
        self.key_bits = max(1, (self.heads * self.slots * chunk_size * num_layers - 1).bit_length())
        self.version = 0
        self._buf = {}

    def _buffer(self, name, numel, dtype):
        b = self._buf.get(name)
        if b is None or b.numel() < numel or b.dtype != dtype:
            b = torch.empty(numel, dtype=dtype, device=self.shard.device)
            self._buf[name] = b
        return b[:numel]

    def epoch(self, q_scores, k_scores, target, beta, log_decay, offset=0):
        """q_scores/k_scores [sequences_local, tokens, heads, 2*half]; returns the readings of
        this rank's tokens and commits every rank's proposals into the owning shards."""
        k, dist, R, K, D = self.k, self.dist, self.world, self.width, self.dim
        tokens = q_scores.shape[1]
        n = q_scores.numel() // q_scores.shape[-1]          # local routing rows
        region = n * K
        # 1. local routes straight into the send buffer [idx_q | idx_k | w_q | w_k]
        send = self._buffer("routes_send", 4 * region, torch.int32)
        k.pk_select_into(q_scores, self.reads, send, 0, 2 * region)
        k.pk_select_into(k_scores, self.reads, send, region, 3 * region)
        routes = self._buffer("routes_all", R * 4 * region, torch.int32)
        dist.all_gather_into_tensor(routes, send, group=self.group)
        # 2. partial readings of every rank's query and write rows over the owned slots
        partial = k.shard_read(self.shard, self.slot_lo, self.slots, routes, 0, 2 * region, R * 2 * n, 2 * n,
                               4 * region, K)
        mine = torch.empty((2 * n, D), dtype=torch.float32, device=self.shard.device)  # returned to the caller
        dist.reduce_scatter_tensor(mine, partial, group=self.group)
        readings = mine[:n].view(*q_scores.shape[:-1], D)
        prediction = mine[n:]
        # 3. write operands to the owning shards, expansion and local commit
        packed = k.write_error(prediction, target, beta, log_decay,
                               self._buffer("error_send", n * (D + 1), torch.float32))
        errors = self._buffer("error_all", R * n * (D + 1), torch.float32)
        dist.all_gather_into_tensor(errors, packed, group=self.group)
        offsets = k.shard_offsets(routes, region, R * n, n, 4 * region, K, self.slot_lo, self.slot_hi)
        entries = int(offsets[-1].item())
        if entries:
            out = (self._buffer("addresses", entries, torch.int64),
                   self._buffer("deltas", entries * D, torch.float32).view(entries, D),
                   self._buffer("keys", entries, torch.int64))
            a, d, s = k.shard_propose(self.shard, self.slot_lo, self.slots, routes, region, 3 * region, 4 * region,
                                      errors, n * (D + 1), None, offsets, entries, R * n, n, tokens, K, offset,
                                      self.chunk_size, self.num_layers, self.layer_index, out)
            flat = self.shard.view(-1, D)
            k.commit_rows(flat, a, d, s, out=flat, key_bits=self.key_bits)
        self.version += 1
        return readings

    def gather_bank(self):
        """The whole bank [1, H, S, D] on every rank (tests and checkpoints)."""
        pieces = [torch.empty_like(self.shard) for _ in range(self.world)]
        self.dist.all_gather(pieces, self.shard, group=self.group)
        return torch.cat(pieces, dim=2)
