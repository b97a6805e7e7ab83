"""Slot-sharded shared bank across the GPUs of one node (one process per GPU, NCCL).

The reference is single-GPU (no torch.distributed anywhere); this is the multi-GPU design of
the same operator. Rank r of R owns the contiguous slot block [r*S/R, (r+1)*S/R) of every head
(and, in dense-key mode, the same block of key rows). Tokens are data-parallel. Per 512-token
commit epoch, all collectives run between kernels, never inside one:

routing, product-key scores (`epoch`): each rank routes its own tokens (their factor scores
  already cover all slots) and all-gathers the K routes per token (int32 slot + fp32 weight,
  query and write side): K candidates per token instead of value rows.
routing, dense keys (`epoch_dense`): the queries are all-gathered (2*dk bytes per token), each
  rank scores ALL tokens against its own key shard on the tensor cores and keeps a partial
  top-k (`glsdm_score_topk`); the K candidates of a token go to the rank that owns the token
  (all-to-all), which merges the R partial lists of its own tokens (`glsdm_topk_merge`: one
  deterministic order, whatever the arrival order); the finished routes (K slots + weights per
  token) are all-gathered, so all ranks hold identical global routes.
read: every rank forms partial readings of all tokens over the rows it owns; a reduce-scatter
  returns each rank the finished readings / write predictions of its own tokens.
commit clock: the write operands go to the owning shard as an all-gather of the per-token
  error vector beta*(target - decay*prediction) and decay-1. The slot owner expands them
  against its own rows into delta rows (delta_k = (decay-1)*row_k + w_k*err,
  gl_sdm/runtime/dense.py:11-14) and commits locally. The factored form moves dim+1 floats
  per token over NVLink instead of K*(dim+4) for expanded deltas.

The factored commit of a shard lists, on the device, the routes whose slot it owns in
(position, sequence, head, route) order, so the stable sort by address sums each address in
the same order as the unsharded operator; no entry count comes back to the host.
"""
import torch

from . import _native


def shard_range(slots, rank, world):
    if slots % world:
        raise ValueError("slots must divide evenly over the ranks")
    per = slots // world
    return rank * per, (rank + 1) * per


def _symmetric_memory(numel, device, dist, group):
    """float32 [numel] that every rank of the group can address, and its address on each rank
    (torch.distributed symmetric memory: one allocation per rank, mapped into all of them). The
    NVLink multicast mapping is not requested: only plain peer stores go there."""
    import os
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    import torch.distributed._symmetric_memory as symm
    world = dist.group.WORLD if group is None else group
    tensor = symm.empty(numel, dtype=torch.float32, device=device)
    handle = symm.rendezvous(tensor, world)
    if getattr(handle, "multicast_ptr", 0):
        import sys
        print("gl_sdm_b200: the symmetric-memory inbox also got an NVLink multicast mapping (unused here)", file=sys.stderr)
    return tensor, [int(p) for p in handle.buffer_ptrs]


class SingleProcess:
    """The collectives of a world of one rank (a single GPU running the sharded code path)."""

    @staticmethod
    def get_world_size(group=None):
        return 1

    @staticmethod
    def get_rank(group=None):
        return 0

    @staticmethod
    def all_gather_into_tensor(out, inp, group=None):
        out.view(-1).copy_(inp.reshape(-1))

    @staticmethod
    def reduce_scatter_tensor(out, inp, group=None):
        out.view(-1).copy_(inp.reshape(-1))

    @staticmethod
    def all_gather(outs, inp, group=None):
        outs[0].copy_(inp)

    @staticmethod
    def all_to_all_single(out, inp, group=None):
        out.view(-1).copy_(inp.reshape(-1))


class ShardedBankOperator:
    """Same epoch interface as SharedBankOperator; `values` is the full bank [1, H, S, D]
    (each rank keeps its slice) or, with ``is_shard=True``, already this rank's slice.
    `keys` [S, dk] (or this rank's [S/R, dk] slice with is_shard) enables dense-key routing."""

    def __init__(self, values, reads, writes, dist=None, chunk_size=512, num_layers=1, layer_index=0,
                 group=None, is_shard=False, slots=None, kernels=_native, keys=None, factored=True):
        if reads != writes:
            raise ValueError("the sharded operator needs equal read and write widths")
        dist = SingleProcess if dist is None else dist
        self.dist, self.group, self.k = dist, group, kernels
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if values.ndim != 4 or values.shape[0] != 1:
            raise ValueError("a shared bank is [1, heads, slots, dim]")
        self.heads, self.dim = values.shape[1], values.shape[3]
        self.slots = slots if is_shard else values.shape[2]
        self.slot_lo, self.slot_hi = shard_range(self.slots, self.rank, self.world)
        self.shard = values if is_shard else values[:, :, self.slot_lo:self.slot_hi].contiguous()
        self.keys = None
        if keys is not None:
            if self.heads != 1:
                raise ValueError("dense-key routing is implemented for single-head banks")
            self.keys = keys if is_shard else keys[self.slot_lo:self.slot_hi].contiguous()
            if self.keys.shape[0] != self.slot_hi - self.slot_lo:
                raise ValueError("key shard does not match the slot shard")
        self.half = int(round(self.slots ** 0.5))
        self.width = reads if keys is not None else kernels.routes_out(reads, self.half)
        self.reads = reads
        self.chunk_size, self.num_layers, self.layer_index = chunk_size, num_layers, layer_index
        self.key_bits = max(1, (self.heads * self.slots * chunk_size * num_layers - 1).bit_length())
        self.version = 0
        # factored: the commit rebuilds every delta row from its token's error vector and the
        # bank row it updates (no [entries, dim] delta array); False keeps the two-step
        # proposal + commit with materialised deltas. Both give bit-identical banks.
        self.factored = factored
        self._buf = {}
        self._floor_state, self._floor_calls = None, 0
        self.marks = None   # set to a list to collect (stage name, CUDA event) pairs for profiling

    def _mark(self, name):
        if self.marks is not None:
            event = torch.cuda.Event(enable_timing=True)
            event.record()
            self.marks.append((name, event))

    def _buffer(self, name, numel, dtype):
        b = self._buf.get(name)
        if b is None or b.numel() < numel or b.dtype != dtype:
            b = torch.empty(numel, dtype=dtype, device=self.shard.device)
            self._buf[name] = b
        return b[:numel]

    # -- routing ---------------------------------------------------------------------------------

    def _routes_product_key(self, q_scores, k_scores, n):
        """Local routes into [idx_q | idx_k | w_q | w_k], all-gathered rank by rank."""
        if self.half * self.half != self.slots:
            raise ValueError("product-key routing needs a square number of slots")
        k, R, K = self.k, self.world, self.width
        region = n * K
        send = self._buffer("routes_send", 4 * region, torch.int32)
        self._mark("route")
        k.pk_select_into(q_scores, self.reads, send, 0, 2 * region)
        k.pk_select_into(k_scores, self.reads, send, region, 3 * region)
        routes = self._buffer("routes_all", R * 4 * region, torch.int32)
        self.dist.all_gather_into_tensor(routes, send, group=self.group)
        return dict(routes=routes, stride=4 * region, read_weights_at=2 * region, write_index_at=region,
                    write_weights_at=3 * region)

    def _routes_dense(self, queries, write_queries, n):
        """All-gather queries, partial top-k on this rank's keys, all-gather the K candidates,
        identical merge on every rank. Rows are ordered (rank, side, token)."""
        k, R, K = self.k, self.world, self.width
        dk = queries.shape[-1]
        send = self._buffer("queries_send", 2 * n * dk, torch.bfloat16).view(2, n, dk)
        send[0].copy_(queries.reshape(n, dk))
        send[1].copy_(write_queries.reshape(n, dk))
        everyone = self._buffer("queries_all", R * 2 * n * dk, torch.bfloat16)
        self.dist.all_gather_into_tensor(everyone, send.view(-1), group=self.group)
        rows = R * 2 * n
        # this rank's candidates: scores then slots in one buffer, so that one all-gather moves both
        mine = self._buffer("cand", 2 * rows * K, torch.int32)
        self._mark("score_topk")
        self._score_all_rows(everyone.view(rows, dk), mine[:rows * K].view(torch.float32).view(rows, K),
                             mine[rows * K:].view(rows, K))
        self._mark("merge")
        region = n * K
        if R == 1:
            routes = self._buffer("routes_all", 4 * region, torch.int32)
            k.topk_merge_packed(mine, 1, rows, K, out=(routes[:2 * region].view(rows, K),
                                                       routes[2 * region:].view(torch.float32).view(rows, K)))
        else:
            # candidates of the tokens of rank o, scores then slots, contiguous per destination
            outgoing = self._buffer("cand_out", 2 * rows * K, torch.int32)
            outgoing.view(R, 2, 2 * region).copy_(mine.view(2, R, 2 * region).transpose(0, 1))
            incoming = self._buffer("cand_in", 2 * rows * K, torch.int32)
            self.dist.all_to_all_single(incoming, outgoing, group=self.group)
            # R partial lists for each of this rank's 2n rows -> its final routes [slots | weights]
            own = self._buffer("routes_send", 4 * region, torch.int32)
            k.topk_merge_packed(incoming, R, 2 * n, K, out=(own[:2 * region].view(2 * n, K),
                                                             own[2 * region:].view(torch.float32).view(2 * n, K)))
            routes = self._buffer("routes_all", R * 4 * region, torch.int32)
            self.dist.all_gather_into_tensor(routes, own, group=self.group)
        # per rank block: [slots of the query rows | slots of the write rows | weights, same order]
        return dict(routes=routes, stride=4 * region, read_weights_at=2 * region, write_index_at=region,
                    write_weights_at=3 * region)

    def _score_all_rows(self, queries, scores, slots):
        """Partial top-k of ALL rows on this rank's keys, the ranks telling each other what they
        have reached while their kernels run (glsdm_score_topk_shared). A streaming top-k spends
        about K * (1 + ln(n / K)) list insertions per row before its threshold is tight, whatever
        the shard size, so R shards pay that R times. Here every rank walks the rows from a
        different starting point (a rotated copy of the queries): after the first R-th of its
        rows, whatever row a rank begins has usually been finished by another rank, whose K-th
        best score - the K-th best over a part of the bank, so never above the true one - arrives
        through peer memory and lets this rank drop nearly all of its candidates at once. Nobody
        waits; without peer memory (or alone) this is the plain kernel."""
        k, R, K = self.k, self.world, self.width
        rows = queries.shape[0]
        inbox = self._floor_inbox(rows) if R > 1 else None
        if inbox is None:
            k.score_topk(queries, self.keys, K, col_base=self.slot_lo, out=(scores, slots))
            return
        boxes, peers = inbox
        call = self._floor_calls
        self._floor_calls += 1
        # The other half was written during the previous call. Every peer finished that call
        # before it entered the collective this rank has just completed (the all-gather of the
        # queries), and none starts the next one before this rank enters the next all-gather:
        # clearing here can neither lose a bound of this call nor leave one of an older call.
        boxes[(call + 1) % 2].fill_(float("-inf"))
        mine_at = ((call % 2) * R + self.rank) * rows * 4
        shift = (rows // R // 128) * 128 * self.rank
        if shift:
            turned = self._buffer("queries_turned", queries.numel(), queries.dtype).view_as(queries)
            turned.copy_(torch.roll(queries, -shift, 0))
            out_scores = self._buffer("cand_turned_scores", scores.numel(), scores.dtype).view_as(scores)
            out_slots = self._buffer("cand_turned_slots", slots.numel(), slots.dtype).view_as(slots)
        else:
            turned, out_scores, out_slots = queries, scores, slots
        k.score_topk(turned, self.keys, K, col_base=self.slot_lo, out=(out_scores, out_slots),
                     floor_in=boxes[call % 2], floor_out=[p + mine_at for i, p in enumerate(peers) if i != self.rank],
                     row_shift=shift)
        if shift:
            scores.copy_(torch.roll(out_scores, shift, 0))
            slots.copy_(torch.roll(out_slots, shift, 0))

    def _floor_inbox(self, rows):
        """([2, R, rows] float32 in memory the peers can store into, [its address on every rank]),
        or None where peer memory is not to be had (then the ranks simply do not share bounds)."""
        if self._floor_state is not None and self._floor_state[0] == rows:
            return self._floor_state[1]
        self._floor_state = (rows, None)
        import os
        if self.world - 1 > 7 or os.environ.get("GLSDM_SHARED_BOUNDS", "1") == "0":
            return None
        numel = 2 * self.world * rows
        try:
            if hasattr(self.dist, "peer_memory"):              # ranks that share one process and GPU (tests)
                boxes, peers = self.dist.peer_memory(numel, self.shard.device, self.group)
            else:
                boxes, peers = _symmetric_memory(numel, self.shard.device, self.dist, self.group)
        except Exception as error:                             # noqa: BLE001 - any failure only costs the saving
            import sys
            print(f"gl_sdm_b200: no peer memory for shared routing bounds ({type(error).__name__}: {error})", file=sys.stderr)
            return None
        boxes = boxes[:numel].view(2, self.world, rows)
        boxes.fill_(float("-inf"))
        self._floor_calls = 0
        # nobody may store into a box that its owner has not cleared yet
        token = torch.zeros(1, device=self.shard.device)
        everyone = torch.empty(self.world, device=self.shard.device)
        self.dist.all_gather_into_tensor(everyone, token, group=self.group)
        self._floor_state = (rows, (boxes, peers))
        return self._floor_state[1]

    # -- read, proposal, commit --------------------------------------------------------------------

    def _finish(self, plan, n, lead, target, beta, log_decay, tokens, offset):
        k, dist, R, K, D = self.k, self.dist, self.world, self.width, self.dim
        routes, stride = plan["routes"], plan["stride"]
        self._last_plan, self._last_n = plan, n
        self._mark("read")
        # partial readings of every rank's query and write rows over the owned slots
        partial = k.shard_read(self.shard, self.slot_lo, self.slots, routes, 0, plan["read_weights_at"], R * 2 * n,
                               2 * n, stride, K)
        if R > 1:
            mine = torch.empty((2 * n, D), dtype=torch.float32, device=self.shard.device)
            dist.reduce_scatter_tensor(mine, partial, group=self.group)
        else:
            mine = partial
        readings = mine[:n].view(*lead, D)
        prediction = mine[n:]
        # write operands to the owning shards, expansion and local commit
        self._mark("propose")
        packed = k.write_error(prediction, target, beta, log_decay,
                               self._buffer("error_send", n * (D + 1), torch.float32))
        if R > 1:
            errors = self._buffer("error_all", R * n * (D + 1), torch.float32)
            dist.all_gather_into_tensor(errors, packed, group=self.group)
        else:
            errors = packed
        if self.factored:
            # every route of every rank is shown to the commit, which lists the ones this shard owns
            # on the device: nothing to count here, no host synchronisation in the epoch
            offsets, entries = None, R * n * K
        else:
            offsets = k.shard_offsets(routes, plan["write_index_at"], R * n, n, stride, K, self.slot_lo, self.slot_hi)
            entries = int(offsets[-1].item())
        if entries and self.factored:
            self._mark("commit")
            k.commit_factored(self.shard, self.slot_lo, self.slots, routes, plan["write_index_at"],
                              plan["write_weights_at"], stride, errors, n * (D + 1), None, offsets, entries, R * n, n,
                              tokens, K, offset, self.chunk_size, self.num_layers, self.layer_index, self.key_bits)
        elif entries:
            out = (self._buffer("addresses", entries, torch.int64),
                   self._buffer("deltas", entries * D, torch.float32).view(entries, D),
                   self._buffer("keys", entries, torch.int64))
            a, d, s = k.shard_propose(self.shard, self.slot_lo, self.slots, routes, plan["write_index_at"],
                                      plan["write_weights_at"], stride, errors, n * (D + 1), None, offsets, entries,
                                      R * n, n, tokens, K, offset, self.chunk_size, self.num_layers,
                                      self.layer_index, out)
            flat = self.shard.view(-1, D)
            self._mark("commit")
            k.commit_rows(flat, a, d, s, out=flat, key_bits=self.key_bits)
        self._mark("end")
        self.last_entries = entries // R if self.factored else entries   # owned entries (expected, when listed on the device)
        self.version += 1
        return readings

    def epoch(self, q_scores, k_scores, target, beta, log_decay, offset=0):
        """Product-key scores [sequences_local, tokens, heads, 2*half] in; returns the readings
        of this rank's tokens and commits every rank's proposals into the owning shards."""
        n = q_scores.numel() // q_scores.shape[-1]
        plan = self._routes_product_key(q_scores, k_scores, n)
        return self._finish(plan, n, q_scores.shape[:-1], target, beta, log_decay, q_scores.shape[1], offset)

    def epoch_dense(self, queries, write_queries, target, beta, log_decay, offset=0):
        """Dense-key routing: queries / write_queries [sequences_local, tokens, dk] bf16."""
        if self.keys is None:
            raise ValueError("this operator was built without keys")
        n = queries.numel() // queries.shape[-1]
        plan = self._routes_dense(queries, write_queries, n)
        lead = (*queries.shape[:-1], 1)
        return self._finish(plan, n, lead, target, beta, log_decay, queries.shape[1], offset)

    def validate_peers(self, rows):
        """Optional start-of-epoch check (one small all-gather and a host synchronisation, so not
        part of the timed path): every rank must be at the same bank version and bring the same
        number of routing rows and routes per row, or the fixed-size exchanges of the epoch
        would pair a rank's buffers with another epoch's or with truncated candidate lists.
        Raises the reference's error for a stale transaction (gl_sdm/memory/transactions.py:72-73)."""
        mine = torch.tensor([self.version, rows, self.width, self.slots], dtype=torch.int64, device=self.shard.device)
        everyone = torch.empty(self.world * 4, dtype=torch.int64, device=self.shard.device)
        self.dist.all_gather_into_tensor(everyone, mine, group=self.group)
        table = everyone.view(self.world, 4).cpu()
        if (table[:, 0] != table[0, 0]).any():
            raise ValueError(f"stale memory transaction: ranks are at bank versions {table[:, 0].tolist()}")
        if (table[:, 1:] != table[0, 1:]).any():
            raise ValueError("ranks disagree on the epoch's candidate lists (rows, routes per row, slots): "
                             f"{table[:, 1:].tolist()}")

    def last_routes(self):
        """Routes of the last epoch as every rank holds them: (read slots, read weights, write
        slots, write weights), each [ranks * n, K] in global row order (rank, sequence, token,
        head). For checks; identical on every rank by construction."""
        plan, n, K, R = self._last_plan, self._last_n, self.width, self.world
        blocks = plan["routes"][:R * plan["stride"]].view(R, plan["stride"])
        region = n * K

        def take(at, as_float):
            part = blocks[:, at:at + region]
            part = part.view(torch.float32) if as_float else part
            return part.reshape(R * n, K).clone()

        return (take(0, False), take(plan["read_weights_at"], True), take(plan["write_index_at"], False),
                take(plan["write_weights_at"], True))

    def gather_bank(self):
        """The whole bank [1, H, S, D] on every rank (tests and checkpoints)."""
        pieces = [torch.empty_like(self.shard) for _ in range(self.world)]
        self.dist.all_gather(pieces, self.shard, group=self.group)
        return torch.cat(pieces, dim=2)
