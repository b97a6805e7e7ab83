"""Chunk-clock memory operator over one bank shared by every sequence of the batch.

The reference clones the learned bank once per request (gl_sdm/memory/state.py:61-62) and
copies the whole bank at every commit (gl_sdm/memory/transactions.py:96). That is fine at
16,384 slots and impossible at 16,777,216, so the large-bank configurations run one shared
bank, updated in place at the commit clock. The arithmetic per 512-token epoch is the
reference's: query read (layers/global_layer.py:22-27), write proposal (global_layer.py:41-54
with runtime/dense.py:11-14) against the frozen snapshot, then one buffered commit
(layers/stack.py:64-65).
"""
import torch

from . import _native


class SharedBankOperator:
    """values [1, heads, slots, dim] (fp32 or bf16); product-key factor scores in, readings out.

    An epoch holds `sequences x tokens` tokens, rows laid out [sequence, token, head]; every
    row reads `reads` routes and proposes `writes` deltas against the epoch-start bank; the
    commit then applies all deltas in (address, position, layer, arrival) order in place.
    """

    def __init__(self, values, reads, writes, chunk_size=512, num_layers=1, layer_index=0, factored=True):
        if values.ndim != 4 or values.shape[0] != 1:
            raise ValueError("a shared bank is [1, heads, slots, dim]")
        _native.require_cuda(values)
        self.values = values
        self.heads, self.slots, self.dim = values.shape[1:]
        self.half = int(round(self.slots ** 0.5))
        if self.half * self.half != self.slots:
            raise ValueError("product-key routing needs a square number of slots")
        self.reads, self.writes = reads, writes
        self.chunk_size, self.num_layers, self.layer_index = chunk_size, num_layers, layer_index
        self.version = 0
        self.key_bits = max(1, (self.heads * self.slots * chunk_size * num_layers - 1).bit_length())
        self._buffers = None
        # factored: the epoch's commit rebuilds each delta row from the token's error vector and
        # the bank row it updates instead of reading a materialised [entries, dim] delta array
        # (bit-identical result, a third of the HBM traffic on the write side).
        self.factored = factored
        self._packed = None
        self._side = None

    def _proposal_buffers(self, rows):
        k = _native.routes_out(self.writes, self.half)
        need = rows * k
        if self._buffers is None or self._buffers[0].numel() < need:
            dev = self.values.device
            self._buffers = (torch.empty(need, dtype=torch.int64, device=dev),
                             torch.empty((need, self.dim), dtype=torch.float32, device=dev),
                             torch.empty(need, dtype=torch.int64, device=dev))
        a, d, s = self._buffers
        return a[:need], d[:need], s[:need]

    def read(self, q_scores, want_routes=False):
        """q_scores [sequences, tokens, heads, 2*half] fp32 -> readings [.., dim] fp32."""
        rows_per_bank = q_scores.shape[1] * self.heads
        out = _native.pk_select_read(self.values, q_scores, self.reads, rows_per_bank, want_routes=want_routes)
        return out if want_routes else out[0]

    def propose(self, k_scores, target, beta, log_decay, offset=0, mass=None):
        """Write proposal of this epoch's rows against the current (frozen) bank."""
        rows = k_scores.numel() // k_scores.shape[-1]
        return _native.pk_propose(self.values, k_scores, target, beta, log_decay, mass, k_scores.shape[1],
                                  self.writes, offset, self.chunk_size, self.num_layers, self.layer_index,
                                  out=self._proposal_buffers(rows))

    def commit(self, addresses, deltas, keys):
        _native.commit_rows(self.values, addresses, deltas, keys, out=self.values, key_bits=self.key_bits)
        self.version += 1

    def write_operands(self, k_scores, target, beta, log_decay):
        """Write side without delta rows, first half: write routes, prediction read and the
        per-token error vector beta * (target - decay * prediction) with decay - 1
        (reference layers/global_layer.py:41-51). -> (index int32, weights, packed errors)."""
        tokens = k_scores.shape[1]
        prediction, index, weights = _native.pk_select_read(self.values, k_scores, self.writes, tokens * self.heads,
                                                            index_dtype=torch.int32)
        rows = index.numel() // index.shape[-1]
        if self._packed is None or self._packed.numel() != rows * (self.dim + 1):
            self._packed = torch.empty(rows * (self.dim + 1), dtype=torch.float32, device=self.values.device)
        return index, weights, _native.write_error(prediction, target, beta, log_decay, self._packed)

    def commit_operands(self, index, weights, packed, offset=0, phases=_native.COMMIT_ORDER | _native.COMMIT_APPLY):
        """Second half: the factored commit (reference layers/global_layer.py:52-54 and
        memory/transactions.py:90-96 in one pass; every route is an entry, no host sync).
        ``phases`` selects its two steps: ordering the entries (leaves the bank alone) and
        applying them."""
        tokens, width = index.shape[1], index.shape[-1]
        rows = index.numel() // width
        _native.commit_factored(self.values, 0, self.slots, (index, weights), 0, 0, 0, packed, 0, None, None,
                                rows * width, rows, rows, tokens, width, offset, self.chunk_size, self.num_layers,
                                self.layer_index, self.key_bits, phases=phases, owner=("operator", id(self)))
        if phases & _native.COMMIT_APPLY:
            self.version += 1

    def epoch(self, q_scores, k_scores, target, beta, log_decay, offset=0):
        """One full commit epoch: read, propose, commit. Returns the readings."""
        if not self.factored:
            readings = self.read(q_scores)
            self.commit(*self.propose(k_scores, target, beta, log_decay, offset))
            return readings
        # Write side first; ordering its entries (a chain of small sort kernels that only fills
        # the commit's workspace) then runs on a second stream beside the query-side read, and
        # the rows are updated once both are done. Reads and proposal see the same snapshot.
        device = self.values.device
        if self._side is None:
            self._side = torch.cuda.Stream(device)
        main = torch.cuda.current_stream(device)
        operands = self.write_operands(k_scores, target, beta, log_decay)
        ready = torch.cuda.Event()
        ready.record(main)
        with torch.cuda.stream(self._side):
            self._side.wait_event(ready)
            self.commit_operands(*operands, offset, phases=_native.COMMIT_ORDER)
            ordered = torch.cuda.Event()
            ordered.record(self._side)
        readings = self.read(q_scores)
        main.wait_event(ordered)
        self.commit_operands(*operands, offset, phases=_native.COMMIT_APPLY)
        return readings
