"""CPU stand-ins (numpy oracle) for the kernel entry points the sharded operator calls.

Used ONLY by tests/test_sharded_cpu.py to run the exchange logic of ShardedBankOperator on
gloo ranks without a GPU; the product always binds the CUDA library."""
import numpy as np
import torch

from oracle import sdm_oracle as oracle


def routes_out(width, half):
    f = min(width, half)
    return min(width, f * f)


def pk_select_into(scores, width, routes, index_at, weights_at):
    idx, w = oracle.select_routes(scores.numpy(), width)
    n = idx.size
    routes[index_at:index_at + n] = torch.from_numpy(idx.reshape(-1).astype(np.int32))
    routes[weights_at:weights_at + n] = torch.from_numpy(w.reshape(-1)).view(torch.int32)


def score_topk(queries, keys, width, col_base=0, out=None, row_floor=None, floor_in=None, floor_out=(), row_shift=0):
    """Dense-key routing of one shard with row bounds, as glsdm_score_topk_shared defines it: best
    `width` (score, slot) per row, larger slot first on equal scores; candidates below the row's
    bound are dropped (padding: -inf, slot -1); the width-th best score of every full list is
    stored at the given addresses under the row's name (row + row_shift) % rows."""
    import ctypes
    scores = queries.float() @ keys.float().T
    rows, slots = scores.shape
    names = (torch.arange(rows) + row_shift) % rows
    bound = torch.full((rows,), float("-inf")) if row_floor is None else row_floor.clone()
    if floor_in is not None:
        bound = torch.maximum(bound, floor_in[:, names].amax(0))
    order = torch.argsort(scores.flip(1), dim=1, descending=True, stable=True)[:, :width]
    slot = slots - 1 - order
    best = scores.gather(1, slot)
    keep = best >= bound.unsqueeze(1)
    best = torch.where(keep, best, torch.full_like(best, float("-inf")))
    slot = torch.where(keep, slot + col_base, torch.full_like(slot, -1))
    told = keep[:, width - 1]
    for address in floor_out:
        box = np.ctypeslib.as_array((ctypes.c_float * rows).from_address(int(address)))
        box[names[told].numpy()] = best[told, width - 1].numpy()
    if out is None:
        return best, slot.int()
    out[0].copy_(best)
    out[1].copy_(slot.int())
    return out


def topk_merge_packed(packed, parts, rows, width, out):
    """parts x (scores [rows, width] as float32 bits | slots [rows, width]) -> (slots ascending, softmax
    weights): reference tie rule gl_sdm/memory/routing.py:21-26 over the union of the lists."""
    region = rows * width
    blocks = packed.view(parts, 2, region)
    score = blocks[:, 0].view(torch.float32).view(parts, rows, width).permute(1, 0, 2).reshape(rows, parts * width)
    slot = blocks[:, 1].view(parts, rows, width).permute(1, 0, 2).reshape(rows, parts * width).long()
    score = torch.where(slot >= 0, score, torch.full_like(score, float("-inf")))
    by_slot = torch.argsort(slot, dim=1, descending=True, stable=True)          # larger slot first among equals
    score, slot = score.gather(1, by_slot), slot.gather(1, by_slot)
    chosen = torch.argsort(score, dim=1, descending=True, stable=True)[:, :width]
    score, slot = score.gather(1, chosen), slot.gather(1, chosen)
    canonical = torch.argsort(slot, dim=1)
    out[0].copy_(slot.gather(1, canonical).to(out[0].dtype))
    out[1].copy_(score.gather(1, canonical).softmax(-1))
    return out


def _blocked(buf, at, rows, block_rows, stride, width):
    out = []
    for b in range(rows // block_rows):
        lo = at + b * stride
        out.append(buf[lo:lo + block_rows * width].view(block_rows, width))
    return torch.cat(out)


def shard_read(shard, slot_lo, slots, routes, index_at, weights_at, rows, block_rows, block_stride, width):
    idx = _blocked(routes, index_at, rows, block_rows, block_stride, width).numpy().astype(np.int64)
    w = _blocked(routes, weights_at, rows, block_rows, block_stride, width).view(torch.float32).numpy()
    H, local, D = shard.shape[1:]
    owned = (idx >= slot_lo) & (idx < slot_lo + local)
    head = (np.arange(rows) % H)[:, None]
    rows_v = shard.float().numpy()[0][head, np.where(owned, idx - slot_lo, 0)]
    return torch.from_numpy((rows_v * (w * owned)[..., None]).sum(1).astype(np.float32))


def write_error(prediction, target, beta, log_decay, packed):
    rows, dim = prediction.shape
    decay = np.exp(log_decay.numpy().reshape(-1, 1).astype(np.float32))
    err = beta.numpy().reshape(-1, 1) * (target.float().numpy().reshape(rows, dim) - decay * prediction.numpy())
    packed[:rows * dim] = torch.from_numpy(err.astype(np.float32).reshape(-1))
    packed[rows * dim:] = torch.from_numpy((decay - np.float32(1)).reshape(-1))
    return packed


def shard_offsets(routes, index_at, rows, block_rows, block_stride, width, slot_lo, slot_hi):
    idx = _blocked(routes, index_at, rows, block_rows, block_stride, width)
    counts = ((idx >= slot_lo) & (idx < slot_hi)).sum(1)
    return torch.cat([torch.zeros(1, dtype=torch.int64), counts.cumsum(0)]).int()


def shard_propose(shard, slot_lo, slots, routes, index_at, weights_at, route_stride, errors, error_stride, mass,
                  offsets, entries, rows, block_rows, tokens, width, chunk_offset, chunk_size, num_layers,
                  layer_index, out):
    idx = _blocked(routes, index_at, rows, block_rows, route_stride, width).numpy().astype(np.int64)
    w = _blocked(routes, weights_at, rows, block_rows, route_stride, width).view(torch.float32).numpy()
    H, local, D = shard.shape[1:]
    bank = shard.float().numpy()[0]
    addresses, deltas, keys = out
    e = 0
    for row in range(rows):
        b, inner = divmod(row, block_rows)
        block = errors[b * error_stride:(b + 1) * error_stride].numpy()
        err = block[inner * D:(inner + 1) * D]
        gate = block[block_rows * D + inner]
        head, token = row % H, row // H
        for k in range(width):
            s = idx[row, k]
            if slot_lo <= s < slot_lo + local:
                deltas[e] = torch.from_numpy(gate * bank[head, s - slot_lo] + w[row, k] * err)
                addresses[e] = head * local + (s - slot_lo)
                keys[e] = (head * slots + s) * (chunk_size * num_layers) + (chunk_offset + token % tokens) * num_layers + layer_index
                e += 1
    assert e == entries
    return addresses[:entries], deltas[:entries], keys[:entries]


def commit_rows(values, addresses, deltas, keys=None, out=None, key_bits=0, row_base=0):
    new = oracle.commit(values.float().numpy(), addresses.numpy(), deltas.numpy(), None if keys is None else keys.numpy())
    out.copy_(torch.from_numpy(new).to(out.dtype))
    return out


def commit_factored(shard, slot_lo, slots, routes, index_at, weights_at, route_stride, errors, error_stride, mass,
                    offsets, entries, rows, block_rows, tokens, width, chunk_offset, chunk_size, num_layers,
                    layer_index, key_bits=0):
    """The factored commit is defined as proposal expansion followed by the in-place commit.
    Without offsets every route of every rank is shown and the shard lists the ones it owns."""
    D = shard.shape[-1]
    if offsets is None:
        local = shard.shape[2]
        offsets = shard_offsets(routes, index_at, rows, block_rows, route_stride, width, slot_lo, slot_lo + local)
        entries = int(offsets[-1])
        if entries == 0:
            return
    out = (torch.empty(entries, dtype=torch.int64), torch.empty(entries, D), torch.empty(entries, dtype=torch.int64))
    a, d, s = shard_propose(shard, slot_lo, slots, routes, index_at, weights_at, route_stride, errors, error_stride,
                            mass, offsets, entries, rows, block_rows, tokens, width, chunk_offset, chunk_size,
                            num_layers, layer_index, out)
    flat = shard.view(-1, D)
    commit_rows(flat, a, d, s, out=flat, key_bits=key_bits)


# --- stand-ins for the entry points gl_sdm_b200.memory calls (chunk-clock API) ---------------
# Used by tests/test_ref_stack_cpu.py to run the host side of the package shim (views, caches,
# pending proposals, the commit clock, autograd wiring) under the unmodified reference stack
# on a machine without a GPU. They are built from oracle/torch_port.py.

def memory_api_standins():
    from oracle import torch_port as port

    def require_cuda(*tensors):
        return None

    def pk_select_read(values, scores, width, rows_per_bank, want_routes=True, index_dtype=torch.int64,
                       slot_lo=0, slots=None):
        readings, index, weights = port.routed_read(values, scores, width)
        return readings, index.to(index_dtype), weights

    def gather_rows(flat, addresses):
        return flat[addresses]

    def commit_rows(values, addresses, deltas, keys=None, out=None, key_bits=0, row_base=0):
        new = port.commit(values, addresses, deltas, keys)
        if out is None:
            return new
        out.copy_(new)
        return out

    def pk_propose(values, scores, target, beta, log_decay, mass, tokens, width, chunk_offset, chunk_size,
                   num_layers, layer_index, out=None):
        B, T, H, _ = scores.shape
        made = port.propose(values, scores, width, target.float().view(B, T, H, -1), beta.view(B, T, H),
                            log_decay.view(B, T, H), mass, chunk_offset, layer_index, chunk_size, num_layers)
        if out is None:
            return made
        for buffer, tensor in zip(out, made):
            buffer.copy_(tensor.view_as(buffer))
        return out

    def pk_propose_backward(values, scores, target, beta, log_decay, mass, addresses, grad_deltas, tokens, width,
                            logs=()):
        # autograd through the port's expression, on the rows of the version that was read
        B, T, H, _ = scores.shape
        dim = values.shape[-1]
        old = values.detach().clone()
        for undo_addresses, undo_rows in reversed(list(logs)):
            undo_apply(old, undo_addresses, undo_rows)
        bank = old.float().requires_grad_()
        leaves = [scores.detach().clone().requires_grad_(), target.detach().float().view(B, T, H, dim).requires_grad_(),
                  beta.detach().view(B, T, H).clone().requires_grad_(), log_decay.detach().view(B, T, H).clone().requires_grad_()]
        with torch.enable_grad():
            made_addresses, deltas, _ = port.propose(bank, leaves[0], width, leaves[1], leaves[2], leaves[3], mass, 0, 0, 1, 1)
            assert torch.equal(made_addresses, addresses)
            rows = bank.flatten(0, 2)[addresses]              # for the compact bank gradient
            grads = torch.autograd.grad(deltas, [bank] + leaves, grad_deltas.view_as(deltas))
        grad_rows = grads[0].flatten(0, 2)[addresses]
        # one row per route: a bank row written by several routes must not be counted several times
        order = torch.argsort(addresses, stable=True)
        first = torch.ones_like(addresses, dtype=torch.bool)
        first[order[1:]] = addresses[order[1:]] != addresses[order[:-1]]
        grad_rows = grad_rows * first.unsqueeze(-1)
        del rows
        return grads[1], grads[2].reshape(-1, dim), grads[3].reshape(-1), grads[4].reshape(-1), grad_rows

    def commit_undo(values, addresses, deltas, keys=None, key_bits=0):
        # the layout of the CUDA call: sorted addresses, the old row at the head of every run
        order = torch.argsort(addresses if keys is None else keys, stable=True)
        undo_addresses = addresses[order]
        flat = values.view(-1, values.shape[-1])
        undo_rows = torch.zeros(addresses.numel(), values.shape[-1], dtype=values.dtype)
        head = torch.ones_like(undo_addresses, dtype=torch.bool)
        head[1:] = undo_addresses[1:] != undo_addresses[:-1]
        undo_rows[head] = flat[undo_addresses[head]]
        values.copy_(port.commit(values, addresses, deltas, keys))
        return undo_addresses, undo_rows

    def undo_apply(values, undo_addresses, undo_rows):
        head = torch.ones_like(undo_addresses, dtype=torch.bool)
        head[1:] = undo_addresses[1:] != undo_addresses[:-1]
        values.view(-1, values.shape[-1])[undo_addresses[head]] = undo_rows[head]
        return values

    def version_rows(values, addresses, logs):
        """Rows of the version that preceded ``logs`` (oldest commit first)."""
        rows = values.flatten(0, 2)[addresses].float()
        found = torch.zeros(addresses.shape, dtype=torch.bool)
        for undo_addresses, undo_rows in logs:
            pos = torch.searchsorted(undo_addresses, addresses.reshape(-1)).reshape(addresses.shape)
            pos = pos.clamp(max=undo_addresses.numel() - 1)
            hit = (undo_addresses[pos] == addresses) & ~found
            rows[hit] = undo_rows[pos[hit]].float()
            found |= hit
        return rows

    def read_backward(values, grad_out, grad_weights, index, weights, rows_per_bank, half, logs=()):
        lead, width, dim = index.shape[:-1], index.shape[-1], values.shape[-1]
        if index.ndim == 4:
            addresses = port.flat_rows(values, index.long())
        else:
            raise ValueError("stand-in expects [B, T, H, K] routes")
        rows = version_rows(values, addresses, logs)
        grad_w = (rows * grad_out.unsqueeze(-2)).sum(-1)
        if grad_weights is not None:
            grad_w = grad_w + grad_weights
        grad_sum = weights * (grad_w - (grad_w * weights).sum(-1, keepdim=True))   # softmax backward
        grad_scores = torch.zeros(*lead, 2 * half)
        idx = index.long()
        grad_scores.scatter_add_(-1, idx // half, grad_sum)
        grad_scores.scatter_add_(-1, half + idx % half, grad_sum)
        grad_rows = (weights.unsqueeze(-1) * grad_out.unsqueeze(-2)).reshape(-1, dim)
        return grad_scores, addresses.reshape(-1), grad_rows

    return dict(require_cuda=require_cuda, require_device=require_cuda, pk_select_read=pk_select_read, gather_rows=gather_rows,
                commit_rows=commit_rows, read_backward=read_backward, commit_undo=commit_undo, undo_apply=undo_apply,
                pk_propose=pk_propose, pk_propose_backward=pk_propose_backward)
