"""Multi-threaded CPU port (PyTorch tensor ops) of the GL-SDM memory operator.

TEST INFRASTRUCTURE ONLY: the timed CPU baseline of bench.py (cpu_baseline and
`--impl reference`) and a second checker in tests/. The functions follow the device of
their inputs, so bench.py can also time the same library-op sequence on CUDA tensors as a
comparison (never as the product). The reference's own CPU path for this
operator is PyTorch tensor code (projects/gl-sdm/src/gl_sdm/memory/routing.py:10-42,
memory/transactions.py:69-97, runtime/dense.py:11-14), so its faithful CPU timing is the
same sequence of library sorts, gathers and segmented sums run on all host threads. The
reference checkout itself cannot travel to the benchmark machine; this port is pinned
against the reference's outputs in tests/test_oracle_golden.py.
"""
import torch


def _rank_desc_prefer_high(values, keep):
    """Positions of the `keep` largest entries along the last axis, equal values preferring
    the higher position (routing.py:15-17,21-24): rank the reversed axis stably."""
    last = values.shape[-1]
    reversed_rank = torch.sort(values.flip(-1), dim=-1, descending=True, stable=True).indices[..., :keep]
    return last - 1 - reversed_rank


def select_routes(scores, width):
    """routing.py:10-26 -> (address int64 ascending, softmax weights)."""
    lead, half = scores.shape[:-1], scores.shape[-1] // 2
    factors = scores.reshape(*lead, 2, half)
    picked = _rank_desc_prefer_high(factors, width)
    best = torch.gather(factors, -1, picked)
    sums = (best[..., 0, :].unsqueeze(-1) + best[..., 1, :].unsqueeze(-2)).flatten(-2)
    slots = (picked[..., 0, :].unsqueeze(-1) * half + picked[..., 1, :].unsqueeze(-2)).flatten(-2)
    # candidates in descending slot order, then a stable ranking of the sums
    slots, by_slot = torch.sort(slots, dim=-1, descending=True, stable=True)
    sums = torch.gather(sums, -1, by_slot)
    winners = torch.sort(sums, dim=-1, descending=True, stable=True).indices[..., :width]
    slots, sums = torch.gather(slots, -1, winners), torch.gather(sums, -1, winners)
    slots, ascending = torch.sort(slots, dim=-1)
    return slots, torch.softmax(torch.gather(sums, -1, ascending), dim=-1)


def flat_rows(memory, index):
    """routing.py:31-34: (b*H + h)*S + slot; a single shared bank uses partition = head."""
    B, T, H, _ = index.shape
    S = memory.shape[2]
    if memory.shape[0] == 1 and B > 1:
        part = torch.arange(H, device=index.device).view(1, 1, H, 1)
    else:
        part = torch.arange(B * H, device=index.device).view(B, 1, H, 1)
    return part * S + index


def routed_read(memory, scores, width):
    """routing.py:10-28 -> (readings, index, weights)."""
    index, weights = select_routes(scores.float(), width)
    rows = memory.flatten(0, 2)[flat_rows(memory, index)].float()
    return (rows * weights.unsqueeze(-1)).sum(-2), index, weights


def delta_rows(rows, weights, prediction, target, beta, log_decay, mass):
    """runtime/dense.py:11-14."""
    decay = log_decay.exp()
    error = beta * (target.float() - decay * prediction)
    return mass[..., None, None, None] * ((decay.unsqueeze(-1) - 1) * rows + weights.unsqueeze(-1) * error.unsqueeze(-2))


def propose(memory, scores, width, target, beta, log_decay, mass, offset, layer_index, chunk_size, num_layers):
    """layers/global_layer.py:41-54 from the factor scores on -> (addresses, deltas, keys)."""
    B, T, H, _ = scores.shape
    prediction, index, weights = routed_read(memory, scores, width)
    addresses = flat_rows(memory, index)
    rows = memory.flatten(0, 2)[addresses].float()
    mass = torch.ones(B, T, device=scores.device) if mass is None else mass
    delta = delta_rows(rows, weights, prediction, target, beta.unsqueeze(-1), log_decay.unsqueeze(-1), mass)
    position = torch.arange(offset, offset + T, device=scores.device).view(1, T, 1, 1)
    keys = addresses * (chunk_size * num_layers) + position * num_layers + layer_index
    return addresses.flatten(), delta.flatten(0, 3), keys.flatten()


def commit(memory, addresses, deltas, keys=None, in_place=False):
    """memory/transactions.py:80,90-96: new bank = old + per-address ordered sums.

    in_place=True skips the reference's whole-bank copy (index_copy_ on the input), which is
    how the large shared banks are committed; it only makes this CPU baseline faster.
    """
    flat = memory.reshape(-1, memory.shape[-1])
    if addresses.numel() == 0:
        return memory if in_place else memory.clone()
    order = torch.sort(addresses if keys is None else keys, stable=True).indices
    rows, runs = torch.unique_consecutive(addresses[order], return_counts=True)
    totals = torch.segment_reduce(deltas.float()[order], "sum", lengths=runs)
    updated = (flat[rows].float() + totals).to(flat.dtype)
    if in_place:
        flat.index_copy_(0, rows, updated)
        return memory
    return flat.index_copy(0, rows, updated).view_as(memory)


def flat_routes(queries, keys, width, chunk=262144):
    """Flat-key mode (no counterpart in the reference): q @ keys^T, then the slot-sum
    selection rule (routing.py:21-26). -> (slot ascending, softmax weights).

    Keys are visited in chunks so the [tokens, slots] score matrix is never held whole: per
    chunk a library top-k keeps `width` candidates, and the surviving candidates are ranked
    with the exact rule (score descending, larger slot first). Equal scores inside one chunk
    are cut by torch.topk's own order, which only matters for bit-equal scores.
    """
    q = queries.float()
    cand_score, cand_slot = [], []
    for lo in range(0, keys.shape[0], chunk):
        block = keys[lo:lo + chunk].float()
        scores = q @ block.T
        top = torch.topk(scores, min(width, block.shape[0]), dim=-1)
        cand_score.append(top.values)
        cand_slot.append(top.indices + lo)
    score, slot = torch.cat(cand_score, -1), torch.cat(cand_slot, -1)
    slot, by_slot = torch.sort(slot, dim=-1, descending=True, stable=True)
    score = torch.gather(score, -1, by_slot)
    winners = torch.sort(score, dim=-1, descending=True, stable=True).indices[..., :width]
    slot, score = torch.gather(slot, -1, winners), torch.gather(score, -1, winners)
    slot, ascending = torch.sort(slot, dim=-1)
    return slot, torch.softmax(torch.gather(score, -1, ascending), dim=-1)


def dense_epoch(memory, keys, queries, write_queries, width, target, beta, log_decay, chunk_size, in_place=True):
    """One commit epoch with flat-key routing on a single-head shared bank [1,1,S,D]:
    read, write proposal (global_layer.py:44-54 with dense.py:11-14) and commit.
    queries [B,T,dk]. Returns (readings [B,T,1,D], memory)."""
    B, T, dk = queries.shape
    flat = memory.flatten(0, 2)
    index, weights = flat_routes(queries.reshape(-1, dk), keys, width)
    readings = (flat[index].float() * weights.unsqueeze(-1)).sum(-2).view(B, T, 1, -1)
    windex, wweights = flat_routes(write_queries.reshape(-1, dk), keys, width)
    rows = flat[windex].float()
    prediction = (rows * wweights.unsqueeze(-1)).sum(-2)
    delta = delta_rows(rows.view(B, T, 1, width, -1), wweights.view(B, T, 1, width), prediction.view(B, T, 1, -1),
                       target.view(B, T, 1, -1), beta.view(B, T, 1, 1), log_decay.view(B, T, 1, 1),
                       torch.ones(B, T, device=queries.device))
    address = windex.view(B, T, 1, width)
    position = torch.arange(T, device=queries.device).view(1, T, 1, 1)
    key = address * chunk_size + position
    memory = commit(memory, address.flatten(), delta.flatten(0, 3), key.flatten(), in_place=in_place)
    return readings, memory
