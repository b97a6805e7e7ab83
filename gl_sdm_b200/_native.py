"""ctypes binding of the C-ABI library (include/glsdm.h) and tensor-level wrappers.

There is exactly one implementation behind these functions: the sm_100a kernels in
``libglsdm_b200.so``. If the library has not been built, or a tensor is not a contiguous
CUDA tensor, the call raises; nothing here computes on the CPU.

The wrappers mirror the three native functions the reference's "urm" backend calls
(gl_sdm/memory/backends/urm.py:49-82,109-122 and gl_sdm/memory/backends/commit.py:57-58).
"""
import ctypes
import os
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIBRARY_PATH = os.path.join(_HERE, "libglsdm_b200.so")

F32, BF16 = 0, 1
DEV_ADDRESS_OUT_OF_RANGE = 1
DEV_WAIT_EXPIRED = 2
DEV_LOG_NOT_ASCENDING = 4
MAX_WIDTH = 32

_lock = threading.Lock()
_lib = None


class Bank(ctypes.Structure):
    """glsdm_bank of include/glsdm.h."""
    _fields_ = [("values", ctypes.c_void_p), ("dtype", ctypes.c_int), ("banks", ctypes.c_int64),
                ("heads", ctypes.c_int32), ("slots", ctypes.c_int64), ("dim", ctypes.c_int32),
                ("slot_lo", ctypes.c_int64), ("slot_hi", ctypes.c_int64)]


_p, _i, _i32, _i64, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_int32, ctypes.c_int64, ctypes.c_size_t
_BANK = ctypes.POINTER(Bank)
SIGNATURES = {
    "glsdm_abi_version": (ctypes.c_int, []),
    "glsdm_status_string": (ctypes.c_char_p, [_i]),
    "glsdm_last_cuda_error": (ctypes.c_char_p, []),
    "glsdm_kernel_launches": (ctypes.c_uint64, []),
    "glsdm_pk_select": (_i, [_p, _i64, _i32, _i32, _p, _i, _p, _p]),
    "glsdm_snapshot_read": (_i, [_BANK, _p, _i, _p, _p, _i64, _i64, _i32, _p, _p, _p]),
    "glsdm_pk_select_read": (_i, [_BANK, _p, _i64, _i64, _i32, _i32, _p, _p, _i, _p, _p, _p]),
    "glsdm_pk_propose": (_i, [_BANK, _p, _p, _i, _p, _p, _p, _i64, _i64, _i64, _i32, _i32, _i64,
                              _i64, _i32, _i32, _p, _p, _p, _p, _p]),
    "glsdm_read_backward": (_i, [_BANK, _p, _p, _p, _i, _p, _i64, _i64, _i32, _i32, _p, _p, _p, _p]),
    "glsdm_pk_propose_backward": (_i, [_BANK, _p, _p, _i, _p, _p, _p, _p, _p, _i64, _i64, _i32, _i32, _i32, _p, _p, _p,
                                       _p, _p, _p, _p, _p, _p]),
    "glsdm_read_backward_version": (_i, [_BANK, _p, _p, _p, _i, _p, _i64, _i64, _i32, _i32, _i32, _p, _p, _p,
                                         _p, _p, _p, _p]),
    "glsdm_gather_rows": (_i, [_p, _i, _i64, _i32, _p, _i64, _p, _p, _p]),
    "glsdm_token_propose": (_i, [_BANK, _p, _p, _i, _p, _p, _p, _p, _p, _i64, _i32, _p, _p, _p, _p]),
    "glsdm_write_error": (_i, [_p, _p, _i, _p, _p, _i64, _i32, _p, _p, _p]),
    "glsdm_shard_read": (_i, [_BANK, _p, _p, _i64, _i64, _i64, _i32, _p, _p, _p]),
    "glsdm_shard_offsets": (_i, [_p, _i64, _i64, _i64, _i32, _i64, _i64, _p, _p]),
    "glsdm_shard_propose": (_i, [_BANK, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i32, _i64, _i64,
                                 _i32, _i32, _p, _p, _p, _p]),
    "glsdm_commit_workspace_bytes": (_sz, [_i64, _i32]),
    "glsdm_commit": (_i, [_p, _p, _i, _i64, _i64, _i32, _p, _p, _p, _i64, _i32, _p, _sz, _p, _p]),
    "glsdm_commit_undo": (_i, [_p, _i, _i64, _i64, _i32, _p, _p, _p, _i64, _i32, _p, _sz, _p, _p, _p, _p]),
    "glsdm_undo_apply": (_i, [_p, _i, _i64, _i64, _i32, _p, _p, _i64, _p]),
    "glsdm_overlay_read": (_i, [_BANK, _p, _i, _p, _i64, _i64, _i32, _i32, _p, _p, _p, _p, _p, _p]),
    "glsdm_commit_factored_workspace_bytes": (_sz, [_i64, _i32]),
    "glsdm_commit_factored": (_i, [_BANK, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _i64, _i64,
                                   _i32, _i32, _i32, _p, _sz, _p, _p]),
    "glsdm_commit_factored_phased": (_i, [_BANK, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _i64,
                                          _i64, _i32, _i32, _i32, _i32, _p, _sz, _p, _p]),
    "glsdm_commit_static": (_i, [_p, _p, _i, _i64, _i64, _i32, _p, _p, _p, _i64, _i32, _p, _p]),
    "glsdm_commit_static_max_entries": (_i64, []),
    "glsdm_wait_probe": (_i, [_p, _i64, _p, _p, _p]),
    "glsdm_score_topk_workspace_bytes": (_sz, [_i64, _i64, _i32, _i32]),
    "glsdm_score_topk": (_i, [_p, _p, _i64, _i64, _i32, _i32, _i64, _p, _p, _p, _sz, _p, _p]),
    "glsdm_score_topk_variant": (_i, [_i]),
    "glsdm_commit_factored_mode": (_i, [_i]),
    "glsdm_score_topk_plan": (_i, [_i64, _i64, _i32, _i32, _i32, _p]),
    "glsdm_score_topk_pitched": (_i, [_p, _i64, _p, _i64, _i64, _i64, _i32, _i32, _i64, _p, _p, _p, _sz, _p, _p]),
    "glsdm_score_topk_bounded": (_i, [_p, _i64, _p, _i64, _i64, _i64, _i32, _i32, _i64, _p, _p, _p, _p, _sz, _p, _p]),
    "glsdm_score_topk_shared": (_i, [_p, _i64, _p, _i64, _i64, _i64, _i32, _i32, _i64, _p, _i64, _p, _i32, _p, _i32, _p, _p,
                                     _p, _sz, _p, _p]),
    "glsdm_pk_combine": (_i, [_p, _p, _p, _p, _i64, _i32, _i32, _p, _i, _p, _p]),
    "glsdm_topk_merge": (_i, [_p, _p, _i32, _i64, _i32, _p, _i, _p, _p]),
    "glsdm_topk_merge_strided": (_i, [_p, _p, _i32, _i64, _i64, _i32, _p, _i, _p, _p]),
}


def library():
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIBRARY_PATH):
                    raise RuntimeError(
                        f"{LIBRARY_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; "
                        "g.build()'` (nvcc, sm_100a). There is no CPU or PyTorch fallback for the GL-SDM memory operator.")
                lib = ctypes.CDLL(LIBRARY_PATH)
                for name, (restype, argtypes) in SIGNATURES.items():
                    fn = getattr(lib, name)
                    fn.restype, fn.argtypes = restype, argtypes
                _lib = lib
    return _lib


def _check(status):
    if status == 0:
        return
    lib = library()
    text = lib.glsdm_status_string(status).decode()
    if status == 4:
        text += ": " + lib.glsdm_last_cuda_error().decode()
        raise RuntimeError(f"glsdm: {text}")
    raise ValueError(f"glsdm: {text}")


def require_cuda(*tensors):
    """Reference gl_sdm/memory/backends/primitives.py:7-11: no silent CPU path."""
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda or not t.is_contiguous():
            raise ValueError("GL-SDM native kernels require contiguous CUDA tensors")


def require_device(*tensors):
    """Operands that the wrappers make contiguous themselves still have to live on a GPU."""
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("GL-SDM native kernels require contiguous CUDA tensors")


def _stream(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _ptr(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _dtype_code(t):
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise ValueError("GL-SDM banks are float32 or bfloat16")


def bank_of(values, slot_lo=0, slot_hi=None, slots=None):
    """Describe values [banks, heads, local_slots, dim]; a shard passes its global range."""
    if values.ndim != 4:
        raise ValueError("bank values must be [banks, heads, slots, dim]")
    require_cuda(values)
    banks, heads, local, dim = values.shape
    slots = local if slots is None else slots
    slot_hi = slot_lo + local if slot_hi is None else slot_hi
    if slot_hi - slot_lo != local:
        raise ValueError("shard range does not match the values tensor")
    return Bank(values.data_ptr(), _dtype_code(values), banks, heads, slots, dim, slot_lo, slot_hi)


def routes_out(width, half):
    factor = min(width, half)
    return min(width, factor * factor)


_status_words = {}


def status_word(device):
    """A zeroed per-device uint32 the kernels OR error bits into."""
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    word = _status_words.get(key)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device=f"cuda:{key}")
        _status_words[key] = word
    return word


def raise_on_device_status(device):
    """Synchronising check of the device status word (tests and debug paths)."""
    word = status_word(device)
    bits = int(word.item())
    if bits:
        word.zero_()
        names = [n for b, n in ((DEV_ADDRESS_OUT_OF_RANGE, "address out of range"),
                                (DEV_WAIT_EXPIRED, "bounded wait expired"),
                                (DEV_LOG_NOT_ASCENDING, "undo log addresses not ascending")) if bits & b]
        raise RuntimeError("glsdm device status: " + ", ".join(names))


def wait_probe(words, position):
    """Run the commit kernels' bounded look-back over `words` (int64 chain words) up to
    `position`; returns the count it reached (a one-element int32 tensor). A word that is never
    published makes the wait run out: the status word then carries DEV_WAIT_EXPIRED."""
    require_cuda(words)
    if words.dtype != torch.int64:
        raise ValueError("chain words are int64")
    out = torch.zeros(1, dtype=torch.int32, device=words.device)
    _check(library().glsdm_wait_probe(_ptr(words), position, _ptr(status_word(words.device)), _ptr(out),
                                      _stream(words.device)))
    return out


def pk_select_into(scores, width, routes, index_at, weights_at):
    """Routes of `scores` written into an int32 buffer: indices at element index_at, weight
    bits at element weights_at (the send buffer of the shard all-gather)."""
    require_cuda(scores, routes)
    half = scores.shape[-1] // 2
    rows = scores.numel() // (2 * half)
    _check(library().glsdm_pk_select(_ptr(scores), rows, half, width, _at(routes, index_at), 0,
                                     _at(routes, weights_at), _stream(scores.device)))


def pk_select(scores, width, index_dtype=torch.int64):
    """scores [..., 2*half] fp32 -> (index [..., k], weights [..., k])."""
    require_cuda(scores)
    if scores.dtype != torch.float32:
        raise ValueError("factor scores must be float32")
    half = scores.shape[-1] // 2
    if half * 2 != scores.shape[-1] or half < 1:
        raise ValueError("scores must hold two factors of equal width")
    k = routes_out(width, half)
    rows = scores.numel() // (2 * half)
    index = torch.empty((*scores.shape[:-1], k), dtype=index_dtype, device=scores.device)
    weights = torch.empty((*scores.shape[:-1], k), dtype=torch.float32, device=scores.device)
    _check(library().glsdm_pk_select(_ptr(scores), rows, half, width, _ptr(index),
                                     int(index_dtype == torch.int64), _ptr(weights), _stream(scores.device)))
    return index, weights


def snapshot_read(values, index, weights, rows_per_bank, requests=None, slot_lo=0, slots=None):
    """Weighted sum of supplied routes; index/weights [..., k] with rows laid out [bank, token, head]."""
    require_cuda(values, index, weights, requests)
    if index.dtype not in (torch.int64, torch.int32) or weights.dtype != torch.float32:
        raise ValueError("routes are int32/int64 indices with float32 weights")
    if requests is not None and requests.dtype != torch.int64:
        raise ValueError("requests must be int64")
    bank = bank_of(values, slot_lo, None, slots)
    width = index.shape[-1]
    rows = index.numel() // width
    out = torch.empty((*index.shape[:-1], values.shape[-1]), dtype=torch.float32, device=values.device)
    _check(library().glsdm_snapshot_read(ctypes.byref(bank), _ptr(index), int(index.dtype == torch.int64),
                                         _ptr(weights), _ptr(requests), rows, rows_per_bank, width,
                                         _ptr(out), _ptr(status_word(values.device)), _stream(values.device)))
    return out


def pk_select_read(values, scores, width, rows_per_bank, want_routes=True, index_dtype=torch.int64,
                   slot_lo=0, slots=None):
    """Fused route + read. scores [..., 2*half] fp32 -> readings [..., dim] (+ routes)."""
    require_cuda(values, scores)
    if scores.dtype != torch.float32:
        raise ValueError("factor scores must be float32")
    half = scores.shape[-1] // 2
    bank = bank_of(values, slot_lo, None, slots)
    k = routes_out(width, half)
    rows = scores.numel() // (2 * half)
    lead = scores.shape[:-1]
    out = torch.empty((*lead, values.shape[-1]), dtype=torch.float32, device=values.device)
    index = weights = None
    if want_routes:
        index = torch.empty((*lead, k), dtype=index_dtype, device=values.device)
        weights = torch.empty((*lead, k), dtype=torch.float32, device=values.device)
    _check(library().glsdm_pk_select_read(ctypes.byref(bank), _ptr(scores), rows, rows_per_bank, half, width,
                                          _ptr(out), _ptr(index), int(index_dtype == torch.int64),
                                          _ptr(weights), _ptr(status_word(values.device)),
                                          _stream(values.device)))
    return out, index, weights


def pk_propose(values, scores, target, beta, log_decay, mass, tokens, width, chunk_offset, chunk_size,
               num_layers, layer_index, out=None):
    """Fused write proposal for rows laid out [bank, token, head].

    Returns (addresses [rows*k] int64, deltas [rows*k, dim] fp32, keys [rows*k] int64); ``out`` may
    supply preallocated views of an epoch-wide buffer.
    """
    require_cuda(values, scores, target, beta, log_decay, mass)
    half = scores.shape[-1] // 2
    bank = bank_of(values)
    k = routes_out(width, half)
    rows = scores.numel() // (2 * half)
    dim = values.shape[-1]
    if target.dtype not in (torch.float32, torch.bfloat16) or target.numel() != rows * dim:
        raise ValueError("target must be [rows, dim] float32 or bfloat16")
    if beta.dtype != torch.float32 or log_decay.dtype != torch.float32 or beta.numel() != rows or log_decay.numel() != rows:
        raise ValueError("beta and log_decay must be float32 with one value per row")
    heads = values.shape[1]
    if mass is not None and (mass.dtype != torch.float32 or mass.numel() != rows // heads):
        raise ValueError("mass must be float32 with one value per token")
    if out is None:
        addresses = torch.empty(rows * k, dtype=torch.int64, device=values.device)
        deltas = torch.empty((rows * k, dim), dtype=torch.float32, device=values.device)
        keys = torch.empty(rows * k, dtype=torch.int64, device=values.device)
    else:
        addresses, deltas, keys = out
        require_cuda(addresses, deltas, keys)
        if addresses.numel() != rows * k or deltas.numel() != rows * k * dim or keys.numel() != rows * k:
            raise ValueError("preallocated proposal buffers have the wrong size")
    rows_per_bank = tokens * heads
    _check(library().glsdm_pk_propose(ctypes.byref(bank), _ptr(scores), _ptr(target), _dtype_code(target),
                                      _ptr(beta), _ptr(log_decay), _ptr(mass), rows, rows_per_bank, tokens,
                                      half, width, chunk_offset, chunk_size, num_layers, layer_index,
                                      _ptr(addresses), _ptr(deltas), _ptr(keys),
                                      _ptr(status_word(values.device)), _stream(values.device)))
    return addresses, deltas, keys


def pk_propose_backward(values, scores, target, beta, log_decay, mass, addresses, grad_deltas, tokens, width, logs=()):
    """Backward of ``pk_propose``: (grad_scores [..., 2*half], grad_target [rows, dim] fp32, grad_beta
    [rows], grad_log_decay [rows], grad_rows [rows*k, dim]); the compact bank gradient belongs to
    ``addresses``. ``logs`` as for ``read_backward``."""
    require_cuda(values, scores, target, beta, log_decay, mass, addresses, grad_deltas)
    half = scores.shape[-1] // 2
    bank = bank_of(values)
    k = routes_out(width, half)
    rows = scores.numel() // (2 * half)
    dim = values.shape[-1]
    if addresses.dtype != torch.int64 or addresses.numel() != rows * k:
        raise ValueError("addresses must be the int64 routes the forward returned")
    if grad_deltas.dtype != torch.float32 or grad_deltas.numel() != rows * k * dim:
        raise ValueError("grad_deltas must be float32 [rows*k, dim]")
    n, log_addresses, log_rows, log_entries = _log_arrays(values, logs)
    dev = values.device
    grad_scores = torch.empty(scores.shape, dtype=torch.float32, device=dev)
    grad_target = torch.empty((rows, dim), dtype=torch.float32, device=dev)
    grad_beta = torch.empty(rows, dtype=torch.float32, device=dev)
    grad_log_decay = torch.empty(rows, dtype=torch.float32, device=dev)
    grad_rows = torch.empty((rows * k, dim), dtype=torch.float32, device=dev)
    _check(library().glsdm_pk_propose_backward(
        ctypes.byref(bank), _ptr(scores), _ptr(target), _dtype_code(target), _ptr(beta), _ptr(log_decay), _ptr(mass),
        _ptr(addresses), _ptr(grad_deltas), rows, tokens * values.shape[1], half, width, n, log_addresses, log_rows,
        log_entries, _ptr(grad_scores), _ptr(grad_target), _ptr(grad_beta), _ptr(grad_log_decay), _ptr(grad_rows),
        _stream(dev)))
    return grad_scores, grad_target, grad_beta, grad_log_decay, grad_rows


def gather_rows(flat, addresses):
    """flat [rows, dim], addresses [...] int64 -> [..., dim] in the bank dtype."""
    require_cuda(flat, addresses)
    if addresses.dtype != torch.int64:
        raise ValueError("addresses must be int64")
    rows, dim = flat.shape
    out = torch.empty((*addresses.shape, dim), dtype=flat.dtype, device=flat.device)
    _check(library().glsdm_gather_rows(_ptr(flat), _dtype_code(flat), rows, dim, _ptr(addresses),
                                       addresses.numel(), _ptr(out), _ptr(status_word(flat.device)),
                                       _stream(flat.device)))
    return out


def token_propose(values, requests, index, weights, target, beta, log_decay, mass):
    """Token-clock proposal: routes [A, H, K] -> (addresses [A*H*K] int64, deltas [A*H*K, dim])."""
    require_cuda(values, requests, index, weights, target, beta, log_decay, mass)
    bank = bank_of(values)
    width = index.shape[-1]
    rows = index.numel() // width
    dim = values.shape[-1]
    if target.numel() != rows * dim or beta.numel() != rows or log_decay.numel() != rows:
        raise ValueError("targets, beta and log_decay must have one entry per (request, head)")
    if requests.numel() * values.shape[1] != rows or mass.numel() != requests.numel():
        raise ValueError("requests and mass must have one entry per active request")
    addresses = torch.empty(rows * width, dtype=torch.int64, device=values.device)
    deltas = torch.empty((rows * width, dim), dtype=torch.float32, device=values.device)
    _check(library().glsdm_token_propose(ctypes.byref(bank), _ptr(requests), _ptr(index),
                                         int(index.dtype == torch.int64), _ptr(weights), _ptr(target),
                                         _ptr(beta), _ptr(log_decay), _ptr(mass), rows, width,
                                         _ptr(addresses), _ptr(deltas), _ptr(status_word(values.device)),
                                         _stream(values.device)))
    return addresses, deltas


def write_error(prediction, target, beta, log_decay, packed=None):
    """Token-owner half of the proposal. Returns `packed`, a float32 buffer of rows*(dim+1)
    elements: the error rows [rows, dim] followed by (decay - 1) [rows]."""
    require_cuda(prediction, target, beta, log_decay, packed)
    dim = prediction.shape[-1]
    rows = prediction.numel() // dim
    if packed is None:
        packed = torch.empty(rows * (dim + 1), dtype=torch.float32, device=prediction.device)
    elif packed.numel() != rows * (dim + 1) or packed.dtype != torch.float32:
        raise ValueError("packed error buffer must hold rows*(dim+1) float32 values")
    _check(library().glsdm_write_error(_ptr(prediction), _ptr(target), _dtype_code(target), _ptr(beta),
                                       _ptr(log_decay), rows, dim, _at(packed, 0), _at(packed, rows * dim),
                                       _stream(prediction.device)))
    return packed


def _at(tensor, offset):
    """Device address of element `offset` of a 4-byte-element tensor."""
    return ctypes.c_void_p(tensor.data_ptr() + 4 * offset)


def shard_read(shard, slot_lo, slots, routes, index_at, weights_at, rows, block_rows, block_stride, width):
    """Partial readings [rows, dim] of this rank's shard for all-gathered routes.

    `routes` is the int32 all-gather buffer; block b's indices start at element
    index_at + b*block_stride and its weights (float32 bits) at weights_at + b*block_stride.
    """
    require_cuda(shard, routes)
    bank = bank_of(shard, slot_lo, None, slots)
    out = torch.empty((rows, shard.shape[-1]), dtype=torch.float32, device=shard.device)
    _check(library().glsdm_shard_read(ctypes.byref(bank), _at(routes, index_at), _at(routes, weights_at), rows,
                                      block_rows, block_stride, width, _ptr(out),
                                      _ptr(status_word(shard.device)), _stream(shard.device)))
    return out


def shard_offsets(routes, index_at, rows, block_rows, block_stride, width, slot_lo, slot_hi):
    """Exclusive prefix of owned routes per row; element `rows` is the shard's entry count."""
    require_cuda(routes)
    offsets = torch.empty(rows + 1, dtype=torch.int32, device=routes.device)
    _check(library().glsdm_shard_offsets(_at(routes, index_at), rows, block_rows, block_stride, width, slot_lo,
                                         slot_hi, _ptr(offsets), _stream(routes.device)))
    return offsets


def shard_propose(shard, slot_lo, slots, routes, index_at, weights_at, route_stride, errors, error_stride, mass,
                  offsets, entries, rows, block_rows, tokens, width, chunk_offset, chunk_size, num_layers,
                  layer_index, out):
    """Slot-owner half of the proposal; fills the first `entries` rows of the `out` buffers.

    `errors` is the float32 all-gather buffer of write errors: per block, block_rows error rows
    [block_rows, dim] followed by block_rows (decay - 1) values, error_stride elements per block.
    """
    require_cuda(shard, routes, errors, mass, offsets)
    bank = bank_of(shard, slot_lo, None, slots)
    dim = shard.shape[-1]
    addresses, deltas, keys = out
    if addresses.numel() < entries or deltas.numel() < entries * dim or keys.numel() < entries:
        raise ValueError("proposal buffers are smaller than the shard's entry count")
    _check(library().glsdm_shard_propose(ctypes.byref(bank), _at(routes, index_at), _at(routes, weights_at),
                                         _at(errors, 0), _at(errors, block_rows * dim), _ptr(mass), _ptr(offsets),
                                         rows, block_rows, route_stride, error_stride, tokens, width, chunk_offset,
                                         chunk_size, num_layers, layer_index, _ptr(addresses), _ptr(deltas),
                                         _ptr(keys), _stream(shard.device)))
    return addresses[:entries], deltas[:entries], keys[:entries]


COMMIT_ORDER, COMMIT_APPLY = 1, 2


def commit_factored(shard, slot_lo, slots, routes, index_at, weights_at, route_stride, errors, error_stride, mass,
                    offsets, entries, rows, block_rows, tokens, width, chunk_offset, chunk_size, num_layers,
                    layer_index, key_bits=0, phases=COMMIT_ORDER | COMMIT_APPLY, owner=None):
    """Commit the proposal of these write routes into ``shard`` in place without ever writing
    its delta rows: the reducer rebuilds them from ``errors`` (the write_error buffer, laid out
    as for shard_propose) and the bank rows it updates. ``offsets=None`` (unsharded bank):
    every route is an entry and ``entries`` must be rows * width. ``routes`` is the int32
    all-gather buffer addressed by index_at / weights_at, or a pair (index int32, weights).
    ``phases`` = COMMIT_ORDER (entries + sort into the workspace; leaves the bank alone, so it may
    run beside kernels that still read the bank), COMMIT_APPLY (sums + row updates), or both."""
    if isinstance(routes, tuple):
        index, weights = routes
        require_cuda(index, weights)
        if index.dtype != torch.int32 or weights.dtype != torch.float32:
            raise ValueError("write routes are int32 indices with float32 weights")
        index_ptr, weights_ptr = _ptr(index), _ptr(weights)
    else:
        require_cuda(routes)
        index_ptr, weights_ptr = _at(routes, index_at), _at(routes, weights_at)
    require_cuda(shard, errors, mass, offsets)
    bank = bank_of(shard, slot_lo, None, slots)
    dim = shard.shape[-1]
    lib = library()
    work = _workspace(shard.device, lib.glsdm_commit_factored_workspace_bytes(entries, dim), owner)
    _check(lib.glsdm_commit_factored_phased(ctypes.byref(bank), index_ptr, weights_ptr,
                                            _at(errors, 0), _ptr(mass), _ptr(offsets), entries, rows, block_rows,
                                            route_stride, error_stride, tokens, width, chunk_offset, chunk_size,
                                            num_layers, layer_index, key_bits, phases, _ptr(work), work.numel(),
                                            _ptr(status_word(shard.device)), _stream(shard.device)))


_workspaces = threading.local()


def _workspace(device, nbytes, owner=None):
    """Scratch for the commit's sort, one buffer per (host thread, device, stream): two threads
    that enqueue commits on the same stream must not share it (their launches interleave), and
    neither may two streams of one thread (their kernels overlap). A caller that runs the two
    phases of one commit on different streams, ordered by events, names the buffer by ``owner``."""
    table = getattr(_workspaces, "table", None)
    if table is None:
        table = _workspaces.table = {}
    key = (torch.device(device).index, owner if owner is not None else torch.cuda.current_stream(device).cuda_stream)
    buf = table.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        table[key] = buf
    return buf


def commit_rows(values, addresses, deltas, keys=None, out=None, key_bits=0, row_base=0):
    """Apply buffered deltas to a flat bank [rows, dim]; ``out is values`` updates in place.

    Returns the updated bank (a new tensor unless ``out`` is given).
    """
    require_cuda(values, addresses, deltas, keys, out)
    dim = values.shape[-1]
    flat = values.view(-1, dim)
    if addresses.dtype != torch.int64 or (keys is not None and keys.dtype != torch.int64):
        raise ValueError("addresses and sort keys must be int64")
    if deltas.dtype != torch.float32:
        raise ValueError("deltas must be float32")
    entries = addresses.numel()
    if deltas.numel() != entries * dim or (keys is not None and keys.numel() != entries):
        raise ValueError("addresses, deltas and keys disagree on the number of entries")
    if out is None:
        out = torch.empty_like(values)
    elif out.shape != values.shape or out.dtype != values.dtype:
        raise ValueError("output bank must match the input bank")
    lib = library()
    nbytes = lib.glsdm_commit_workspace_bytes(entries, dim)
    work = _workspace(values.device, nbytes)
    _check(lib.glsdm_commit(_ptr(flat), _ptr(out), _dtype_code(values), row_base, flat.shape[0], dim,
                            _ptr(addresses), _ptr(deltas), _ptr(keys), entries, key_bits, _ptr(work),
                            work.numel(), _ptr(status_word(values.device)), _stream(values.device)))
    return out


MAX_UNDO_LOGS = 8


def commit_undo(values, addresses, deltas, keys=None, key_bits=0):
    """In-place commit that also records the touched rows' previous contents.

    Returns (undo_addresses [entries] int64 sorted, undo_rows [entries, dim] in the bank dtype;
    the first position of each run of equal addresses holds that address's old row)."""
    require_cuda(values, addresses, deltas, keys)
    dim = values.shape[-1]
    flat = values.view(-1, dim)
    if addresses.dtype != torch.int64 or (keys is not None and keys.dtype != torch.int64):
        raise ValueError("addresses and sort keys must be int64")
    if deltas.dtype != torch.float32:
        raise ValueError("deltas must be float32")
    entries = addresses.numel()
    if deltas.numel() != entries * dim or (keys is not None and keys.numel() != entries):
        raise ValueError("addresses, deltas and keys disagree on the number of entries")
    undo_addresses = torch.empty(entries, dtype=torch.int64, device=values.device)
    undo_rows = torch.empty((entries, dim), dtype=values.dtype, device=values.device)
    lib = library()
    work = _workspace(values.device, lib.glsdm_commit_workspace_bytes(entries, dim))
    _check(lib.glsdm_commit_undo(_ptr(flat), _dtype_code(values), 0, flat.shape[0], dim, _ptr(addresses),
                                 _ptr(deltas), _ptr(keys), entries, key_bits, _ptr(work), work.numel(),
                                 _ptr(undo_addresses), _ptr(undo_rows), _ptr(status_word(values.device)),
                                 _stream(values.device)))
    return undo_addresses, undo_rows


def undo_apply(values, undo_addresses, undo_rows):
    """Write the logged old rows back into ``values`` (in place)."""
    require_cuda(values, undo_addresses, undo_rows)
    dim = values.shape[-1]
    flat = values.view(-1, dim)
    if undo_rows.dtype != values.dtype or undo_rows.shape[-1] != dim:
        raise ValueError("the undo log does not match the bank")
    _check(library().glsdm_undo_apply(_ptr(flat), _dtype_code(values), 0, flat.shape[0], dim, _ptr(undo_addresses),
                                      _ptr(undo_rows), undo_addresses.numel(), _stream(values.device)))
    return values


def overlay_read(values, index, weights, rows_per_bank, logs):
    """snapshot_read of an older version: ``logs`` = [(undo_addresses, undo_rows), ...] of the
    commits applied to ``values`` since that version, oldest commit first."""
    require_cuda(values, index, weights)
    if index.dtype not in (torch.int64, torch.int32) or weights.dtype != torch.float32:
        raise ValueError("routes are int32/int64 indices with float32 weights")
    n, addresses, log_rows, entries = _log_arrays(values, logs)
    bank = bank_of(values)
    width = index.shape[-1]
    rows = index.numel() // width
    out = torch.empty((*index.shape[:-1], values.shape[-1]), dtype=torch.float32, device=values.device)
    _check(library().glsdm_overlay_read(ctypes.byref(bank), _ptr(index), int(index.dtype == torch.int64),
                                        _ptr(weights), rows, rows_per_bank, width, n, addresses, log_rows, entries,
                                        _ptr(out), _ptr(status_word(values.device)), _stream(values.device)))
    return out


def topk_merge(cand_score, cand_slot, index_dtype=torch.int64, out=None):
    """cand_* [parts, rows..., k] -> (index [rows..., k] ascending, softmax weights)."""
    require_cuda(cand_score, cand_slot)
    if cand_score.dtype != torch.float32 or cand_slot.dtype != torch.int32:
        raise ValueError("candidates are float32 scores with int32 slots")
    parts, width = cand_score.shape[0], cand_score.shape[-1]
    rows = cand_score.numel() // (parts * width)
    if out is None:
        index = torch.empty(cand_score.shape[1:], dtype=index_dtype, device=cand_score.device)
        weights = torch.empty(cand_score.shape[1:], dtype=torch.float32, device=cand_score.device)
    else:
        index, weights = out
        require_cuda(index, weights)
        index_dtype = index.dtype
        if index.numel() != rows * width or weights.numel() != rows * width or weights.dtype != torch.float32:
            raise ValueError("preallocated route buffers have the wrong size")
    _check(library().glsdm_topk_merge(_ptr(cand_score), _ptr(cand_slot), parts, rows, width, _ptr(index),
                                      int(index_dtype == torch.int64), _ptr(weights),
                                      _stream(cand_score.device)))
    return index, weights


def topk_merge_packed(packed, parts, rows, width, out):
    """Merge candidates that arrive as one int32 buffer of `parts` blocks, each holding a
    shard's scores [rows, width] (float32 bits) followed by its slots [rows, width]: the
    receive buffer of a single all-gather. ``out`` = (index int32/int64, weights)."""
    index, weights = out
    require_cuda(packed, index, weights)
    region = rows * width
    if packed.numel() != parts * 2 * region or packed.dtype != torch.int32:
        raise ValueError("packed candidates are parts x (scores, slots) x rows x width int32 words")
    _check(library().glsdm_topk_merge_strided(_at(packed, 0), _at(packed, region), parts, 2 * region, rows, width,
                                              _ptr(index), int(index.dtype == torch.int64), _ptr(weights),
                                              _stream(packed.device)))
    return index, weights


def score_topk(queries, keys, width, col_base=0, out=None, row_floor=None, floor_in=None, floor_out=(), row_shift=0):
    """Dense-key routing of one shard: best `width` (score, slot) per query row, best first.
    ``row_floor`` [rows] float32: a score each row's width-th best over the WHOLE bank is known
    to reach; candidates below it are dropped (lists may come back short, padded with slot -1).
    ``floor_in`` [sources, rows] float32 (this GPU) / ``floor_out`` (device addresses of this
    shard's [rows] float32 row in each peer's floor_in) / ``row_shift``: bounds exchanged with
    the other shards while the kernels run, see glsdm_score_topk_shared."""
    require_cuda(queries, keys, row_floor, floor_in)
    if queries.dtype != torch.bfloat16 or keys.dtype != torch.bfloat16:
        raise ValueError("queries and keys must be bfloat16")
    rows, dk = queries.shape
    slots = keys.shape[0]
    lib = library()
    nbytes = lib.glsdm_score_topk_workspace_bytes(rows, slots, dk, width)
    work = _workspace(queries.device, nbytes)
    if out is None:
        score = torch.empty((rows, width), dtype=torch.float32, device=queries.device)
        slot = torch.empty((rows, width), dtype=torch.int32, device=queries.device)
    else:
        score, slot = out
        require_cuda(score, slot)
        if score.numel() != rows * width or slot.numel() != rows * width or score.dtype != torch.float32 or slot.dtype != torch.int32:
            raise ValueError("preallocated candidate buffers have the wrong size or type")
    if row_floor is not None and (row_floor.dtype != torch.float32 or row_floor.numel() != rows):
        raise ValueError("row_floor must be float32 with one value per query row")
    sources = 0
    if floor_in is not None:
        if floor_in.dtype != torch.float32 or floor_in.ndim != 2 or floor_in.shape[1] != rows:
            raise ValueError("floor_in must be float32 [sources, rows]")
        sources = floor_in.shape[0]
    peers = (ctypes.c_void_p * max(len(floor_out), 1))(*[int(a) for a in floor_out])
    _check(lib.glsdm_score_topk_shared(_ptr(queries), dk, _ptr(keys), dk, rows, slots, dk, width, col_base,
                                       _ptr(row_floor), row_shift, _ptr(floor_in), sources, peers, len(floor_out),
                                       _ptr(score), _ptr(slot), _ptr(work), work.numel(),
                                       _ptr(status_word(queries.device)), _stream(queries.device)))
    return score, slot


def pk_gemm_select(queries, codebooks, width, index_dtype=torch.int64):
    """Product-key routing without materialising factor scores.

    queries [rows, dk] bf16 (left sub-query in the first dk/2 columns), codebooks
    [2, half, dk/2] bf16. Each factor's scores are computed on the tensor cores with a fused
    top-k (glsdm_score_topk_pitched), then combined (glsdm_pk_combine).
    Returns (index [rows, k] ascending, softmax weights [rows, k]).
    """
    require_cuda(queries, codebooks)
    if queries.dtype != torch.bfloat16 or codebooks.dtype != torch.bfloat16:
        raise ValueError("queries and codebooks must be bfloat16")
    rows, dk = queries.shape
    _, half, sub = codebooks.shape
    if codebooks.shape[0] != 2 or sub * 2 != dk:
        raise ValueError("codebooks must be [2, half, dk/2]")
    lib = library()
    kf = min(width, half)
    k = routes_out(width, half)
    dev = queries.device
    lists = []
    for f in range(2):
        score = torch.empty((rows, kf), dtype=torch.float32, device=dev)
        index = torch.empty((rows, kf), dtype=torch.int32, device=dev)
        nbytes = lib.glsdm_score_topk_workspace_bytes(rows, half, sub, kf)
        work = _workspace(dev, nbytes)
        _check(lib.glsdm_score_topk_pitched(ctypes.c_void_p(queries.data_ptr() + 2 * f * sub), dk, _ptr(codebooks[f]), sub,
                                            rows, half, sub, kf, 0, _ptr(score), _ptr(index), _ptr(work), work.numel(),
                                            _ptr(status_word(dev)), _stream(dev)))
        lists.append((score, index))
    out_index = torch.empty((rows, k), dtype=index_dtype, device=dev)
    out_weights = torch.empty((rows, k), dtype=torch.float32, device=dev)
    _check(lib.glsdm_pk_combine(_ptr(lists[0][0]), _ptr(lists[0][1]), _ptr(lists[1][0]), _ptr(lists[1][1]), rows, half,
                                width, _ptr(out_index), int(index_dtype == torch.int64), _ptr(out_weights), _stream(dev)))
    return out_index, out_weights


def _log_arrays(values, logs):
    """ctypes arrays (addresses, rows, entries) of undo logs [(addresses, rows), ...]."""
    if len(logs) > MAX_UNDO_LOGS:
        raise ValueError(f"at most {MAX_UNDO_LOGS} undo logs per read")
    for a, r in logs:
        require_cuda(a, r)
        if a.dtype != torch.int64 or r.dtype != values.dtype or r.shape[-1] != values.shape[-1]:
            raise ValueError("the undo log does not match the bank")
    n = len(logs)
    addresses = (ctypes.c_void_p * max(n, 1))(*[a.data_ptr() for a, _ in logs])
    rows = (ctypes.c_void_p * max(n, 1))(*[r.data_ptr() for _, r in logs])
    entries = (ctypes.c_int64 * max(n, 1))(*[a.numel() for a, _ in logs])
    return n, addresses, rows, entries


def read_backward(values, grad_out, grad_weights, index, weights, rows_per_bank, half, logs=()):
    """Backward of the routed read: (grad_scores [..., 2*half], addresses [rows*k] int64,
    grad_rows [rows*k, dim]) - the bank gradient stays compact, one row per route. ``logs``
    = [(undo_addresses, undo_rows), ...] of the copy-free commits applied to ``values`` since
    the version that was read (oldest first); empty when ``values`` still is that version."""
    require_cuda(values, grad_out, grad_weights, index, weights)
    bank = bank_of(values)
    width = index.shape[-1]
    rows = index.numel() // width
    dim = values.shape[-1]
    n, log_addresses, log_rows, log_entries = _log_arrays(values, logs)
    grad_scores = torch.empty((*index.shape[:-1], 2 * half), dtype=torch.float32, device=values.device)
    grad_rows = torch.empty((rows * width, dim), dtype=torch.float32, device=values.device)
    addresses = torch.empty(rows * width, dtype=torch.int64, device=values.device)
    _check(library().glsdm_read_backward_version(
        ctypes.byref(bank), _ptr(grad_out), _ptr(grad_weights), _ptr(index), int(index.dtype == torch.int64),
        _ptr(weights), rows, rows_per_bank, width, half, n, log_addresses, log_rows, log_entries,
        _ptr(grad_scores), _ptr(grad_rows), _ptr(addresses), _stream(values.device)))
    return grad_scores, addresses, grad_rows
