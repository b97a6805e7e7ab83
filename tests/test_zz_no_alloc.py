"""glsdm_commit_static: the commit for hosts that cannot hand in a workspace.

The entry point keeps its scratch in a fixed device array inside the library, so it must
give the same bank as glsdm_commit (which gets its scratch from the caller), call after
call, although the array still holds the previous call's leftovers. The file name sorts
last on purpose: a run that stops at the first failure has then already run everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _entries(seed, rows, entries, dim):
    g = torch.Generator().manual_seed(seed)
    addresses = torch.randint(0, rows, (entries,), generator=g)
    keys = addresses * 64 + torch.randint(0, 64, (entries,), generator=g)
    deltas = torch.randn(entries, dim, generator=g)
    return addresses.to(DEV), deltas.to(DEV), keys.to(DEV)


def _commit_static(native, bank, addresses, deltas, keys):
    lib = native.library()
    out = torch.empty_like(bank)
    status = native.status_word(bank.device)
    code = lib.glsdm_commit_static(bank.data_ptr(), out.data_ptr(), native._dtype_code(bank), 0, bank.shape[0],
                                   bank.shape[1], addresses.data_ptr(), deltas.data_ptr(), keys.data_ptr(),
                                   addresses.numel(), 0, status.data_ptr(),
                                   ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return code, out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_commit_matches_the_workspace_commit_twice(native, dtype):
    rows, dim = 3000, 128
    bank = torch.randn(rows, dim, generator=torch.Generator().manual_seed(1)).to(dtype).to(DEV)
    # two different calls in a row: the second one starts from the first one's leftovers
    for seed, entries in ((11, 40000), (12, 9000)):
        addresses, deltas, keys = _entries(seed, rows, entries, dim)
        want = native.commit_rows(bank, addresses, deltas, keys)
        code, got = _commit_static(native, bank, addresses, deltas, keys)
        assert code == 0
        torch.cuda.synchronize()
        assert torch.equal(got, want)          # same kernels, same order: bit-identical
        native.raise_on_device_status(DEV)


def test_static_scratch_commit_at_its_documented_limit(native):
    """65,536 entries of 256 values, the largest request the built-in array covers, with hot
    addresses (segments longer than 256 entries take the chunked path and its partial sums)."""
    rows, dim, entries = 5000, 256, 65536
    bank = torch.randn(rows, dim, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).to(DEV)
    addresses, deltas, keys = _entries(13, rows, entries, dim)
    addresses[:3000] = 7                        # one address receives 3000+ entries
    keys[:3000] = 7 * 64 + (keys[:3000] % 64)
    want = native.commit_rows(bank, addresses, deltas, keys)
    for _ in range(2):
        code, got = _commit_static(native, bank, addresses, deltas, keys)
        assert code == 0
        torch.cuda.synchronize()
        assert torch.equal(got, want)
    native.raise_on_device_status(DEV)


def test_static_scratch_commit_rejects_oversized_requests(native):
    lib = native.library()
    limit = lib.glsdm_commit_static_max_entries()
    assert limit == 65536
    bank = torch.zeros(16, 8, device=DEV)
    addresses = torch.zeros(limit + 1, dtype=torch.long, device=DEV)
    deltas = torch.zeros(limit + 1, 8, device=DEV)
    code, _ = _commit_static(native, bank, addresses, deltas, addresses)
    assert code == 5 and b"capacity" in lib.glsdm_status_string(code)
    wide = torch.zeros(4, 512, device=DEV)
    code, _ = _commit_static(native, wide, addresses[:4], torch.zeros(4, 512, device=DEV), addresses[:4])
    assert code == 5
