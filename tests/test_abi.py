"""The C-ABI library loads and exports every symbol include/glsdm.h declares; argument
checks that run before any launch work without a GPU."""
import ctypes
import os
import re

from conftest import ROOT


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "glsdm.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(glsdm_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(native):
    lib = ctypes.CDLL(native.LIBRARY_PATH)
    names = declared_symbols()
    assert len(names) >= 12
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in glsdm.h but not exported"
    assert set(native.SIGNATURES) == set(names), "ctypes signatures and header disagree"


def test_status_strings_and_version(native):
    lib = native.library()
    assert lib.glsdm_abi_version() >= 1
    assert lib.glsdm_status_string(0) == b"ok"
    for code in range(1, 6):
        assert len(lib.glsdm_status_string(code)) > 4
    assert lib.glsdm_status_string(99) == b"unknown status"


def test_argument_errors_need_no_device(native):
    lib = native.library()
    null = ctypes.c_void_p(0)
    # null scores
    assert lib.glsdm_pk_select(null, 4, 8, 2, null, 1, null, null) == 1
    # width beyond the 32 routes a warp keeps
    fake = ctypes.c_void_p(4096)
    assert lib.glsdm_pk_select(fake, 4, 64, 33, fake, 1, fake, null) == 2
    # zero rows is a successful no-op and launches nothing
    assert lib.glsdm_pk_select(fake, 0, 64, 8, fake, 1, fake, null) == 0
    bank = native.Bank(4096, 0, 1, 1, 16, 8, 0, 16)
    assert lib.glsdm_snapshot_read(ctypes.byref(bank), fake, 1, fake, null, 0, 1, 2, fake, null, null) == 0
    bad = native.Bank(4096, 0, 1, 1, 16, 8, 4, 2)  # empty slot range
    assert lib.glsdm_snapshot_read(ctypes.byref(bad), fake, 1, fake, null, 1, 1, 2, fake, null, null) == 1
    assert lib.glsdm_commit_workspace_bytes(1000, 64) > 1000 * 28
    # commit with a workspace that is too small
    assert lib.glsdm_commit(fake, fake, 0, 0, 16, 8, fake, fake, null, 10, 0, ctypes.c_void_p(256), 16, null, null) == 3
    assert lib.glsdm_topk_merge(fake, fake, 2, 0, 8, fake, 1, fake, null) == 0
    assert lib.glsdm_topk_merge(fake, fake, 2, 4, 40, fake, 1, fake, null) == 2


def test_rows_beyond_the_banks_are_rejected_before_any_launch(native):
    """Per-request banks: routing row r reads bank r / rows_per_bank, so a call whose rows do
    not fit banks * rows_per_bank would read past the last bank. Every entry that takes
    rows_per_bank must refuse it on the host (nothing is launched; the pointers are fake)."""
    lib = native.library()
    null, fake = ctypes.c_void_p(0), ctypes.c_void_p(4096)
    two = native.Bank(4096, 0, 2, 1, 16, 8, 0, 16)       # 2 banks, 1 head, 16 slots (half 4), dim 8
    one = native.Bank(4096, 0, 1, 1, 16, 8, 0, 16)
    ok, bad = 2 * 5, 2 * 5 + 1                            # rows_per_bank = 5
    assert lib.glsdm_snapshot_read(ctypes.byref(two), fake, 1, fake, null, bad, 5, 2, fake, null, null) == 1
    assert lib.glsdm_pk_select_read(ctypes.byref(two), fake, bad, 5, 4, 2, fake, fake, 1, fake, null, null) == 1
    assert lib.glsdm_pk_propose(ctypes.byref(two), fake, fake, 0, fake, fake, null, bad, 5, 5, 4, 2, 0, 8, 1, 0,
                                fake, fake, fake, null, null) == 1
    assert lib.glsdm_read_backward(ctypes.byref(two), fake, null, fake, 1, fake, bad, 5, 2, 4, fake, fake, fake,
                                   null) == 1
    assert lib.glsdm_overlay_read(ctypes.byref(two), fake, 1, fake, bad, 5, 2, 0, null, null, null, fake, null,
                                  null) == 1
    assert lib.glsdm_read_backward_version(ctypes.byref(two), fake, null, fake, 1, fake, bad, 5, 2, 4, 0, null, null,
                                           null, fake, fake, fake, null) == 1
    backward = lambda bank, rows, logs: lib.glsdm_pk_propose_backward(                     # noqa: E731
        ctypes.byref(bank), fake, fake, 0, fake, fake, null, fake, fake, rows, 5, 4, 2, logs, null, null, null,
        fake, fake, fake, fake, fake, null)
    assert backward(two, bad, 0) == 1
    assert backward(two, ok, 1) == 1                      # logs announced, none given
    assert backward(two, ok, native.MAX_UNDO_LOGS + 1) == lib.glsdm_read_backward_version(
        ctypes.byref(two), fake, null, fake, 1, fake, ok, 5, 2, 4, native.MAX_UNDO_LOGS + 1, null, null, null,
        fake, fake, fake, null) != 0
    wide = native.Bank(4096, 0, 1, 1, 16, 512, 0, 16)     # rows of 512 values: the backward kernel holds 256
    assert backward(wide, 5, 0) == 2
    del one


def test_score_topk_plans_cover_every_block_and_tile_once():
    """Host-side work decomposition of the dense-key routing kernels (no GPU involved): the
    uniform parts and the extra cuts of the last wave's row blocks tile rows x key tiles exactly."""
    import ctypes
    from gl_sdm_b200 import _native
    lib = _native.library()
    out = (ctypes.c_int32 * 8)()
    for which in (0, 2):
        for sms in (148, 132, 8):
            for rows in (1, 127, 128, 129, 5000, 19000, 65536, 70001):
                for slots in (1, 255, 4096, 70000, 1 << 20, (1 << 24) - 3):
                    assert lib.glsdm_score_topk_plan(rows, slots, 32, which, sms, out) == 0
                    blocks_u, parts, per, tiles, tail_blocks, tail_parts, tail_per, block_rows = list(out)
                    tile_cols = 128 if which == 0 else 256
                    assert tiles == -(-slots // tile_cols)
                    assert (blocks_u + tail_blocks) * block_rows >= rows > (blocks_u + tail_blocks - 1) * block_rows
                    assert parts >= 1 and (parts - 1) * per < tiles <= parts * per
                    if tail_blocks:
                        assert which == 2 and parts == 1 and blocks_u % sms == 0
                        assert tail_parts >= 2 and (tail_parts - 1) * tail_per < tiles <= tail_parts * tail_per
                        assert tail_blocks * tail_parts <= sms
    assert lib.glsdm_score_topk_plan(0, 10, 32, 2, 148, out) != 0
