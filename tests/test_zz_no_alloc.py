"""The allocation-free pair counter (``stbpe_rows_count_pairs_noalloc``) against the regular one.

Some users of this library cannot let a call allocate device memory: the reference trainer hands
all of the device to its workspaces before the merge loop (so a late allocation is the one that
runs out), and it keeps three streams per device busy, which the device-wide synchronisation of a
``cudaMalloc`` / ``cudaFree`` would stall.  For them the library carries a fixed scratch block and
this entry point, which must give exactly what ``stbpe_rows_count_pairs`` gives.  Integer work: the
comparison is bit-exact.  Two calls in a row on different inputs check that nothing of the first
call's table or counters leaks into the second.  The file name sorts last so that a run which
stops at the first failure has already run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from supertoken_b200 import _lib

pytestmark = pytest.mark.gpu


def _run(fn_name, tokens, valid, cap):
    lib = _lib.load()
    B, L = tokens.shape
    keys = torch.full((cap, 2), 7, dtype=torch.int32, device="cuda")
    counts = torch.full((cap,), 7, dtype=torch.int64, device="cuda")
    length = torch.full((1,), 7, dtype=torch.int64, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    args = [tokens.data_ptr(), valid.data_ptr(), B, L, keys.data_ptr(), counts.data_ptr(), cap,
            length.data_ptr(), stream]
    err = None
    if fn_name.endswith("noalloc"):
        err = ctypes.create_string_buffer(256)
        args += [err, 256]
    status = getattr(lib, fn_name)(*args)
    torch.cuda.synchronize()
    return status, keys.cpu(), counts.cpu(), int(length.item()), (err.value.decode() if err else "")


def _batch(seed, B, L, alphabet):
    g = torch.Generator().manual_seed(seed)
    tokens = torch.randint(0, alphabet, (B, L), generator=g, dtype=torch.int32).cuda()
    valid = (torch.rand((B, L), generator=g) < 0.85).to(torch.uint8).cuda()
    return tokens, valid


def test_noalloc_matches_allocating_entry_point_on_two_calls_in_a_row():
    # first a batch with many distinct pairs, then one with few: stale entries would show up
    for seed, B, L, alphabet in ((1, 37, 400, 5000), (2, 64, 1000, 3)):
        tokens, valid = _batch(seed, B, L, alphabet)
        cap = B * (L - 1)
        s0, k0, c0, n0, _ = _run("stbpe_rows_count_pairs", tokens, valid, cap)
        s1, k1, c1, n1, msg = _run("stbpe_rows_count_pairs_noalloc", tokens, valid, cap)
        assert s0 == _lib.OK and s1 == _lib.OK, msg
        assert n0 == n1 and n0 > 0
        assert torch.equal(k0, k1) and torch.equal(c0, c1)
        assert int(c1[:n1].sum()) == int((valid[:, :-1] & valid[:, 1:]).sum())


def test_noalloc_rejects_oversized_batches_and_small_buffers():
    tokens, valid = _batch(3, 33, 2001, 10)          # 33 * 2000 = 66 000 positions > 65 536
    status, _, _, _, msg = _run("stbpe_rows_count_pairs_noalloc", tokens, valid, 100)
    assert status == _lib.E_CAPACITY and "65536" in msg.replace(" ", "")
    tokens, valid = _batch(4, 8, 200, 5000)
    status, _, _, _, msg = _run("stbpe_rows_count_pairs_noalloc", tokens, valid, 10)
    assert status == _lib.E_CAPACITY and "capacity exceeded" in msg
    # and it still works afterwards
    tokens, valid = _batch(5, 4, 50, 4)
    s0, k0, c0, n0, _ = _run("stbpe_rows_count_pairs", tokens, valid, 4 * 49)
    s1, k1, c1, n1, _ = _run("stbpe_rows_count_pairs_noalloc", tokens, valid, 4 * 49)
    assert s0 == s1 == _lib.OK and n0 == n1 and torch.equal(k0, k1) and torch.equal(c0, c1)


def test_noalloc_at_the_size_limit_with_all_pairs_distinct():
    # 65 536 pair positions, every pair different: the largest number of unique keys the fixed block
    # has to sort (its sort runs through the block's own double buffers, whatever the count)
    tokens = torch.arange(65537, dtype=torch.int32).reshape(1, -1).cuda()
    valid = torch.ones((1, 65537), dtype=torch.uint8).cuda()
    cap = 65536
    s0, k0, c0, n0, _ = _run("stbpe_rows_count_pairs", tokens, valid, cap)
    s1, k1, c1, n1, msg = _run("stbpe_rows_count_pairs_noalloc", tokens, valid, cap)
    assert s0 == _lib.OK and s1 == _lib.OK, msg
    assert n0 == n1 == 65536 and torch.equal(k0, k1) and torch.equal(c0, c1)
    assert k1[:, 0].tolist() == list(range(65536)) and torch.all(c1 == 1)
    # a small batch right after it must not see the large one's leftovers
    tokens, valid = _batch(6, 3, 40, 6)
    s0, k0, c0, n0, _ = _run("stbpe_rows_count_pairs", tokens, valid, 3 * 39)
    s1, k1, c1, n1, _ = _run("stbpe_rows_count_pairs_noalloc", tokens, valid, 3 * 39)
    assert s0 == s1 == _lib.OK and n0 == n1 and torch.equal(k0, k1) and torch.equal(c0, c1)


def test_noalloc_against_the_reference_made_fixtures():
    # the histograms the reference's own count_pairs produced (tests/golden/ops.json)
    from tests.helpers import load_golden
    for case in load_golden("ops.json")["count"]:
        tokens = torch.tensor(case["tokens"], dtype=torch.int32).cuda()
        valid = torch.tensor(case["valid"], dtype=torch.uint8).cuda()
        B, L = tokens.shape
        cap = max(B * max(L - 1, 0), 1)
        status, keys, counts, n, msg = _run("stbpe_rows_count_pairs_noalloc", tokens, valid, cap)
        assert status == _lib.OK, msg
        assert n == len(case["keys"])
        packed = (keys[:n, 0].to(torch.int64) << 32) | keys[:n, 1].to(torch.int64)
        assert packed.tolist() == case["keys"] and counts[:n].tolist() == case["counts"]
