"""The multi-rank merge loop's protocol on CPU: sharding, owner hashing, bounded exchange chunks
with exchange-only rounds, candidate gathering, identical decisions on every rank.  World size 2
and 3 over gloo (one process per rank) and the in-process LocalComm; the result must equal the
single-process oracle."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle as O
from supertoken_b200 import _lib as L
from supertoken_b200 import synth
from supertoken_b200.dist import LocalComm, ShardedBPE, TorchDistComm, owner_of, shard_rows
from tests.cpu_worker import CpuWorker
from tests.helpers import corpus_rows


def _corpus():
    c = synth.config2_mixed(24 << 10, seed=5, lexicon=800, mean_doc_bytes=300)
    return [r.tolist() for r in corpus_rows(c)], np.asarray(c.row_offsets)


def test_shard_rows_contiguous_and_balanced():
    rows, off = _corpus()
    for world in (1, 2, 3, 8):
        parts = shard_rows(off, world)
        assert parts[0][0] == 0 and parts[-1][1] == len(rows)
        assert all(parts[i][1] == parts[i + 1][0] for i in range(world - 1))
        sizes = [off[hi] - off[lo] for lo, hi in parts]
        assert max(sizes) - min(sizes) <= 2 * np.diff(off).max()
    assert shard_rows(np.array([0, 5]), 4) == [(0, 0), (0, 0), (0, 0), (0, 1)] or \
        sum(hi - lo for lo, hi in shard_rows(np.array([0, 5]), 4)) == 1


def test_owner_hash_is_spread():
    keys = [(a << 32) | b for a in range(60) for b in range(60)]
    for world in (2, 8):
        hist = np.bincount([owner_of(k, world) for k in keys], minlength=world)
        assert hist.min() > 0.7 * len(keys) / world


@pytest.mark.parametrize("world,cap", [(2, 4096), (2, 7), (3, 50)])
def test_local_comm_matches_oracle(world, cap):
    rows, off = _corpus()
    target = 40
    om, oc, reason = O.train_flat(*O.flatten_rows(rows), 256, target, 1)
    parts = shard_rows(off, world)
    workers = [CpuWorker(rows[lo:hi], r, world, 256, target, cap) for r, (lo, hi) in enumerate(parts)]
    loop = ShardedBPE(workers, LocalComm())
    done, stop = loop.train(check_every=8)
    assert stop == L.STOP_TARGET and done == target
    for w in workers:
        assert w.merges == om and w.counts == oc
    if cap < 100:
        assert loop.rounds > target + 1      # the small chunks forced exchange-only rounds


def _gloo_rank(rank, world, port, cap, target, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rows, off = _corpus()
        lo, hi = shard_rows(off, world)[rank]
        w = CpuWorker(rows[lo:hi], rank, world, 256, target, cap)
        loop = ShardedBPE([w], TorchDistComm())
        done, stop = loop.train(check_every=16)
        q.put((rank, w.merges, w.counts, done, stop, loop.rounds))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,cap", [(2, 64), (3, 9)])
def test_gloo_ranks_agree_with_oracle(world, cap):
    rows, off = _corpus()
    target = 25
    om, oc, _ = O.train_flat(*O.flatten_rows(rows), 256, target, 1)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_gloo_rank, args=(r, world, port, cap, target, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, merges, counts, done, stop, rounds in results:
        assert merges == om and counts == oc and done == target and stop == L.STOP_TARGET


def test_stop_rules_across_ranks():
    # no pair anywhere -> stop without merges; all counts 1 -> low-count stop
    for rows, expect in (([[1], [2], [3]], L.STOP_NO_PAIRS), ([[1, 2], [3, 4], [5, 6, 7]], L.STOP_LOW_COUNT)):
        workers = [CpuWorker(rows[r::2], r, 2, 256, 5, 16) for r in range(2)]
        done, stop = ShardedBPE(workers, LocalComm()).train(check_every=2)
        assert done == 0 and stop == expect


def _reducer_rank(rank, world, port, q):
    from supertoken_b200.dist import get_histogram_reducer, register_histogram_reducer
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rows, off = _corpus()
        lo, hi = shard_rows(off, world)[rank]
        ids, o2 = O.flatten_rows(rows[lo:hi]) if hi > lo else (np.zeros(0, np.int32), np.zeros(1, np.int64))
        k, c = O.count_pairs_flat(ids, o2, 1) if hi > lo else (np.zeros(0, np.uint64), np.zeros(0, np.int64))
        # unsorted input with a duplicated key: the reducer merges duplicates as well
        keys = torch.from_numpy(np.concatenate([k[::-1], k[:1]]).astype(np.int64))
        counts = torch.from_numpy(np.concatenate([c[::-1], np.array([5], np.int64)[:len(k[:1])]]))
        register_histogram_reducer(None)
        gk, gc = get_histogram_reducer()(keys, counts)
        q.put((rank, gk.tolist(), gc.tolist(), int(k[0]) if len(k) else -1))
    finally:
        dist.destroy_process_group()


def test_histogram_reducer_hook_sums_over_gloo_ranks():
    # mirror of the reference's reducer hook: every rank gets the same sorted global histogram
    from supertoken_b200.dist import get_histogram_reducer, reduce_pair_histograms, register_histogram_reducer
    rows, off = _corpus()
    world = 2
    gk, gc = O.count_pairs_flat(*O.flatten_rows(rows), 1)
    want = dict(zip(gk.astype(np.int64).tolist(), gc.tolist()))
    # a pair that straddles the two shards does not exist (rows are never split), so the sum of the
    # shard histograms is the histogram of the corpus; each rank added 5 to its first key
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_reducer_rank, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for _, _, _, first in results:
        if first >= 0:
            want[first] += 5
    for _, keys, counts, _ in results:
        assert keys == sorted(want) and counts == [want[k] for k in keys]
    # the hook itself
    marker = lambda k, c: (k, c)
    register_histogram_reducer(marker)
    assert get_histogram_reducer() is marker
    register_histogram_reducer(None)
    assert get_histogram_reducer() is reduce_pair_histograms
    k, c = reduce_pair_histograms(torch.tensor([7, 3, 7]), torch.tensor([1, 2, 4]))   # no group: local merge only
    assert k.tolist() == [3, 7] and c.tolist() == [2, 5]
