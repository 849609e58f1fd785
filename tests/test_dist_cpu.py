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
