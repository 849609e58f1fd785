"""Multi-GPU merge loop: rows sharded by contiguous document ranges, pair keys by hash owner.

Replaces the reference's cross-rank histogram reduction (``utils.reduce_pair_histograms``,
``gpu_tokenizer/utils.py:863-978``: all-gather of every rank's key list plus a dense all-reduce
over the union, once per recount) with an exchange of the +-deltas of each merge:

    round:  local merge kernel -> per-owner outbox chunks -> all-to-all (equal splits)
            -> owners add into their table slice -> local best candidate
            -> all-gather of ``world`` candidates -> every rank commits the same decision

A chunk has a fixed capacity; deltas that do not fit stay on the sender and the candidates carry an
"incomplete" flag, in which case every rank agrees to run another exchange-only round before a
merge is chosen.  Nothing in a round needs the host to look at device data, so rounds are enqueued
back to back and the host reads the state only every ``check_every`` rounds.

The round logic is written against a small worker interface so that the same code drives
(a) one ``EngineWorker`` per process over ``torch.distributed`` (NCCL), (b) several workers of one
process on one GPU (tests: the device kernels of every rank run one after the other, no kernel
waits for another), and (c) CPU stand-in workers over ``gloo`` (tests of the protocol itself).
"""
from __future__ import annotations

import ctypes
import os
from typing import Callable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import _lib as L

_M64 = (1 << 64) - 1


def mix64(x: int) -> int:
    """The 64-bit finaliser the kernels use to place and to own keys."""
    x &= _M64
    x ^= x >> 33
    x = (x * 0xFF51AFD7ED558CCD) & _M64
    x ^= x >> 33
    x = (x * 0xC4CEB9FE1A85EC53) & _M64
    x ^= x >> 33
    return x


_M32 = (1 << 32) - 1


def mix32(x: int) -> int:
    """The invertible 32-bit mix that names a key's partition (``mix32`` in ``csrc/common.cuh``)."""
    x &= _M32
    x ^= x >> 16
    x = (x * 0x7FEB352D) & _M32
    x ^= x >> 15
    x = (x * 0x846CA68B) & _M32
    x ^= x >> 16
    return x


def part_of(key: int) -> int:
    """Partition (0..255) of a packed pair key: top bits of its slot in the pair table, partition of
    the first count of a 16-bit vocabulary, and - modulo the number of ranks - its owner."""
    a, b = (key >> 32) & _M32, key & _M32
    folded = ((a << 16) ^ b ^ ((a >> 16) * 0x9E3779B1) ^ ((b >> 16) * 0x85EBCA77)) & _M32
    return mix32(folded) >> 24


def owner_of(key: int, world: int) -> int:
    """Rank that owns a packed pair key (``owner_of`` in ``csrc/common.cuh``)."""
    return part_of(key) % world


def shard_rows(row_offsets: np.ndarray, world: int) -> List[Tuple[int, int]]:
    """Contiguous row ranges ``[lo, hi)`` per rank, balanced by bytes; a row never spans ranks
    (so no halo crosses GPUs).  The reference shards whole files per rank
    (``gpu_tokenizer/cli_train_bpe.py:124-140``)."""
    off = np.asarray(row_offsets, dtype=np.int64)
    n_rows = len(off) - 1
    total = int(off[-1] - off[0])
    cuts = [0]
    for r in range(1, world):
        target = off[0] + total * r // world
        k = int(np.searchsorted(off, target, side="left"))
        cuts.append(min(max(k, cuts[-1]), n_rows))
    cuts.append(n_rows)
    return [(cuts[r], cuts[r + 1]) for r in range(world)]


# ----------------------------------------------------------------------------- reducer hook
# The reference lets a launcher install the function that sums sparse pair histograms over the
# ranks (``gpu_tokenizer/dist/launcher.py:25``, ``:98-110``; default ``utils.reduce_pair_histograms``,
# ``gpu_tokenizer/utils.py:863-978``).  The engine here never ships whole histograms (it exchanges
# per-merge deltas by key owner), but callers of the hook find the same three names with the same
# contract: (keys int64[n], counts int64[n]) -> (sorted unique keys, summed counts), identical on
# every rank.
ReducerFn = Callable[[torch.Tensor, torch.Tensor], Tuple[torch.Tensor, torch.Tensor]]
_histogram_reducer: Optional[ReducerFn] = None


def register_histogram_reducer(fn: Optional[ReducerFn]) -> None:
    global _histogram_reducer
    _histogram_reducer = fn


def get_histogram_reducer() -> ReducerFn:
    return _histogram_reducer if _histogram_reducer is not None else reduce_pair_histograms


def _aggregate(keys: torch.Tensor, counts: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    if keys.numel() == 0:
        return keys.to(torch.int64), counts.to(torch.int64)
    keys, order = torch.sort(keys.to(torch.int64))
    uniq, inverse = torch.unique_consecutive(keys, return_inverse=True)
    out = torch.zeros(uniq.numel(), dtype=torch.int64, device=keys.device)
    out.index_add_(0, inverse, counts.to(torch.int64)[order])
    return uniq, out


def reduce_pair_histograms(keys: torch.Tensor, counts: torch.Tensor, group=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Sum sparse histograms over the ranks of the process group (all ranks get the same sorted
    result); without an initialised group, or with one rank, only duplicate keys are merged."""
    import torch.distributed as dist
    keys, counts = _aggregate(keys, counts)
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return keys, counts
    world = dist.get_world_size(group)
    n = torch.tensor([keys.numel()], dtype=torch.int64, device=keys.device)
    sizes = [torch.zeros_like(n) for _ in range(world)]
    dist.all_gather(sizes, n, group=group)
    sizes = [int(x.item()) for x in sizes]
    cap = max(sizes)
    if cap == 0:
        return keys, counts
    pad_k = torch.zeros(cap, dtype=torch.int64, device=keys.device)
    pad_c = torch.zeros(cap, dtype=torch.int64, device=keys.device)
    pad_k[:keys.numel()], pad_c[:keys.numel()] = keys, counts
    all_k = [torch.empty_like(pad_k) for _ in range(world)]
    all_c = [torch.empty_like(pad_c) for _ in range(world)]
    dist.all_gather(all_k, pad_k, group=group)
    dist.all_gather(all_c, pad_c, group=group)
    return _aggregate(torch.cat([k[:m] for k, m in zip(all_k, sizes)]),
                      torch.cat([c[:m] for c, m in zip(all_c, sizes)]))


def rounds_until_next_check(done: int, target: int, check_every: int) -> int:
    """Rounds to enqueue before the host looks at the device state again.  Every rank must enqueue
    the same number, so this depends only on what all ranks agree on (merges committed, target).
    Early in a run the host looks more often: that is where each rank decides to start keeping its
    pair filter (tile skipping) and to re-pack.  Never more rounds than the target still needs
    (one per merge plus the round that applies the last one); exchange-only rounds, if any, are
    caught by the next check."""
    n = check_every if done >= 512 else min(check_every, 32)
    return max(1, min(n, target - done + 1))


# ----------------------------------------------------------------------------- first count, 16-bit vocabulary
def wide_count(engine, group=None) -> bool:
    """First count of an id stream over at most 65 536 ids, one process per GPU on one NVLink domain:
    every rank partitions the pairs of its rows, the owner of a partition counts it out of all ranks'
    buffers over peer memory (``stbpe_mg_wide_*``).  Call it before the loop's count round, which then
    finds the table filled.  Returns False - and leaves the counting to that round - when the stream
    of any rank does not qualify.  ``torch.distributed`` carries the IPC handles (first call on an
    engine only: the peers' buffers stay mapped until ``wide_close``), the agreement and the barrier
    between the two passes."""
    import torch.distributed as dist
    lib = L.load()
    world = engine.world_size
    if engine.base_vocab > 65536 or world < 2:
        return False
    dev = engine.device
    if not getattr(engine, "_wide_mapped", False):
        buf = (ctypes.c_ubyte * 64)()
        with torch.cuda.device(dev):
            st = lib.stbpe_mg_wide_export(engine._h, buf)
        have = torch.tensor([1 if st == L.OK else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(have, op=dist.ReduceOp.MIN, group=group)
        if int(have.item()) == 0:     # a rank has no room for the buffers: the ordinary round counts
            return False
        mine = torch.tensor(list(buf), dtype=torch.uint8, device=dev)
        every = torch.empty(world * 64, dtype=torch.uint8, device=dev)
        dist.all_gather_into_tensor(every, mine, group=group)
        raw = bytes(every.cpu().tolist())
        with torch.cuda.device(dev):
            engine._check(lib.stbpe_mg_wide_open(engine._h, raw, world))
        engine._wide_mapped = True
    ok = ctypes.c_int32(0)
    with torch.cuda.device(dev):
        engine._check(lib.stbpe_mg_wide_pass1(engine._h, ctypes.byref(ok), engine._s))
    agreed = torch.tensor([ok.value], dtype=torch.int32, device=dev)
    dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=group)   # also the barrier between the passes
    good = int(agreed.item()) == 1
    if good:
        with torch.cuda.device(dev):
            engine._check(lib.stbpe_mg_wide_pass2(engine._h, engine._s))
    dist.barrier(group=group)     # nobody starts the next first pass while a peer still reads this one
    return good


def wide_close(engine, group=None) -> None:
    """Unmap the peers' partition buffers and wait for every rank to have done so; call before the
    engine is closed (its buffers must outlive the peers' mappings)."""
    import torch.distributed as dist
    if getattr(engine, "_wide_mapped", False):
        with torch.cuda.device(engine.device):
            engine._check(L.load().stbpe_mg_wide_close(engine._h))
        dist.barrier(group=group)
        engine._wide_mapped = False


# ----------------------------------------------------------------------------- workers
class EngineWorker:
    """One rank's engine plus its exchange buffers (torch tensors on the engine's device)."""

    def __init__(self, engine, cap_per_peer: int = 8192):
        self.e = engine
        self.world, self.rank = engine.world_size, engine.rank
        self.cap = int(cap_per_peer)
        dev = engine.device
        shape = (self.world, self.cap + 1, 2)
        self.outbox = torch.zeros(shape, dtype=torch.int64, device=dev)
        self.inbox = torch.zeros(shape, dtype=torch.int64, device=dev)
        self.cand = torch.zeros(4, dtype=torch.int64, device=dev)
        self.all_cands = torch.zeros((self.world, 4), dtype=torch.int64, device=dev)
        self._lib = L.load()
        self._check(self._lib.stbpe_mg_set_buffers(engine._h, self.outbox.data_ptr(), self.inbox.data_ptr(), self.cap))

    def _check(self, st):
        self.e._check(st)

    @property
    def _s(self):
        return self.e._s

    def count_local(self):
        with torch.cuda.device(self.e.device):
            self._check(self._lib.stbpe_mg_count_local(self.e._h, self._s))

    def merge_local(self):
        with torch.cuda.device(self.e.device):
            self._check(self._lib.stbpe_mg_merge_local(self.e._h, self._s))

    def apply_inbox(self):
        with torch.cuda.device(self.e.device):
            self._check(self._lib.stbpe_mg_apply_inbox(self.e._h, self._s))

    def candidate(self):
        with torch.cuda.device(self.e.device):
            self._check(self._lib.stbpe_mg_candidate(self.e._h, self.cand.data_ptr(), self._s))

    def commit(self):
        with torch.cuda.device(self.e.device):
            self._check(self._lib.stbpe_mg_commit(self.e._h, self.all_cands.data_ptr(), self._s))

    def progress(self) -> Tuple[int, int]:
        """(merges done, stop reason); synchronises.  Also the point where this rank re-packs its
        own tiles when they have become sparse (a purely local decision)."""
        self.e.repack()
        st = self.e.state()
        if st.device_error:
            self.e.count_error()
        return int(st.merges_done), int(st.stop_reason)

    def merges(self):
        return self.e.merges()


class TorchDistComm:
    """The two collectives of a round over ``torch.distributed`` (NCCL on GPUs, gloo in CPU tests)."""

    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist = dist
        self.group = group

    def exchange(self, workers: Sequence):
        (w,) = workers
        self.dist.all_to_all_single(w.inbox.view(-1), w.outbox.view(-1), group=self.group)

    def gather(self, workers: Sequence):
        (w,) = workers
        self.dist.all_gather_into_tensor(w.all_cands.view(-1), w.cand, group=self.group)


class LocalComm:
    """All ranks live in this process (one GPU or CPU): chunks are copied between the workers."""

    def exchange(self, workers: Sequence):
        for dst in workers:
            for src in workers:
                dst.inbox[src.rank].copy_(src.outbox[dst.rank])

    def gather(self, workers: Sequence):
        for dst in workers:
            for src in workers:
                dst.all_cands[src.rank].copy_(src.cand)


class ShardedBPE:
    """Drives the rounds.  ``workers`` are the ranks that live in this process (normally one)."""

    def __init__(self, workers: Sequence, comm):
        self.workers = list(workers)
        self.comm = comm
        self.rounds = 0
        self._counted = False

    def _round(self, first: bool):
        for w in self.workers:
            w.count_local() if first else w.merge_local()
        self.comm.exchange(self.workers)
        for w in self.workers:
            w.apply_inbox()
            w.candidate()
        self.comm.gather(self.workers)
        for w in self.workers:
            w.commit()
        self.rounds += 1

    def train(self, check_every: int = 64, max_rounds: Optional[int] = None):
        """Run rounds until a stop rule fires on the device: the merge target the engines were
        created with (``max_merges``), no pair left, or best count below 2.  A round applies the
        merge committed by the previous round and commits the next one, so the last committed merge
        is applied by one more round before the target stop is raised.  Returns (merges committed,
        stop reason) as every rank sees them; the host reads device state only every
        ``check_every`` rounds."""
        left = max_rounds if max_rounds is not None else 1 << 62
        if not self._counted:
            self._round(True)
            self._counted = True
            left -= 1
        while True:
            states = [w.progress() for w in self.workers]   # every rank may re-pack its own tiles here
            done, reason = states[0]
            if reason != L.RUNNING or left <= 0:
                return done, reason
            w0 = self.workers[0]
            target = w0.max_merges if hasattr(w0, "max_merges") else w0.e.max_merges
            n = min(rounds_until_next_check(done, target, check_every), left)
            for _ in range(n):
                self._round(False)
            left -= n


class NativeLoop:
    """The same rounds issued by the library itself (``stbpe_mg_run``): kernels, grouped
    ncclSend/ncclRecv and ncclAllGather on one stream from C++, no Python and no host
    synchronisation per round.  ``torch.distributed`` is used once, to hand the NCCL id to every
    rank.  One engine (one GPU) per process."""

    _joined = set()   # (device index, world, rank) whose communicator exists in this process

    def __init__(self, engine, cap_per_peer: int = 4096, group=None):
        import torch.distributed as dist
        self.e = engine
        self._lib = L.load()
        key = (engine.device.index, engine.world_size, engine.rank)
        raw = bytes(128)
        if key not in NativeLoop._joined:
            ident = torch.zeros(128, dtype=torch.uint8)
            if dist.get_rank(group) == 0:
                buf = (ctypes.c_ubyte * 128)()
                engine._check(self._lib.stbpe_mg_nccl_unique_id(buf))
                ident = torch.tensor(list(buf), dtype=torch.uint8)
            ident = ident.to(engine.device)
            dist.broadcast(ident, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
            raw = bytes(ident.cpu().tolist())
            NativeLoop._joined.add(key)
        with torch.cuda.device(engine.device):
            engine._check(self._lib.stbpe_mg_nccl_init(engine._h, raw, int(cap_per_peer)))
        self.rounds = 0
        self._counted = False

    def run(self, n_rounds: int):
        first = 0 if self._counted else 1
        with torch.cuda.device(self.e.device):
            self.e._check(self._lib.stbpe_mg_run(self.e._h, first, int(n_rounds), self.e._s))
        self._counted = True
        self.rounds += n_rounds

    def progress(self) -> Tuple[int, int]:
        self.e.repack()
        st = self.e.state()
        if st.device_error:
            self.e.count_error()
        return int(st.merges_done), int(st.stop_reason)

    def train(self, check_every: int = 256):
        if not self._counted:
            self.run(1)
        while True:
            done, reason = self.progress()
            if reason != L.RUNNING:
                return done, reason
            self.run(rounds_until_next_check(done, self.e.max_merges, check_every))


class PeerLoop:
    """Rounds whose exchange the kernels do themselves over NVLink peer memory
    (``stbpe_mg_peer_run``): every rank's mailbox is mapped by its peers through CUDA IPC, a round
    is six kernel launches and no collective, and batches of rounds replay as one CUDA graph.
    ``torch.distributed`` is used on the host only: once to hand round the IPC handles, and for a
    barrier before each batch so that the ranks start it together (a kernel waits at most two
    seconds for a peer).  One engine (one GPU) per process; never two ranks on one GPU."""

    def __init__(self, engine, cap_per_peer: int = 4096, group=None):
        import torch.distributed as dist
        self.dist, self.group = dist, group
        self.e = engine
        self._lib = L.load()
        world = engine.world_size
        if dist.get_world_size(group) != world or dist.get_rank(group) != engine.rank:
            raise ValueError("the engine's world size / rank differ from the process group's")
        buf = (ctypes.c_ubyte * 64)()
        with torch.cuda.device(engine.device):
            engine._check(self._lib.stbpe_mg_peer_export(engine._h, int(cap_per_peer), buf))
        mine = torch.tensor(list(buf), dtype=torch.uint8, device=engine.device)
        every = torch.empty(world * 64, dtype=torch.uint8, device=engine.device)
        dist.all_gather_into_tensor(every, mine, group=group)
        raw = bytes(every.cpu().tolist())
        with torch.cuda.device(engine.device):
            engine._check(self._lib.stbpe_mg_peer_open(engine._h, raw, world))
        self._open = True
        self.rounds = 0
        self._counted = False

    def run(self, n_rounds: int):
        first = 0 if self._counted else 1
        self.dist.barrier(group=self.group)
        with torch.cuda.device(self.e.device):
            self.e._check(self._lib.stbpe_mg_peer_run(self.e._h, first, int(n_rounds), self.e._s))
        self._counted = True
        self.rounds += n_rounds

    def progress(self) -> Tuple[int, int]:
        self.e.repack()
        st = self.e.state()
        if st.device_error:
            self.e.count_error()
        return int(st.merges_done), int(st.stop_reason)

    def train(self, check_every: int = 256):
        if not self._counted:
            self.run(1)
        while True:
            done, reason = self.progress()
            if reason != L.RUNNING:
                return done, reason
            self.run(rounds_until_next_check(done, self.e.max_merges, check_every))

    def close(self):
        """Unmap the peers' mailboxes and wait for every rank to have done so; only then may a
        rank destroy its engine (its mailbox must outlive the peers' mappings)."""
        if self._open:
            with torch.cuda.device(self.e.device):
                self.e._check(self._lib.stbpe_mg_peer_close(self.e._h))
            self.dist.barrier(group=self.group)
            self._open = False


# ----------------------------------------------------------------------------- bench (N > 1)
def run_bench_multi(args, wl, rank: int, local_rank: int, world: int) -> None:
    """``bench.py`` at N > 1: the same corpus as N = 1, rows sharded over the ranks (strong
    scaling), one process per GPU over NCCL.  Rank 0 prints the JSON line."""
    import json
    import sys
    import time

    import torch.distributed as dist

    from . import synth
    from .engine import Engine

    gen, n_bytes, seed, merges, desc = wl
    K, W = args.steps, args.warmup
    dev = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=dev)
    t_start = time.perf_counter()

    def phase(name: str) -> None:     # STBPE_BENCH_VERBOSE=1: wall-clock marks on stderr (rank 0)
        if rank == 0 and os.environ.get("STBPE_BENCH_VERBOSE"):
            print(f"[bench {time.perf_counter() - t_start:7.1f} s] {name}", file=sys.stderr, flush=True)

    if args.workload == "c3":
        run_count_bench_multi(args, wl, rank, local_rank, world)
        dist.barrier()
        dist.destroy_process_group()
        return
    corpus = getattr(synth, gen)(n_bytes=n_bytes, seed=seed, device=str(dev))
    off = corpus.row_offsets.cpu().numpy()
    lo, hi = shard_rows(off, world)[rank]
    shard = corpus.data[off[lo]:off[hi]].clone()
    shard_off = off[lo:hi + 1] - off[lo]
    del corpus
    torch.cuda.empty_cache()
    n_local = int(shard.numel())
    phase("corpus generated and sharded")

    # round driver: kernels over peer memory (default), the native NCCL loop, or Python rounds
    driver = os.environ.get("STBPE_MG_DRIVER", "peer")
    if os.environ.get("STBPE_MG_PYTHON_ROUNDS"):
        driver = "python"
    native = driver != "python"
    launches_per_round = {"peer": 6, "nccl": 7, "python": 7}[driver]

    def make(max_merges):
        e = Engine(max(n_local, 1), base_vocab=256, max_merges=max(max_merges, 1), device=dev,
                   world_size=world, rank=rank)
        if driver == "peer":
            return e, PeerLoop(e, cap_per_peer=4096)
        if driver == "nccl":
            return e, NativeLoop(e, cap_per_peer=4096)
        return e, ShardedBPE([EngineWorker(e, cap_per_peer=4096)], TorchDistComm())

    def finish(e, loop):
        if hasattr(loop, "close"):
            loop.close()
        e.close()

    def ev():
        x = torch.cuda.Event(enable_timing=True)
        x.record()
        return x

    def synced_max(ms: float) -> float:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # warm-up on a throw-away engine
    e, loop = make(W)
    e.append_bytes(shard, shard_off)
    loop.train(check_every=8)
    finish(e, loop)
    del e, loop
    phase("warm-up done")

    e, loop = make(K)
    e.append_bytes(shard, shard_off)
    torch.cuda.synchronize()
    dist.barrier()
    sampler = None
    if rank == 0:
        from bench import ClockSampler  # type: ignore
        sampler = ClockSampler(local_rank)
        sampler.start()
    t0 = ev()
    if native:                      # initial histogram + exchange + first decision
        loop.run(1)
    else:
        loop._round(True)
        loop._counted = True
    t1 = ev()
    done, stop = loop.train(check_every=256)
    t2 = ev()
    torch.cuda.synchronize()
    clocks = sampler.stop() if sampler is not None else None
    dist.barrier()
    phase(f"timed run done ({done} merges, {loop.rounds} rounds)")
    count_ms = synced_max(t0.elapsed_time(t1))
    loop_ms = synced_max(t1.elapsed_time(t2))
    merges_gpu, counts_gpu, live_before = e.merges(0, done)
    live_all = torch.tensor(live_before.astype(np.float64).sum(), dtype=torch.float64, device=dev)
    dist.all_reduce(live_all)
    tokens_all = torch.tensor([float(n_local)], dtype=torch.float64, device=dev)
    dist.all_reduce(tokens_all)
    rounds = loop.rounds
    finish(e, loop)
    del e, loop

    # end to end from pinned host memory through the same public pieces
    host = torch.empty(n_local, dtype=torch.uint8, pin_memory=True)
    host.copy_(shard)
    torch.cuda.synchronize()
    del shard
    dist.barrier()
    t = time.perf_counter()
    e, loop2 = make(K)
    e.append_bytes(host, shard_off)
    done2, _ = loop2.train(check_every=256)
    m2, _, _ = e.merges(0, done2)
    torch.cuda.synchronize()
    e2e_s = synced_max((time.perf_counter() - t) * 1000.0) / 1000.0
    assert m2 == merges_gpu, "merge list changed between two runs on the same input"
    finish(e, loop2)
    phase("end-to-end run done")

    if rank == 0:
        from bench import merges_sha256, peaks  # type: ignore
        peak, peak_kind = peaks()
        algo = 4.0 * float(live_all.item())
        line = {
            "metric": "bpe_merges_per_sec", "value": done / (loop_ms / 1e3), "unit": "merges/s",
            "n_gpus": world, "steps": done, "warmup": W, "ms_per_step": loop_ms / max(done, 1),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int32",
            "data": "synthetic",
            "config": {"workload": desc, "name": args.workload, "corpus_bytes": int(tokens_all.item()),
                       "rows": len(off) - 1, "merges_timed": done, "first_merge": 0, "stop_reason": int(stop),
                       "merges_sha256": merges_sha256(merges_gpu, counts_gpu),
                       "sharding": "contiguous document ranges by bytes; pair keys by hash owner",
                       "rounds": rounds, "chunk_entries": 4096,
                       "round_driver": {"peer": "kernels over NVLink peer memory, CUDA graph of 16 rounds (stbpe_mg_peer_run)",
                                        "nccl": "native NCCL loop (stbpe_mg_run)",
                                        "python": "python rounds over torch.distributed"}[driver],
                       "l2": "inputs larger than L2 (4 bytes x tokens per merge)", "tile_tokens": 1024},
            "pair_count": {"ms": count_ms, "gbs": 4.0 * float(tokens_all.item()) / (count_ms / 1e3) / 1e9,
                           "note": "local histogram + all-to-all + owner insert + first decision"},
            "roofline": {"bound": "hbm", "kernel": "merge round (all kernels and the exchange)",
                         "achieved": algo / (loop_ms / 1e3) / 1e9, "peak": peak * world, "peak_kind": peak_kind,
                         "unit": "GB/s", "frac": algo / (loop_ms / 1e3) / 1e9 / (peak * world),
                         "algorithmic_bytes": algo, "traffic": None},
            "e2e": {"value": done2 / e2e_s, "unit": "merges/s", "seconds": e2e_s,
                    "h2d_bytes_per_step": float(tokens_all.item()) / max(done2, 1), "d2h_bytes_per_step": 24.0},
            "gpu_launches": rounds * launches_per_round,
            "clocks": clocks, "cpu_baseline": None,
        }
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()


def run_count_bench_multi(args, wl, rank: int, local_rank: int, world: int) -> None:
    """``bench.py --workload c3`` at N > 1: the id stream sharded by rows over the ranks, one histogram
    pass per step.  A step = first pass on every rank, second pass on the owners over peer memory, and
    the count round that selects the best pair (timed together with CUDA events, maximum over ranks)."""
    import json
    import time

    import torch.distributed as dist

    from . import synth
    from .engine import Engine

    gen, n_tokens, seed, _, desc = wl
    K, W = args.steps, max(args.warmup, 1)
    dev = torch.device("cuda", local_rank)
    ids, off = synth.config3_ids(n_tokens, seed=seed, device=str(dev))
    off = off.cpu().numpy()
    lo, hi = shard_rows(off, world)[rank]
    local = ids[off[lo]:off[hi]].clone()
    local_off = off[lo:hi + 1] - off[lo]
    del ids
    torch.cuda.empty_cache()
    n_local = int(local.numel())
    slots = 1 << max(20, int(np.ceil(np.log2(max(n_tokens // 4 // world, 1)))))
    e = Engine(max(n_local, 1), base_vocab=65536, max_merges=1, device=dev, table_slots=slots,
               world_size=world, rank=rank)
    loop = PeerLoop(e, cap_per_peer=4096)

    def synced_max(x: float) -> float:
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def step(src):
        e.reset()
        e.append_ids(src, local_off)
        torch.cuda.synchronize()
        dist.barrier()
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        t = time.perf_counter()
        a.record()
        good = wide_count(e)
        loop._counted = False
        loop.run(1)
        b.record()
        torch.cuda.synchronize()
        return good, a.elapsed_time(b), time.perf_counter() - t

    ms, used = [], True
    for it in range(W + K):
        good, dev_ms, _ = step(local)
        used = used and good
        if it >= W:
            ms.append(synced_max(dev_ms))
    st = e.state()
    keys = torch.tensor([float(st.table_keys)], dtype=torch.float64, device=dev)
    dist.all_reduce(keys)
    best, counts, _ = e.merges(0, 1)
    kernel_ms = synced_max(float(st.count_kernel_ms))
    # end to end from pinned host ids
    host = torch.empty(n_local, dtype=torch.int32, pin_memory=True)
    host.copy_(local)
    del local
    torch.cuda.empty_cache()
    e.reset()
    dist.barrier()
    t = time.perf_counter()
    e.append_ids(host, local_off)
    wide_count(e)
    loop._counted = False
    loop.run(1)
    torch.cuda.synchronize()
    e2e_s = synced_max(time.perf_counter() - t)
    wide_close(e)
    loop.close()
    e.close()
    if rank == 0:
        from bench import peaks  # type: ignore
        peak, peak_kind = peaks()
        med = float(np.median(ms))
        gbs = 4.0 * n_tokens / (med / 1e3) / 1e9
        print(json.dumps({
            "metric": "pair_count_gbs", "value": gbs, "unit": "GB/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": med, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int32", "data": "synthetic",
            "config": {"workload": desc, "name": "c3", "tokens": n_tokens, "rows": len(off) - 1,
                       "distinct_pairs": int(keys.item()),
                       "best_pair": [int(best[0][0]), int(best[0][1]), int(counts[0])] if best else None,
                       "partitioned_path": bool(used), "l2": "inputs larger than L2", "bytes_per_token": 4,
                       "sharding": "contiguous row ranges by tokens; partitions (and keys) owned by partition % ranks"},
            "roofline": {"bound": "hbm", "kernel": "both passes of the partitioned count + the count round "
                                                   "(host barrier between the passes included)",
                         "achieved": gbs, "peak": peak * world, "peak_kind": peak_kind, "unit": "GB/s",
                         "frac": gbs / (peak * world), "kernels_only_ms": kernel_ms, "traffic": None},
            "e2e": {"value": 4.0 * n_tokens / e2e_s / 1e9, "unit": "GB/s", "seconds": e2e_s,
                    "h2d_bytes_per_step": 4.0 * n_tokens, "d2h_bytes_per_step": 24.0},
            "gpu_launches": (3 + 6) * K,   # first pass, hot pairs, second pass; the six launches of the count round
             "clocks": None, "cpu_baseline": None}), flush=True)
