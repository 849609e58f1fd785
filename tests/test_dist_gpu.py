"""Multi-rank engine kernels (rank-local delta table, per-owner outbox, inbox apply, candidate,
commit) against the single-process oracle.  With one GPU the ranks are emulated as several engines
of one process whose kernels run one after the other (LocalComm copies the chunks); with two or
more GPUs the same loop runs as one process per GPU: over NCCL (Python rounds and the native loop)
and with the exchange done by the kernels over NVLink peer memory.  The peer-memory kernels wait for
one another and therefore never run with two ranks on one GPU."""
import os
import socket

import numpy as np
import pytest
import torch

from oracle import oracle as O
from supertoken_b200 import _lib as L
from supertoken_b200 import synth
from supertoken_b200.dist import EngineWorker, LocalComm, ShardedBPE, TorchDistComm, shard_rows
from supertoken_b200.engine import Engine
from tests.helpers import corpus_rows

pytestmark = pytest.mark.gpu


def _make_worker(data, off, lo, hi, rank, world, target, cap, device="cuda"):
    n = int(off[hi] - off[lo])
    e = Engine(max(n, 1), base_vocab=256, max_merges=target, device=device, table_slots=1 << 18,
               world_size=world, rank=rank)
    if n:
        e.append_bytes(data[off[lo]:off[hi]], off[lo:hi + 1] - off[lo])
    return EngineWorker(e, cap_per_peer=cap)


@pytest.mark.parametrize("world,cap", [(2, 8192), (3, 40), (4, 500)])
def test_emulated_ranks_on_one_gpu_match_oracle(world, cap):
    c = synth.config5_adversarial(1 << 20, seed=11)
    rows = corpus_rows(c)
    off = np.asarray(c.row_offsets)
    target = 60
    om, oc, _ = O.train_flat(*O.flatten_rows(rows), 256, target, 1)
    workers = [_make_worker(c.data, off, lo, hi, r, world, target, cap)
               for r, (lo, hi) in enumerate(shard_rows(off, world))]
    loop = ShardedBPE(workers, LocalComm())
    done, stop = loop.train(check_every=16)
    assert done == target and stop == L.STOP_TARGET
    for w in workers:
        m, cnt, _ = w.merges()
        assert m == om and cnt.tolist() == oc
    if cap < 100:
        assert loop.rounds > target + 1   # small chunks forced exchange-only rounds
    # the union of the owners' table slices is the histogram of the rewritten corpus
    ids, o2 = O.flatten_rows(rows)
    for i, (a, b) in enumerate(om):
        O.apply_merge_flat(ids, o2, a, b, 256 + i)
    ok, okc = O.count_pairs_flat(ids[:o2[-1]].copy(), o2, 1)
    got = {}
    for w in workers:
        k, cnt = w.e.export_histogram()
        for kk, cc in zip(k.cpu().numpy().astype(np.uint64).tolist(), cnt.cpu().tolist()):
            assert kk not in got
            got[kk] = cc
    assert got == dict(zip(ok.tolist(), okc.tolist()))
    for w in workers:
        w.e.close()


def test_emulated_ranks_repack_between_commit_and_apply():
    """A rank re-packs its sparse tiles when the host looks at the progress, i.e. after a merge has
    been committed and before the next round applies it: the worklist of that merge must be built
    on the re-packed layout."""
    world, target = 2, 80
    c = synth.config2_mixed(2 << 20, seed=3, lexicon=5000, mean_doc_bytes=2048)
    off = np.asarray(c.row_offsets)
    om, oc, _ = O.train_flat(*O.flatten_rows(corpus_rows(c)), 256, target, 1)
    workers = [_make_worker(c.data, off, lo, hi, r, world, target, 4096)
               for r, (lo, hi) in enumerate(shard_rows(off, world))]
    done, stop = ShardedBPE(workers, LocalComm()).train(check_every=8)
    assert done == target and stop == L.STOP_TARGET
    assert sum(w.e.state().repacks for w in workers) > 0
    for w in workers:
        m, cnt, _ = w.merges()
        assert m == om and cnt.tolist() == oc
        w.e.close()


def test_peer_wait_runs_out_when_the_other_rank_never_sends():
    # failure detection of the peer-memory rounds: rank 0 runs one round while rank 1 (an engine of
    # the same process that never launches anything) raises no flag.  The wait in rank 0's kernels
    # gives up after its two-second limit, the kernels that follow return at once, the host reads
    # the time-out status, and the CUDA context stays usable.
    import ctypes
    import time
    lib = L.load()
    data = np.frombuffer(b"abcabcabd" * 2000, dtype=np.uint8).copy()
    engines = []
    for r in range(2):
        e = Engine(len(data), base_vocab=256, max_merges=4, table_slots=1 << 16, world_size=2, rank=r)
        e.append_bytes(data, None)
        engines.append(e)
    boxes = (ctypes.c_void_p * 2)()
    for r, e in enumerate(engines):
        buf = (ctypes.c_ubyte * 64)()
        e._check(lib.stbpe_mg_peer_export(e._h, 256, buf))
        box = ctypes.c_void_p()
        e._check(lib.stbpe_mg_peer_mailbox(e._h, ctypes.byref(box)))
        boxes[r] = box.value
    e0 = engines[0]
    e0._check(lib.stbpe_mg_peer_set(e0._h, boxes, 2))
    t = time.perf_counter()
    e0._check(lib.stbpe_mg_peer_run(e0._h, 1, 2, e0._s))   # two rounds: the second must not wait again
    torch.cuda.synchronize()
    waited = time.perf_counter() - t
    assert 1.5 < waited < 6.0
    st = e0.state()
    assert st.device_error & 32
    with pytest.raises(RuntimeError, match="wait gave up"):
        e0.count_error()
    # the device still works: a fresh single-rank engine trains as usual
    e = Engine(len(data), base_vocab=256, max_merges=3, table_slots=1 << 16)
    e.append_bytes(data, None)
    e.count_initial()
    e.train(3)
    om, _, _ = O.train_flat(data.astype(np.int32), np.array([0, len(data)], dtype=np.int64), 256, 3, 1)
    assert e.merges()[0] == om
    e.close()
    for x in engines:
        x.close()


def _nccl_rank(rank, world, port, target, q, native=False):
    import datetime
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=90))
    try:
        c = synth.config2_mixed(2 << 20, seed=3, lexicon=5000, mean_doc_bytes=2048)
        off = np.asarray(c.row_offsets)
        lo, hi = shard_rows(off, world)[rank]
        if native:
            from supertoken_b200.dist import NativeLoop, PeerLoop
            n = int(off[hi] - off[lo])
            e = Engine(max(n, 1), base_vocab=256, max_merges=target, device=f"cuda:{rank}",
                       table_slots=1 << 18, world_size=world, rank=rank)
            e.append_bytes(c.data[off[lo]:off[hi]], off[lo:hi + 1] - off[lo])
            cls = PeerLoop if native == "peer" else NativeLoop
            loop = cls(e, cap_per_peer=64)                    # small chunks: extra rounds
            done, stop = loop.train(check_every=32)
            m, cnt, _ = e.merges()
            if native == "peer":
                assert loop.rounds > target + 1
                loop.close()
        else:
            w = _make_worker(c.data, off, lo, hi, rank, world, target, 4096, device=f"cuda:{rank}")
            done, stop = ShardedBPE([w], TorchDistComm()).train(check_every=32)
            m, cnt, _ = w.merges()
        q.put((rank, m, cnt.tolist(), done, stop))
    except Exception as exc:   # the parent ends the other rank instead of waiting for it
        q.put((rank, "error", repr(exc), 0, 0))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("native", [False, True, "peer"])
def test_ranks_on_separate_gpus_match_oracle(native, world):
    # one process per GPU over NCCL: python rounds over torch.distributed (False), the library's own
    # NCCL loop (True), and rounds whose exchange the kernels do over peer memory ("peer")
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    if native is False and world > 2:
        pytest.skip("the python round driver is covered at two ranks")
    import torch.multiprocessing as mp
    target = 80
    c = synth.config2_mixed(2 << 20, seed=3, lexicon=5000, mean_doc_bytes=2048)
    om, oc, _ = O.train_flat(*O.flatten_rows(corpus_rows(c)), 256, target, 1)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_nccl_rank, args=(r, world, port, target, q, native)) for r in range(world)]
    for p in procs:
        p.start()
    results = []
    for _ in range(world):
        results.append(q.get(timeout=240))
        if results[-1][1] == "error":
            break
    failed = [r for r in results if r[1] == "error"]
    for p in procs:
        p.join(timeout=5 if failed else 60)
        if p.is_alive():
            p.terminate()
    assert not failed, failed
    for rank, m, cnt, done, stop in results:
        assert m == om and cnt == oc and done == target and stop == L.STOP_TARGET


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_trainer_with_two_devices_in_one_process():
    # GPUBPETrainer(devices=(...)): the rows are split over the devices, one engine per device, the
    # exchange is a copy between the devices; merges equal the single-stream oracle
    from supertoken_b200 import GPUBPETrainer
    c = synth.config2_mixed(2 << 20, seed=5, lexicon=3000, mean_doc_bytes=1500)
    target = 70
    om, oc, _ = O.train_flat(*O.flatten_rows(corpus_rows(c)), 256, target, 1)
    tr = GPUBPETrainer(base_vocab=256, merges=target, devices=("cuda:0", "cuda:1"))
    res = tr.fit_bytes(np.asarray(c.data), np.asarray(c.row_offsets))
    assert res["merges"] == om and tr.merge_counts == oc and res["vocab_size"] == 256 + target
    # the padded-batch entry point takes the same route
    rows = corpus_rows(c)[:40]
    Lmax = max(len(r) for r in rows)
    tok = torch.full((len(rows), Lmax), -1, dtype=torch.int32)
    val = torch.zeros((len(rows), Lmax), dtype=torch.uint8)
    for i, r in enumerate(rows):
        tok[i, :len(r)] = torch.from_numpy(np.asarray(r, dtype=np.int32))
        val[i, :len(r)] = 1
    lens = torch.tensor([len(r) for r in rows], dtype=torch.int32)
    om2, _, _ = O.train_flat(*O.flatten_rows(rows), 256, 25, 1)
    tr2 = GPUBPETrainer(base_vocab=256, merges=25, devices=("cuda:0", "cuda:1"))
    assert tr2.fit([(tok[:20], val[:20], lens[:20]), (tok[20:], val[20:], lens[20:])], log_every=0)["merges"] == om2


def _trainer_rank(rank, world, port, target, q):
    import datetime
    import torch.distributed as dist
    from supertoken_b200 import GPUBPETrainer
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), LOCAL_WORLD_SIZE=str(world))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=90))
    try:
        c = synth.config2_mixed(2 << 20, seed=5, lexicon=3000, mean_doc_bytes=1500)
        off = np.asarray(c.row_offsets)
        lo, hi = shard_rows(off, world)[rank]
        tr = GPUBPETrainer(base_vocab=256, merges=target, device=f"cuda:{rank}")
        res = tr.fit_bytes(np.asarray(c.data)[off[lo]:off[hi]], off[lo:hi + 1] - off[lo])
        q.put((rank, res["merges"], tr.merge_counts, res["vocab_size"], 0))
    except Exception as exc:
        q.put((rank, "error", repr(exc), 0, 0))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_trainer_in_a_process_group_of_two_ranks():
    # one process per GPU, process group initialised by the caller: every rank passes its own rows
    # to the unchanged trainer call and all ranks return the merges of the whole corpus
    import torch.multiprocessing as mp
    world, target = 2, 70
    c = synth.config2_mixed(2 << 20, seed=5, lexicon=3000, mean_doc_bytes=1500)
    om, oc, _ = O.train_flat(*O.flatten_rows(corpus_rows(c)), 256, target, 1)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_trainer_rank, args=(r, world, port, target, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = []
    for _ in range(world):
        results.append(q.get(timeout=240))
        if results[-1][1] == "error":
            break
    failed = [r for r in results if r[1] == "error"]
    for p in procs:
        p.join(timeout=5 if failed else 60)
        if p.is_alive():
            p.terminate()
    assert not failed, failed
    for rank, m, cnt, vocab, _ in results:
        assert m == om and cnt == oc and vocab == 256 + target


def _wide_rank(rank, world, port, q):
    import datetime
    import torch.distributed as dist
    from supertoken_b200.dist import PeerLoop, wide_close, wide_count
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), STBPE_DENSE32_MIN_TOKENS="1")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=90))
    try:
        ids, off = synth.config3_ids(1 << 21, seed=2)
        lo, hi = shard_rows(off, world)[rank]
        e = Engine(int(off[hi] - off[lo]), base_vocab=65536, max_merges=3, device=f"cuda:{rank}",
                   table_slots=1 << 22, world_size=world, rank=rank)
        e.append_ids(np.ascontiguousarray(ids[off[lo]:off[hi]]), off[lo:hi + 1] - off[lo])
        loop = PeerLoop(e, cap_per_peer=4096)
        assert wide_count(e)                       # both passes ran: the table holds this rank's keys
        k, c = e.export_histogram(cap=1 << 22)
        done, stop = loop.train(check_every=8)
        m, cnt, _ = e.merges()
        wide_close(e)
        loop.close()
        q.put((rank, k.cpu().numpy().astype(np.uint64), c.cpu().numpy(), m, cnt.tolist(), done, stop))
    except Exception as exc:
        q.put((rank, "error", repr(exc), 0, 0, 0, 0))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_first_count_of_a_16_bit_vocabulary_over_ranks(world):
    # every rank partitions the pairs of its rows, the owner of a partition counts it out of all
    # ranks' buffers over peer memory: the union of the ranks' tables is the histogram of the whole
    # stream, every key on the rank that owns it, and the merges that follow are the oracle's
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    from supertoken_b200.dist import owner_of
    ids, off = synth.config3_ids(1 << 21, seed=2)
    ok, oc = O.count_pairs_flat(ids, off, 1)
    om, ocnt, _ = O.train_flat(ids, off, 65536, 3, 1)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_wide_rank, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = []
    try:
        for _ in range(world):
            results.append(q.get(timeout=240))
            if isinstance(results[-1][1], str):
                break
    finally:
        failed = [r for r in results if isinstance(r[1], str)] or len(results) < world
        for p in procs:
            p.join(timeout=5 if failed else 60)
            if p.is_alive():
                p.terminate()
    assert not failed, failed
    keys = np.concatenate([r[1] for r in results])
    counts = np.concatenate([r[2] for r in results])
    order = np.argsort(keys, kind="stable")
    assert np.array_equal(keys[order], ok) and np.array_equal(counts[order], oc)
    for rank, k, _, m, cnt, done, stop in results:
        assert all(owner_of(int(x), world) == rank for x in k[:2000])
        assert m == om and cnt == ocnt and done == 3 and stop == L.STOP_TARGET
