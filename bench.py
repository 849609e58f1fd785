#!/usr/bin/env python
"""Benchmark of the BPE merge loop on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload c2|c1|c5|c3]

One *step* is one merge of the loop (select best pair, rewrite the stream, update the pair
histogram by deltas).  The workload at N=1 is the 1 GiB mixed-script corpus with a 32 000-merge
target (seeded synthetic stand-in, generated on the device); ``--steps K`` times the first K
merges of that job, the default K is the whole job.  Warm-up merges run first and the engine is
then reloaded from the device-resident bytes, so the timed merges start from merge 0
(``--first-merge M``: from merge M, after M untimed merges, to look at the late phase of a job).

Printed JSON (one line, rank 0):
  value      merges/s with the corpus already packed in HBM (device time, CUDA events)
  e2e        merges/s through ``GPUBPETrainer.fit_bytes`` from pinned host bytes: H2D copy, pack,
             initial histogram, K merges, merge list back to the host
  pair_count GB/s of the initial histogram pass at 4 bytes per token
  roofline   merge kernel: 4 bytes x live tokens per launch / its average device time
  cpu_baseline  the CPU oracle (C restatement of the reference's recount loop) on a bounded sample

``--impl reference`` times that CPU restatement on the host cores instead (the reference is a
Python package whose source tree is not present on the benchmark machine).
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import struct
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (generator, bytes, seed, merges, description)
    "c2": ("config2_mixed", 1 << 30, 1, 32000, "1 GiB mixed ASCII/Cyrillic/CJK Zipf(1.1) text, docs ~4 KiB, 32000 merges"),
    "c1": ("config1_text", 16 << 20, 0, 1000, "16 MiB lowercase Zipf(1.07) text, 16 rows of 1 MiB, 1000 merges"),
    "c5": ("config5_adversarial", 512 << 20, 4, 8000, "512 MiB runs/text/random bytes, 8000 merges"),
    "c4": ("config2_mixed", 8 << 30, 3, 50000, "8 GiB mixed text (as c2), 50000 merges"),
    # count-only microbenchmark: a step is one full histogram pass (N = 1 only); "bytes" = tokens here
    "c3": ("config3_ids", 1 << 31, 2, 5, "2^31 int32 ids Zipf(1.1) over 65 536, rows ~2048 tokens, one histogram pass per step"),
}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "200"], stdout=fd, stderr=subprocess.DEVNULL)
            os.close(fd)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        try:
            sm, reasons = [], set()
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                sm.append(float(f[1]))
                out["sm_max_mhz"] = float(f[2])
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            if sm:
                out["sm_mhz"] = float(np.median(sm))
                out["samples"] = len(sm)
            out["reasons"] = sorted(reasons)
            os.unlink(self.path)
        except Exception:
            pass
        return out


def merges_sha256(merges, counts) -> str:
    """SHA-256 over the ordered (a, b, count) triples of a merge list (little-endian int32, int32,
    int64): equal hashes at every N mean every GPU count learned the same merges with the same counts."""
    h = hashlib.sha256()
    for (a, b), c in zip(merges, counts):
        h.update(struct.pack("<iiq", int(a), int(b), int(c)))
    return h.hexdigest()


def rank_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


# ----------------------------------------------------------------------------- CPU arm
def cpu_sample(corpus_np: np.ndarray, offsets_np: np.ndarray, n_bytes: int):
    """First rows of the corpus up to n_bytes (rows are never split)."""
    k = int(np.searchsorted(offsets_np, n_bytes, side="right")) - 1
    k = max(k, 1)
    end = int(offsets_np[k])
    return corpus_np[:end].astype(np.int32), offsets_np[:k + 1].astype(np.int64)


def time_oracle(ids: np.ndarray, off: np.ndarray, steps: int, warmup: int):
    """Seconds for exactly `steps` merges of the oracle's recount loop, started from merge 0 of a fresh
    copy of the stream after `warmup` untimed merges on another copy (the GPU arm does the same: it
    warms up, reloads the corpus and times the first merges).  The stream is restarted when a stop rule
    fires before `steps`.  Returns (seconds, threads, merges of the first timed pass, their counts).
    The thread count is set here to the cores this process may use (torch.distributed.run exports
    OMP_NUM_THREADS=1 to its children)."""
    from oracle import oracle as O
    O.lib()
    cores = O.set_threads()
    if warmup:
        O.train_flat(ids.copy(), off.copy(), 256, warmup, 1, copy=False)
    done, total = 0, 0.0
    first_merges, first_counts = None, None
    while done < steps:
        cur_ids, cur_off = ids.copy(), off.copy()
        t = time.perf_counter()
        m, c, reason = O.train_flat(cur_ids, cur_off, 256, steps - done, 1, copy=False)
        total += time.perf_counter() - t
        if not m:
            raise RuntimeError("oracle sample too small to learn a merge")
        if first_merges is None:
            first_merges, first_counts = list(m), list(c)
        done += len(m)
    return total, cores, first_merges, first_counts


def make_corpus(gen: str, n_bytes: int, seed: int):
    """The workload's bytes and row offsets as numpy arrays (generated on a GPU when there is one:
    the generators give the same bytes on either backend, the GPU is just faster)."""
    from supertoken_b200 import synth
    try:
        import torch
        if torch.cuda.is_available():
            c = getattr(synth, gen)(n_bytes=n_bytes, seed=seed, device="cuda:0")
            data, off = c.data.cpu().numpy(), c.row_offsets.cpu().numpy()
            del c
            torch.cuda.empty_cache()
            return data, off
    except ImportError:
        pass
    c = getattr(synth, gen)(n_bytes=n_bytes, seed=seed)
    return np.asarray(c.data), np.asarray(c.row_offsets)


def run_reference_arm(args, wl):
    """The reference's algorithm (full recount per merge, as gpu_tokenizer/bpe_trainer.py:4193-4517
    does in recount mode) restated in C and run on the host cores, on a bounded sample."""
    rank, _, world = rank_env()
    if rank != 0:
        return
    from supertoken_b200 import synth
    gen, n_bytes, seed, merges, desc = wl
    if args.workload == "c3":
        from oracle import oracle as O
        O.set_threads()
        n = min(1 << 25, n_bytes)
        ids, off = synth.config3_ids(n, seed=seed)
        ids, off = np.asarray(ids), np.asarray(off)
        ts = []
        for it in range(args.warmup + args.steps):
            t = time.perf_counter()
            O.count_pairs_flat(ids, off, 1)
            if it >= args.warmup:
                ts.append(time.perf_counter() - t)
        med = float(np.median(ts))
        gbs = 4.0 * n / med / 1e9
        print(json.dumps({
            "impl": "reference", "metric": "pair_count_gbs", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": med * 1e3 * (n_bytes / n),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int32", "data": "synthetic",
            "config": {"workload": desc, "name": "c3"},
            "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": O.num_threads(), "kind": "port",
                             "sample": f"first {n} ids; threaded hash recount + sort by key"},
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}), flush=True)
        return
    # The whole workload when W + K merges of it fit the time a bench run may take on this
    # machine's cores; otherwise a prefix of the corpus, with the rate scaled to the full size.
    budget_s = 150.0
    probe = getattr(synth, gen)(n_bytes=1 << 20, seed=seed)
    ids, off = cpu_sample(np.asarray(probe.data), np.asarray(probe.row_offsets), 1 << 20)
    t, cores, _, _ = time_oracle(ids, off, 3, 0)
    early = t / 3 / len(ids)                      # seconds per token and merge, first merges
    n_steps = args.steps + args.warmup
    whole = n_bytes <= (2 << 30) and n_steps <= 64 and 1.5 * early * n_bytes * n_steps <= budget_s
    if whole:
        data, off_all = make_corpus(gen, n_bytes, seed)
        ids, off = data.astype(np.int32), off_all.astype(np.int64)
        del data
        sample = f"the whole corpus ({len(ids)} bytes), merges 0..{args.steps - 1} after {args.warmup} warm-up merges"
    else:
        # the recount costs up to 8x more per token late in a run (distinct pairs of the order of the
        # tokens) than on the first merges, so a long run is sized for the late regime
        rate = max(early, 2.0e-8) if n_steps > 64 else 1.5 * early
        sample_bytes = int(min(max(budget_s / n_steps / rate, 64 << 10), 256 << 20, n_bytes))
        c = getattr(synth, gen)(n_bytes=sample_bytes, seed=seed)
        ids, off = cpu_sample(np.asarray(c.data), np.asarray(c.row_offsets), sample_bytes)
        sample = (f"first {len(ids)} bytes of the corpus, {args.steps} merges; rate scaled by "
                  f"{len(ids) / float(n_bytes):.5f} to the full corpus (a recount is linear in tokens)")
    t, cores, m, c = time_oracle(ids, off, args.steps, args.warmup)
    scale = len(ids) / float(n_bytes)
    value = args.steps / t * scale
    line = {
        "impl": "reference", "metric": "bpe_merges_per_sec", "value": value, "unit": "merges/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1000.0 * t / args.steps / scale, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int32", "data": "synthetic",
        "config": {"workload": desc, "name": args.workload, "merges_timed": args.steps,
                   "same_workload": bool(whole), "measured_seconds": t,
                   "merges_sha256": merges_sha256(m[:args.steps], c[:args.steps]) if whole else None},
        "cpu_baseline": {"value": value, "unit": "merges/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "merges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- count-only workload
def run_count_bench(args, wl, dev):
    print(json.dumps(count_bench(wl, dev, args.steps, max(args.warmup, 1))), flush=True)


def count_bench(wl, dev, K, W, with_e2e=True):
    """Initial pair-count microbenchmark on an id stream (16-bit vocabulary): every step loads the
    resident ids again (pack, untimed) and runs one full histogram pass.  `value` is GB/s at 4 bytes
    per token over the device time of all kernels of the count, from the first read of the stream
    until the pair table holds the histogram; the share of the second pass is reported beside it."""
    import torch
    from supertoken_b200 import synth
    from supertoken_b200.engine import Engine
    gen, n_tokens, seed, _, desc = wl
    ids, off = synth.config3_ids(n_tokens, seed=seed, device=str(dev))
    torch.cuda.synchronize()
    off_np = off.cpu().numpy()
    slots = 1 << max(20, int(np.ceil(np.log2(max(n_tokens // 4, 1)))))
    eng = Engine(n_tokens, base_vocab=65536, max_merges=1, device=dev, table_slots=slots)
    sampler = ClockSampler(dev.index)
    ms, conv, call = [], [], []
    for it in range(W + K):
        eng.reset()
        eng.append_ids(ids, off_np)
        torch.cuda.synchronize()
        if it == W:
            sampler.start()
        t = time.perf_counter()
        eng.count_initial()
        torch.cuda.synchronize()
        if it >= W:
            st = eng.state()
            call.append((time.perf_counter() - t) * 1e3)
            ms.append(float(st.count_kernel_ms))
            conv.append(float(st.count_convert_ms))
    clocks = sampler.stop()
    st = eng.state()
    key, count, ties = eng.select_best(True)
    # size-independent check of the whole histogram: every pair position is counted exactly once
    # (tokens minus non-empty rows), and the exported keys are strictly ascending (no key twice)
    hk, hc = eng.export_histogram()
    n_pairs = n_tokens - int(np.count_nonzero(np.diff(off_np)))
    sum_ok = bool(int(hc.sum().item()) == n_pairs and hk.numel() == st.table_keys
                  and bool((hk[1:] > hk[:-1]).all().item()))
    del hk, hc
    torch.cuda.empty_cache()
    peak, peak_kind = peaks()
    med = float(np.median(ms))
    gbs = 4.0 * n_tokens / (med / 1e3) / 1e9
    # end to end: pinned host ids -> device -> pack -> histogram -> best pair back on the host
    e2e_s = None
    if with_e2e:
        host = torch.empty(n_tokens, dtype=torch.int32, pin_memory=True)
        host.copy_(ids)
        del ids
        torch.cuda.empty_cache()
        torch.cuda.synchronize()
        t = time.perf_counter()
        eng.reset()
        eng.append_ids(host, off_np)
        eng.count_initial()
        k2, c2, _ = eng.select_best(False)
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t
        assert (k2, c2) == (key, count)
        del host
    eng.close()
    line = {
        "metric": "pair_count_gbs", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": med, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int32", "data": "synthetic",
        "config": {"workload": desc, "name": "c3", "tokens": n_tokens, "rows": len(off_np) - 1,
                   "distinct_pairs": int(st.table_keys), "best_pair": [int(key >> 32), int(key & 0xFFFFFFFF), int(count)],
                   "sum_of_counts_equals_pair_positions": sum_ok,
                   "l2": "inputs larger than L2", "bytes_per_token": 4},
        "roofline": {"bound": "hbm",
                     "kernel": ("partition_pairs_kernel + partition_table_kernel (all 256 partitions in one launch): both passes, until the "
                                "pair table is complete") if conv and conv[0] > 0 else "count_kernel",
                     "achieved": gbs, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": gbs / peak,
                     "frac_of_8tbs": gbs / 8000.0, "kernel_ms": med, "second_pass_ms": float(np.median(conv)),
                     "call_ms": float(np.median(call)), "traffic": None},
        "e2e": None if e2e_s is None else {"value": 4.0 * n_tokens / e2e_s / 1e9, "unit": "GB/s", "seconds": e2e_s,
                                           "h2d_bytes_per_step": 4.0 * n_tokens + off_np.nbytes,
                                           "d2h_bytes_per_step": 24.0},
        "gpu_launches": 3 * K, "clocks": clocks, "cpu_baseline": None,   # first pass, hot pairs, second pass
    }
    return line


# ----------------------------------------------------------------------------- GPU arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--bytes", type=int, default=None, help="override the corpus size (debugging)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-c3", action="store_true", help="skip the config-3 pair-count block of the default run")
    ap.add_argument("--first-merge", type=int, default=0,
                    help="single GPU: run this many merges untimed after the count and time the --steps merges that "
                         "follow (the late phase of a job); the end-to-end figure then covers all of them")
    args = ap.parse_args()
    wl = list(WORKLOADS[args.workload])
    if args.bytes:
        wl[1] = args.bytes
    gen, n_bytes, seed, merges, desc = wl
    if args.steps is None:
        args.steps = merges
    args.warmup = max(args.warmup, 0)
    if args.impl == "reference":
        run_reference_arm(args, wl)
        return

    import torch
    rank, local_rank, world = rank_env()
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback for the product path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        from supertoken_b200.dist import run_bench_multi
        run_bench_multi(args, wl, rank, local_rank, world)
        return

    from supertoken_b200 import GPUBPETrainer, synth
    from supertoken_b200.engine import Engine

    if args.workload == "c3":
        run_count_bench(args, wl, dev)
        return

    K, W, M = args.steps, args.warmup, max(args.first_merge, 0)
    if M:
        args.no_cpu_baseline = True   # the oracle would have to run the untimed merges first
    corpus = getattr(synth, gen)(n_bytes=n_bytes, seed=seed, device=str(dev))
    torch.cuda.synchronize()
    data_dev, off_np = corpus.data, corpus.row_offsets.cpu().numpy()
    n_tokens = int(data_dev.numel())

    def ev():
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return e

    eng = Engine(n_tokens, base_vocab=256, max_merges=max(M + K, W, 1), device=dev)

    def load():
        eng.reset()
        eng.append_bytes(data_dev, off_np)

    # warm-up: pack, count, W merges, then start over from the resident bytes
    load()
    eng.count_initial()
    eng.train(W)
    torch.cuda.synchronize()

    # timed: initial histogram (reported on its own) and K merges
    load()
    sampler = ClockSampler(local_rank)
    sampler.start()
    t0 = ev()
    eng.count_initial()
    tc = ev()
    if M:
        eng.train(M)
    t1 = ev()
    eng.train(K)
    t2 = ev()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    count_call_ms = t0.elapsed_time(tc)
    loop_ms = t1.elapsed_time(t2)
    st = eng.state()
    count_ms = float(st.count_kernel_ms)   # histogram kernel(s) only; the call also clears the table,
    # builds the tile records, the pair filter and the block maxima
    done = st.merges_done - M
    merges_gpu, counts_gpu, live_before = eng.merges(M, done)
    if done < 1:
        raise SystemExit("no merge was learned")
    value = done / (loop_ms / 1000.0)

    # per-kernel device time of the same K merges (events around every launch)
    load()
    eng.count_initial()
    if M:
        eng.train(M)
    st_b = eng.state()
    sel_ms, mrg_ms, ref_ms, repack_ms = eng.train_timed(K)
    torch.cuda.synchronize()
    st_t = eng.state()
    # what the merge kernel's bulk copies moved during the timed merges
    tile_bytes = float(st_t.tile_bytes_in + st_t.tile_bytes_out) - float(st_b.tile_bytes_in + st_b.tile_bytes_out)
    merges_again, _, _ = eng.merges(M, eng.state().merges_done - M)
    assert merges_again == merges_gpu, "merge list changed between two runs on the same input"
    algo_bytes = 4.0 * float(live_before.sum())
    peak, peak_kind = peaks()
    achieved = algo_bytes / (mrg_ms / 1000.0) / 1e9
    eng.close()
    del eng

    # end to end through the public API from pinned host memory
    host = torch.empty(n_tokens, dtype=torch.uint8, pin_memory=True)
    host.copy_(data_dev)
    torch.cuda.synchronize()
    del data_dev, corpus
    torch.cuda.empty_cache()
    t = time.perf_counter()
    trainer = GPUBPETrainer(base_vocab=256, merges=M + K, device=str(dev))
    res = trainer.fit_bytes(host, off_np, log_every=0)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t
    learned = trainer.merge_counts
    assert res["merges"][M:len(learned)] == merges_gpu[:max(len(learned) - M, 0)]
    e2e = len(learned) / e2e_s

    cpu = None
    oracle_ok, oracle_n = None, 0
    if not args.no_cpu_baseline:
        # The oracle on this machine's cores: the first merges of the WHOLE corpus when a few of them
        # fit about 25 s (then the same run also checks the GPU's merges and counts against the oracle),
        # else a prefix of the corpus with the rate scaled by its share of the tokens.
        ids, off = cpu_sample(host.numpy(), off_np, min(32 << 20, n_bytes))
        t_probe, cores, _, _ = time_oracle(ids, off, 3, 0)
        per_merge_full = t_probe / 3 / len(ids) * n_tokens * 1.3
        if n_tokens <= (2 << 30) and 2 * per_merge_full <= 60.0:
            n_cpu = int(min(max(25.0 / per_merge_full, 2), 8, len(learned)))
            ids, off = host.numpy().astype(np.int32), off_np.astype(np.int64)
            t_cpu, cores, om, oc = time_oracle(ids, off, n_cpu, 0)
            oracle_n = min(len(om), len(merges_gpu))
            oracle_ok = bool(om[:oracle_n] == merges_gpu[:oracle_n] and
                             list(oc[:oracle_n]) == [int(x) for x in counts_gpu[:oracle_n]])
            cpu = {"value": n_cpu / t_cpu, "unit": "merges/s", "cores": cores, "kind": "port",
                   "sample": f"the whole corpus ({n_tokens} bytes), merges 0..{n_cpu - 1}, {t_cpu:.1f} s, not scaled"}
        else:
            n_cpu = 12
            t_cpu, cores, _, _ = time_oracle(ids, off, n_cpu, 0)
            scale = len(ids) / float(n_tokens)
            cpu = {"value": n_cpu / t_cpu * scale, "unit": "merges/s", "cores": cores, "kind": "port",
                   "sample": f"first {len(ids)} bytes, first {n_cpu} merges, {t_cpu:.1f} s; rate scaled by "
                             f"{scale:.4f} to the full corpus (recount cost is linear in tokens)"}
        del ids, off

    # the initial pair count that is the path's microbenchmark (config 3: 2^31 ids over a
    # 65 536 vocabulary), two passes beside the merge job so that it reaches the same record
    pair_count_c3 = None
    if args.workload == "c2" and not args.bytes and not args.no_c3:
        del host
        torch.cuda.empty_cache()
        c3 = count_bench(list(WORKLOADS["c3"]), dev, 2, 1, with_e2e=False)
        pair_count_c3 = {"workload": c3["config"]["workload"], "gbs": c3["value"], "ms": c3["ms_per_step"],
                         "second_pass_ms": c3["roofline"]["second_pass_ms"], "kernel": c3["roofline"]["kernel"],
                         "frac_of_measured_peak": c3["roofline"]["frac"], "frac_of_8tbs": c3["roofline"]["frac_of_8tbs"],
                         "distinct_pairs": c3["config"]["distinct_pairs"], "best_pair": c3["config"]["best_pair"],
                         "sum_of_counts_equals_pair_positions": c3["config"]["sum_of_counts_equals_pair_positions"],
                         "bytes_per_token": 4}

    line = {
        "metric": "bpe_merges_per_sec", "value": value, "unit": "merges/s", "n_gpus": 1, "steps": done,
        "warmup": W, "ms_per_step": loop_ms / done, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int32", "data": "synthetic",
        "config": {"workload": desc, "name": args.workload, "corpus_bytes": n_tokens, "rows": len(off_np) - 1,
                   "merges_timed": done, "first_merge": M, "stop_reason": int(st.stop_reason),
                   "merges_sha256": merges_sha256(merges_gpu, counts_gpu),
                   "oracle_prefix_ok": oracle_ok, "oracle_prefix_merges": oracle_n,
                   "l2": "inputs larger than L2 (4 bytes x tokens per merge)", "tile_tokens": 1024},
        "pair_count": {"kernel": "count_dense_kernel (byte-level path)", "call_ms": count_call_ms, "ms": count_ms, "gbs": 4.0 * n_tokens / (count_ms / 1e3) / 1e9,
                       "frac_of_measured_peak": 4.0 * n_tokens / (count_ms / 1e3) / 1e9 / peak,
                       "frac_of_8tbs": 4.0 * n_tokens / (count_ms / 1e3) / 1e9 / 8000.0,
                       "bytes_per_token": 4, "distinct_pairs": None},
        "pair_count_c3": pair_count_c3,
        "roofline": {"bound": "hbm", "kernel": "merge_kernel", "achieved": achieved, "peak": peak,
                     "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                     "algorithmic_bytes": algo_bytes, "kernel_ms": mrg_ms, "launches": done,
                     "other_kernels_ms": {"select_kernel": sel_ms, "refresh_kernel": ref_ms, "repack": repack_ms},
                     "traffic": tile_bytes / done,
                     "traffic_note": "bytes per launch that the kernel's own bulk copies moved in this run (tiles and tile "
                                     "records read + rewritten tile parts and records stored, counted by the kernel); "
                                     "the ncu summaries under profiles/ give dram__bytes for the same kernel"},
        "e2e": {"value": e2e, "unit": "merges/s", "seconds": e2e_s,
                "h2d_bytes_per_step": (n_tokens + off_np.nbytes) / max(len(learned), 1),
                "d2h_bytes_per_step": 24.0},
        "gpu_launches": 4 * done + 2,   # select, worklist, merge, refresh per merge; the count and the final selection
        "clocks": clocks,
        "cpu_baseline": cpu,
    }
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
