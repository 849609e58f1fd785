#!/usr/bin/env python
"""Benchmark of the BPE merge loop on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload c2|c1|c5|c3]

One *step* is one merge of the loop (select best pair, rewrite the stream, update the pair
histogram by deltas).  The workload at N=1 is the 1 GiB mixed-script corpus with a 32 000-merge
target (seeded synthetic stand-in, generated on the device); ``--steps K`` times the first K
merges of that job, the default K is the whole job.  Warm-up merges run first and the engine is
then reloaded from the device-resident bytes, so the timed merges start from merge 0.

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
import json
import os
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
    """Seconds for exactly `steps` merges of the oracle's recount loop (after `warmup` merges);
    the stream is restarted from a fresh copy when a stop rule fires before `steps`."""
    from oracle import oracle as O
    O.lib()
    done, total = 0, 0.0
    first = True
    while done < steps:
        cur_ids, cur_off = ids.copy(), off.copy()
        w = warmup if first else 0
        first = False
        if w:
            m, _, reason = O.train_flat(cur_ids, cur_off, 256, w, 1, copy=False)
            base = 256 + len(m)
        else:
            base = 256
        want = steps - done
        t = time.perf_counter()
        m, _, reason = O.train_flat(cur_ids, cur_off, base, want, 1, copy=False)
        total += time.perf_counter() - t
        if not m:
            raise RuntimeError("oracle sample too small to learn a merge")
        done += len(m)
    return total, O.num_threads()


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
    # time per step such that the whole run ends within a few minutes
    total_s = 150.0
    per_step = total_s / max(args.steps + args.warmup, 1)
    probe = getattr(synth, gen)(n_bytes=1 << 20, seed=seed)
    ids, off = cpu_sample(np.asarray(probe.data), np.asarray(probe.row_offsets), 1 << 20)
    t, cores = time_oracle(ids, off, 3, 0)
    # the recount costs about 2.5 ns per token on the first merges (a few thousand distinct pairs)
    # and up to 20 ns per token late in a run (distinct pairs of the order of the tokens; measured
    # with this oracle on 8 cores), so the sample is sized for the late regime
    sec_per_token_merge = max(t / 3 / len(ids), 2.0e-8)
    sample_bytes = int(min(max(per_step / sec_per_token_merge, 64 << 10), 256 << 20, n_bytes))
    c = getattr(synth, gen)(n_bytes=sample_bytes, seed=seed)
    ids, off = cpu_sample(np.asarray(c.data), np.asarray(c.row_offsets), sample_bytes)
    t, cores = time_oracle(ids, off, args.steps, args.warmup)
    scale = len(ids) / float(n_bytes)          # recount cost is linear in the corpus size
    value = args.steps / t * scale
    line = {
        "impl": "reference", "metric": "bpe_merges_per_sec", "value": value, "unit": "merges/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1000.0 * t / args.steps / scale, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int32", "data": "synthetic",
        "config": {"workload": desc, "name": args.workload, "merges_timed": args.steps},
        "cpu_baseline": {"value": value, "unit": "merges/s", "cores": cores, "kind": "port",
                         "sample": f"first {len(ids)} bytes of the corpus, {args.steps} merges; "
                                   f"rate scaled by {scale:.5f} to the full corpus (a recount is linear in tokens; "
                                   f"a small sample has more distinct pairs per token than the full corpus, which "
                                   f"costs the recount up to 8x more per token than the first merges at full size)"},
        "e2e": {"value": value, "unit": "merges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- count-only workload
def run_count_bench(args, wl, dev):
    """Initial pair-count microbenchmark on an id stream (16-bit vocabulary): every step loads the
    resident ids again (pack, untimed) and runs one full histogram pass.  `value` is GB/s at 4 bytes
    per token over the histogram kernel; the time to move the directly indexed counters into the pair
    table is reported beside it."""
    import torch
    from supertoken_b200 import synth
    from supertoken_b200.engine import Engine
    gen, n_tokens, seed, _, desc = wl
    K, W = args.steps, max(args.warmup, 1)
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
    peak, peak_kind = peaks()
    med = float(np.median(ms))
    gbs = 4.0 * n_tokens / (med / 1e3) / 1e9
    # end to end: pinned host ids -> device -> pack -> histogram -> best pair back on the host
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
    line = {
        "metric": "pair_count_gbs", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": med, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int32", "data": "synthetic",
        "config": {"workload": desc, "name": "c3", "tokens": n_tokens, "rows": len(off_np) - 1,
                   "distinct_pairs": int(st.table_keys), "best_pair": [int(key >> 32), int(key & 0xFFFFFFFF), int(count)],
                   "l2": "inputs larger than L2", "bytes_per_token": 4},
        "roofline": {"bound": "hbm", "kernel": "count_dense32_kernel" if med and conv and conv[0] > 0 else "count_kernel",
                     "achieved": gbs, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": gbs / peak,
                     "frac_of_8tbs": gbs / 8000.0, "kernel_ms": med, "to_pair_table_ms": float(np.median(conv)),
                     "call_ms": float(np.median(call)), "traffic": None},
        "e2e": {"value": 4.0 * n_tokens / e2e_s / 1e9, "unit": "GB/s", "seconds": e2e_s,
                "h2d_bytes_per_step": 4.0 * n_tokens + off_np.nbytes, "d2h_bytes_per_step": 24.0},
        "gpu_launches": 2 * K, "clocks": clocks, "cpu_baseline": None,
    }
    print(json.dumps(line), flush=True)


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

    K, W = args.steps, args.warmup
    corpus = getattr(synth, gen)(n_bytes=n_bytes, seed=seed, device=str(dev))
    torch.cuda.synchronize()
    data_dev, off_np = corpus.data, corpus.row_offsets.cpu().numpy()
    n_tokens = int(data_dev.numel())

    def ev():
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return e

    eng = Engine(n_tokens, base_vocab=256, max_merges=max(K, W, 1), device=dev)

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
    t1 = ev()
    eng.train(K)
    t2 = ev()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    count_call_ms = t0.elapsed_time(t1)
    loop_ms = t1.elapsed_time(t2)
    st = eng.state()
    count_ms = float(st.count_kernel_ms)   # histogram kernel(s) only; the call also clears the table,
    # builds the tile records, the pair filter and the block maxima
    done = st.merges_done
    merges_gpu, counts_gpu, live_before = eng.merges(0, done)
    if done < 1:
        raise SystemExit("no merge was learned")
    value = done / (loop_ms / 1000.0)

    # per-kernel device time of the same K merges (events around every launch)
    load()
    eng.count_initial()
    sel_ms, mrg_ms, ref_ms, repack_ms = eng.train_timed(K)
    torch.cuda.synchronize()
    merges_again, _, _ = eng.merges(0, eng.state().merges_done)
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
    trainer = GPUBPETrainer(base_vocab=256, merges=K, device=str(dev))
    res = trainer.fit_bytes(host, off_np, log_every=0)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t
    learned = trainer.merge_counts
    assert res["merges"][:len(learned)] == merges_gpu[:len(learned)]
    e2e = len(learned) / e2e_s

    cpu = None
    if not args.no_cpu_baseline:
        sample_bytes = min(64 << 20, n_bytes)
        ids, off = cpu_sample(host.numpy(), off_np, sample_bytes)
        n_cpu = 12
        t_cpu, cores = time_oracle(ids, off, n_cpu, 0)
        if t_cpu < 8.0:  # aim at about 12 s of CPU work on this machine's cores
            n_cpu = int(min(max(12.0 / (t_cpu / 12), 12), 600))
            t_cpu, cores = time_oracle(ids, off, n_cpu, 0)
        scale = len(ids) / float(n_tokens)
        cpu = {"value": n_cpu / t_cpu * scale, "unit": "merges/s", "cores": cores, "kind": "port",
               "sample": f"first {len(ids)} bytes, first {n_cpu} merges, {t_cpu:.1f} s; rate scaled by "
                         f"{scale:.4f} to the full corpus (recount cost is linear in tokens)"}

    line = {
        "metric": "bpe_merges_per_sec", "value": value, "unit": "merges/s", "n_gpus": 1, "steps": done,
        "warmup": W, "ms_per_step": loop_ms / done, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int32", "data": "synthetic",
        "config": {"workload": desc, "name": args.workload, "corpus_bytes": n_tokens, "rows": len(off_np) - 1,
                   "merges_timed": done, "first_merge": 0, "stop_reason": int(st.stop_reason),
                   "l2": "inputs larger than L2 (4 bytes x tokens per merge)", "tile_tokens": 1024},
        "pair_count": {"kernel": "count_dense_kernel (byte-level path)", "call_ms": count_call_ms, "ms": count_ms, "gbs": 4.0 * n_tokens / (count_ms / 1e3) / 1e9,
                       "frac_of_measured_peak": 4.0 * n_tokens / (count_ms / 1e3) / 1e9 / peak,
                       "frac_of_8tbs": 4.0 * n_tokens / (count_ms / 1e3) / 1e9 / 8000.0,
                       "bytes_per_token": 4, "distinct_pairs": None},
        "roofline": {"bound": "hbm", "kernel": "merge_kernel", "achieved": achieved, "peak": peak,
                     "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                     "algorithmic_bytes": algo_bytes, "kernel_ms": mrg_ms, "launches": done,
                     "other_kernels_ms": {"select_kernel": sel_ms, "refresh_kernel": ref_ms, "repack": repack_ms},
                     "traffic": 0.711 * algo_bytes / done,
                     "traffic_note": "DRAM read+write per launch = 0.711 x algorithmic bytes: ncu over merges 1-1500 of a "
                                     "64 MiB slice (115.7 GB of traffic for 162.7 GB algorithmic), scaled by live tokens; "
                                     "later merges visit fewer tiles, so the factor of the full job is lower"},
        "e2e": {"value": e2e, "unit": "merges/s", "seconds": e2e_s,
                "h2d_bytes_per_step": (n_tokens + off_np.nbytes) / max(len(learned), 1),
                "d2h_bytes_per_step": 24.0},
        "gpu_launches": 4 * done + 1,
        "clocks": clocks,
        "cpu_baseline": cpu,
    }
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
