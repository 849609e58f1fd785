"""``GPUBPETrainer`` -- drop-in for the reference trainer's BPE merge loop.

Mirrors the public surface of ``gpu_tokenizer/bpe_trainer.py:691-4790`` that sits on the
merge-loop path: constructor (``:694-708``), ``fit`` (``:2501-2518``) with its return
dictionary (``:4582-4607``), merge log / vocabulary attributes, checkpoint and artifact
methods.  The loop itself (``:4193-4517``) runs on the GPU through the C-ABI library; there
is no CPU path here -- ``device="cpu"`` raises.

Semantics kept bit-for-bit (see ``supertoken_b200/csrc/kernels.cuh`` for the kernels):
rows are the only pair boundary, every adjacent position counts, best pair = highest count
then smallest ``(a << 32) | b``, stop when the best count is below 2 (then pad with
``random.randint`` pairs as the reference does) or when no pair is left (no padding),
``new_id = base_vocab + len(merges)``, simultaneous-match merge with run collapse.
"""
from __future__ import annotations

import json
import logging
import os
import random
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Iterable, List, Mapping, Optional, Sequence, Tuple

import numpy as np
import torch

from . import _lib as L
from .base import BaseTrainer
from .engine import Engine
from .export import GPUBPETokenizer, build_artifacts, bytes_to_unicode, write_artifacts

logger = logging.getLogger(__name__)
UINT32_MAX = (1 << 32) - 1
CHECKPOINT_SCHEMA_VERSION = 1


@dataclass
class StageTiming:
    """Timing samples of a named stage (``gpu_tokenizer/bpe_trainer.py:85-107``)."""

    name: str
    samples: List[float] = field(default_factory=list)

    def record(self, duration_s: float) -> None:
        if duration_s >= 0:
            self.samples.append(float(duration_s))

    def summary(self) -> dict:
        total = float(sum(self.samples))
        n = len(self.samples)
        return {"stage": self.name, "count": n, "total_s": total, "avg_s": total / n if n else 0.0,
                "samples": list(self.samples)}


class _NullAutoScaler:
    """Batch size does not influence merges; the controller is kept only as an attribute."""

    def state_dict(self) -> dict:
        return {}


def hash_merge_pair(pair: Tuple[int, int], salt: bytes = b"") -> str:
    """Salted SHA-256 digest of a merge pair (``gpu_tokenizer/utils.py:137-157``)."""
    import hashlib
    d = hashlib.sha256()
    d.update(salt)
    d.update(int(pair[0]).to_bytes(8, "big", signed=False))
    d.update(int(pair[1]).to_bytes(8, "big", signed=False))
    return d.hexdigest()


def _flatten_batch(batch) -> Tuple[torch.Tensor, np.ndarray]:
    """``(tokens[B,L], valid[B,L], lengths[B])`` -> flat int32 ids + row offsets.

    The reference's batchers only emit prefix-valid rows (``gpu_tokenizer/datasets.py:83-84``);
    anything else is outside the parity contract and rejected."""
    tokens, valid = batch[0], batch[1]
    if tokens.dim() != 2 or valid.shape != tokens.shape:
        raise ValueError("expected tokens[B, L] and valid[B, L]")
    vb = valid.to(torch.bool)
    lens = vb.sum(dim=1, dtype=torch.int64)
    L_ = tokens.shape[1]
    prefix = torch.arange(L_, device=vb.device)[None, :] < lens[:, None]
    if not torch.equal(prefix, vb):
        raise ValueError("valid must mark a prefix of every row")
    ids = tokens[vb].to(torch.int32).contiguous()
    off = np.zeros(tokens.shape[0] + 1, dtype=np.int64)
    np.cumsum(lens.cpu().numpy(), out=off[1:])
    return ids, off


class GPUBPETrainer(BaseTrainer):
    """B200 implementation of the reference's ``GPUBPETrainer`` merge loop."""

    def __init__(self, base_vocab: int = 256, merges: int = 50_000, device: str | None = None,
                 devices: Optional[Sequence[str]] = None, autoscaler: Any = None, sync_every: int = 1,
                 warm_start_merges: Optional[Sequence[Tuple[int, int]]] = None,
                 freeze_warm_start: bool = False, privacy_mode: bool = False,
                 randomize_ties: bool | None = None, tie_seed: int | None = None,
                 privacy_salt: bytes | bytearray | str | None = None) -> None:
        super().__init__()
        self.base_vocab = int(base_vocab)
        self.target_merges = int(merges)
        resolved: List[torch.device] = []
        if devices is not None:
            if not devices:
                raise ValueError("devices must be a non-empty sequence when provided")
            resolved = [torch.device(d) for d in devices]
        if device is not None:
            primary = torch.device(device)
            if resolved and primary not in resolved:
                raise ValueError("primary device must be included in devices sequence")
            if not resolved:
                resolved = [primary]
        if not resolved:
            resolved = [torch.device("cuda")]
        if any(d.type != "cuda" for d in resolved):
            raise RuntimeError("supertoken_b200.GPUBPETrainer runs on CUDA devices only "
                               "(the CPU path belongs to the reference implementation)")
        self.devices = resolved
        self.device = str(resolved[0])
        self.vocab_size = self.base_vocab
        self.merges: List[Tuple[int, int]] = []
        self.merge_counts: List[int] = []
        self._seed_warm_start_merges = list(warm_start_merges) if warm_start_merges is not None else []
        self.freeze_warm_start = bool(freeze_warm_start)
        self.privacy_mode = bool(privacy_mode)
        self.randomize_ties = self.privacy_mode if randomize_ties is None else bool(randomize_ties)
        self.tie_seed = int(tie_seed) if tie_seed is not None else None
        self._tie_seed_value = int(self.tie_seed if self.tie_seed is not None else 0)
        if privacy_salt is None:
            self._privacy_hash_salt = b""
        elif isinstance(privacy_salt, (bytes, bytearray)):
            self._privacy_hash_salt = bytes(privacy_salt)
        else:
            self._privacy_hash_salt = str(privacy_salt).encode("utf-8")
        self._tie_rng: random.Random | None = None
        self._reset_tie_rng()
        self.autoscaler = autoscaler if autoscaler is not None else _NullAutoScaler()
        self.sync_every = max(1, int(sync_every))
        self._enable_histogram_cache = False  # the engine always keeps an exact histogram
        self._top_pairs_limit = 0
        self._cpu_fallback_batches = 0
        self._active_batch_size: Optional[int] = None
        self.bytes_h2d = self.bytes_d2h = 0
        self.h2d_events = self.d2h_events = 0
        self.throughput_metrics: dict = {}
        self.table_slots = 0  # 0 = sized from the token count
        # a process group initialised by the caller (one process per GPU) shards the corpus over the
        # ranks: every rank passes its own rows to fit() and all ranks learn the same merges
        self.use_process_group = True
        self.exchange_entries = 4096  # delta entries per peer and round
        self._engine: Optional[Engine] = None
        self._last_stats: dict = {}

    # ------------------------------------------------------------------ small helpers
    def _reset_tie_rng(self) -> None:
        self._tie_rng = random.Random(self._tie_seed_value) if self.randomize_ties else None

    def metrics(self) -> Mapping[str, Any]:
        return self._metrics_mapping()

    def handle_chunk_start(self, chunk_id: int, *, reprocessed: bool = False, attempts: int = 1) -> None:
        """Lease bookkeeping hook of the reference (``bpe_trainer.py:836-856``): static
        document sharding has no leases, so there is nothing to invalidate."""

    @staticmethod
    def _bytes_to_unicode() -> dict:
        return bytes_to_unicode()

    def import_merges(self, merges, *, vocab_size: int | None = None, base_vocab: int | None = None,
                      source: str | None = None, freeze: bool = False) -> None:
        """``gpu_tokenizer/bpe_trainer.py:2254-2300``."""
        if merges is None:
            raise ValueError("merges must be provided when importing external artifacts")
        coerced = []
        for entry in merges:
            if not isinstance(entry, Sequence) or len(entry) != 2:
                raise ValueError("merge entries must contain exactly two token ids")
            coerced.append((int(entry[0]), int(entry[1])))
        self.base_vocab = int(base_vocab) if base_vocab is not None else self.base_vocab
        self.vocab_size = int(vocab_size) if vocab_size is not None else self.base_vocab + len(coerced)
        self.target_merges = max(self.target_merges, len(coerced))
        self.merges = coerced
        self._seed_warm_start_merges = list(coerced)
        self.freeze_warm_start = bool(freeze)

    @classmethod
    def precompute_warm_start_plan(cls, batches: Iterable, top_k: int, device=None) -> dict:
        """Warm-start plan from the bigram histogram of the batches: the ``top_k`` most frequent
        pairs (``gpu_tokenizer/bpe_trainer.py:2165-2252`` over ``ngram_stats.compute_ngram_histograms``,
        order 2 = the adjacent-pair histogram the engine builds anyway).  Equal counts are ordered by
        the smaller packed key, which makes the plan deterministic."""
        empty = {"merges": [], "counts": [], "top_k": 0, "requested_top_k": int(top_k or 0), "order": 2,
                 "histogram_size": 0, "source": "ngram"}
        if top_k is None or top_k <= 0:
            return empty
        flat = [_flatten_batch(b) for b in batches]
        total = sum(int(ids.numel()) for ids, _ in flat)
        eng = Engine(max(total, 1), base_vocab=0, max_merges=1,
                     device=torch.device(device) if device is not None else None)
        try:
            for ids, off in flat:
                if ids.numel():
                    eng.append_ids(ids, off)
            eng.count_initial()
            keys, counts = eng.export_histogram()
        finally:
            eng.close()
        if keys.numel() == 0:
            return empty
        limit = min(int(top_k), int(keys.numel()))
        # keys come out ascending: a stable sort by descending count keeps ties in key order
        order = torch.argsort(counts, descending=True, stable=True)[:limit]
        ks, cs = keys[order].cpu().tolist(), counts[order].cpu().tolist()
        merges = [((k >> 32) & 0xFFFFFFFF, k & 0xFFFFFFFF) for k in ks]
        return {"merges": merges, "counts": [int(c) for c in cs], "top_k": len(merges),
                "requested_top_k": int(top_k), "order": 2, "histogram_size": int(keys.numel()), "source": "ngram"}

    # ------------------------------------------------------------------ the loop
    def _make_engine(self, n_tokens: int, first_new_id: Optional[int] = None) -> Engine:
        """``first_new_id``: id the engine gives its first merge (a stream restored from a checkpoint
        already holds the ids of the merges made before it was written)."""
        dev = torch.device(self.device)
        if self._engine is not None:
            self._engine.close()
        base = self.base_vocab if first_new_id is None else int(first_new_id)
        self._engine = Engine(max(int(n_tokens), 1), base_vocab=base,
                              max_merges=max(self.target_merges - (base - self.base_vocab), 1), device=dev,
                              table_slots=self.table_slots)
        return self._engine

    def fit(self, batches: Iterable, log_every: int = 100, profile_streams: bool = False,
            on_batch_size_change: Optional[Callable] = None, warm_start_merges=None,
            freeze_warm_start: Optional[bool] = None, overlap_transfers: bool = True,
            warm_start_plan=None, warm_start_ngrams=None, warm_start_device=None,
            checkpoint_interval: Optional[int] = None, checkpoint_dir: Optional[str] = None,
            resume_state=None, on_iteration_summary=None, dataset_state=None) -> dict:
        """Train on an iterable of ``(tokens[B,L] int32, valid[B,L] uint8, lengths[B])`` CPU or
        CUDA tensors, as the reference's batchers yield them (``gpu_tokenizer/datasets.py:88-92``)."""
        if checkpoint_interval is not None and checkpoint_dir is None:
            raise ValueError("checkpoint_interval requires checkpoint_dir")
        restored_rows = None
        if resume_state is not None:
            # resume (bpe_trainer.py:2938-2986).  A checkpoint that holds the rewritten rows continues
            # from them; otherwise its merges are replayed on the batches without counting.  Merges
            # are a pure function of the corpus (and of the restored tie-break generator), so either
            # way the result equals an uninterrupted run.
            record = self.load_state_dict(resume_state)
            restored_rows = record.get("sequences")
            warm_start_merges = list(self.merges)
        elif warm_start_merges is None and warm_start_plan is not None:
            warm_start_merges = [tuple(p) for p in warm_start_plan.get("merges", [])]
        elif warm_start_merges is None and warm_start_ngrams:
            batches = list(batches)
            plan = self.precompute_warm_start_plan(batches, int(warm_start_ngrams), device=warm_start_device or self.device)
            warm_start_merges = plan["merges"]
        t0 = time.perf_counter()
        if restored_rows is not None:
            if self._sharded_mode() is not None:
                self._reject_in_sharded_mode(warm_start_merges, checkpoint_interval)
            lens = np.fromiter((len(r) for r in restored_rows), dtype=np.int64, count=len(restored_rows))
            off = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
            ids = np.fromiter((t for r in restored_rows for t in r), dtype=np.int32, count=int(off[-1]))
            eng = self._make_engine(len(ids), first_new_id=self.base_vocab + len(self.merges))
            if len(ids):
                eng.append_ids(ids, off)
                self.bytes_h2d += ids.nbytes
                self.h2d_events += 1
            return self._run_loop(eng, log_every, t0, None, checkpoint_interval, checkpoint_dir,
                                  already=list(self.merges), dataset_state=dataset_state)
        flat: List[Tuple[torch.Tensor, np.ndarray]] = [_flatten_batch(b) for b in batches]
        total = sum(int(ids.numel()) for ids, _ in flat)
        mode = self._sharded_mode()
        if mode is not None:
            self._reject_in_sharded_mode(warm_start_merges, checkpoint_interval)
            return self._fit_sharded(mode, flat, False, log_every, t0)
        eng = self._make_engine(total)
        for ids, off in flat:
            if ids.numel():
                eng.append_ids(ids, off)
                if not ids.is_cuda:
                    self.bytes_h2d += ids.numel() * 4
                    self.h2d_events += 1
        return self._run_loop(eng, log_every, t0, warm_start_merges, checkpoint_interval, checkpoint_dir,
                              dataset_state=dataset_state)

    def fit_bytes(self, data, row_offsets=None, log_every: int = 0, *, warm_start_merges=None,
                  checkpoint_interval: Optional[int] = None, checkpoint_dir: Optional[str] = None,
                  resume_state=None, dataset_state=None) -> dict:
        """Fast ingest: one uint8 buffer (host or device) plus row offsets; rows are what
        the reference calls files / documents.  Not part of the reference API: padded
        ``[B, L]`` int32 batches cost five host bytes per input byte.  Warm start, checkpoint
        interval and resume behave as in ``fit``."""
        if checkpoint_interval is not None and checkpoint_dir is None:
            raise ValueError("checkpoint_interval requires checkpoint_dir")
        if isinstance(data, np.ndarray):
            data = torch.from_numpy(np.ascontiguousarray(data, dtype=np.uint8))
        if resume_state is not None:
            record = self.load_state_dict(resume_state)
            if record.get("sequences") is not None:
                return self.fit([], log_every=log_every, checkpoint_interval=checkpoint_interval,
                                checkpoint_dir=checkpoint_dir, resume_state=resume_state,
                                dataset_state=dataset_state)
            warm_start_merges = list(self.merges)
        t0 = time.perf_counter()
        mode = self._sharded_mode()
        if mode is not None:
            self._reject_in_sharded_mode(warm_start_merges, checkpoint_interval)
            off = Engine._offsets(row_offsets, int(data.numel()))
            return self._fit_sharded(mode, [(data, off)], True, log_every, t0)
        eng = self._make_engine(data.numel())
        eng.append_bytes(data, row_offsets)
        if not data.is_cuda:
            self.bytes_h2d += data.numel()
            self.h2d_events += 1
        return self._run_loop(eng, log_every, t0, warm_start_merges, checkpoint_interval, checkpoint_dir,
                              dataset_state=dataset_state)

    def _run_loop(self, eng: Engine, log_every: int, t0: float, warm_start_merges,
                  checkpoint_interval, checkpoint_dir, already: Optional[List[Tuple[int, int]]] = None,
                  dataset_state=None) -> dict:
        """``already``: merges that the loaded stream holds already (resume from the rows of a
        checkpoint); the engine numbers its own merges after them."""
        timings = {k: StageTiming(k) for k in ("pair_count", "apply_merge", "host_sync")}
        events: List[dict] = []
        self.merges = list(already) if already else []
        self.merge_counts = []
        self._readbacks: List[dict] = []
        self.vocab_size = self.base_vocab + len(self.merges)
        skip = len(self.merges)   # merges the engine's own log does not hold
        if already:
            warm: List[Tuple[int, int]] = []
        else:
            warm = list(warm_start_merges) if warm_start_merges is not None else list(self._seed_warm_start_merges)

        t = time.perf_counter()
        eng.count_initial()
        torch.cuda.synchronize(eng.device)
        timings["pair_count"].record(time.perf_counter() - t)
        events.append({"stage": "pair_count", "duration_s": timings["pair_count"].samples[-1],
                       "mode": "gpu", "merge": 0, "type": "merge", "timestamp": time.time()})

        # warm start: seeded merges are applied without selection (bpe_trainer.py:4058-4182)
        warm_applied = 0
        for a, b in warm[: self.target_merges]:
            if max(a, b, self.vocab_size) > UINT32_MAX:
                raise OverflowError(f"Token id overflow: encountered id above UINT32_MAX (limit {UINT32_MAX}).")
            eng.apply_merge(int(a), int(b), self.vocab_size)
            self.merges.append((int(a), int(b)))
            self.vocab_size += 1
            warm_applied += 1

        def checkpoint():
            self.save_checkpoint(checkpoint_dir, dataset_state=dataset_state)

        t = time.perf_counter()
        remaining = self.target_merges - len(self.merges)
        reason = L.RUNNING
        if remaining > 0:
            if self.randomize_ties:
                reason = self._loop_random_ties(eng, remaining, checkpoint_interval,
                                                checkpoint if checkpoint_dir else None)
            else:
                step = checkpoint_interval if checkpoint_interval else remaining
                while remaining > 0 and reason in (L.RUNNING, L.STOP_TARGET):
                    n = min(step, remaining)
                    eng.train(n)
                    th = time.perf_counter()
                    st = eng.state()
                    have = len(self.merges) - skip
                    got, counts, _ = eng.merges(have, st.merges_done - have)
                    timings["host_sync"].record(time.perf_counter() - th)   # merge log back to the host
                    self.bytes_d2h += len(got) * 24
                    self.d2h_events += 1
                    if got:
                        self._readbacks.append({"merge": len(self.merges) + len(got) - 1, "merges": len(got),
                                                "bytes_d2h": len(got) * 24})
                    self.merges.extend(got)
                    self.merge_counts.extend(int(c) for c in counts)
                    self.vocab_size = self.base_vocab + len(self.merges)
                    remaining = self.target_merges - len(self.merges)
                    reason = st.stop_reason
                    if checkpoint_interval and checkpoint_dir and remaining > 0:
                        checkpoint()
                    if len(got) < n:
                        break
        loop_s = time.perf_counter() - t
        return self._finalize(eng.state(), reason, timings, events, warm_applied + skip, loop_s, t0, log_every)

    def _finalize(self, st, reason, timings, events, warm_applied, loop_s, t0, log_every) -> dict:
        timings["apply_merge"].record(loop_s)
        if log_every and log_every > 0:
            for step, ((a, b), c) in enumerate(zip(self.merges[warm_applied:], self.merge_counts)):
                if step % log_every == 0:
                    print(f"merge {step:6d}: ({a},{b}) -> {self.base_vocab + warm_applied + step}  count={c}")
        if reason == L.STOP_NO_PAIRS:
            print("No pairs left to merge.")  # bpe_trainer.py:4304-4308: stop, no padding
        elif reason == L.STOP_LOW_COUNT:
            # bpe_trainer.py:4347-4353: pad with random pairs up to the target
            while len(self.merges) < self.target_merges:
                self.merges.append((random.randint(0, self.vocab_size - 1), random.randint(0, self.vocab_size - 1)))
                self.vocab_size += 1
            if log_every and log_every > 0:
                logger.info("Stopping: no frequent pairs.")
        self._last_stats = {"live_tokens": int(st.live_tokens), "table_keys": int(st.table_keys),
                            "table_slots": int(st.table_slots), "loop_s": loop_s,
                            "total_s": time.perf_counter() - t0, "stop_reason": int(reason)}
        # The loop runs on the device: nothing is copied to the host per merge.  The merge log comes
        # back once per train call (24 bytes per merge: pair, count, live tokens); merge_stats holds
        # one record per such read-back, named after the last merge it brought.
        n_learned = len(self.merge_counts)
        return {
            "base_vocab": self.base_vocab,
            "vocab_size": self.vocab_size,
            "merges": self.merges,
            "warm_start": {"applied": warm_applied, "source": "constructor" if warm_applied else None},
            "transfer_metrics": {
                "bytes_h2d": self.bytes_h2d, "bytes_d2h": self.bytes_d2h,
                "h2d_events": self.h2d_events, "d2h_events": self.d2h_events,
                "merge_stats": list(getattr(self, "_readbacks", [])), "sync_intervals": [],
                "per_device": {self.device: {"bytes_h2d": self.bytes_h2d, "bytes_d2h": self.bytes_d2h}},
                "per_stage": {"pair_count": {"h2d": self.bytes_h2d, "d2h": 0}, "apply_merge": {"h2d": 0, "d2h": 0},
                              "host_sync": {"h2d": 0, "d2h": self.bytes_d2h}},
                "avg_d2h_bytes_per_merge": (self.bytes_d2h / n_learned) if n_learned else 0.0,
                "cpu_fallback": {"batches": 0, "ratio": 0.0},
            },
            "telemetry": {
                "timings": {k: v.summary() for k, v in timings.items()},
                "events": events, "host_sync_events": [], "device_snapshots": [],
                "autoscaler": {"window": []},
                "iteration_metrics": {"ewma": {}, "iterations": []},
                "engine": dict(self._last_stats),
            },
        }

    # ------------------------------------------------------------------ several GPUs
    def _sharded_mode(self) -> Optional[str]:
        """``"devices"``: this process drives every GPU of ``devices=(...)`` itself
        (``gpu_tokenizer/bpe_trainer.py:716-731``, rows split over the devices ``:541-576``);
        ``"ranks"``: one process per GPU, process group initialised by the caller
        (``docs/performance.md:70-81`` of the reference); ``None``: one GPU."""
        if len(self.devices) > 1:
            return "devices"
        if self.use_process_group:
            import torch.distributed as dist
            if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
                return "ranks"
        return None

    def _reject_in_sharded_mode(self, warm_start_merges, checkpoint_interval) -> None:
        if warm_start_merges or self._seed_warm_start_merges or self.randomize_ties or checkpoint_interval:
            raise NotImplementedError("warm start / resume, randomised ties and checkpoint intervals drive the "
                                      "merge loop from the host and are available on one GPU only")

    def _fit_sharded(self, mode: str, pieces, as_bytes: bool, log_every: int, t0: float) -> dict:
        """Merge loop over several GPUs: rows stay where they are loaded, pair keys are owned by
        hash, every round exchanges the deltas of one merge and all ranks commit the same winner
        (``supertoken_b200/dist.py``).  ``pieces`` = [(flat ids or bytes, row offsets)] in row order."""
        from . import dist as D
        timings = {k: StageTiming(k) for k in ("pair_count", "apply_merge", "host_sync")}
        events: List[dict] = []
        self.merges, self.merge_counts, self.vocab_size = [], [], self.base_vocab

        def load(engine, lo_row, hi_row):
            # rows [lo_row, hi_row) of the concatenation of the pieces
            r0 = 0
            for data, off in pieces:
                n = len(off) - 1
                a, b = max(lo_row - r0, 0), min(hi_row - r0, n)
                if a < b:
                    part, poff = data[int(off[a]):int(off[b])], off[a:b + 1] - off[a]
                    (engine.append_bytes if as_bytes else engine.append_ids)(part, poff)
                    if not part.is_cuda:
                        self.bytes_h2d += part.numel() * (1 if as_bytes else 4)
                        self.h2d_events += 1
                r0 += n

        lens = np.concatenate([np.diff(off) for _, off in pieces]) if pieces else np.zeros(0, np.int64)
        goff = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
        n_rows = len(goff) - 1
        t = time.perf_counter()
        engines: List[Engine] = []
        closer = None
        if mode == "devices":
            world = len(self.devices)
            cuts = D.shard_rows(goff, world)
            workers = []
            for r, dev in enumerate(self.devices):
                lo, hi = cuts[r]
                e = Engine(max(int(goff[hi] - goff[lo]), 1), base_vocab=self.base_vocab,
                           max_merges=max(self.target_merges, 1), device=dev, table_slots=self.table_slots,
                           world_size=world, rank=r)
                load(e, lo, hi)
                engines.append(e)
                workers.append(D.EngineWorker(e, cap_per_peer=self.exchange_entries))
            loop = D.ShardedBPE(workers, D.LocalComm())
        else:
            import torch.distributed as dist
            world, rank = dist.get_world_size(), dist.get_rank()
            e = Engine(max(int(goff[-1]), 1), base_vocab=self.base_vocab, max_merges=max(self.target_merges, 1),
                       device=torch.device(self.device), table_slots=self.table_slots, world_size=world, rank=rank)
            load(e, 0, n_rows)
            engines.append(e)
            same_node = int(os.environ.get("LOCAL_WORLD_SIZE", "0")) == world
            driver = os.environ.get("STBPE_MG_DRIVER", "peer" if same_node and world <= 16 else "nccl")
            loop = D.PeerLoop(e, self.exchange_entries) if driver == "peer" else D.NativeLoop(e, self.exchange_entries)
            closer = getattr(loop, "close", None)
            if not as_bytes and self.base_vocab <= 65536 and same_node:
                # a large id stream over a 16-bit vocabulary: the ranks partition their pairs and the
                # owners count them over peer memory before the first round (supertoken_b200/dist.py)
                total = torch.tensor([float(goff[-1])], dtype=torch.float64, device=e.device)
                dist.all_reduce(total)
                if total.item() >= float(1 << 24):
                    D.wide_count(e)
        try:
            timings["pair_count"].record(time.perf_counter() - t)
            t = time.perf_counter()
            done, reason = loop.train()
            loop_s = time.perf_counter() - t
            got, counts, _ = engines[0].merges(0, done)
            self.merges = list(got)
            self.merge_counts = [int(c) for c in counts]
            self.vocab_size = self.base_vocab + len(self.merges)
            st = engines[0].state()
            if mode == "ranks":
                D.wide_close(engines[0])
            if closer is not None:
                closer()
        finally:
            for e in engines:
                e.close()
        return self._finalize(st, reason, timings, events, 0, loop_s, t0, log_every)


    def _loop_random_ties(self, eng: Engine, remaining: int, checkpoint_interval=None, checkpoint=None) -> int:
        """Host-driven loop for ``randomize_ties``: the seeded ``random.Random`` picks an index
        into the tied candidates in ascending key order (``bpe_trainer.py:915-923``,
        ``trainers/bpe_gpu.py:112-123``).  ``checkpoint`` is called every ``checkpoint_interval``
        merges (the checkpoint carries the generator's state, so a resumed run draws on)."""
        since = 0
        while remaining > 0:
            key, count, ties = eng.select_best(with_ties=True)
            if key is None:
                return L.STOP_NO_PAIRS
            if count < 2:
                return L.STOP_LOW_COUNT
            if ties > 1 and self._tie_rng is not None:
                cands = eng.tied_keys(count, ties)
                key = cands[self._tie_rng.randrange(len(cands))]
            a, b = key >> 32, key & 0xFFFFFFFF
            eng.apply_merge(a, b, self.vocab_size)
            self.merges.append((a, b))
            self.merge_counts.append(count)
            self.vocab_size += 1
            remaining -= 1
            since += 1
            if checkpoint is not None and checkpoint_interval and since >= checkpoint_interval and remaining > 0:
                checkpoint()
                since = 0
        return L.STOP_TARGET

    # ------------------------------------------------------------------ state / artifacts
    def _merges_for_metadata(self) -> list:
        if not self.privacy_mode:
            return [list(map(int, p)) for p in self.merges]
        return [hash_merge_pair(p, self._privacy_hash_salt) for p in self.merges]

    def _privacy_summary(self) -> dict:
        mode = "tie-randomize" if self.randomize_ties else ("hash-merges" if self.privacy_mode else "none")
        s: dict = {"mode": mode, "merges_redacted": bool(self.privacy_mode),
                   "randomize_ties": bool(self.randomize_ties)}
        if self.randomize_ties or self.tie_seed is not None:
            s["tie_seed_effective"] = int(self._tie_seed_value)
            if self.tie_seed is not None:
                s["tie_seed"] = int(self.tie_seed)
        if self._privacy_hash_salt:
            s["salt_configured"] = True
        return s

    # Checkpoints follow the reference's layout (``gpu_tokenizer/bpe_trainer.py:1450-1601``,
    # ``:1890-1948``; ``gpu_tokenizer/trainers/base.py:17-41``): ``state_dict`` returns
    # ``{"payload": <schema v1: version / trainer / autoscaler / dataset / rng>, "tensors": {...}}``,
    # ``save_checkpoint`` writes the payload as ``state.json`` and the tensors as ``tensors.pt``.
    # The tensors are the pair histogram (ascending keys, int64 counts), which the reference keeps as
    # its cached histogram; ``dataset.batches.sequences`` are the rewritten rows, from which a
    # resumed ``fit`` continues without replaying the merges.
    SEQUENCE_DUMP_LIMIT = 1 << 24  # rows are written as Python int lists, as the reference does

    @staticmethod
    def _encode_random_state(state):
        if isinstance(state, (tuple, list)):
            return [GPUBPETrainer._encode_random_state(x) for x in state]
        return state

    @staticmethod
    def _decode_random_state(state):
        if isinstance(state, (tuple, list)):
            return tuple(GPUBPETrainer._decode_random_state(x) for x in state)
        return state

    def _current_rows(self) -> Optional[List[List[int]]]:
        """Rows of the engine's stream as it stands (after the merges applied so far)."""
        eng = self._engine
        if eng is None or not getattr(eng, "_h", None) or not eng._h.value:
            return None
        st = eng.state()
        if st.live_tokens > self.SEQUENCE_DUMP_LIMIT:
            return None
        ids, off = eng.export_stream()
        return [ids[int(off[i]):int(off[i + 1])].tolist() for i in range(len(off) - 1)]

    def state_dict(self, *, current_batches=None, include_batches: bool = True, stage_timings=None,
                   stage_event_log=None, host_sync_events=None, device_snapshot_log=None,
                   dataset_state=None) -> dict:
        model = {"base_vocab": int(self.base_vocab), "target_merges": int(self.target_merges),
                 "vocab_size": int(self.vocab_size), "merges": [list(map(int, p)) for p in self.merges],
                 "merge_step": len(self.merges), "privacy_mode": bool(self.privacy_mode),
                 "randomize_ties": bool(self.randomize_ties),
                 "tie_seed": int(self.tie_seed) if self.tie_seed is not None else None,
                 "tie_seed_effective": int(self._tie_seed_value)}
        if self._privacy_hash_salt:
            model["privacy_salt"] = self._privacy_hash_salt.hex()
        logs: dict = {"merge_transfer_log": [], "sync_intervals": [], "transfer_stage_totals": {}}
        progress = {}
        if stage_timings is not None:
            progress["stage_timings"] = {k: list(v.samples) for k, v in stage_timings.items()}
        for name, val in (("stage_event_log", stage_event_log), ("host_sync_events", host_sync_events),
                          ("device_snapshot_log", device_snapshot_log)):
            if val is not None:
                progress[name] = [dict(x) for x in val]
        if progress:
            logs["telemetry_progress"] = progress
        trainer = {
            "model": model,
            "warm_start": {"plan": None, "applied": bool(self._seed_warm_start_merges),
                           "freeze": bool(self.freeze_warm_start),
                           "seed_merges": [list(map(int, p)) for p in self._seed_warm_start_merges],
                           "frozen_pair_keys": []},
            "histogram_cache": {"enable": False, "valid": False, "force_recount": False,
                                "sizes": {"keys": 0, "counts": 0}},
            "counters": {"bytes_h2d": int(self.bytes_h2d), "bytes_d2h": int(self.bytes_d2h),
                         "h2d_events": int(self.h2d_events), "d2h_events": int(self.d2h_events)},
            "logs": logs,
            "privacy": self._privacy_summary(),
        }
        dataset: dict = {"cpu_fallback_batches": 0, "last_cpu_fallback_ratio": 0.0}
        if self._active_batch_size is not None:
            dataset["active_batch_size"] = int(self._active_batch_size)
        if include_batches:
            rows = None
            if current_batches is not None:
                rows = []
                for b in current_batches:
                    ids, off = _flatten_batch(b)
                    flat = ids.cpu().numpy()
                    rows.extend(flat[int(off[i]):int(off[i + 1])].tolist() for i in range(len(off) - 1))
            else:
                rows = self._current_rows()
            if rows is not None:
                dataset["batches"] = {"sequences": rows, "has_gpu": True,
                                      "active_batch_size": self._active_batch_size}
        if isinstance(dataset_state, Mapping):
            offsets = dataset_state.get("stream_offsets")
            if isinstance(offsets, Mapping) and offsets:
                dataset["stream_offsets"] = {str(k): int(v) for k, v in offsets.items() if isinstance(k, str)}
            try:
                bs = int(dataset_state.get("batch_size")) if dataset_state.get("batch_size") is not None else None
            except (TypeError, ValueError):
                bs = None
            if bs and bs > 0:
                dataset["stream_batch_size"] = bs
        rng: dict = {}
        if self.randomize_ties and self._tie_rng is not None:
            rng["tie_breaker"] = {"seed": int(self._tie_seed_value),
                                  "state": self._encode_random_state(self._tie_rng.getstate())}
        auto_state = self.autoscaler.state_dict() if hasattr(self.autoscaler, "state_dict") else {}
        payload = {"version": CHECKPOINT_SCHEMA_VERSION, "trainer": trainer,
                   "autoscaler": {"state": auto_state}, "dataset": dataset}
        if rng:
            payload["rng"] = rng
        tensors = {"cached_pair_keys": torch.empty((0,), dtype=torch.long),
                   "cached_pair_counts": torch.empty((0,), dtype=torch.int64)}
        eng = self._engine
        if eng is not None and getattr(eng, "_h", None) and eng._h.value:
            st = eng.state()
            if 0 < st.table_keys <= self.SEQUENCE_DUMP_LIMIT:
                keys, counts = eng.export_histogram()
                tensors = {"cached_pair_keys": keys.cpu(), "cached_pair_counts": counts.cpu()}
                trainer["histogram_cache"]["sizes"] = {"keys": int(keys.numel()), "counts": int(counts.numel())}
        return {"payload": payload, "tensors": tensors}

    def load_state_dict(self, state_dict: Mapping[str, Any], *, device_contexts=None, use_cuda: bool = False) -> dict:
        """Restore merges, privacy settings and the tie-break generator (``bpe_trainer.py:1603-1888``).
        Accepts the reference layout (``payload`` / ``tensors``), a bare payload, and this package's
        earlier flat layout.  Returns the resume record ``fit`` works from."""
        empty = {"current_batches": None, "gpu_batches": None, "scale_state": None, "step": len(self.merges),
                 "stage_timings": None, "stage_event_log": [], "host_sync_events": [],
                 "device_snapshot_log": [], "dataset_state": None, "sequences": None}
        if not state_dict:
            return empty
        payload = state_dict.get("payload", state_dict)
        trainer = dict(payload.get("trainer", {}) or {})
        model = trainer.get("model") if isinstance(trainer.get("model"), Mapping) else trainer
        self.base_vocab = int(model.get("base_vocab", self.base_vocab))
        self.target_merges = int(model.get("target_merges", self.target_merges))
        self.merges = [tuple(map(int, p)) for p in model.get("merges", [])]
        self.merge_counts = []
        self.vocab_size = int(model.get("vocab_size", self.base_vocab + len(self.merges)))
        if model.get("privacy_mode") is not None:
            self.privacy_mode = bool(model["privacy_mode"])
        if model.get("randomize_ties") is not None:
            self.randomize_ties = bool(model["randomize_ties"])
        elif model.get("privacy_mode") is not None:
            self.randomize_ties = self.privacy_mode
        if "tie_seed" in model:
            self.tie_seed = int(model["tie_seed"]) if model["tie_seed"] is not None else None
        if model.get("tie_seed_effective") is not None:
            self._tie_seed_value = int(model["tie_seed_effective"])
        elif self.tie_seed is not None:
            self._tie_seed_value = int(self.tie_seed)
        if model.get("privacy_salt") is not None:
            try:
                self._privacy_hash_salt = bytes.fromhex(str(model["privacy_salt"]))
            except ValueError:
                self._privacy_hash_salt = str(model["privacy_salt"]).encode("utf-8")
        privacy = trainer.get("privacy")
        if isinstance(privacy, Mapping):
            mode = str(privacy.get("mode", "")).lower()
            if mode == "none":
                self.privacy_mode = False
            elif mode in ("hash-merges", "tie-randomize"):
                self.privacy_mode = True
            if privacy.get("randomize_ties") is not None:
                self.randomize_ties = bool(privacy["randomize_ties"])
            if privacy.get("tie_seed_effective") is not None:
                self._tie_seed_value = int(privacy["tie_seed_effective"])
        warm = trainer.get("warm_start") if isinstance(trainer.get("warm_start"), Mapping) else {}
        self.freeze_warm_start = bool(warm.get("freeze", self.freeze_warm_start))
        self._seed_warm_start_merges = list(self.merges)
        rng_state = None
        tie = (payload.get("rng") or {}).get("tie_breaker") if isinstance(payload.get("rng"), Mapping) else None
        if isinstance(tie, Mapping):
            if tie.get("seed") is not None:
                self._tie_seed_value = int(tie["seed"])
            if tie.get("state") is not None:
                rng_state = self._decode_random_state(tie["state"])
        self._reset_tie_rng()
        if rng_state is not None and self._tie_rng is not None:
            self._tie_rng.setstate(rng_state)
        dataset = payload.get("dataset") if isinstance(payload.get("dataset"), Mapping) else {}
        if dataset.get("active_batch_size") is not None:
            self._active_batch_size = int(dataset["active_batch_size"])
        sequences = None
        batches = dataset.get("batches")
        if isinstance(batches, Mapping) and isinstance(batches.get("sequences"), list):
            sequences = [[int(t) for t in row] for row in batches["sequences"]]
        stream_state = {k: dataset[k] for k in ("stream_offsets", "stream_batch_size") if k in dataset} or None
        progress = ((trainer.get("logs") or {}).get("telemetry_progress") or {}) if isinstance(trainer.get("logs"), Mapping) else {}
        out = dict(empty)
        out.update({"step": int(model.get("merge_step", len(self.merges))), "sequences": sequences,
                    "dataset_state": stream_state, "stage_timings": progress.get("stage_timings"),
                    "stage_event_log": list(progress.get("stage_event_log", [])),
                    "host_sync_events": list(progress.get("host_sync_events", [])),
                    "device_snapshot_log": list(progress.get("device_snapshot_log", []))})
        return out

    def save_checkpoint(self, path, include_batches: bool = True, *, current_batches=None, stage_timings=None,
                        stage_event_log=None, host_sync_events=None, device_snapshot_log=None,
                        dataset_state=None) -> dict:
        state = self.state_dict(current_batches=current_batches, include_batches=include_batches,
                                stage_timings=stage_timings, stage_event_log=stage_event_log,
                                host_sync_events=host_sync_events, device_snapshot_log=device_snapshot_log,
                                dataset_state=dataset_state)
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, "state.json"), "w", encoding="utf-8") as f:
            json.dump(state["payload"], f, indent=2, sort_keys=True)
        torch.save({k: v.detach().clone().cpu() for k, v in state["tensors"].items()},
                   os.path.join(path, "tensors.pt"))
        return state

    def load_checkpoint(self, path) -> dict:
        """Read ``state.json`` / ``tensors.pt`` of a checkpoint directory and return them as
        ``{"payload", "tensors"}`` for ``fit(resume_state=...)``; nothing is applied here
        (``bpe_trainer.py:1938-1948``)."""
        with open(os.path.join(path, "state.json"), encoding="utf-8") as f:
            payload = json.load(f)
        tensors: dict = {}
        tp = os.path.join(path, "tensors.pt")
        if os.path.exists(tp):
            loaded = torch.load(tp, map_location="cpu")
            if isinstance(loaded, dict):
                tensors = loaded
        return {"payload": payload, "tensors": tensors}

    def export_tokenizer(self, out_dir: str | None = None) -> GPUBPETokenizer:
        """A runtime tokenizer for the learned merges (``bpe_trainer.py:4758-4773``); with ``out_dir``
        the artifacts are written there first and the tokenizer is loaded from ``tokenizer.json``."""
        if out_dir is not None:
            return GPUBPETokenizer.from_file(self.save_artifacts(out_dir)["tokenizer"])
        _, _, config, _ = build_artifacts(self.base_vocab, self.merges, self.vocab_size)
        return GPUBPETokenizer.from_config(config)

    def save_artifacts(self, out_dir) -> dict:
        extra: dict = {"privacy": self._privacy_summary()}
        if self.privacy_mode:
            extra.update({"privacy_mode": True, "merge_count": len(self.merges),
                          "randomize_ties": bool(self.randomize_ties), "tie_seed": int(self._tie_seed_value)})
        return write_artifacts(os.fspath(out_dir), self.base_vocab, self.merges, self.vocab_size,
                               metadata_merges=self._merges_for_metadata(), extra_meta=extra)

    def save(self, out_dir) -> None:
        p = self.save_artifacts(out_dir)
        print("Saved tokenizer artifacts → "
              f"{p['vocab']}, {p['merges']}, {p['tokenizer']}, {p['tiktoken_merges']}")


__all__ = ["GPUBPETokenizer", "GPUBPETrainer", "StageTiming", "hash_merge_pair"]
