"""CPU stand-in for one rank of the multi-GPU merge loop (test infrastructure).

It implements the worker interface of ``supertoken_b200.dist`` with the CPU oracle doing the local
work, so that the exchange protocol (owner hashing, chunk capacity and exchange-only rounds,
candidate gathering, the commit decision and the stop rules) can be run over ``gloo`` without a GPU.
The decision logic mirrors ``commit_kernel`` / ``advance_or_stop`` in ``csrc/kernels.cuh``.
"""
from __future__ import annotations

import numpy as np
import torch

from oracle import oracle as O
from supertoken_b200 import _lib as L
from supertoken_b200.dist import owner_of


class CpuWorker:
    def __init__(self, rows, rank: int, world: int, base_vocab: int, max_merges: int, cap_per_peer: int):
        self.ids, self.off = O.flatten_rows(rows)
        self.rank, self.world, self.cap = rank, world, cap_per_peer
        self.base_vocab, self.max_merges = base_vocab, max_merges
        shape = (world, cap_per_peer + 1, 2)
        self.outbox = torch.zeros(shape, dtype=torch.int64)
        self.inbox = torch.zeros(shape, dtype=torch.int64)
        self.cand = torch.zeros(4, dtype=torch.int64)
        self.all_cands = torch.zeros((world, 4), dtype=torch.int64)
        self.table = {}      # keys this rank owns -> count
        self.pending = {}    # local deltas not yet sent
        self.merges, self.counts = [], []
        self.cur = None
        self.exchange_only = False
        self.stop_reason = L.RUNNING
        self.incomplete = False

    # -- local work ---------------------------------------------------------------------
    def _hist(self):
        k, c = O.count_pairs_flat(self.ids[:self.off[-1]].copy(), self.off, 1)
        return {int(a): int(b) for a, b in zip(k, c)}

    def _drain(self):
        self.outbox.zero_()
        self.incomplete = False
        fill = [0] * self.world
        kept = {}
        for key in sorted(self.pending):
            d = self.pending[key]
            if d == 0:
                continue
            o = owner_of(key, self.world)
            if fill[o] >= self.cap:
                kept[key] = d
                self.incomplete = True
                fill[o] += 1
                continue
            self.outbox[o, 1 + fill[o], 0] = np.int64(np.uint64(key))
            self.outbox[o, 1 + fill[o], 1] = d
            fill[o] += 1
        for o in range(self.world):
            self.outbox[o, 0, 0] = fill[o]
        self.pending = kept

    def count_local(self):
        for k, c in self._hist().items():
            self.pending[k] = self.pending.get(k, 0) + c
        self._drain()

    def merge_local(self):
        if self.stop_reason == L.RUNNING and not self.exchange_only and self.cur is not None:
            a, b, new = self.cur
            before = self._hist()
            O.apply_merge_flat(self.ids, self.off, a, b, new)
            after = self._hist()
            merged = (a << 32) | b
            for k in set(before) | set(after):
                if k == merged:
                    continue  # the owner zeroes the merged pair's entry when it commits
                d = after.get(k, 0) - before.get(k, 0)
                if d:
                    self.pending[k] = self.pending.get(k, 0) + d
        self._drain()

    def apply_inbox(self):
        for p in range(self.world):
            n = int(self.inbox[p, 0, 0])
            if n > self.cap:
                n = self.cap
                self.incomplete = True
            for i in range(n):
                key = int(np.uint64(np.int64(self.inbox[p, 1 + i, 0].item())))
                self.table[key] = self.table.get(key, 0) + int(self.inbox[p, 1 + i, 1])

    def candidate(self):
        best_k, best_c = 0, 0
        for k, c in self.table.items():
            if c > best_c or (c == best_c and c > 0 and k < best_k):
                best_k, best_c = k, c
        self.cand[0] = np.int64(np.uint64(best_k))
        self.cand[1] = best_c
        self.cand[2] = int(self.incomplete)
        self.cand[3] = 0

    def commit(self):
        if self.stop_reason != L.RUNNING:
            return
        best_k, best_c, incomplete = 0, 0, False
        for r in range(self.world):
            k = int(np.uint64(np.int64(self.all_cands[r, 0].item())))
            c = int(self.all_cands[r, 1])
            incomplete |= bool(self.all_cands[r, 2])
            if c > 0 and (c > best_c or (c == best_c and k < best_k)):
                best_k, best_c = k, c
        if incomplete:
            self.exchange_only = True
            return
        self.exchange_only = False
        if len(self.merges) >= self.max_merges:
            self.stop_reason = L.STOP_TARGET
        elif best_c <= 0:
            self.stop_reason = L.STOP_NO_PAIRS
        elif best_c < 2:
            self.stop_reason = L.STOP_LOW_COUNT
        else:
            a, b = best_k >> 32, best_k & 0xFFFFFFFF
            self.cur = (a, b, self.base_vocab + len(self.merges))
            self.merges.append((a, b))
            self.counts.append(best_c)
            if best_k in self.table:
                self.table[best_k] = 0

    def progress(self):
        return len(self.merges), self.stop_reason
