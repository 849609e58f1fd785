"""ctypes/numpy front end of the C oracle (``bpe_oracle.c``).

TEST INFRASTRUCTURE ONLY.  Only tests, the smoke check and the bench's CPU
baseline may import this module; the product package never does.

Parity status: pinned -- see the header of ``bpe_oracle.c``.
"""
from __future__ import annotations

import ctypes
import os
import random
import subprocess
from typing import List, Optional, Sequence, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liborc.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile ``liborc.so`` next to its source if missing or stale."""
    src = os.path.join(_HERE, "bpe_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    if force or stale:
        base = ["gcc", "-O3", "-fPIC", "-fvisibility=hidden", "-shared", "-o", _LIB_PATH, src]
        # OpenMP only speeds up the "fast" recount; fall back to a serial build without it
        if subprocess.call(base + ["-fopenmp"], stderr=subprocess.DEVNULL) != 0:
            subprocess.check_call(base)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        i64, i32, vp = ctypes.c_int64, ctypes.c_int32, ctypes.c_void_p
        L.orc_count_pairs_rows.restype = i64
        L.orc_count_pairs_rows.argtypes = [vp, vp, i64, i64, vp, vp, i64]
        L.orc_apply_merge_rows.restype = None
        L.orc_apply_merge_rows.argtypes = [vp, vp, vp, i64, i64, i32, i32, i32, vp]
        L.orc_select_best.restype = i64
        L.orc_select_best.argtypes = [vp, vp, i64, vp, vp]
        L.orc_count_pairs_flat.restype = i64
        L.orc_count_pairs_flat.argtypes = [vp, vp, i64, ctypes.c_int, vp, vp, i64]
        L.orc_apply_merge_flat.restype = i64
        L.orc_apply_merge_flat.argtypes = [vp, vp, i64, i32, i32, i32]
        L.orc_train_flat.restype = i64
        L.orc_train_flat.argtypes = [vp, vp, i64, i32, i64, ctypes.c_int, vp, vp, vp]
        L.orc_num_threads.restype = ctypes.c_int
        L.orc_set_threads.restype = None
        L.orc_set_threads.argtypes = [ctypes.c_int]
        _lib = L
    return _lib


def _p(a: np.ndarray) -> ctypes.c_void_p:
    return ctypes.c_void_p(a.ctypes.data)


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_threads(n: Optional[int] = None) -> int:
    """Threads of the threaded recount; default = the cores this process may run on."""
    if n is None:
        try:
            n = len(os.sched_getaffinity(0))
        except AttributeError:
            n = os.cpu_count() or 1
    lib().orc_set_threads(int(n))
    return num_threads()


# --------------------------------------------------------------------------- rows API
def count_pairs_rows(tokens: np.ndarray, valid: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """Histogram of adjacent valid pairs of a padded ``[B, L]`` batch.

    Follows ``gpu_tokenizer/utils.py:558-635``.  Returns (keys uint64 ascending,
    counts int64)."""
    tokens = np.ascontiguousarray(tokens, dtype=np.int32)
    valid = np.ascontiguousarray(valid, dtype=np.uint8)
    B, L = tokens.shape
    cap = max(B * max(L - 1, 0), 1)
    keys = np.empty(cap, dtype=np.uint64)
    counts = np.empty(cap, dtype=np.int64)
    n = lib().orc_count_pairs_rows(_p(tokens), _p(valid), B, L, _p(keys), _p(counts), cap)
    if n < 0:
        raise RuntimeError("pair workspace capacity exceeded" if n == -1 else "oracle alloc failure")
    return keys[:n].copy(), counts[:n].copy()


def apply_merge_rows(tokens: np.ndarray, valid: np.ndarray, a: int, b: int, new_id: int):
    """In-place merge + stable compaction of a padded batch
    (``gpu_tokenizer/utils.py:515-555``, ``:347-410``).  Returns (lengths, spans)."""
    assert tokens.dtype == np.int32 and valid.dtype == np.uint8
    assert tokens.flags.c_contiguous and valid.flags.c_contiguous
    B, L = tokens.shape
    lengths = np.zeros(B, dtype=np.int64)
    spans = np.zeros((B, max(L - 1, 0)), dtype=np.uint8)
    lib().orc_apply_merge_rows(_p(tokens), _p(valid), _p(lengths), B, L, a, b, new_id, _p(spans))
    return lengths, spans.astype(bool)


def select_best(keys: np.ndarray, counts: np.ndarray) -> Tuple[Optional[int], int]:
    """Max count, ties to the smallest packed key (``trainers/bpe_gpu.py:96-130``)."""
    keys = np.ascontiguousarray(keys, dtype=np.uint64)
    counts = np.ascontiguousarray(counts, dtype=np.int64)
    bk = ctypes.c_uint64(0)
    bc = ctypes.c_int64(0)
    i = lib().orc_select_best(_p(keys), _p(counts), len(keys), ctypes.byref(bk), ctypes.byref(bc))
    if i < 0:
        return None, 0
    return int(bk.value), int(bc.value)


# --------------------------------------------------------------------------- flat API
def flatten_rows(rows: Sequence[Sequence[int]]) -> Tuple[np.ndarray, np.ndarray]:
    off = np.zeros(len(rows) + 1, dtype=np.int64)
    for i, r in enumerate(rows):
        off[i + 1] = off[i] + len(r)
    ids = np.empty(int(off[-1]), dtype=np.int32)
    for i, r in enumerate(rows):
        ids[off[i]:off[i + 1]] = np.asarray(r, dtype=np.int32)
    return ids, off


def count_pairs_flat(ids: np.ndarray, off: np.ndarray, mode: int = 1):
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    off = np.ascontiguousarray(off, dtype=np.int64)
    cap = max(int(off[-1] - off[0]), 1)
    keys = np.empty(cap, dtype=np.uint64)
    counts = np.empty(cap, dtype=np.int64)
    n = lib().orc_count_pairs_flat(_p(ids), _p(off), len(off) - 1, mode, _p(keys), _p(counts), cap)
    if n < 0:
        raise RuntimeError(f"oracle count failed ({n})")
    return keys[:n].copy(), counts[:n].copy()


def apply_merge_flat(ids: np.ndarray, off: np.ndarray, a: int, b: int, new_id: int) -> int:
    """In place on ``ids``/``off``; live data is ``ids[:off[-1]]`` afterwards."""
    assert ids.dtype == np.int32 and off.dtype == np.int64
    return int(lib().orc_apply_merge_flat(_p(ids), _p(off), len(off) - 1, a, b, new_id))


def train_flat(ids: np.ndarray, off: np.ndarray, base_vocab: int, target: int, mode: int = 1,
               copy: bool = True):
    """Run the recount merge loop (``gpu_tokenizer/bpe_trainer.py:4193-4517``).

    Returns ``(merges list[(a, b)], counts list[int], reason)`` with reason
    0 = target reached, 1 = no pairs left, 2 = best count < 2."""
    ids = np.array(ids, dtype=np.int32, copy=True) if copy else ids
    off = np.array(off, dtype=np.int64, copy=True) if copy else off
    merges = np.zeros(2 * max(target, 1), dtype=np.int32)
    counts = np.zeros(max(target, 1), dtype=np.int64)
    reason = ctypes.c_int32(0)
    n = lib().orc_train_flat(_p(ids), _p(off), len(off) - 1, base_vocab, target, mode,
                             _p(merges), _p(counts), ctypes.byref(reason))
    if n < 0:
        raise RuntimeError(f"oracle train failed ({n})")
    m = [(int(merges[2 * i]), int(merges[2 * i + 1])) for i in range(n)]
    return m, [int(c) for c in counts[:n]], int(reason.value)


def pad_merges(merges: List[Tuple[int, int]], base_vocab: int, target: int, reason: int,
               rng=random) -> List[Tuple[int, int]]:
    """Host-side padding of ``gpu_tokenizer/bpe_trainer.py:4344-4353``: when the
    best count falls below 2 the reference appends random pairs, two
    ``randint(0, vocab-1)`` draws per pad with the vocabulary growing by one each
    time; when no pairs are left at all it stops without padding (:4304-4308)."""
    out = list(merges)
    if reason == 2:
        vocab = base_vocab + len(out)
        while len(out) < target:
            out.append((rng.randint(0, vocab - 1), rng.randint(0, vocab - 1)))
            vocab += 1
    return out
