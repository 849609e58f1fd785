"""Run the *reference itself* (imported from its source tree) on CPU.

TEST INFRASTRUCTURE ONLY, and usable only where the reference checkout exists: it
is how the golden fixtures under ``tests/golden/`` were produced and how the C
oracle was pinned.  Nothing that runs on a GPU box imports this module.

The reference trainer must be driven in its "recount" mode
(``SUPERTOKEN_PARITY_ALWAYS_RECOUNT=1``, read at ``gpu_tokenizer/bpe_trainer.py:812``):
its default histogram-cache path leaves the pair list empty after the first merge
and pads with random pairs (``bpe_trainer.py:4224-4239``, ``:4344-4353``).  ``fit``
also appends to ``./.artifacts/temp_debug.txt`` (``:4194-4196``), so it is run from a
scratch directory that has that folder.
"""
from __future__ import annotations

import contextlib
import io
import os
import sys
import tempfile
from typing import List, Sequence, Tuple

import numpy as np


def _import_reference(root: str):
    os.environ["SUPERTOKEN_PARITY_ALWAYS_RECOUNT"] = "1"
    if root not in sys.path:
        sys.path.insert(0, root)
    import torch  # noqa: F401
    from gpu_tokenizer import cpu_fastpath, utils  # type: ignore
    from gpu_tokenizer.bpe_trainer import GPUBPETrainer  # type: ignore
    from gpu_tokenizer.trainers import bpe_gpu  # type: ignore
    return GPUBPETrainer, cpu_fastpath, utils, bpe_gpu


def make_batch(rows: Sequence[Sequence[int]]):
    """Padded ``(tokens, valid, lengths)`` as the reference's batchers emit them
    (``gpu_tokenizer/datasets.py:42-92``): pad id -1, valid 0/1, prefix-valid."""
    import torch
    width = max(1, max((len(r) for r in rows), default=0))
    tokens = torch.full((len(rows), width), -1, dtype=torch.int32)
    valid = torch.zeros((len(rows), width), dtype=torch.uint8)
    lengths = torch.zeros((len(rows),), dtype=torch.int32)
    for i, r in enumerate(rows):
        if len(r):
            tokens[i, :len(r)] = torch.tensor(list(r), dtype=torch.int32)
            valid[i, :len(r)] = 1
            lengths[i] = len(r)
    return tokens, valid, lengths


def reference_fit(root: str, row_batches: Sequence[Sequence[Sequence[int]]], base_vocab: int,
                  merges: int, **ctor) -> Tuple[List[Tuple[int, int]], int]:
    """Train the reference on CPU in recount mode.  Returns (merges, vocab_size)."""
    GPUBPETrainer, _, _, _ = _import_reference(root)
    batches = [make_batch(rows) for rows in row_batches]
    cwd = os.getcwd()
    with tempfile.TemporaryDirectory() as tmp:
        os.makedirs(os.path.join(tmp, ".artifacts"))
        os.chdir(tmp)
        try:
            trainer = GPUBPETrainer(base_vocab=base_vocab, merges=merges, device="cpu", **ctor)
            trainer._enable_histogram_cache = False
            with contextlib.redirect_stdout(io.StringIO()):
                trainer.fit(batches, log_every=0)
        finally:
            os.chdir(cwd)
    return [(int(a), int(b)) for a, b in trainer.merges], int(trainer.vocab_size)


def reference_count_pairs(root: str, tokens: np.ndarray, valid: np.ndarray):
    """``cpu_fastpath.count_pairs_fastpath`` (``gpu_tokenizer/cpu_fastpath.py:59-92``)."""
    import torch
    _, cpu_fastpath, _, _ = _import_reference(root)
    k, c = cpu_fastpath.count_pairs_fastpath(torch.from_numpy(tokens.copy()),
                                             torch.from_numpy(valid.copy()))
    return k.numpy().astype(np.uint64), c.numpy().astype(np.int64)


def reference_apply_merge(root: str, tokens: np.ndarray, valid: np.ndarray, a: int, b: int,
                          new_id: int):
    """``utils.apply_merge_once`` CPU branch (``gpu_tokenizer/utils.py:413-555``)."""
    import torch
    _, _, utils, _ = _import_reference(root)
    t = torch.from_numpy(tokens.copy())
    v = torch.from_numpy(valid.copy())
    lengths = v.sum(dim=1).to(torch.int32)
    t, v, lengths, spans = utils.apply_merge_once(t, v, lengths, a, b, new_id)
    return t.numpy(), v.numpy(), lengths.numpy().astype(np.int64), spans.numpy().astype(bool)


def reference_select(root: str, keys: np.ndarray, counts: np.ndarray):
    """``select_best_pair`` (``gpu_tokenizer/trainers/bpe_gpu.py:96-130``)."""
    import torch
    _, _, _, bpe_gpu = _import_reference(root)
    h = bpe_gpu.PairHistogramResult(torch.from_numpy(keys.astype(np.int64)),
                                    torch.from_numpy(counts.astype(np.int64)))
    key, count, _ = bpe_gpu.select_best_pair(h)
    return key, count
