"""Shared helpers for the parity tests."""
from __future__ import annotations

import json
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_golden(name: str):
    with open(os.path.join(GOLDEN, name)) as f:
        return json.load(f)


def corpus_rows(c):
    d = np.asarray(c.data.cpu() if hasattr(c.data, "cpu") else c.data)
    off = np.asarray(c.row_offsets.cpu() if hasattr(c.row_offsets, "cpu") else c.row_offsets)
    return [d[off[i]:off[i + 1]].astype(np.int32) for i in range(len(off) - 1)]


def learned_prefix(case, oracle_merges, reason):
    """Split a reference run into learned merges and random pads.

    The reference pads with unseeded random pairs once the best count is below 2
    (gpu_tokenizer/bpe_trainer.py:4347-4353).  The learned part is the prefix that the
    oracle reproduces; the checks here are that this prefix is identical and that the
    reference's total length follows the stop rule."""
    raw = [tuple(m) for m in case["merges_raw"]]
    n = len(oracle_merges)
    assert raw[:n] == [tuple(m) for m in oracle_merges]
    if reason == 0:
        assert len(raw) == case["target"] == n
    elif reason == 1:  # no pairs at all: stop, no padding (bpe_trainer.py:4304-4308)
        assert len(raw) == n
    else:  # count < 2: padded up to the target
        assert len(raw) == case["target"]
    return raw[:n]
