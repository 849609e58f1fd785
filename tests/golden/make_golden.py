"""Regenerate the golden fixtures in this directory from the reference itself.

    python tests/golden/make_golden.py --reference <path to the reference checkout>

Runs only where the reference source tree is available (CPU torch is enough).  It
imports the reference, drives it in recount mode through ``oracle/ref_harness.py``
and stores inputs and outputs as JSON.  The GPU box never runs this script; it
only reads the JSON files.

Fixtures:
  ops.json       operator level: count_pairs_fastpath, apply_merge_once and
                 select_best_pair on seeded random padded batches (non-prefix valid
                 masks included, as in the reference's own count test).
  train.json     trainer level: merges learned by the reference trainer on seeded
                 random rows (tiny alphabets, long equal-token runs, empty rows,
                 several batches), on the reference's adversarial corpora (imported,
                 not transcribed) and on small prefixes of the synthetic configs
                 (inputs regenerated from supertoken_b200.synth; only SHA-256 and
                 merges are stored for those).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import ref_harness as R  # noqa: E402
from supertoken_b200 import synth  # noqa: E402


def random_rows(rng: np.random.Generator, n_rows: int, max_len: int, alphabet: int, run_p: float):
    rows = []
    for _ in range(n_rows):
        n = int(rng.integers(0, max_len + 1))
        row = []
        while len(row) < n:
            if rng.random() < run_p:
                sym = int(rng.integers(0, alphabet))
                if rng.random() < 0.5:
                    row += [sym] * int(rng.integers(2, 40))
                else:
                    sym2 = int(rng.integers(0, alphabet))
                    row += [sym, sym2] * int(rng.integers(1, 20))
            else:
                row.append(int(rng.integers(0, alphabet)))
        rows.append(row[:n])
    return rows


def corpus_rows(c):
    d = np.asarray(c.data)
    off = np.asarray(c.row_offsets)
    return [d[off[i]:off[i + 1]].astype(int).tolist() for i in range(len(off) - 1)]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    ref = os.path.abspath(args.reference)

    # ------------------------------------------------------------------ operator level
    ops = {"count": [], "apply": [], "select": []}
    rng = np.random.default_rng(20240)
    for case in range(12):
        B, L = int(rng.integers(1, 7)), int(rng.integers(2, 48))
        alphabet = int(rng.choice([2, 3, 8, 512]))
        tokens = rng.integers(0, alphabet, (B, L)).astype(np.int32)
        if case % 3 == 0:
            valid = rng.integers(0, 2, (B, L)).astype(np.uint8)  # arbitrary mask
        else:
            lens = rng.integers(0, L + 1, B)
            valid = (np.arange(L)[None, :] < lens[:, None]).astype(np.uint8)
        k, c = R.reference_count_pairs(ref, tokens, valid)
        ops["count"].append({"tokens": tokens.tolist(), "valid": valid.tolist(),
                             "keys": [int(x) for x in k], "counts": [int(x) for x in c]})
        if len(k):
            bk, bc = R.reference_select(ref, k, c)
            ops["select"].append({"keys": [int(x) for x in k], "counts": [int(x) for x in c],
                                  "best_key": bk, "best_count": bc})
        a, b = int(tokens[0, 0]), int(tokens[0, min(1, L - 1)])
        if case % 2 == 0:
            b = a
        t2, v2, lens2, spans = R.reference_apply_merge(ref, tokens, valid, a, b, 1000 + case)
        ops["apply"].append({"tokens": tokens.tolist(), "valid": valid.tolist(), "a": a, "b": b,
                             "new": 1000 + case, "out_tokens": t2.tolist(),
                             "out_valid": v2.tolist(), "out_lengths": lens2.tolist(),
                             "spans": spans.astype(int).tolist()})
    # hand-made ties for the selector
    for keys, counts in ([[5, 3, 9], [4, 4, 4]], [[(1 << 32) | 2, (0 << 32) | 7, 3], [2, 9, 9]],
                         [[8, 1], [1, 1]]):
        bk, bc = R.reference_select(ref, np.array(keys, dtype=np.uint64), np.array(counts))
        ops["select"].append({"keys": keys, "counts": counts, "best_key": bk, "best_count": bc})
    with open(os.path.join(HERE, "ops.json"), "w") as f:
        json.dump(ops, f, separators=(",", ":"))

    # ------------------------------------------------------------------ trainer level
    train = {"random": [], "adversarial": [], "synthetic": []}
    rng = np.random.default_rng(777)
    for case in range(40):
        alphabet = int(rng.choice([1, 2, 3, 4, 16, 200]))
        n_batches = int(rng.integers(1, 4))
        batches = [random_rows(rng, int(rng.integers(1, 6)), int(rng.choice([4, 33, 150])),
                               alphabet, float(rng.choice([0.0, 0.2, 0.6])))
                   for _ in range(n_batches)]
        target = int(rng.integers(1, 25))
        merges, vocab = R.reference_fit(ref, batches, 256, target)
        # the reference pads with unseeded random pairs once the best count drops
        # below 2; keep only the learned prefix (a learned merge never repeats)
        rows = [r for b in batches for r in b]
        train["random"].append({"rows": rows, "n_batches": n_batches, "base_vocab": 256,
                                "target": target, "merges_raw": merges, "vocab_size": vocab})

    sys.path.insert(0, ref)
    from tests.adversarial_corpora import iter_adversarial_corpora  # type: ignore
    for corpus in iter_adversarial_corpora():
        rows = [list(s.encode("utf-8")) for s in corpus.iter_corpus()]
        merges, vocab = R.reference_fit(ref, [rows], 256, corpus.target_merge_operations)
        train["adversarial"].append({"name": corpus.name, "rows": rows, "base_vocab": 256,
                                     "target": corpus.target_merge_operations,
                                     "merges_raw": merges, "vocab_size": vocab})

    specs = [("config1_text", dict(n_bytes=192 << 10, seed=0, file_bytes=12 << 10), 48),
             ("config2_mixed", dict(n_bytes=128 << 10, seed=1, mean_doc_bytes=1024, lexicon=5000), 48),
             ("config5_adversarial", dict(n_bytes=160 << 10, seed=4), 32)]
    for fn, kw, target in specs:
        c = getattr(synth, fn)(**kw)
        rows = corpus_rows(c)
        merges, vocab = R.reference_fit(ref, [rows], 256, target)
        train["synthetic"].append({"generator": fn, "kwargs": kw, "sha256": c.sha256(),
                                   "n_rows": len(rows), "base_vocab": 256, "target": target,
                                   "merges_raw": merges, "vocab_size": vocab})
        print(fn, "done", len(merges), flush=True)
    with open(os.path.join(HERE, "train.json"), "w") as f:
        json.dump(train, f, separators=(",", ":"))
    print("wrote fixtures")


if __name__ == "__main__":
    main()
