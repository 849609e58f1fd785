"""More fixtures made by the reference itself, written to ``extra.json`` in this directory.

    python tests/golden/make_golden_extra.py --reference <path to the reference checkout>

Runs only where the reference source tree is available (CPU torch is enough); tests read the JSON.

  artifacts   the five files the reference's own writer produces (``GPUBPETrainer.save_artifacts``,
              ``gpu_tokenizer/bpe_trainer.py:4615-4756``) for given merge lists, one of them over a base
              vocabulary above 256, as text; ``bpe_merges.json`` with its absolute path field removed.
  ties        merges the reference learns with ``randomize_ties=True`` and a ``tie_seed`` on rows that
              hold many equally frequent pairs, so that several merges in a row are decided by the
              seeded generator (``bpe_trainer.py:915-923``, ``trainers/bpe_gpu.py:112-123``); one case is
              interrupted, written to a checkpoint, and resumed by the reference.
  checkpoint  ``state.json`` of a checkpoint the reference wrote in the middle of a run, with the
              merges the uninterrupted reference run learns in the end.
"""
from __future__ import annotations

import argparse
import contextlib
import io
import json
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import ref_harness as R  # noqa: E402


def tie_rows(rng: np.random.Generator, n_pairs: int, reps: int, alphabet: int):
    """Rows in which ``n_pairs`` different pairs occur ``reps`` times each, separated by unique
    symbols so that no other pair repeats: every selection starts as an ``n_pairs``-way tie."""
    pairs = set()
    while len(pairs) < n_pairs:
        a, b = int(rng.integers(0, alphabet)), int(rng.integers(0, alphabet))
        if a != b:
            pairs.add((a, b))
    pairs = sorted(pairs)
    rows, sep = [], alphabet
    units = [p for p in pairs for _ in range(reps)]
    rng.shuffle(units)
    row = []
    for i, (a, b) in enumerate(units):
        row += [a, b, sep]
        sep += 1
        if len(row) > 60:
            rows.append(row)
            row = []
    if row:
        rows.append(row)
    return rows


def fit(GPUBPETrainer, rows_batches, base_vocab, merges, fit_kw=None, **kw):
    batches = [R.make_batch(rows) for rows in rows_batches]
    t = GPUBPETrainer(base_vocab=base_vocab, merges=merges, device="cpu", **kw)
    t._enable_histogram_cache = False
    with contextlib.redirect_stdout(io.StringIO()):
        t.fit(batches, log_every=0, **(fit_kw or {}))
    return t


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    ref = os.path.abspath(args.reference)
    GPUBPETrainer, _, _, _ = R._import_reference(ref)
    out = {"artifacts": [], "ties": [], "checkpoint": None}
    cwd = os.getcwd()
    with tempfile.TemporaryDirectory() as tmp:
        os.makedirs(os.path.join(tmp, ".artifacts"))
        os.chdir(tmp)
        try:
            # ---------------------------------------------------------------- artifacts
            for base_vocab, merges in ((256, [(104, 101), (108, 108), (256, 257), (258, 111), (32, 259), (0, 255), (10, 13)]),
                                       (300, [(65, 66), (300, 67), (299, 301), (226, 130), (303, 172), (257, 258)])):
                t = GPUBPETrainer(base_vocab=base_vocab, merges=len(merges), device="cpu")
                t.merges = list(merges)
                t.vocab_size = base_vocab + len(merges)
                d = os.path.join(tmp, f"art{base_vocab}")
                paths = t.save_artifacts(d)
                files = {}
                for key, p in paths.items():
                    raw = open(p, "rb").read().decode("utf-8")
                    if key == "metadata":
                        meta = json.loads(raw)
                        meta.pop("tiktoken_merges_path", None)
                        raw = json.dumps(meta, sort_keys=True)
                    files[os.path.basename(p)] = raw
                out["artifacts"].append({"base_vocab": base_vocab, "merges": [list(m) for m in merges], "files": files})
            # ---------------------------------------------------------------- randomised ties
            rng = np.random.default_rng(4242)
            for seed, n_pairs, reps, target in ((7, 9, 3, 8), (123, 14, 2, 12), (0, 6, 4, 6), (99, 20, 2, 16)):
                rows = tie_rows(rng, n_pairs, reps, 40)
                t = fit(GPUBPETrainer, [rows], 256, target, randomize_ties=True, tie_seed=seed)
                plain = fit(GPUBPETrainer, [rows], 256, target)
                out["ties"].append({"rows": rows, "base_vocab": 256, "target": target, "tie_seed": seed,
                                    "merges": [list(m) for m in t.merges],
                                    "merges_without_randomisation": [list(m) for m in plain.merges]})
            # interrupted by the reference: checkpoint after 6 of 12 merges
            rows = out["ties"][1]["rows"]
            half = fit(GPUBPETrainer, [rows], 256, 6, randomize_ties=True, tie_seed=123)
            ck = os.path.join(tmp, "ck_ties")
            half.save_checkpoint(ck, include_batches=False)
            payload = json.load(open(os.path.join(ck, "state.json")))
            out["ties"][1]["checkpoint_after_6"] = payload
            # ---------------------------------------------------------------- a plain checkpoint
            rng = np.random.default_rng(5)
            rows = [rng.integers(0, 6, int(rng.integers(20, 120))).tolist() for _ in range(8)]
            full = fit(GPUBPETrainer, [rows], 256, 18)
            # the reference writes this one itself, inside fit, after merge 7 of a 13-merge run (the
            # next interval would fall past the target), with the rows as they stand at that point
            ck = os.path.join(tmp, "ck_plain")
            fit(GPUBPETrainer, [rows], 256, 13, fit_kw=dict(checkpoint_interval=7, checkpoint_dir=ck))
            state = json.load(open(os.path.join(ck, "state.json")))
            out["checkpoint"] = {"rows": rows, "base_vocab": 256, "target": 18, "state_json": state,
                                 "merges_at_checkpoint": state["trainer"]["model"]["merges"],
                                 "merges_final": [list(m) for m in full.merges]}
        finally:
            os.chdir(cwd)
    with open(os.path.join(HERE, "extra.json"), "w") as f:
        json.dump(out, f, separators=(",", ":"))
    print("wrote extra.json:", {k: (len(v) if isinstance(v, list) else "1") for k, v in out.items()})


if __name__ == "__main__":
    main()
