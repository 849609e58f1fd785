"""``train-bpe`` with the reference's flags on top of the B200 engine.

    python -m supertoken_b200.cli train-bpe --data 'corpus/*.txt' --merges 32000 --out-dir out

Mirrors ``main.py train-bpe`` of the reference (``main.py:2194-2356``; ``_cmd_train_bpe``
``:1182-1646``): one file is one row (``gpu_tokenizer/datasets.py:167-172``), bytes map to ids
unchanged, optional BOS / EOS ids are added per row (``gpu_tokenizer/cpu_packer.py:52-61``), the
trainer's artifacts are written to ``--out-dir``.  Flags that steer parts of the reference outside
the merge loop (streaming workers, autoscaler targets, morphology, code mode, augmentation) are
accepted so that existing command lines keep parsing; they do not influence the merges.
``--warm-start`` names a JSON manifest or TikToken bundle of seed merges that are applied before the
loop (``main.py:2351-2356``, loader ``:501-575``); ``--checkpoint-dir`` / ``--checkpoint-every`` write
``state.json`` + ``tensors.pt`` during training and ``--resume-from`` continues from such a directory
(``main.py:1397-1571``).
"""
from __future__ import annotations

import argparse
import glob
import os
import sys
from typing import List, Sequence

import numpy as np


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="supertoken_b200")
    sub = ap.add_subparsers(dest="command", required=True)
    p = sub.add_parser("train-bpe", help="train a byte-level BPE tokenizer on the GPU")
    p.add_argument("--data", nargs="+", required=True, help="files or glob patterns; one file = one row")
    p.add_argument("--bos", type=int, default=None)
    p.add_argument("--eos", type=int, default=None)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--device", default="cuda")
    p.add_argument("--merges", type=int, default=50_000)
    p.add_argument("--base-vocab", type=int, default=256)
    p.add_argument("--log-every", type=int, default=100)
    p.add_argument("--out-dir", default="out")
    p.add_argument("--privacy", type=str, default="none", choices=["none", "hash-merges", "tie-randomize"])
    p.add_argument("--privacy-salt", default=None)
    p.add_argument("--tie-seed", type=int, default=None)
    p.add_argument("--checkpoint-dir", default=None)
    p.add_argument("--checkpoint-every", type=int, default=None)
    p.add_argument("--resume-from", default=None)
    p.add_argument("--dry-run", action="store_true")
    p.add_argument("--warm-start", type=str, default=None,
                   help="JSON manifest or TikToken bundle containing seed merges")
    # accepted for command-line compatibility; outside the merge loop
    for flag, kw in (("--target-util", dict(type=float, default=0.9)), ("--min-batch", dict(type=int, default=1)),
                     ("--max-batch", dict(type=int, default=65536)), ("--token-bytes", dict(type=int, default=8192)),
                     ("--compression", dict(default=None)),
                     ("--io-workers", dict(type=int, default=1)), ("--prefetch-batches", dict(type=int, default=2)),
                     ("--prefetch-jitter", dict(type=float, default=0.0)), ("--code-mode", dict(action="store_true")),
                     ("--code-langs", dict(nargs="*", default=None)), ("--meta-compress", dict(action="store_true")),
                     ("--augmentation", dict(default=None)), ("--aug-strength", dict(type=float, default=0.0))):
        p.add_argument(flag, **kw)
    return ap


def expand_patterns(patterns: Sequence[str]) -> List[str]:
    paths: List[str] = []
    for pat in patterns:
        hits = sorted(glob.glob(pat, recursive=True))
        paths.extend(hits if hits else ([pat] if os.path.exists(pat) else []))
    return sorted(dict.fromkeys(p for p in paths if os.path.isfile(p)))


def load_rows(paths: Sequence[str], bos, eos):
    """Concatenate the files into one id buffer with row offsets (a row per file)."""
    chunks, offsets = [], [0]
    wide = (bos is not None and bos > 255) or (eos is not None and eos > 255)
    for p in paths:
        b = np.fromfile(p, dtype=np.uint8)
        parts = []
        if bos is not None:
            parts.append(np.array([bos], dtype=np.int32))
        parts.append(b.astype(np.int32) if (wide or bos is not None or eos is not None) else b)
        if eos is not None:
            parts.append(np.array([eos], dtype=np.int32))
        row = np.concatenate(parts) if len(parts) > 1 else parts[0]
        chunks.append(row)
        offsets.append(offsets[-1] + len(row))
    data = np.concatenate(chunks) if chunks else np.zeros(0, dtype=np.uint8)
    return data, np.asarray(offsets, dtype=np.int64)


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    paths = expand_patterns(args.data)
    if not paths:
        print("No input files matched --data", file=sys.stderr)
        return 2
    if args.dry_run:
        print(f"{len(paths)} files, {sum(os.path.getsize(p) for p in paths)} bytes; nothing trained (--dry-run)")
        return 0
    from .bpe_trainer import GPUBPETrainer
    data, off = load_rows(paths, args.bos, args.eos)
    # privacy modes as the reference's factory maps them (main.py:674-689)
    trainer = GPUBPETrainer(base_vocab=args.base_vocab, merges=args.merges, device=args.device,
                            privacy_mode=args.privacy != "none", randomize_ties=args.privacy == "tie-randomize",
                            tie_seed=args.tie_seed, privacy_salt=args.privacy_salt)
    from .export import load_warm_start_merges
    warm = load_warm_start_merges(args.warm_start)
    resume_state = None
    if args.resume_from:
        resume_state = trainer.load_checkpoint(args.resume_from)
        model = resume_state["payload"].get("trainer", {}).get("model", {})
        print(f"[checkpoint] Restored checkpoint from {args.resume_from} at merge {model.get('merge_step')}")
        if model.get("target_merges") is not None and int(model["target_merges"]) != int(args.merges):
            # the reference refuses to resume towards another target (main.py:1465-1483)
            print("[checkpoint] Error: CLI --merges does not match checkpoint target_merges", file=sys.stderr)
            return 2
    every = args.checkpoint_every if args.checkpoint_dir else None
    if data.dtype == np.uint8:
        trainer.fit_bytes(data, off, log_every=args.log_every, warm_start_merges=warm,
                          checkpoint_interval=every, checkpoint_dir=args.checkpoint_dir, resume_state=resume_state)
    else:
        import torch
        L = int(np.diff(off).max()) if len(off) > 1 else 1
        tokens = torch.full((len(off) - 1, max(L, 1)), -1, dtype=torch.int32)
        valid = torch.zeros_like(tokens, dtype=torch.uint8)
        for r in range(len(off) - 1):
            n = int(off[r + 1] - off[r])
            tokens[r, :n] = torch.from_numpy(data[off[r]:off[r + 1]])
            valid[r, :n] = 1
        trainer.fit([(tokens, valid, valid.sum(dim=1).to(torch.int32))], log_every=args.log_every,
                    warm_start_merges=warm, checkpoint_interval=every, checkpoint_dir=args.checkpoint_dir,
                    resume_state=resume_state)
    if args.checkpoint_dir:
        trainer.save_checkpoint(args.checkpoint_dir)
    trainer.save(args.out_dir)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
