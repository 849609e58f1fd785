"""Tokenizer artifact writers with the reference's file formats.

Restates ``GPUBPETrainer._build_tokenizer_artifacts`` / ``_write_tokenizer_artifacts``
(``gpu_tokenizer/bpe_trainer.py:4615-4756``) and the byte-level / TikToken helpers
(``gpu_tokenizer/export/artifacts.py:705-725``, ``:743-781``): identical merges give
byte-identical ``vocab.json``, ``merges.txt``, ``tokenizer.json`` and ``merges.tiktoken``.
"""
from __future__ import annotations

import base64
import json
import os
from typing import Dict, List, Sequence, Tuple


def bytes_to_unicode() -> Dict[int, str]:
    """The byte -> printable unicode alphabet of byte-level BPE tokenizers: printable
    Latin-1 bytes map to themselves, the rest to code points from 256 upwards."""
    keep = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
    mapping = {b: chr(b) for b in keep}
    extra = 0
    for b in range(256):
        if b not in mapping:
            mapping[b] = chr(256 + extra)
            extra += 1
    return mapping


def build_artifacts(base_vocab: int, merges: Sequence[Tuple[int, int]], vocab_size: int):
    enc = bytes_to_unicode()
    tokens: List[str] = []
    added = []
    for tid in range(base_vocab):
        if tid < 256:
            tokens.append(enc[tid])
        else:
            content = f"<|{tid}|>"
            tokens.append(content)
            added.append({"id": tid, "content": content, "single_word": False, "lstrip": False,
                          "rstrip": False, "normalized": False, "special": True})
    for idx, (left, right) in enumerate(merges):
        if not (0 <= left < len(tokens) and 0 <= right < len(tokens)):
            raise ValueError(f"Invalid merge pair {(left, right)} at position {idx}")
        tokens.append(tokens[left] + tokens[right])
    expected = base_vocab + len(merges)
    if vocab_size != expected:
        raise ValueError(f"Mismatch between vocab_size and merges: expected {expected}, found {vocab_size}")
    vocab = {tok: i for i, tok in enumerate(tokens)}
    merge_lines = [f"{tokens[l]} {tokens[r]}" for l, r in merges]
    byte_level = {"type": "ByteLevel", "add_prefix_space": False, "trim_offsets": True, "use_regex": True}
    config = {
        "version": "1.0", "truncation": None, "padding": None, "added_tokens": added,
        "normalizer": None, "pre_tokenizer": dict(byte_level), "post_processor": None,
        "decoder": dict(byte_level),
        "model": {"type": "BPE", "dropout": None, "unk_token": None, "continuing_subword_prefix": "",
                  "end_of_word_suffix": "", "fuse_unk": False, "byte_fallback": False,
                  "vocab": vocab, "merges": merge_lines},
    }
    dec = {v: k for k, v in enc.items()}
    special = {e["content"] for e in added}
    ranks: Dict[bytes, int] = {}
    for tok, rank in sorted(vocab.items(), key=lambda kv: kv[1]):
        if tok in special:
            continue
        ranks[bytes(dec[ch] for ch in tok)] = rank
    return vocab, merge_lines, config, ranks


def write_artifacts(out_dir: str, base_vocab: int, merges: Sequence[Tuple[int, int]], vocab_size: int,
                    metadata_merges=None, extra_meta=None) -> Dict[str, str]:
    vocab, merge_lines, config, ranks = build_artifacts(base_vocab, merges, vocab_size)
    os.makedirs(out_dir, exist_ok=True)
    paths = {k: os.path.join(out_dir, v) for k, v in
             (("vocab", "vocab.json"), ("merges", "merges.txt"), ("tokenizer", "tokenizer.json"),
              ("metadata", "bpe_merges.json"), ("tiktoken_merges", "merges.tiktoken"))}
    with open(paths["vocab"], "w", encoding="utf-8") as f:
        json.dump(vocab, f, ensure_ascii=False)
    with open(paths["merges"], "w", encoding="utf-8") as f:
        f.write("#version: 0.2\n")
        for line in merge_lines:
            f.write(f"{line}\n")
    with open(paths["tokenizer"], "w", encoding="utf-8") as f:
        json.dump(config, f, ensure_ascii=False)
    with open(paths["tiktoken_merges"], "wb") as f:
        for tok, rank in sorted(ranks.items(), key=lambda kv: kv[1]):
            f.write(base64.b64encode(tok) + b" " + str(rank).encode("ascii") + b"\n")
    meta = {"base_vocab": base_vocab, "vocab_size": vocab_size,
            "merges": metadata_merges if metadata_merges is not None else [list(map(int, p)) for p in merges],
            "tiktoken_merges_path": paths["tiktoken_merges"]}
    meta.update(extra_meta or {})
    with open(paths["metadata"], "w", encoding="utf-8") as f:
        json.dump(meta, f)
    return paths
