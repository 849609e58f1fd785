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


# ----------------------------------------------------------------------------- imports of merges
def tiktoken_ranks_to_merges(ranks: Dict[bytes, int], base_vocab: int | None = None) -> List[Tuple[int, int]]:
    """Merge pairs behind a TikToken rank table (``export/artifacts.py:800-858`` of the reference):
    tokens in rank order; every token past the base vocabulary is the concatenation of two earlier
    tokens, and the split tried first (shortest left part) is the one taken."""
    enc = bytes_to_unicode()
    ordered = sorted(ranks.items(), key=lambda kv: int(kv[1]))
    strings = ["".join(enc[b] for b in tok) for tok, _ in ordered]
    if base_vocab is None:
        base_vocab = next((i for i, s in enumerate(strings) if len(s) > 1), len(strings))
    index = {s: i for i, s in enumerate(strings)}
    merges: List[Tuple[int, int]] = []
    for i in range(int(base_vocab), len(strings)):
        s = strings[i]
        if len(s) <= 1:
            raise ValueError("single-character token beyond the base vocabulary in a TikToken table")
        for cut in range(1, len(s)):
            l, r = index.get(s[:cut]), index.get(s[cut:])
            if l is not None and r is not None and l < i and r < i:
                merges.append((l, r))
                break
        else:
            raise ValueError(f"TikToken symbol {s!r} at rank {i} is not a pair of earlier tokens")
    return merges


def load_tiktoken_merges(path: str, base_vocab: int | None = None) -> List[Tuple[int, int]]:
    ranks: Dict[bytes, int] = {}
    with open(path, "rb") as f:
        for raw in f:
            line = raw.strip()
            if not line:
                continue
            tok, rank = line.split()
            ranks[base64.b64decode(tok)] = int(rank)
    return tiktoken_ranks_to_merges(ranks, base_vocab)


def load_warm_start_merges(source: str | None) -> List[Tuple[int, int]] | None:
    """Seed merges of ``train-bpe --warm-start`` (``main.py:501-575`` of the reference): a JSON
    manifest holding a ``merges`` list (at the top level or under ``trainer``), a bare JSON list, a
    ``.tiktoken`` rank table, or a directory that contains ``merges.tiktoken`` /
    ``tokenizer.tiktoken`` / ``bpe_merges.json``."""
    if not source:
        return None
    if not os.path.exists(source):
        raise SystemExit(f"Warm-start plan not found at {source}")
    if os.path.isdir(source):
        for name in ("merges.tiktoken", "tokenizer.tiktoken", "bpe_merges.json"):
            cand = os.path.join(source, name)
            if os.path.exists(cand):
                return load_warm_start_merges(cand)
        raise SystemExit("Warm-start directories must contain merges.tiktoken or bpe_merges.json")
    ext = os.path.splitext(source)[1].lower()
    if ext == ".tiktoken":
        try:
            return load_tiktoken_merges(source)
        except Exception as exc:
            raise SystemExit(f"Failed to parse TikToken merges from {source}: {exc}") from exc
    if ext not in (".json", ".jsonl"):
        raise SystemExit("Warm-start plans must be JSON manifests or TikToken bundles containing a 'merges' list")
    with open(source, encoding="utf-8") as f:
        payload = json.load(f)
    raw = None
    if isinstance(payload, dict):
        raw = payload.get("merges")
        if raw is None and isinstance(payload.get("trainer"), dict):
            raw = payload["trainer"].get("merges")
            if raw is None and isinstance(payload["trainer"].get("model"), dict):
                raw = payload["trainer"]["model"].get("merges")
    elif isinstance(payload, list):
        raw = payload
    if not isinstance(raw, list):
        raise SystemExit(f"Warm-start manifest {source} does not contain a 'merges' sequence")
    merges = []
    for entry in raw:
        if not isinstance(entry, (list, tuple)) or len(entry) != 2:
            raise SystemExit(f"Warm-start manifest {source} holds an entry that is not a pair of ids")
        merges.append((int(entry[0]), int(entry[1])))
    return merges


# ----------------------------------------------------------------------------- runtime tokenizer
class GPUBPETokenizer:
    """What ``GPUBPETrainer.export_tokenizer`` returns (``gpu_tokenizer/bpe_trainer.py:604-689``): the
    Hugging Face ``tokenizers.Tokenizer`` built from the exported configuration, with the
    configuration, vocabulary and merge lines kept beside it.  Other attributes pass through to the
    wrapped tokenizer."""

    def __init__(self, tokenizer, *, config: dict, vocab: Dict[str, int], merges: List[str],
                 artifact_path: str | None = None) -> None:
        if tokenizer is None:
            raise RuntimeError("The `tokenizers` library is required to construct GPUBPETokenizer")
        self._tokenizer = tokenizer
        self.config = json.loads(json.dumps(config))
        self.vocab = dict(vocab)
        self.merges = list(merges)
        self.artifact_path = artifact_path

    @staticmethod
    def _hf():
        try:
            from tokenizers import Tokenizer
        except ImportError as exc:  # pragma: no cover
            raise RuntimeError("The `tokenizers` library is required to use GPUBPETokenizer") from exc
        return Tokenizer

    @classmethod
    def from_config(cls, config: dict) -> "GPUBPETokenizer":
        tok = cls._hf().from_str(json.dumps(config))
        model = dict(config.get("model", {}))
        return cls(tok, config=config, vocab=dict(model.get("vocab", {})), merges=list(model.get("merges", [])))

    @classmethod
    def from_file(cls, path: str) -> "GPUBPETokenizer":
        tok = cls._hf().from_file(path)
        with open(path, encoding="utf-8") as f:
            config = json.load(f)
        model = dict(config.get("model", {}))
        return cls(tok, config=config, vocab=dict(model.get("vocab", {})), merges=list(model.get("merges", [])),
                   artifact_path=path)

    def encode(self, *args, **kwargs):
        return self._tokenizer.encode(*args, **kwargs)

    def decode(self, *args, **kwargs):
        return self._tokenizer.decode(*args, **kwargs)

    @property
    def tokenizer(self):
        return self._tokenizer

    def __getattr__(self, name: str):
        return getattr(self._tokenizer, name)
