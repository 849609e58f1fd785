"""Seeded synthetic corpora for the benchmark configurations.

Every generator is a pure integer function of ``(seed, stream, index)`` built on a
counter-based 64-bit mixer, so the same bytes come out of numpy on the host and
of torch on a GPU (the formulas below are written once against a tiny array shim
and run on either backend).  No floating point touches a sampled value: the
categorical draws compare a 63-bit uniform integer with integer thresholds that
are computed once on the host.

These corpora are stand-ins with the shapes, sizes and value distributions of the
configurations the benchmark is quoted on; no external dataset is involved.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np

try:  # torch is only needed for device-side generation
    import torch
except Exception:  # pragma: no cover
    torch = None

_M64 = (1 << 64) - 1


def _s64(x: int) -> int:
    """Two's complement view of an unsigned 64-bit constant."""
    x &= _M64
    return x - (1 << 64) if x >= (1 << 63) else x


_GOLD = _s64(0x9E3779B97F4A7C15)
_C1 = _s64(0xBF58476D1CE4E5B9)
_C2 = _s64(0x94D049BB133111EB)


def _mix_py(x: int) -> int:
    x &= _M64
    x ^= x >> 30
    x = (x * 0xBF58476D1CE4E5B9) & _M64
    x ^= x >> 27
    x = (x * 0x94D049BB133111EB) & _M64
    x ^= x >> 31
    return x


def _stream_key(seed: int, stream: int) -> int:
    return _s64(_mix_py((seed + 1) * 0x9E3779B97F4A7C15 + stream * 0xD1B54A32D192ED03))


class _XP:
    """Minimal array shim: int64 arithmetic with wrap-around on numpy or torch."""

    def __init__(self, device: Optional[str] = None):
        self.torch = device is not None
        self.device = device
        if self.torch and torch is None:
            raise RuntimeError("torch is required for device-side generation")

    def arange(self, lo: int, hi: int):
        if self.torch:
            return torch.arange(lo, hi, dtype=torch.int64, device=self.device)
        return np.arange(lo, hi, dtype=np.int64)

    def asarray(self, a):
        if self.torch:
            return torch.as_tensor(np.ascontiguousarray(a), device=self.device)
        return np.asarray(a)

    def lsr(self, x, s: int):
        mask = (1 << (64 - s)) - 1
        return (x >> s) & mask

    def mix(self, x):
        with np.errstate(over="ignore"):
            x = x ^ self.lsr(x, 30)
            x = x * _C1
            x = x ^ self.lsr(x, 27)
            x = x * _C2
            x = x ^ self.lsr(x, 31)
        return x

    def rand63(self, key: int, idx):
        """63-bit non-negative uniform integers for the given indices."""
        with np.errstate(over="ignore"):
            x = (idx + 1) * _GOLD + key
        return self.lsr(self.mix(x), 1)

    def searchsorted_right(self, sorted_arr, v):
        if self.torch:
            return torch.searchsorted(sorted_arr, v, right=True)
        return np.searchsorted(sorted_arr, v, side="right").astype(np.int64)

    def cumsum(self, x):
        return torch.cumsum(x, 0) if self.torch else np.cumsum(x)

    def repeat_interleave(self, x, reps, total: int):
        if self.torch:
            return torch.repeat_interleave(x, reps, output_size=total)
        return np.repeat(x, reps)

    def where(self, c, a, b):
        return torch.where(c, a, b) if self.torch else np.where(c, a, b)

    def to_u8(self, x):
        return x.to(torch.uint8) if self.torch else x.astype(np.uint8)

    def to_i32(self, x):
        return x.to(torch.int32) if self.torch else x.astype(np.int32)

    def zeros_i64(self, n: int):
        if self.torch:
            return torch.zeros(n, dtype=torch.int64, device=self.device)
        return np.zeros(n, dtype=np.int64)

    def cat(self, xs):
        return torch.cat(xs) if self.torch else np.concatenate(xs)

    def item(self, x) -> int:
        return int(x.item()) if self.torch else int(x)

    def nonzero(self, c):
        return torch.nonzero(c).flatten() if self.torch else np.nonzero(c)[0].astype(np.int64)


def zipf_thresholds(n: int, s: float) -> np.ndarray:
    """Integer CDF thresholds (scaled to 2**63) of p_r proportional to r**-s, r=1..n."""
    w = np.arange(1, n + 1, dtype=np.float64) ** (-s)
    cdf = np.cumsum(w) / np.sum(w)
    thr = np.minimum(np.floor(cdf * float(1 << 63)), float((1 << 63) - 1024)).astype(np.int64)
    thr[-1] = (1 << 63) - 1
    return thr


def _sample_categorical(xp: _XP, thr, u):
    idx = xp.searchsorted_right(thr, u)
    n = thr.shape[0]
    return xp.where(idx >= n, idx * 0 + (n - 1), idx)


# stream identifiers (any distinct integers)
_S_LEXLEN, _S_LEXCH, _S_LEXTYPE, _S_WORD, _S_SEP, _S_DOC, _S_ID, _S_BOUND = range(1, 9)
_S_DTYPE, _S_DLEN, _S_DPAT, _S_RBYTE = range(9, 13)


@dataclass
class Corpus:
    """A byte corpus with row (document / file) offsets; ``data`` is uint8."""

    data: object  # np.ndarray or torch.Tensor (uint8)
    row_offsets: object  # int64, n_rows + 1
    name: str = ""

    def sha256(self) -> str:
        d = self.data.cpu().numpy() if hasattr(self.data, "cpu") else self.data
        return hashlib.sha256(np.ascontiguousarray(d).tobytes()).hexdigest()


# --------------------------------------------------------------------------- lexicons
def _lexicon_ascii(seed: int, n_words: int, max_len: int) -> Tuple[np.ndarray, np.ndarray]:
    """Lowercase words with uniform lengths 1..max_len.  Returns (bytes, offsets)."""
    xp = _XP()
    lens = 1 + xp.rand63(_stream_key(seed, _S_LEXLEN), xp.arange(0, n_words)) % max_len
    off = np.zeros(n_words + 1, dtype=np.int64)
    np.cumsum(lens, out=off[1:])
    chars = 97 + xp.rand63(_stream_key(seed, _S_LEXCH), xp.arange(0, int(off[-1]))) % 26
    return chars.astype(np.uint8), off


def _lexicon_mixed(seed: int, n_words: int) -> Tuple[np.ndarray, np.ndarray]:
    """70% ASCII words (1-14 letters), 20% Cyrillic U+0400-04FF (2-10 chars, 2-byte
    UTF-8), 10% CJK U+4E00-9FFF (1-4 chars, 3-byte UTF-8)."""
    xp = _XP()
    w = xp.arange(0, n_words)
    t = xp.rand63(_stream_key(seed, _S_LEXTYPE), w) % 10
    kind = np.where(t < 7, 0, np.where(t < 9, 1, 2))
    r = xp.rand63(_stream_key(seed, _S_LEXLEN), w)
    nchars = np.where(kind == 0, 1 + r % 14, np.where(kind == 1, 2 + r % 9, 1 + r % 4))
    bpc = kind + 1
    coff = np.zeros(n_words + 1, dtype=np.int64)
    np.cumsum(nchars, out=coff[1:])
    total_chars = int(coff[-1])
    ckind = np.repeat(kind, nchars)
    rc = xp.rand63(_stream_key(seed, _S_LEXCH), xp.arange(0, total_chars))
    cp = np.where(ckind == 0, 97 + rc % 26,
                  np.where(ckind == 1, 0x400 + rc % 256, 0x4E00 + rc % (0x9FFF - 0x4E00 + 1)))
    cb = ckind + 1
    boff = np.zeros(total_chars + 1, dtype=np.int64)
    np.cumsum(cb, out=boff[1:])
    out = np.zeros(int(boff[-1]), dtype=np.uint8)
    s = boff[:-1]
    m0, m1, m2 = ckind == 0, ckind == 1, ckind == 2
    out[s[m0]] = cp[m0]
    out[s[m1]] = 0xC0 | (cp[m1] >> 6)
    out[s[m1] + 1] = 0x80 | (cp[m1] & 0x3F)
    out[s[m2]] = 0xE0 | (cp[m2] >> 12)
    out[s[m2] + 1] = 0x80 | ((cp[m2] >> 6) & 0x3F)
    out[s[m2] + 2] = 0x80 | (cp[m2] & 0x3F)
    woff = boff[coff]
    return out, woff.astype(np.int64)


# --------------------------------------------------------------------------- text assembly
_SEP_SIMPLE = (np.array([[32, 0], [10, 0]], dtype=np.uint8), np.array([1, 1], dtype=np.int64))
# separator table for the mixed corpus: (bytes, length); weights below
_SEP_MIXED_BYTES = np.array(
    [[32, 0], [44, 32], [46, 32], [10, 0], [59, 32], [58, 32], [9, 0], [33, 32], [63, 32], [45, 0]],
    dtype=np.uint8)
_SEP_MIXED_LEN = np.array([1, 2, 2, 1, 2, 2, 1, 2, 2, 1], dtype=np.int64)
_SEP_MIXED_W = np.array([780, 80, 60, 30, 10, 10, 5, 5, 5, 15], dtype=np.float64)


def _weights_to_thr(w: np.ndarray) -> np.ndarray:
    cdf = np.cumsum(w) / np.sum(w)
    thr = np.floor(cdf * float(1 << 63)).astype(np.float64)
    thr = np.minimum(thr, float((1 << 63) - 1024)).astype(np.int64)
    thr[-1] = (1 << 63) - 1
    return thr


def _assemble_text(xp: _XP, seed: int, n_bytes: int, lex_bytes: np.ndarray, lex_off: np.ndarray,
                   zipf_s: float, sep_bytes: np.ndarray, sep_len: np.ndarray, sep_thr: np.ndarray,
                   doc_end_prob_thr: int, chunk_words: int = 1 << 24):
    """Concatenate Zipf-drawn words and separators until ``n_bytes`` are produced.

    Returns (data uint8[n_bytes], doc_end_positions int64) where a position p in
    the second array means "a document ends after byte p-1" (p in 1..n_bytes)."""
    n_lex = len(lex_off) - 1
    thr = xp.asarray(zipf_thresholds(n_lex, zipf_s))
    lexlen = xp.asarray((lex_off[1:] - lex_off[:-1]).astype(np.int64))
    lexoff = xp.asarray(lex_off[:-1].astype(np.int64))
    lexb = xp.asarray(lex_bytes.astype(np.int64))
    sepb = xp.asarray(sep_bytes.astype(np.int64).reshape(-1))
    sepl = xp.asarray(sep_len)
    sthr = xp.asarray(sep_thr)
    kw, ks, kd = (_stream_key(seed, s) for s in (_S_WORD, _S_SEP, _S_DOC))

    pieces, ends = [], []
    produced, k0 = 0, 0
    while produced < n_bytes:
        k = xp.arange(k0, k0 + chunk_words)
        wid = _sample_categorical(xp, thr, xp.rand63(kw, k))
        sid = _sample_categorical(xp, sthr, xp.rand63(ks, k))
        wl = lexlen[wid]
        sl = sepl[sid]
        tl = wl + sl
        cs = xp.cumsum(tl)
        total = xp.item(cs[-1])
        starts = cs - tl
        slot = xp.repeat_interleave(xp.arange(0, chunk_words), tl, total)
        pos = xp.arange(0, total) - starts[slot]
        w_of = wid[slot]
        inword = pos < wl[slot]
        lex_idx = xp.where(inword, lexoff[w_of] + pos, pos * 0)
        sep_idx = xp.where(inword, pos * 0, sid[slot] * 2 + (pos - wl[slot]))
        byte = xp.where(inword, lexb[lex_idx], sepb[sep_idx])
        pieces.append(xp.to_u8(byte))
        if doc_end_prob_thr > 0:
            is_end = xp.rand63(kd, k) < doc_end_prob_thr
            ends.append(cs[xp.nonzero(is_end)] + produced)
        produced += total
        k0 += chunk_words
        del slot, pos, w_of, inword, lex_idx, sep_idx, byte
    data = xp.cat(pieces)[:n_bytes]
    doc_ends = xp.cat(ends) if ends else xp.zeros_i64(0)
    return data, doc_ends


def _offsets_from_ends(xp: _XP, ends, n_bytes: int):
    ends = ends[ends < n_bytes]
    z = xp.zeros_i64(1)
    return xp.cat([z, ends, z + n_bytes])


def config1_text(n_bytes: int = 16 << 20, seed: int = 0, file_bytes: int = 1 << 20,
                 device: Optional[str] = None) -> Corpus:
    """Lowercase Zipf(1.07) text over a 20 000-word lexicon (lengths 1-12), single
    spaces, a newline instead after a geometric(mean 40) number of words; rows are
    files of ``file_bytes`` (the reference makes one row per file)."""
    xp = _XP(device)
    lex_b, lex_o = _lexicon_ascii(seed, 20000, 12)
    sep_thr = _weights_to_thr(np.array([39.0, 1.0]))
    chunk = 1 << 24 if n_bytes >= (64 << 20) else max(1 << 12, min(1 << 22, n_bytes // 4 + 16))
    data, _ = _assemble_text(xp, seed, n_bytes, lex_b, lex_o, 1.07, _SEP_SIMPLE[0], _SEP_SIMPLE[1],
                             sep_thr, 0, chunk_words=chunk)
    n_rows = (n_bytes + file_bytes - 1) // file_bytes
    off = np.minimum(np.arange(n_rows + 1, dtype=np.int64) * file_bytes, n_bytes)
    return Corpus(data, xp.asarray(off), f"c1_text_{n_bytes}_s{seed}")


def config2_mixed(n_bytes: int = 1 << 30, seed: int = 1, mean_doc_bytes: int = 4096,
                  lexicon: int = 200000, device: Optional[str] = None) -> Corpus:
    """Mixed ASCII / Cyrillic / CJK Zipf(1.1) text over a 200 000-word lexicon with
    whitespace and punctuation separators; a document (row) ends after a word with a
    fixed probability chosen so that documents average ``mean_doc_bytes``."""
    xp = _XP(device)
    lex_b, lex_o = _lexicon_mixed(seed, lexicon)
    # expected bytes per word slot under the Zipf weights, to convert bytes -> word probability
    w = np.arange(1, lexicon + 1, dtype=np.float64) ** (-1.1)
    w /= w.sum()
    mean_word = float(np.sum(w * (lex_o[1:] - lex_o[:-1])))
    mean_sep = float(np.sum(_SEP_MIXED_W / _SEP_MIXED_W.sum() * _SEP_MIXED_LEN))
    p_end = min(1.0, (mean_word + mean_sep) / float(mean_doc_bytes))
    p_thr = int(p_end * float(1 << 63))
    chunk = 1 << 24 if n_bytes >= (64 << 20) else max(1 << 12, min(1 << 22, n_bytes // 4 + 16))
    data, ends = _assemble_text(xp, seed, n_bytes, lex_b, lex_o, 1.1, _SEP_MIXED_BYTES,
                                _SEP_MIXED_LEN, _weights_to_thr(_SEP_MIXED_W), p_thr,
                                chunk_words=chunk)
    return Corpus(data, _offsets_from_ends(xp, ends, n_bytes), f"c2_mixed_{n_bytes}_s{seed}")


def config3_ids(n_tokens: int = 1 << 31, seed: int = 2, vocab: int = 65536, mean_row: int = 2048,
                device: Optional[str] = None, chunk: int = 1 << 26):
    """int32 ids Zipf(1.1) over ``vocab`` with row boundaries at geometric(mean
    ``mean_row``) gaps.  Returns (ids int32[n], row_offsets int64)."""
    xp = _XP(device)
    thr = xp.asarray(zipf_thresholds(vocab, 1.1))
    kid, kb = _stream_key(seed, _S_ID), _stream_key(seed, _S_BOUND)
    bthr = (1 << 63) // mean_row
    ids, bounds = [], []
    for lo in range(0, n_tokens, chunk):
        i = xp.arange(lo, min(lo + chunk, n_tokens))
        ids.append(xp.to_i32(_sample_categorical(xp, thr, xp.rand63(kid, i))))
        b = xp.nonzero(xp.rand63(kb, i) < bthr) + lo
        bounds.append(b[b > 0])
    z = xp.zeros_i64(1)
    return xp.cat(ids), xp.cat([z] + bounds + [z + n_tokens])


def config5_adversarial(n_bytes: int = 512 << 20, seed: int = 4,
                        device: Optional[str] = None) -> Corpus:
    """30% long runs (2-4096 bytes) of one byte or a two-byte pattern, 40% text as in
    ``config1_text``, 30% uniform random bytes in documents of 256-65 536 bytes (shares
    by bytes).  Every document is a row."""
    xp = _XP(device)
    # document type probabilities proportional to share / mean length
    mean_run, mean_other = (2 + 4096) / 2.0, (256 + 65536) / 2.0
    wts = np.array([0.3 / mean_run, 0.4 / mean_other, 0.3 / mean_other])
    tthr = xp.asarray(_weights_to_thr(wts))
    kt, kl, kp, kr = (_stream_key(seed, s) for s in (_S_DTYPE, _S_DLEN, _S_DPAT, _S_RBYTE))
    exp_doc = float(np.sum(wts / wts.sum() * np.array([mean_run, mean_other, mean_other])))
    n_docs = int(n_bytes / exp_doc * 1.25) + 64
    while True:
        d = xp.arange(0, n_docs)
        kind = _sample_categorical(xp, tthr, xp.rand63(kt, d))
        rl = xp.rand63(kl, d)
        dlen = xp.where(kind == 0, 2 + rl % 4095, 256 + rl % 65281)
        cs = xp.cumsum(dlen)
        if xp.item(cs[-1]) >= n_bytes:
            break
        n_docs *= 2
    starts = cs - dlen
    n_used = xp.item((starts < n_bytes).sum())
    kind, dlen, starts, d = kind[:n_used], dlen[:n_used], starts[:n_used], d[:n_used]
    total = xp.item(dlen.sum())
    rp = xp.rand63(kp, d)
    pat0 = rp & 0xFF
    pat1 = xp.where((xp.lsr(rp, 8) & 1) == 0, pat0, xp.lsr(rp, 16) & 0xFF)  # one byte or two
    # text bytes are taken consecutively from a config-1 style stream
    is_text = kind == 1
    tlen = xp.where(is_text, dlen, dlen * 0)
    tstart = xp.cumsum(tlen) - tlen
    n_text = xp.item(tlen.sum())
    text = config1_text(max(n_text, 1), seed=seed + 1000, device=device).data
    out = []
    step = 1 << 14
    for lo in range(0, n_used, step):  # chunks of documents bound the temporaries
        hi = min(lo + step, n_used)
        dl = dlen[lo:hi]
        tot = xp.item(dl.sum())
        slot = xp.repeat_interleave(xp.arange(lo, hi), dl, tot)
        first = xp.item(starts[lo])
        q = xp.arange(first, first + tot) - starts[slot]
        k = kind[slot]
        run_b = xp.where((q & 1) == 0, pat0[slot], pat1[slot])
        rnd_b = xp.rand63(kr, xp.arange(first, first + tot)) & 0xFF
        t_idx = xp.where(k == 1, tstart[slot] + q, q * 0)
        txt_b = text[t_idx].to(torch.int64) if xp.torch else text[t_idx].astype(np.int64)
        out.append(xp.to_u8(xp.where(k == 0, run_b, xp.where(k == 1, txt_b, rnd_b))))
    data = xp.cat(out)[:n_bytes]
    off = xp.cat([starts[starts < n_bytes], xp.zeros_i64(1) + n_bytes])
    del total
    return Corpus(data, off, f"c5_adversarial_{n_bytes}_s{seed}")


def bytes_to_ids(corpus: Corpus):
    """uint8 bytes -> int32 ids (identity map, as the reference's byte packer)."""
    d = corpus.data
    return d.to(torch.int32) if hasattr(d, "cpu") else d.astype(np.int32)
