"""Operator seam of the reference on CUDA tensors: ``count_pairs``, ``apply_merge_once``,
``select_best_pair`` with the reference's names, argument meaning and errors
(``gpu_tokenizer/utils.py:691-706``, ``:413-555``; ``gpu_tokenizer/trainers/bpe_gpu.py:14-130``).
Each call is one C-ABI call into ``libstbpe.so``; CPU tensors are rejected (the CPU path is
the reference's own)."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Callable, Optional, Sequence, Tuple

import torch

from . import _lib as L

UINT32_MAX = (1 << 32) - 1


def _stream(t: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _need_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("supertoken_b200 operators need CUDA tensors; there is no CPU fallback")
        if not t.is_contiguous():
            raise ValueError("tensors must be contiguous")


def count_pairs(seqs: torch.Tensor, valid: torch.Tensor, pair_keys_buffer: torch.Tensor,
                pair_counts_buffer: torch.Tensor, pair_count_length: torch.Tensor) -> None:
    """Histogram of adjacent valid pairs: unique ``(a, b)`` rows ascending by ``(a<<32)|b`` into
    ``pair_keys_buffer[:n]`` (rest -1), int64 counts into ``pair_counts_buffer[:n]`` (rest 0),
    ``n`` into ``pair_count_length``.  ``RuntimeError("pair workspace capacity exceeded")`` when
    the buffers are too small (``gpu_tokenizer/utils.py:619-620``)."""
    _need_cuda(seqs, valid, pair_keys_buffer, pair_counts_buffer, pair_count_length)
    if seqs.dtype != torch.int32 or valid.dtype != torch.uint8:
        raise TypeError("seqs must be int32 and valid uint8")
    if pair_keys_buffer.dtype != torch.int32 or pair_counts_buffer.dtype != torch.int64:
        raise TypeError("pair_keys_buffer must be int32 [cap, 2] and pair_counts_buffer int64 [cap]")
    if pair_count_length.numel() != 1:
        raise RuntimeError("pair_count_length must be a singleton tensor")
    B = seqs.size(0)
    Lw = seqs.size(1) if seqs.dim() > 1 else 0
    cap = pair_counts_buffer.numel()
    length = pair_count_length if pair_count_length.dtype == torch.int64 else \
        torch.zeros(1, dtype=torch.int64, device=seqs.device)
    with torch.cuda.device(seqs.device):
        st = L.load().stbpe_rows_count_pairs(seqs.data_ptr(), valid.data_ptr(), B, Lw,
                                            pair_keys_buffer.data_ptr(), pair_counts_buffer.data_ptr(),
                                            cap, length.data_ptr(), _stream(seqs))
    if st == L.E_CAPACITY:
        raise RuntimeError("pair workspace capacity exceeded")
    if st != L.OK:
        raise RuntimeError(f"stbpe_rows_count_pairs failed with status {st}")
    if length is not pair_count_length:
        pair_count_length.copy_(length.to(pair_count_length.dtype))


def apply_merge_once(seqs: torch.Tensor, valid: torch.Tensor, lengths: torch.Tensor, a_id: int,
                     b_id: int, new_id: int, pair_workspace: Optional[torch.Tensor] = None,
                     prefix_workspace: Optional[torch.Tensor] = None,
                     span_workspace: Optional[torch.Tensor] = None,
                     overflow_workspace: Optional[torch.Tensor] = None):
    """In-place merge of ``(a_id, b_id) -> new_id`` on a padded batch with stable compaction and a
    zero-filled tail; returns ``(seqs, valid, lengths, spans)`` where ``spans`` is the ``[B, L-1]``
    match mask in pre-compaction coordinates (``gpu_tokenizer/utils.py:413-555``)."""
    if max(a_id, b_id, new_id) > UINT32_MAX:
        raise OverflowError(f"Token id overflow: encountered id above UINT32_MAX (limit {UINT32_MAX}).")
    _need_cuda(seqs, valid, lengths)
    if seqs.dtype != torch.int32 or valid.dtype != torch.uint8:
        raise TypeError("seqs must be int32 and valid uint8")
    if max(a_id, b_id, new_id) > 0x7FFFFFFF:
        raise OverflowError("Token id overflow: int32 token storage holds ids up to 2^31-1")
    B, Lw = seqs.shape
    width = max(Lw - 1, 0)
    spans = pair_workspace if (pair_workspace is not None and pair_workspace.shape == (B, width)
                               and pair_workspace.dtype == torch.bool and pair_workspace.is_cuda) \
        else torch.zeros((B, width), dtype=torch.bool, device=seqs.device)
    if B == 0:
        lengths.zero_()
        return seqs, valid, lengths, spans
    out_len = torch.zeros(B, dtype=torch.int32, device=seqs.device)
    with torch.cuda.device(seqs.device):
        st = L.load().stbpe_rows_apply_merge(seqs.data_ptr(), valid.data_ptr(), out_len.data_ptr(), B, Lw,
                                            int(a_id), int(b_id), int(new_id),
                                            spans.data_ptr() if width > 0 else None, _stream(seqs))
    if st != L.OK:
        raise RuntimeError(f"stbpe_rows_apply_merge failed with status {st}")
    # length storage rule of gpu_tokenizer/dtypes.py:15-41: uint16 clamps and flags overflow
    if lengths.dtype == torch.uint16:
        lengths.copy_(torch.clamp_max(out_len, 65535).to(torch.uint16))
        if overflow_workspace is not None:
            overflow_workspace.copy_(out_len > 65535)
    else:
        lengths.copy_(out_len.to(lengths.dtype))
        if overflow_workspace is not None:
            overflow_workspace.zero_()
    if span_workspace is not None and span_workspace.shape == spans.shape:
        span_workspace.copy_(spans.to(span_workspace.dtype))
        spans = span_workspace
    return seqs, valid, lengths, spans


@dataclass(frozen=True)
class PairHistogramResult:
    """Packed pair histogram (``gpu_tokenizer/trainers/bpe_gpu.py:14-34``)."""

    keys: torch.Tensor
    counts: torch.Tensor

    @property
    def device(self) -> torch.device:
        return self.keys.device

    def is_empty(self) -> bool:
        return self.keys.numel() == 0 or self.counts.numel() == 0


def select_best_pair(histogram: PairHistogramResult, *,
                     tie_breaker: Callable[[Sequence[int], torch.Tensor], int] | None = None
                     ) -> Tuple[Optional[int], int, Optional[int]]:
    """Best ``(key, count, index)`` of an exported histogram: highest count, ties to the smallest
    key or to ``tie_breaker(candidate_indices, keys)`` (``trainers/bpe_gpu.py:96-130``).  Works on
    the small exported tensors; inside the engine the same rule runs in ``select_kernel``."""
    if histogram.is_empty():
        return None, 0, None
    counts, keys = histogram.counts, histogram.keys
    best = int(counts.max().item())
    if best <= 0:
        return None, 0, None
    cand = torch.nonzero(counts == best).flatten()
    if cand.numel() == 1 or tie_breaker is None:
        idx = int(cand[torch.argmin(keys[cand])].item())
    else:
        cl = [int(i) for i in cand.tolist()]
        idx = int(tie_breaker(cl, keys))
        if idx not in cl:
            raise ValueError("tie_breaker must return one of the candidate indices")
    return int(keys[idx].item()), best, idx
