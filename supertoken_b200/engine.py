"""Python handle on one ``stbpe_engine`` (one per GPU / rank)."""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import _lib as L


class CapacityError(RuntimeError):
    pass


def _raise(status: int, msg: str):
    if status == L.E_BADARG:
        raise ValueError(msg)
    if status == L.E_ID_OVERFLOW:
        raise OverflowError(msg)
    if status == L.E_CAPACITY:
        raise CapacityError(msg if "capacity exceeded" in msg else f"pair workspace capacity exceeded: {msg}")
    raise RuntimeError(msg)


def _stream_ptr(device: torch.device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


class Engine:
    """Token stream + pair table of one GPU.  Thin wrapper: every method is one C-ABI call."""

    def __init__(self, max_tokens: int, base_vocab: int = 256, max_merges: int = 50_000,
                 device: Optional[torch.device | str | int] = None, table_slots: int = 0,
                 world_size: int = 1, rank: int = 0):
        if not torch.cuda.is_available():
            raise RuntimeError("supertoken_b200 needs a CUDA device (B200, sm_100a); there is no CPU fallback")
        self._lib = L.load()
        dev = torch.device("cuda" if device is None else device)
        if dev.type != "cuda":
            raise ValueError("Engine runs on CUDA devices only")
        self.device = torch.device("cuda", torch.cuda.current_device() if dev.index is None else dev.index)
        self.base_vocab = int(base_vocab)
        self.max_merges = int(max_merges)
        self.world_size, self.rank = int(world_size), int(rank)
        cfg = L.Config(self.device.index, self.base_vocab, int(max_tokens), int(table_slots),
                       self.max_merges, self.world_size, self.rank, 0)
        self._h = ctypes.c_void_p()
        st = self._lib.stbpe_create(ctypes.byref(self._h), ctypes.byref(cfg))
        if st != L.OK:
            msg = self._lib.stbpe_last_error(None).decode()
            self._h = ctypes.c_void_p()
            _raise(st, msg)

    # ------------------------------------------------------------------ plumbing
    def _check(self, st: int):
        if st != L.OK:
            _raise(st, self._lib.stbpe_last_error(self._h).decode())

    def close(self):
        if getattr(self, "_h", None) and self._h.value:
            self._lib.stbpe_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def _s(self):
        return _stream_ptr(self.device)

    # ------------------------------------------------------------------ ingest
    def reset(self):
        self._check(self._lib.stbpe_reset(self._h))

    @staticmethod
    def _offsets(row_offsets, n: int) -> np.ndarray:
        if row_offsets is None:
            return np.array([0, n], dtype=np.int64)
        if isinstance(row_offsets, torch.Tensor):
            row_offsets = row_offsets.cpu().numpy()
        return np.ascontiguousarray(row_offsets, dtype=np.int64)

    def append_bytes(self, data, row_offsets=None):
        """``data``: uint8 torch tensor (CUDA or CPU, pinned or not) or numpy array."""
        if isinstance(data, np.ndarray):
            data = torch.from_numpy(np.ascontiguousarray(data, dtype=np.uint8))
        assert data.dtype == torch.uint8 and data.is_contiguous()
        off = self._offsets(row_offsets, data.numel())
        self._check(self._lib.stbpe_append_bytes(self._h, data.data_ptr(), data.numel(),
                                                 off.ctypes.data, len(off) - 1, self._s))

    def append_ids(self, ids, row_offsets=None):
        if isinstance(ids, np.ndarray):
            ids = torch.from_numpy(np.ascontiguousarray(ids, dtype=np.int32))
        assert ids.dtype == torch.int32 and ids.is_contiguous()
        off = self._offsets(row_offsets, ids.numel())
        self._check(self._lib.stbpe_append_ids(self._h, ids.data_ptr(), ids.numel(),
                                               off.ctypes.data, len(off) - 1, self._s))

    # ------------------------------------------------------------------ operators
    def count_initial(self):
        self._check(self._lib.stbpe_count_initial(self._h, self._s))

    def select_best(self, with_ties: bool = False) -> Tuple[Optional[int], int, int]:
        key, count, ties = ctypes.c_uint64(0), ctypes.c_int64(0), ctypes.c_int64(0)
        self._check(self._lib.stbpe_select_best(self._h, ctypes.byref(key), ctypes.byref(count),
                                                ctypes.byref(ties) if with_ties else None, self._s))
        if count.value <= 0:
            return None, 0, 0
        return int(key.value), int(count.value), int(ties.value)

    def apply_merge(self, a: int, b: int, new_id: int) -> int:
        if max(a, b, new_id) > 0x7FFFFFFE or min(a, b, new_id) < 0:
            raise OverflowError("Token id overflow: ids must be in [0, 2^31-2]")
        n = ctypes.c_int64(0)
        self._check(self._lib.stbpe_apply_merge(self._h, a, b, new_id, ctypes.byref(n), self._s))
        return int(n.value)

    def train(self, n_merges: int):
        self._check(self._lib.stbpe_train(self._h, int(n_merges), self._s))

    def train_timed(self, n_merges: int):
        """Like ``train`` but returns device milliseconds spent in (select, merge, refresh)."""
        ms = (ctypes.c_float * 4)()
        self._check(self._lib.stbpe_train_timed(self._h, int(n_merges), ms, self._s))
        return float(ms[0]), float(ms[1]), float(ms[2]), float(ms[3])

    def repack(self, force: bool = False) -> bool:
        """Dense re-pack of the stream if at most half of the tile capacity is live (or forced)."""
        did = ctypes.c_int(0)
        self._check(self._lib.stbpe_repack(self._h, int(force), ctypes.byref(did), self._s))
        return bool(did.value)

    def count_error(self):
        """Raise the exception that matches the device error bits, if any are set."""
        st = self.state()
        bits = st.device_error
        if bits & 32:
            raise RuntimeError("a bounded device-side wait gave up (tile pipeline or a peer's flag)")
        if bits & (1 | 2 | 4):
            raise CapacityError("pair workspace capacity exceeded (pair table / delta buffers full)")
        if bits & 16:
            raise OverflowError("Token id overflow: ids must be in [0, 2^31-2]")
        if bits:
            raise RuntimeError(f"device error bits {bits:#x}")

    def state(self) -> L.State:
        st = L.State()
        self._check(self._lib.stbpe_get_state(self._h, ctypes.byref(st), self._s))
        return st

    def merges(self, first: int = 0, n: Optional[int] = None):
        """Returns (merges list[(a,b)], counts int64[n], live_before int64[n])."""
        if n is None:
            n = self.state().merges_done - first
        m = np.zeros((max(n, 0), 2), dtype=np.int32)
        c = np.zeros(max(n, 0), dtype=np.int64)
        lb = np.zeros(max(n, 0), dtype=np.int64)
        if n > 0:
            self._check(self._lib.stbpe_get_merges(self._h, first, n, m.ctypes.data, c.ctypes.data,
                                                   lb.ctypes.data))
        return [(int(x), int(y)) for x, y in m], c, lb

    def export_histogram(self, cap: Optional[int] = None):
        """(keys int64 ascending, counts int64) on the device, zero counts dropped."""
        st = self.state()
        cap = int(cap if cap is not None else max(st.table_keys, 1))
        keys = torch.empty(cap, dtype=torch.int64, device=self.device)
        counts = torch.empty(cap, dtype=torch.int64, device=self.device)
        n = ctypes.c_int64(0)
        self._check(self._lib.stbpe_export_histogram(self._h, keys.data_ptr(), counts.data_ptr(), cap,
                                                     ctypes.byref(n), self._s))
        return keys[:n.value], counts[:n.value]

    def tied_keys(self, count: int, n_ties: int) -> List[int]:
        """Keys holding exactly ``count``, ascending."""
        buf = torch.empty(max(n_ties, 1), dtype=torch.int64, device=self.device)
        n = ctypes.c_int64(0)
        self._check(self._lib.stbpe_export_ties(self._h, count, buf.data_ptr(), buf.numel(),
                                                ctypes.byref(n), self._s))
        return sorted(int(k) for k in buf[:min(n.value, buf.numel())].cpu().numpy().view(np.uint64))

    def export_stream(self):
        """int32 ids on the device with bit 31 marking row starts -> (ids, row_offsets) on CPU."""
        st = self.state()
        cap = max(int(st.live_tokens), 1)
        buf = torch.empty(cap, dtype=torch.int32, device=self.device)
        n = ctypes.c_int64(0)
        self._check(self._lib.stbpe_export_stream(self._h, buf.data_ptr(), cap, ctypes.byref(n), self._s))
        raw = buf[:n.value].cpu().numpy().view(np.uint32)
        starts = np.nonzero(raw >> 31)[0].astype(np.int64)
        ids = (raw & 0x7FFFFFFF).astype(np.int32)
        off = np.concatenate([starts, [len(ids)]]).astype(np.int64) if len(ids) else np.zeros(1, np.int64)
        return ids, off
