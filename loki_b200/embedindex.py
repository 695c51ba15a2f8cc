"""Path-keyed exact index with the reference's interface.

Mirrors ``media-server/embedindex/embedindex.go``: ``New()`` / ``NewCentered()``
return a ``VectorIndex`` with ``Add``, ``Delete``, ``Search``, ``SearchFiltered``,
``SearchScored``, ``SearchShared``, ``SearchSharedScored`` and ``Len``; hits are
``SearchHit(Path, Score)``.  Names, argument meaning and error behaviour follow the
Go package so that the reference's own tests can be read side by side with ours.

All bookkeeping (path table, slot map, swap-remove, allow-set resolution, tie order)
is the C++ of ``include/lokiscan_index.h`` inside ``liblokiscan.so``; all scoring
runs on the GPU.  This module only marshals arguments.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import Iterable, List, Optional, Sequence

import numpy as np

from . import _lib
from ._lib import LK_F16, LK_F32, LK_I8, LokiError, check, lib  # noqa: F401

MinCenterCount = _lib.LK_MIN_CENTER_COUNT  # media-server/embedindex/embedindex.go:55
ScoreDefault = _lib.LK_SCORE_DEFAULT       # media-server/embedindex/embedindex.go:70
ScorePlain = _lib.LK_SCORE_PLAIN           # media-server/embedindex/embedindex.go:76

_vp, _i64, _int = C.c_void_p, C.c_int64, C.c_int
_cpp = C.POINTER(C.c_char_p)


def _sig(name, restype, *argtypes):
    fn = getattr(lib, name)
    fn.restype = restype
    fn.argtypes = list(argtypes)
    return fn


_sig("lkx_new", _int, _int, _int, _int, C.POINTER(_vp))
_sig("lkx_free", _int, _vp)
_sig("lkx_save", _int, _vp, C.c_char_p, C.c_uint64)
_sig("lkx_load", _int, C.c_char_p, C.c_uint64, _int, C.POINTER(_vp))
_sig("lkx_add", _int, _vp, C.c_char_p, _vp, _int)
_sig("lkx_add_batch", _int, _vp, _cpp, _vp, _i64, _int)
_sig("lkx_delete", _int, _vp, C.c_char_p)
_sig("lkx_len", _i64, _vp)
_sig("lkx_search_scored", _int, _vp, _vp, _int, _int, _int, _cpp, _i64, _int, C.POINTER(_vp))
_sig("lkx_search_shared_scored", _int, _vp, C.POINTER(_vp), C.POINTER(_int), _int, _vp, _int,
     C.POINTER(_vp), C.POINTER(_int), _int, _vp, _int, _int, _int, _cpp, _i64, _int, C.POINTER(_vp))
_sig("lkx_hits_len", _i64, _vp)
_sig("lkx_hits_path", C.c_char_p, _vp, _i64)
_sig("lkx_hits_score", C.c_float, _vp, _i64)
_sig("lkx_hits_free", None, _vp)
_sig("lkx_device_index", _vp, _vp)
_sig("lkx_slot_of", _i64, _vp, C.c_char_p)


@dataclass
class SearchHit:  # media-server/embedindex/embedindex.go:58-61
    Path: str
    Score: np.float32


@dataclass
class SharedSpec:  # media-server/embedindex/embedindex.go:83-88
    Pos: Sequence
    PosW: Optional[Sequence] = None
    Neg: Optional[Sequence] = None
    NegW: Optional[Sequence] = None


def _f32(v) -> np.ndarray:
    return np.ascontiguousarray(v, dtype=np.float32).reshape(-1)


def _paths(allow: Optional[Iterable[str]]):
    if allow is None:
        return 0, None, 0
    items = [p.encode("utf-8") for p in allow]
    arr = (C.c_char_p * max(len(items), 1))(*items)
    return 1, arr, len(items)


def _vec_list(vs):
    vs = [_f32(v) for v in (vs or [])]
    n = len(vs)
    ptrs = (_vp * max(n, 1))(*[v.ctypes.data for v in vs])
    lens = (_int * max(n, 1))(*[v.size for v in vs])
    return vs, ptrs, lens, n


class VectorIndex:
    """media-server/embedindex/embedindex.go:93-117.  Not internally synchronised."""

    def __init__(self, centered: bool, store: int = LK_F32, device: int = 0):
        h = _vp()
        check(lib.lkx_new(1 if centered else 0, int(store), int(device), C.byref(h)))
        self._h = h

    def close(self):
        if getattr(self, "_h", None):
            lib.lkx_free(self._h)
            self._h = None

    __del__ = close

    def Add(self, path: str, vec) -> None:
        v = _f32(vec)
        check(lib.lkx_add(self._h, path.encode("utf-8"), _lib.ptr(v), v.size))

    def AddBatch(self, paths: Sequence[str], rows) -> None:
        """n Adds in order with one upload per run of new paths (bulk index build)."""
        rows = np.ascontiguousarray(rows, dtype=np.float32)
        n = len(paths)
        assert rows.ndim == 2 and rows.shape[0] == n
        arr = (C.c_char_p * max(n, 1))(*[p.encode("utf-8") for p in paths])
        check(lib.lkx_add_batch(self._h, arr, _lib.ptr(rows), n, rows.shape[1]))

    def SaveCache(self, path: str, tag: int = 0) -> None:
        """Write the built index and its paths (slot order) to `path` and `path`.paths."""
        check(lib.lkx_save(self._h, os.fsencode(path), C.c_uint64(int(tag))))

    @classmethod
    def LoadCache(cls, path: str, tag: int = 0, device: int = 0) -> "VectorIndex":
        """The index SaveCache wrote, without the row-by-row rebuild; raises when the tag
        (model + row count), the sizes or the checksum do not match."""
        h = _vp()
        check(lib.lkx_load(os.fsencode(path), C.c_uint64(int(tag)), int(device), C.byref(h)))
        self = cls.__new__(cls)
        self._h = h
        return self

    def Delete(self, path: str) -> None:
        check(lib.lkx_delete(self._h, path.encode("utf-8")))

    def Len(self) -> int:
        return int(lib.lkx_len(self._h))

    def Search(self, query, k: int) -> Optional[List[SearchHit]]:
        return self.SearchScored(query, k, None, ScoreDefault)

    def SearchFiltered(self, query, k: int, allow) -> Optional[List[SearchHit]]:
        return self.SearchScored(query, k, allow, ScoreDefault)

    def SearchScored(self, query, k: int, allow, s: int) -> Optional[List[SearchHit]]:
        q = _f32(query)
        has, arr, n = _paths(allow)
        out = _vp()
        check(lib.lkx_search_scored(self._h, _lib.ptr(q), q.size, int(k), has, arr, n, int(s), C.byref(out)))
        return self._take(out)

    def SearchShared(self, spec: SharedSpec, k: int, allow) -> Optional[List[SearchHit]]:
        return self.SearchSharedScored(spec, k, allow, ScoreDefault)

    def SearchSharedScored(self, spec: SharedSpec, k: int, allow, s: int) -> Optional[List[SearchHit]]:
        """Raises ``ValueError`` where the reference returns an error."""
        pos, pptr, plen, npos = _vec_list(spec.Pos)
        neg, nptr, nlen, nneg = _vec_list(spec.Neg)
        pw = None if spec.PosW is None else _f32(spec.PosW)
        nw = None if spec.NegW is None else _f32(spec.NegW)
        has, arr, n = _paths(allow)
        out = _vp()
        st = lib.lkx_search_shared_scored(self._h, pptr, plen, npos, _lib.ptr(pw), 0 if pw is None else pw.size,
                                          nptr, nlen, nneg, _lib.ptr(nw), 0 if nw is None else nw.size,
                                          int(k), has, arr, n, int(s), C.byref(out))
        if st == _lib.LK_EINVAL:
            raise ValueError(lib.lk_last_error().decode("utf-8", "replace"))
        check(st)
        return self._take(out)

    @staticmethod
    def _take(out) -> Optional[List[SearchHit]]:
        if not out:
            return None
        try:
            n = lib.lkx_hits_len(out)
            return [SearchHit(lib.lkx_hits_path(out, i).decode("utf-8"), np.float32(lib.lkx_hits_score(out, i)))
                    for i in range(n)]
        finally:
            lib.lkx_hits_free(out)

    def slot_of(self, path: str) -> int:
        return int(lib.lkx_slot_of(self._h, path.encode("utf-8")))


def New(store: int = LK_F32, device: int = 0) -> VectorIndex:
    """Plain-cosine exact index: media-server/embedindex/embedindex.go:144-146."""
    return VectorIndex(False, store, device)


def NewCentered(device: int = 0) -> VectorIndex:
    """Mean-centering exact index: media-server/embedindex/embedindex.go:151-153."""
    return VectorIndex(True, LK_F32, device)
