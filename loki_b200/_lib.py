"""ctypes binding of ``liblokiscan.so`` (the C ABI declared in ``include/lokiscan.h``).

There is no fallback of any kind: if the shared library is missing this module
raises at import time, and every compute entry point fails with ``LK_ECUDA`` when
no CUDA device is present.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

try:  # if PyTorch is around, let it load its NCCL first so that one copy serves both
    import torch  # noqa: F401
except Exception:  # pragma: no cover - torch is optional for this package
    torch = None

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liblokiscan.so")

LK_OK, LK_EINVAL, LK_EDIM, LK_ENOMEM, LK_ECUDA, LK_ENCCL, LK_ETIMEOUT, LK_ERANGE = range(8)
LK_F32, LK_F16, LK_I8 = 0, 1, 2
LK_SCORE_DEFAULT, LK_SCORE_PLAIN = 0, 1
LK_MIN_CENTER_COUNT = 64

STATUS_NAMES = {0: "LK_OK", 1: "LK_EINVAL", 2: "LK_EDIM", 3: "LK_ENOMEM", 4: "LK_ECUDA",
                5: "LK_ENCCL", 6: "LK_ETIMEOUT", 7: "LK_ERANGE"}


class LokiError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status


if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python -m loki_b200.build` "
        "(this package has no CPU or pure-Python path)")

lib = C.CDLL(LIB_PATH)

_vp = C.c_void_p
_i64 = C.c_int64
_int = C.c_int


class lk_stats_t(C.Structure):
    _fields_ = [("len", _i64), ("capacity", _i64), ("bytes_resident", _i64),
                ("scan_launches", _i64), ("aux_launches", _i64), ("last_search_ms", C.c_float),
                ("grid", _int), ("sm_count", _int)]


def _sig(name, restype, *argtypes):
    fn = getattr(lib, name)
    fn.restype = restype
    fn.argtypes = list(argtypes)
    return fn


_sig("lk_last_error", C.c_char_p)
_sig("lk_version", C.c_char_p)
_sig("lk_device_count", _int)
_sig("lk_index_create", _int, _int, _int, _int, _int, C.POINTER(_vp))
_sig("lk_index_destroy", _int, _vp)
_sig("lk_index_reserve", _int, _vp, _i64)
_sig("lk_index_len", _i64, _vp)
_sig("lk_index_dim", _int, _vp)
_sig("lk_index_kind", _int, _vp, _vp, _vp)
_sig("lk_index_save", _int, _vp, C.c_char_p, C.c_uint64)
_sig("lk_index_load", _int, C.c_char_p, C.c_uint64, _int, C.POINTER(_vp))
_sig("lk_index_upsert_f32", _int, _vp, _i64, _i64, _vp)
_sig("lk_index_upsert_f32_device", _int, _vp, _i64, _i64, _vp)
_sig("lk_index_swap_remove", _int, _vp, _i64)
_sig("lk_index_read_rows", _int, _vp, _i64, _i64, _vp, _vp)
_sig("lk_index_center_state", _int, _vp, C.POINTER(_int), C.POINTER(_i64), C.POINTER(C.c_double), _vp, _vp, _vp)
_sig("lk_search", _int, _vp, _vp, _int, _int, _int, _vp, _i64, _vp, _vp, _vp, _vp)
_sig("lk_search_shared", _int, _vp, _vp, _vp, _int, _vp, _vp, _int, C.c_float, C.c_float, _int, _int,
     _vp, _i64, _vp, _vp, _vp)
_sig("lk_queries_create", _int, _vp, _vp, _int, _int, C.POINTER(_vp))
_sig("lk_queries_destroy", _int, _vp)
_sig("lk_search_resident", _int, _vp, _vp, _int, _int, _int)
_sig("lk_queries_fetch", _int, _vp, _vp, _int, _int, _int, _vp, _vp, _vp, _vp)
_sig("lk_timer_start", _int, _vp)
_sig("lk_timer_stop", _int, _vp, C.POINTER(C.c_float))
_sig("lk_index_sync", _int, _vp)
_sig("lk_comm_unique_id", _int, _vp)
_sig("lk_comm_create", _int, _int, _int, _int, _vp, C.POINTER(_vp))
_sig("lk_comm_destroy", _int, _vp)
_sig("lk_comm_peer_export", _int, _vp, _vp)
_sig("lk_comm_peer_attach", _int, _vp, _vp)
_sig("lk_index_attach_comm", _int, _vp, _vp, _i64)
_sig("lk_index_set_shard_base", _int, _vp, _i64)
_sig("lk_cosine_sim_topk", _int, _vp, _i64, _int, _vp, _int, _vp, _i64, _int, _vp, _vp, _vp)
_sig("lk_hamming_pairs", _int, _vp, _i64, _int, _int, _int, _int, _vp, _i64, C.POINTER(_i64))
_sig("lk_hamming_pairs_sharded", _int, _vp, _vp, _i64, _int, _vp, _i64, C.POINTER(_i64))
_sig("lk_hamming_scan", _int, _vp, _i64, C.c_uint64, _int, _int, _vp, _vp, _i64, C.POINTER(_i64))
_sig("lk_stats", _int, _vp, C.POINTER(lk_stats_t))
_sig("lk_index_set_batch_mode", _int, _vp, _int)
_sig("lk_prescreen_pairs", _int, _vp, _i64, _int, C.c_float, _int, _vp, _vp, _vp)
_sig("lk_pca3", _int, _vp, _i64, _int, _int, _int, _vp, _vp)
_sig("lk_seed_scores", _int, _vp, _i64, _vp, _i64, _int, C.c_float, _i64, _int, _vp, _vp, _vp, _i64, _vp)
_sig("lk_scan_i8_prealloc", _int, _int, _vp, _i64, _int, _i64, _vp, _vp, C.c_float, _int, _vp, _vp, _vp, _vp, _vp)
LK_PREALLOC_MAX_K = 128


def check(status: int):
    if status != LK_OK:
        raise LokiError(status, lib.lk_last_error().decode("utf-8", "replace"))


def ptr(a):
    """Host pointer of a C-contiguous numpy array (None -> NULL)."""
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_vp)


def device_count() -> int:
    return int(lib.lk_device_count())


_NP_STORE = {LK_F32: np.float32, LK_F16: np.uint16, LK_I8: np.int8}


class DeviceIndex:
    """Slot-level index in HBM: a thin, allocation-owning wrapper over the C ABI.

    This is what a cgo binding sees (slot numbers, no strings).  The path-keyed
    interface of the reference lives in :mod:`loki_b200.embedindex`.
    """

    def __init__(self, dim: int, store: int = LK_F32, centered: bool = False, device: int = 0):
        h = _vp()
        check(lib.lk_index_create(int(dim), int(store), 1 if centered else 0, int(device), C.byref(h)))
        self._h = h
        self.dim, self.store, self.centered, self.device = int(dim), int(store), bool(centered), int(device)
        self._comm = None

    def close(self):
        if getattr(self, "_h", None) and lib is not None:  # lib is None during interpreter shutdown
            lib.lk_index_destroy(self._h)
            self._h = None

    def save(self, path: str, tag: int = 0):
        """Write the built index (rows as stored, scales, centering state) to `path`."""
        check(lib.lk_index_save(self._h, os.fsencode(path), C.c_uint64(int(tag))))

    @classmethod
    def load(cls, path: str, tag: int = 0, device: int = 0) -> "DeviceIndex":
        """Read an index written by :meth:`save`; raises when tag, size or checksum do not match."""
        h = _vp()
        check(lib.lk_index_load(os.fsencode(path), C.c_uint64(int(tag)), int(device), C.byref(h)))
        self = cls.__new__(cls)
        self._h = h
        store, centered = _int(0), _int(0)
        check(lib.lk_index_kind(h, C.byref(store), C.byref(centered)))
        self.dim, self.store, self.centered, self.device = int(lib.lk_index_dim(h)), store.value, bool(centered.value), int(device)
        self._comm = None
        return self

    __del__ = close

    def __len__(self) -> int:
        return int(lib.lk_index_len(self._h))

    def reserve(self, n: int):
        check(lib.lk_index_reserve(self._h, int(n)))

    def upsert(self, first_slot: int, rows):
        rows = np.ascontiguousarray(rows, dtype=np.float32)
        if rows.ndim == 1:
            rows = rows.reshape(1, -1)
        if rows.shape[1] != self.dim:
            raise LokiError(LK_EDIM, f"rows have {rows.shape[1]} columns, index has dim {self.dim}")
        check(lib.lk_index_upsert_f32(self._h, int(first_slot), rows.shape[0], ptr(rows)))

    def upsert_device(self, first_slot: int, n: int, device_ptr: int):
        check(lib.lk_index_upsert_f32_device(self._h, int(first_slot), int(n), _vp(device_ptr)))

    def append(self, rows):
        self.upsert(len(self), rows)

    def swap_remove(self, slot: int):
        check(lib.lk_index_swap_remove(self._h, int(slot)))

    def read_rows(self, first: int = 0, n: int | None = None):
        n = len(self) - first if n is None else n
        out = np.empty((n, self.dim), _NP_STORE[self.store])
        scales = np.empty(n, np.float32) if self.store == LK_I8 else None
        check(lib.lk_index_read_rows(self._h, int(first), int(n), ptr(out), ptr(scales)))
        if self.store == LK_F16:
            out = out.view(np.float16)
        return (out, scales) if self.store == LK_I8 else out

    def center_state(self):
        live, nc, n2 = _int(0), _i64(0), C.c_double(0)
        mu = np.zeros(self.dim, np.float32)
        s = np.zeros(self.dim, np.float64)
        cn = np.zeros(max(len(self), 1), np.float32)
        check(lib.lk_index_center_state(self._h, C.byref(live), C.byref(nc), C.byref(n2), ptr(mu),
                                        ptr(s) if self.centered else None, ptr(cn)))
        return dict(live=bool(live.value), n_centered=nc.value, mu_n2=n2.value, mu=mu, sum=s,
                    cnorm=cn[:len(self)])

    def search(self, queries, k: int, scoring: int = LK_SCORE_DEFAULT, allow_slots=None):
        """-> ids[nq,k] int64 (-1 padded), scores[nq,k] f32, iscores[nq,k] i32, counts[nq]."""
        q = np.ascontiguousarray(queries, dtype=np.float32)
        if q.ndim == 1:
            q = q.reshape(1, -1)
        if q.shape[1] != self.dim:
            raise LokiError(LK_EDIM, f"queries have {q.shape[1]} columns, index has dim {self.dim}")
        nq, kk = q.shape[0], max(int(k), 0)
        # the library writes every entry (misses are -1 / 0), so the outputs need no initialisation
        ids = np.empty((nq, kk), np.int64)
        scores = np.empty((nq, kk), np.float32)
        iscores = np.empty((nq, kk), np.int32)
        counts = np.empty(nq, np.int32)
        al, nal = None, 0
        if allow_slots is not None:
            al = np.ascontiguousarray(allow_slots, dtype=np.int32)
            nal = al.size
            if nal == 0:
                al = np.zeros(1, np.int32)  # non-NULL pointer, zero entries: "allow nothing"
        check(lib.lk_search(self._h, q.ctypes.data, nq, int(k), int(scoring), ptr(al), nal,
                            ids.ctypes.data, scores.ctypes.data, iscores.ctypes.data, counts.ctypes.data))
        return ids, scores, iscores, counts

    def search_one(self, query, k: int, scoring: int = LK_SCORE_DEFAULT):
        """One query through lk_search with as little Python around the call as possible: the
        output arrays are kept per k and reused, so the result is valid until the next call.
        -> ids[1,k], scores[1,k], iscores[1,k], counts[1]."""
        cache = self.__dict__.setdefault("_one", {})
        b = cache.get(k)
        if b is None:
            arrs = (np.empty((1, k), np.int64), np.empty((1, k), np.float32), np.empty((1, k), np.int32), np.empty(1, np.int32))
            b = cache[k] = (arrs, tuple(a.ctypes.data for a in arrs))
        q = query if (query.dtype == np.float32 and query.flags["C_CONTIGUOUS"]) else np.ascontiguousarray(query, np.float32)
        if q.size != self.dim:
            raise LokiError(LK_EDIM, f"query has {q.size} elements, index has dim {self.dim}")
        st = lib.lk_search(self._h, q.ctypes.data, 1, k, scoring, None, 0, *b[1])
        if st != LK_OK:
            check(st)
        return b[0]

    def search_shared(self, pos, posw=None, neg=None, negw=None, k: int = 10, scoring: int = LK_SCORE_DEFAULT,
                      allow_slots=None, beta: float = 0.25, lam: float = 1.0):
        pos = np.ascontiguousarray(pos, dtype=np.float32).reshape(-1, self.dim) if len(pos) else np.zeros((0, self.dim), np.float32)
        npos = pos.shape[0]
        pw = None if posw is None else np.ascontiguousarray(posw, np.float32)
        ng = None if neg is None or len(neg) == 0 else np.ascontiguousarray(neg, np.float32).reshape(-1, self.dim)
        nneg = 0 if ng is None else ng.shape[0]
        nw = None if negw is None or len(negw) == 0 else np.ascontiguousarray(negw, np.float32)
        kk = max(int(k), 0)
        ids = np.full(kk, -1, np.int64)
        scores = np.zeros(kk, np.float32)
        count = np.zeros(1, np.int32)
        al, nal = None, 0
        if allow_slots is not None:
            al = np.ascontiguousarray(allow_slots, dtype=np.int32)
            nal = al.size
            if nal == 0:
                al = np.zeros(1, np.int32)
        check(lib.lk_search_shared(self._h, ptr(pos), ptr(pw), npos, ptr(ng), ptr(nw), nneg, float(beta), float(lam),
                                   int(k), int(scoring), ptr(al), nal, ptr(ids), ptr(scores), ptr(count)))
        return ids[:count[0]], scores[:count[0]]

    # ---- device-resident queries ----
    def queries(self, queries, scoring: int = LK_SCORE_DEFAULT) -> "ResidentQueries":
        return ResidentQueries(self, queries, scoring)

    def timer_start(self):
        check(lib.lk_timer_start(self._h))

    def timer_stop(self) -> float:
        ms = C.c_float(0)
        check(lib.lk_timer_stop(self._h, C.byref(ms)))
        return float(ms.value)

    def sync(self):
        check(lib.lk_index_sync(self._h))

    def attach_comm(self, comm: "Comm", shard_base: int):
        check(lib.lk_index_attach_comm(self._h, comm._h if comm is not None else None, int(shard_base)))
        self._comm = comm

    def set_batch_mode(self, tensor_cores: bool):
        """Batches of queries (>= 32 on an int8 index, >= 3 on a float32 index): tensor-core
        kernels (True, default) or consecutive single-query scans (False)."""
        check(lib.lk_index_set_batch_mode(self._h, 1 if tensor_cores else 0))

    def set_shard_base(self, base: int):
        check(lib.lk_index_set_shard_base(self._h, int(base)))

    def stats(self) -> dict:
        st = lk_stats_t()
        check(lib.lk_stats(self._h, C.byref(st)))
        return {f: getattr(st, f) for f, _ in lk_stats_t._fields_}


class ResidentQueries:
    """Prepared queries kept in HBM; scans are enqueued without host synchronisation."""

    def __init__(self, index: DeviceIndex, queries, scoring: int):
        q = np.ascontiguousarray(queries, dtype=np.float32)
        if q.ndim == 1:
            q = q.reshape(1, -1)
        h = _vp()
        check(lib.lk_queries_create(index._h, ptr(q), q.shape[0], int(scoring), C.byref(h)))
        self._h, self.index, self.nq = h, index, q.shape[0]

    def close(self):
        if getattr(self, "_h", None) and lib is not None:
            lib.lk_queries_destroy(self._h)
            self._h = None

    __del__ = close

    def enqueue(self, first: int, count: int, k: int):
        check(lib.lk_search_resident(self.index._h, self._h, int(first), int(count), int(k)))

    def fetch(self, first: int, count: int, k: int):
        ids = np.full((count, k), -1, np.int64)
        scores = np.zeros((count, k), np.float32)
        iscores = np.zeros((count, k), np.int32)
        counts = np.zeros(count, np.int32)
        check(lib.lk_queries_fetch(self.index._h, self._h, int(first), int(count), int(k),
                                   ptr(ids), ptr(scores), ptr(iscores), ptr(counts)))
        return ids, scores, iscores, counts


class Comm:
    """One NCCL communicator rank (one process per GPU)."""

    @staticmethod
    def unique_id() -> bytes:
        buf = C.create_string_buffer(128)
        check(lib.lk_comm_unique_id(buf))
        return buf.raw

    def __init__(self, world: int, rank: int, device: int, unique_id: bytes):
        h = _vp()
        buf = C.create_string_buffer(bytes(unique_id), 128)
        check(lib.lk_comm_create(int(world), int(rank), int(device), buf, C.byref(h)))
        self._h, self.world, self.rank = h, world, rank

    def peer_export(self) -> bytes:
        """This rank's inbox handle (64 bytes) for the in-kernel exchange over peer memory."""
        buf = C.create_string_buffer(64)
        check(lib.lk_comm_peer_export(self._h, buf))
        return buf.raw

    def peer_attach(self, handles):
        """handles: the 64-byte handle of every rank, in rank order."""
        blob = b"".join(bytes(h) for h in handles)
        assert len(blob) == 64 * self.world
        check(lib.lk_comm_peer_attach(self._h, C.create_string_buffer(blob, len(blob))))

    def hamming_pairs(self, hashes, radius: int, cap: int = 1 << 22):
        """All pairs within `radius`, the search split over the ranks (every rank passes the same
        hashes and receives the complete sorted list): -> (pairs[m, 2] uint32, total)."""
        h = np.ascontiguousarray(hashes, dtype=np.uint64)
        pairs = np.empty((max(cap, 1), 2), np.uint32)
        cnt = _i64(0)
        check(lib.lk_hamming_pairs_sharded(self._h, ptr(h), h.size, int(radius), ptr(pairs), int(cap), C.byref(cnt)))
        return pairs[:min(cnt.value, cap)].copy(), int(cnt.value)

    def close(self):
        if getattr(self, "_h", None):
            lib.lk_comm_destroy(self._h)
            self._h = None


def cosine_sim_topk(rows, query, k: int, allow_slots=None, device: int = 0):
    """embedvec.CosineSim of `query` against raw (un-normalised) rows, exact top-k:
    -> (ids[m] int64, scores[m] float32), m = min(k, candidates)."""
    r = np.ascontiguousarray(rows, dtype=np.float32)
    q = np.ascontiguousarray(query, dtype=np.float32).reshape(-1)
    n = r.shape[0]
    dim = r.shape[1] if r.ndim == 2 and n else q.size
    kk = max(int(k), 0)
    ids = np.full(max(kk, 1), -1, np.int64)
    scores = np.zeros(max(kk, 1), np.float32)
    cnt = _int(0)
    al, nal = None, 0
    if allow_slots is not None:
        al = np.ascontiguousarray(allow_slots, dtype=np.int32)
        nal = al.size
        if nal == 0:
            al = np.zeros(1, np.int32)
    check(lib.lk_cosine_sim_topk(ptr(r) if n else None, n, int(dim), ptr(q), int(k), ptr(al), nal, int(device),
                                 ptr(ids), ptr(scores), C.byref(cnt)))
    return ids[:cnt.value].copy(), scores[:cnt.value].copy()


def hamming_pairs(hashes, radius: int, cap: int = 1 << 22, part: int = 0, parts: int = 1, device: int = 0):
    h = np.ascontiguousarray(hashes, dtype=np.uint64)
    pairs = np.empty((max(cap, 1), 2), np.uint32)
    cnt = _i64(0)
    check(lib.lk_hamming_pairs(ptr(h), h.size, int(radius), int(part), int(parts), int(device),
                               ptr(pairs), int(cap), C.byref(cnt)))
    return pairs[:min(cnt.value, cap)].copy(), int(cnt.value)


def hamming_scan(hashes, query: int, radius: int, cap: int | None = None, device: int = 0):
    h = np.ascontiguousarray(hashes, dtype=np.uint64)
    cap = h.size if cap is None else cap
    ids = np.empty(max(cap, 1), np.uint32)
    dist = np.empty(max(cap, 1), np.int32)
    cnt = _i64(0)
    check(lib.lk_hamming_scan(ptr(h), h.size, C.c_uint64(int(query)), int(radius), int(device),
                              ptr(ids), ptr(dist), int(cap), C.byref(cnt)))
    n = min(cnt.value, cap)
    return ids[:n].copy(), dist[:n].copy(), int(cnt.value)


def prescreen_pairs(vecs, threshold: float, device: int = 0):
    """Neighbour prescreen of face clustering: -> (near[n,256] int32, count[n], overflow[n] bool)."""
    v = np.ascontiguousarray(vecs, dtype=np.float32)
    n, dim = v.shape
    near = np.zeros((max(n, 1), 256), np.int32)
    count = np.zeros(max(n, 1), np.int32)
    over = np.zeros(max(n, 1), np.uint8)
    check(lib.lk_prescreen_pairs(ptr(v), n, dim, C.c_float(threshold), int(device), ptr(near), ptr(count), ptr(over)))
    return near[:n], count[:n], over[:n].astype(bool)


def seed_scores(cands, seeds, min_score: float, chunk: int = 0, device: int = 0):
    """Candidate x seed scores of face clustering at or above `min_score`:
    -> (row_start[n_cand + 1] int64, seed[total] int32 ascending per candidate, score[total] float32)."""
    c = np.ascontiguousarray(cands, dtype=np.float32)
    s = np.ascontiguousarray(seeds, dtype=np.float32)
    n_cand, n_seeds = c.shape[0], s.shape[0]
    dim = c.shape[1] if c.ndim == 2 and n_cand else (s.shape[1] if s.ndim == 2 and n_seeds else 1)
    row_start = np.zeros(n_cand + 1, np.int64)
    total = _i64(0)
    cap = max(1024, 8 * n_cand)
    for _ in range(2):  # a second call when the first guess at the output size was too small
        out_seed = np.empty(cap, np.int32)
        out_score = np.empty(cap, np.float32)
        st = lib.lk_seed_scores(ptr(c), n_cand, ptr(s), n_seeds, int(dim), C.c_float(min_score), int(chunk), int(device),
                                ptr(row_start), ptr(out_seed), ptr(out_score), int(cap), C.byref(total))
        if st == LK_ERANGE and total.value > cap:
            cap = int(total.value)
            continue
        check(st)
        break
    n = int(total.value)
    return row_start, out_seed[:n].copy(), out_score[:n].copy()


def pca3(vecs, workers: int = 1, device: int = 0):
    """Three-component PCA projection: -> (coords[n, 3] float32 in [-1, 1], variance[3] float64)."""
    v = np.ascontiguousarray(vecs, dtype=np.float32)
    n = v.shape[0]
    dim = v.shape[1] if v.ndim == 2 else 0
    coords = np.zeros((max(n, 1), 3), np.float32)
    variance = np.zeros(3, np.float64)
    check(lib.lk_pca3(ptr(v) if n and dim else None, n, int(dim), int(workers), int(device), ptr(coords), ptr(variance)))
    return coords[:n], variance
