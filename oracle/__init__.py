"""CPU oracle for the exact vector-scan path (TEST INFRASTRUCTURE ONLY).

Only the tests, ``__graft_entry__.smoke()`` and the CPU-baseline / reference legs
of ``bench.py`` may import this package; the shipped library never does.

``oracle.c`` holds the arithmetic (a C restatement of the reference's Go code, each
function citing the lines it follows); this module loads it through ctypes and
``exact_index.py`` restates the index bookkeeping around it.

Parity status: the fp32 path is pinned by the reference's literal-vector tests
(ported in ``tests/``); the int8 and Hamming functions have no counterpart in the
reference: parity unpinned.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle.so")


def build(force: bool = False) -> str:
    """Compile ``oracle.c`` with the Makefile beside it; returns the .so path."""
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s"] + (["-B"] if force else []))
    return _SO


_lib = None

_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(np.float64, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_i8p = np.ctypeslib.ndpointer(np.int8, flags="C_CONTIGUOUS")
_u64p = np.ctypeslib.ndpointer(np.uint64, flags="C_CONTIGUOUS")
_u32p = np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")


def lib():
    global _lib
    if _lib is not None:
        return _lib
    L = C.CDLL(build())
    L.orc_normalize.argtypes = [_f32p, C.c_int, _f32p]
    L.orc_normalize.restype = None
    L.orc_cosine.argtypes = [_f32p, _f32p, C.c_int]
    L.orc_cosine.restype = C.c_float
    L.orc_cosine_sim.argtypes = [_f32p, _f32p, C.c_int]
    L.orc_cosine_sim.restype = C.c_float
    L.orc_centered_norm.argtypes = [_f32p, _f32p, C.c_int, C.c_double]
    L.orc_centered_norm.restype = C.c_float
    L.orc_mean_from_sum.argtypes = [_f64p, C.c_int, C.c_int64, _f32p]
    L.orc_mean_from_sum.restype = C.c_double
    L.orc_center_query.argtypes = [_f32p, _f32p, C.c_int, _f32p]
    L.orc_center_query.restype = C.c_float
    L.orc_scan_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int, _f32p, C.c_void_p,
                               C.c_float, C.c_void_p, C.c_int64, _f32p, C.c_int]
    L.orc_scan_f32.restype = None
    L.orc_topk_heap_f32.argtypes = [_f32p, C.c_int64, C.c_int, _i32p]
    L.orc_topk_heap_f32.restype = C.c_int
    L.orc_shared_new.argtypes = [_f32p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int,
                                 C.c_int, C.c_float, C.c_float, C.POINTER(C.c_int)]
    L.orc_shared_new.restype = C.c_void_p
    L.orc_shared_free.argtypes = [C.c_void_p]
    L.orc_shared_free.restype = None
    L.orc_shared_rank.argtypes = [C.c_void_p]
    L.orc_shared_rank.restype = C.c_int
    L.orc_shared_export.argtypes = [C.c_void_p, _f32p, _f32p, _f32p, _f32p, _f32p,
                                    C.POINTER(C.c_float)]
    L.orc_shared_export.restype = None
    L.orc_shared_score.argtypes = [C.c_void_p, _f32p]
    L.orc_shared_score.restype = C.c_float
    L.orc_scan_shared.argtypes = [C.c_void_p, _f32p, C.c_int64, C.c_void_p, C.c_void_p,
                                  C.c_void_p, C.c_int64, _f32p]
    L.orc_scan_shared.restype = None
    L.orc_quantize_i8.argtypes = [_f32p, C.c_int, _i8p, C.POINTER(C.c_float)]
    L.orc_quantize_i8.restype = None
    L.orc_build_i8.argtypes = [_f32p, C.c_int64, C.c_int, C.c_int64, _i8p, C.c_int64, _f32p]
    L.orc_build_i8.restype = None
    L.orc_scan_i8.argtypes = [_i8p, C.c_int64, C.c_int, _i8p, C.c_void_p, C.c_int64, _i32p]
    L.orc_scan_i8.restype = None
    L.orc_topk_i32.argtypes = [_i32p, C.c_void_p, C.c_int64, C.c_int, _i32p, _i32p]
    L.orc_topk_i32.restype = C.c_int
    L.orc_topk_f32.argtypes = [_f32p, C.c_void_p, C.c_int64, C.c_int, _i32p, _f32p]
    L.orc_topk_f32.restype = C.c_int
    L.orc_hamming_pairs.argtypes = [_u64p, C.c_int64, C.c_int, _u32p, C.c_int64]
    L.orc_hamming_pairs.restype = C.c_int64
    L.orc_hamming_pairs_rows.argtypes = [_u64p, C.c_int64, C.c_int, C.c_int64, C.c_int64, _u32p, C.c_int64]
    L.orc_hamming_pairs_rows.restype = C.c_int64
    L.orc_hamming_scan.argtypes = [_u64p, C.c_int64, C.c_uint64, _i32p]
    L.orc_hamming_scan.restype = None
    _u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
    L.orc_dotf.argtypes = [_f32p, _f32p, C.c_int]
    L.orc_dotf.restype = C.c_float
    for fn in (L.orc_prescreen, L.orc_prescreen_bruteforce):
        fn.argtypes = [_f32p, C.c_int, C.c_int, C.c_float, _i32p, _i32p, _u8p]
        fn.restype = None
    L.orc_seed_scores.argtypes = [_f32p, C.c_int, _f32p, C.c_int, C.c_int, C.c_int, _f32p]
    L.orc_seed_scores.restype = None
    L.orc_seed_scores_single.argtypes = [_f32p, C.c_int, _f32p, C.c_int, C.c_int, _f32p]
    L.orc_seed_scores_single.restype = None
    L.orc_pca3.argtypes = [_f32p, C.c_int, C.c_int, C.c_int, _f32p, np.ctypeslib.ndpointer(np.float64, flags="C_CONTIGUOUS")]
    L.orc_pca3.restype = None
    L.orc_dot32.argtypes = [_f32p, _f32p, C.c_int]
    L.orc_dot32.restype = C.c_float
    _lib = L
    return L


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


# ---- embedvec ---------------------------------------------------------------

def normalize(v) -> np.ndarray:
    v = _f32(v)
    out = np.empty_like(v)
    lib().orc_normalize(v, v.size, out)
    return out


def normalize_rows(rows) -> np.ndarray:
    rows = _f32(rows)
    out = np.empty_like(rows)
    L = lib()
    for i in range(rows.shape[0]):
        L.orc_normalize(rows[i], rows.shape[1], out[i])
    return out


def cosine(a, b) -> np.float32:
    a, b = _f32(a), _f32(b)
    if a.size != b.size:
        return np.float32(0)
    return np.float32(lib().orc_cosine(a, b, a.size))


def cosine_sim(a, b) -> np.float32:
    a, b = _f32(a), _f32(b)
    if a.size != b.size:
        return np.float32(0)
    return np.float32(lib().orc_cosine_sim(a, b, a.size))


def encode(v) -> bytes:
    """Little-endian float32 BLOB (media-server/embedvec/embedvec.go:13-19)."""
    return _f32(v).astype("<f4").tobytes()


def decode(b: bytes) -> np.ndarray:
    """Inverse of encode; rejects lengths that are not a multiple of 4
    (media-server/embedvec/embedvec.go:22-31)."""
    if len(b) % 4 != 0:
        raise ValueError(f"embedvec: byte length {len(b)} is not a multiple of 4")
    return np.frombuffer(b, dtype="<f4").astype(np.float32)


# ---- scans ------------------------------------------------------------------

def scan_f32(rows, q, cnorm=None, cq=0.0, slots=None, workers=1, rowp=None) -> np.ndarray:
    """scores[t] for every row (or rows[slots[t]]); plain when cnorm is None."""
    rows = _f32(rows)
    q = _f32(q)
    n = rows.shape[0] if slots is None else len(slots)
    scores = np.empty(n, dtype=np.float32)
    if n == 0:
        return scores
    sl = None if slots is None else np.ascontiguousarray(slots, dtype=np.int32)
    cn = None if cnorm is None else _f32(cnorm)
    lib().orc_scan_f32(None if rowp is not None else _ptr(rows), _ptr(rowp), rows.shape[1],
                       q.size, q, _ptr(cn), float(cq), _ptr(sl), n, scores, int(workers))
    return scores


def topk_heap(scores, k) -> np.ndarray:
    scores = _f32(scores)
    h = np.empty(max(k, 1), dtype=np.int32)
    n = lib().orc_topk_heap_f32(scores, scores.size, int(k), h)
    return h[:n]


def topk_f32(scores, k, ids=None):
    scores = _f32(scores)
    kk = max(min(k, scores.size), 0)
    oi = np.empty(max(kk, 1), np.int32)
    os_ = np.empty(max(kk, 1), np.float32)
    idp = None if ids is None else np.ascontiguousarray(ids, np.int32)
    n = lib().orc_topk_f32(scores, _ptr(idp), scores.size, int(k), oi, os_)
    return oi[:n], os_[:n]


def topk_i32(scores, k, ids=None):
    scores = np.ascontiguousarray(scores, np.int32)
    kk = max(min(k, scores.size), 0)
    oi = np.empty(max(kk, 1), np.int32)
    os_ = np.empty(max(kk, 1), np.int32)
    idp = None if ids is None else np.ascontiguousarray(ids, np.int32)
    n = lib().orc_topk_i32(scores, _ptr(idp), scores.size, int(k), oi, os_)
    return oi[:n], os_[:n]


# ---- int8 (parity unpinned) -------------------------------------------------

def build_i8(rows, ld_out=None):
    """normalize + quantise each row -> (codes[n, ld_out] int8, scales[n] f32)."""
    rows = _f32(rows)
    n, d = rows.shape
    ld_out = d if ld_out is None else ld_out
    codes = np.zeros((n, ld_out), np.int8)
    scales = np.zeros(n, np.float32)
    if n:
        lib().orc_build_i8(rows, n, d, d, codes, ld_out, scales)
    return codes, scales


def scan_i8(codes, q, d=None, slots=None, workers=1) -> np.ndarray:
    """int32 dot of every row (or rows[slots[t]]) with q; workers > 1 splits the rows into
    contiguous bands, one host thread each (whole-corpus scans of 1,000,000+ rows)."""
    codes = np.ascontiguousarray(codes, np.int8)
    q = np.ascontiguousarray(q, np.int8)
    d = q.size if d is None else d
    n = codes.shape[0] if slots is None else len(slots)
    out = np.empty(n, np.int32)
    sl = None if slots is None else np.ascontiguousarray(slots, np.int32)
    if n and (workers <= 1 or slots is not None or n < 4 * workers):
        lib().orc_scan_i8(codes, codes.shape[1], d, q, _ptr(sl), n, out)
    elif n:
        from concurrent.futures import ThreadPoolExecutor
        L = lib()
        edges = [n * w // workers for w in range(workers + 1)]

        def band(w):
            lo, hi = edges[w], edges[w + 1]
            L.orc_scan_i8(codes[lo:hi], codes.shape[1], d, q, None, hi - lo, out[lo:hi])

        with ThreadPoolExecutor(workers) as ex:
            list(ex.map(band, range(workers)))
    return out


# ---- Hamming (parity unpinned) ----------------------------------------------

def hamming_pairs(h, radius, cap=None):
    h = np.ascontiguousarray(h, np.uint64)
    cap = 1 << 20 if cap is None else cap
    pairs = np.empty((max(cap, 1), 2), np.uint32)
    n = lib().orc_hamming_pairs(h, h.size, int(radius), pairs.reshape(-1), cap)
    return pairs[:min(n, cap)].copy(), int(n)


def hamming_pairs_threaded(h, radius, cap=None, threads=None):
    """The same all-pairs loop with its rows spread over host threads (row bands of equal
    pair counts, concatenated in order): for inputs of 100,000+ hashes."""
    import os
    from concurrent.futures import ThreadPoolExecutor
    h = np.ascontiguousarray(h, np.uint64)
    n = h.size
    cap = 1 << 20 if cap is None else cap
    threads = threads or os.cpu_count() or 1
    bands = threads * 8
    # row i carries n-1-i pairs: cut the triangle into bands of equal area
    edges = [int(round(n * (1.0 - np.sqrt(1.0 - b / bands)))) for b in range(bands)] + [n]
    L = lib()

    def band(b):
        buf = np.empty((max(cap, 1), 2), np.uint32)
        c = L.orc_hamming_pairs_rows(h, n, int(radius), edges[b], edges[b + 1], buf.reshape(-1), cap)
        return buf[:min(c, cap)].copy(), int(c)

    with ThreadPoolExecutor(threads) as ex:
        parts = list(ex.map(band, range(bands)))
    total = sum(c for _, c in parts)
    allp = np.concatenate([p for p, _ in parts]) if parts else np.zeros((0, 2), np.uint32)
    return allp[:cap], total


def hamming_scan(h, q) -> np.ndarray:
    h = np.ascontiguousarray(h, np.uint64)
    out = np.empty(h.size, np.int32)
    lib().orc_hamming_scan(h, h.size, int(q), out)
    return out


# ---- shared query -----------------------------------------------------------

class SharedQuery:
    """embedvec.SharedQuery (media-server/embedvec/shared.go:45-220)."""

    def __init__(self, pos, posw=None, neg=None, negw=None, beta=0.25, lam=1.0):
        pos = [np.asarray(p, np.float32) for p in (pos or [])]
        neg = [np.asarray(p, np.float32) for p in (neg or [])]
        if len(pos) == 0:
            raise ValueError("embedvec: shared query has no positive terms")
        if posw is not None and len(posw) != len(pos):
            raise ValueError("embedvec: shared query: positives/weights count mismatch")
        if len(neg) != (0 if negw is None else len(negw)):
            raise ValueError("embedvec: shared query: negatives/weights count mismatch")
        d = pos[0].size
        for v in pos + neg:
            if v.size != d:
                raise ValueError("embedvec: shared query length mismatch")
        self.d, self.m, self.nneg = d, len(pos), len(neg)
        P = _f32(np.stack(pos))
        N = _f32(np.stack(neg)) if neg else None
        pw = None if posw is None else _f32(posw)
        nw = None if not neg else _f32(negw)
        err = C.c_int(0)
        self._h = lib().orc_shared_new(P, _ptr(pw), self.m, _ptr(N), _ptr(nw), self.nneg, d,
                                       float(beta), float(lam), C.byref(err))
        if not self._h:
            raise ValueError({1: "embedvec: shared query has no positive terms",
                              2: "embedvec: shared query positive weight must be > 0",
                              3: "embedvec: shared query has too many terms"}[err.value])
        self.rank = lib().orc_shared_rank(self._h)

    def __del__(self):
        if getattr(self, "_h", None):
            lib().orc_shared_free(self._h)
            self._h = None

    def score(self, v) -> np.float32:
        return np.float32(lib().orc_shared_score(self._h, _f32(v)))

    def scan(self, rows, mu=None, cnorm=None, slots=None) -> np.ndarray:
        rows = _f32(rows)
        n = rows.shape[0] if slots is None else len(slots)
        out = np.empty(n, np.float32)
        sl = None if slots is None else np.ascontiguousarray(slots, np.int32)
        muv = None if mu is None else _f32(mu)
        cn = None if cnorm is None else _f32(cnorm)
        if n:
            lib().orc_scan_shared(self._h, rows, rows.shape[1], _ptr(muv), _ptr(cn), _ptr(sl), n, out)
        return out

    def export(self):
        pos = np.empty((self.m, self.d), np.float32)
        basis = np.empty((max(self.rank, 1), self.d), np.float32)
        posw = np.empty(self.m, np.float32)
        posnorm = np.empty(self.m, np.float32)
        qb = np.empty((self.m, max(self.rank, 1)), np.float32)
        g = C.c_float(0)
        lib().orc_shared_export(self._h, pos, basis, posw, posnorm, qb.reshape(-1), C.byref(g))
        return dict(pos=pos, basis=basis[:self.rank], posw=posw, posnorm=posnorm,
                    qb=qb.reshape(-1)[:self.m * self.rank].reshape(self.m, self.rank) if self.rank else qb[:, :0],
                    gamma=np.float32(g.value))


# ---- face-clustering prescreen (media-server/tasks/face_cluster.go:1189-1285) --------

MAX_FORM_CANDIDATES = 256


def dotf(a, b) -> np.float32:
    a, b = _f32(a), _f32(b)
    return np.float32(lib().orc_dotf(a, b, a.size)) if a.size == b.size else np.float32(0)


def prescreen(vecs, threshold: float, brute_force: bool = False):
    """-> (near[n, 256] int32, count[n] int32, overflow[n] bool) for unit rows `vecs`."""
    v = _f32(vecs)
    n, d = v.shape
    near = np.zeros((max(n, 1), MAX_FORM_CANDIDATES), np.int32)
    count = np.zeros(max(n, 1), np.int32)
    over = np.zeros(max(n, 1), np.uint8)
    fn = lib().orc_prescreen_bruteforce if brute_force else lib().orc_prescreen
    if n:
        fn(v, n, d, float(threshold), near.reshape(-1), count, over)
    return near[:n], count[:n], over[:n].astype(bool)


# ---- face-clustering candidate x seed scores (media-server/tasks/face_cluster.go:1315-1462) ----

def seed_scores(cands, seeds, chunk: int = 0, grouped: bool = True) -> np.ndarray:
    """Dense n_cand x n_seeds float32 scores: four candidates at a time within worker chunks of
    `chunk` candidates (`grouped`), or every pair one at a time."""
    c, s = _f32(cands), _f32(seeds)
    out = np.zeros((c.shape[0], s.shape[0]), np.float32)
    if c.shape[0] and s.shape[0]:
        if grouped:
            lib().orc_seed_scores(c, c.shape[0], s, s.shape[0], c.shape[1], int(chunk), out.reshape(-1))
        else:
            lib().orc_seed_scores_single(c, c.shape[0], s, s.shape[0], c.shape[1], out.reshape(-1))
    return out


def dot32(a, b) -> np.float32:
    a, b = _f32(a), _f32(b)
    return np.float32(lib().orc_dot32(a, b, a.size))


# ---- PCA projection (media-server/embedvec/pca.go:22-182) -----------------------------------

def pca3(vecs, workers: int = 1):
    """embedvec.ProjectPCA3 as it runs on a machine with `workers` CPUs:
    -> (coords[n, 3] float32, variance[3] float64)."""
    v = _f32(vecs)
    n = v.shape[0]
    d = v.shape[1] if v.ndim == 2 else 0
    coords = np.zeros((max(n, 1), 3), np.float32)
    variance = np.zeros(3, np.float64)
    if n and d:
        lib().orc_pca3(v, n, d, int(workers), coords.reshape(-1), variance)
    return coords[:n], variance
