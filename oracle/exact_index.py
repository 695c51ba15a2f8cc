"""Oracle restatement of the reference's in-RAM exact index (TEST INFRASTRUCTURE ONLY).

Bookkeeping (paths, slot map, swap-remove delete, f64 running column sum, lazy
re-centering, allow-set resolution, heap top-k, tie order) follows
media-server/embedindex/embedindex.go line by line; the arithmetic is delegated to
the C functions in oracle.c.  Method names are the reference's.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional

import numpy as np

import oracle as O

MinCenterCount = 64  # media-server/embedindex/embedindex.go:55
ScoreDefault = 0     # media-server/embedindex/embedindex.go:70
ScorePlain = 1       # media-server/embedindex/embedindex.go:76
DefaultSharedBeta = 0.25   # media-server/embedvec/shared.go:20
DefaultSharedLambda = 1.0  # media-server/embedvec/shared.go:26


@dataclass
class SearchHit:  # media-server/embedindex/embedindex.go:58-61
    Path: str
    Score: np.float32


@dataclass
class SharedSpec:  # media-server/embedindex/embedindex.go:83-88
    Pos: list
    PosW: Optional[list] = None
    Neg: Optional[list] = None
    NegW: Optional[list] = None


class ExactIndex:
    """media-server/embedindex/embedindex.go:122-140."""

    def __init__(self, centering: bool = False):
        self.paths: List[str] = []
        self.vecs: List[np.ndarray] = []
        self.slot: Dict[str, int] = {}
        self.centering = centering
        self.sum: Optional[np.ndarray] = None
        self.mu: Optional[np.ndarray] = None
        self.muN2 = 0.0
        self.cnorm: Optional[List[np.float32]] = None
        self.nCentered = 0

    # -- :155-174
    def _sum_add(self, v):
        if not self.centering:
            return
        if self.sum is None:
            self.sum = np.zeros(v.size, np.float64)
        self.sum[: v.size] += v.astype(np.float64)

    def _sum_sub(self, v):
        if not self.centering or self.sum is None:
            return
        self.sum[: v.size] -= v.astype(np.float64)

    # -- :176-194
    def Add(self, path: str, vec):
        v = O.normalize(vec)
        i = self.slot.get(path)
        if i is not None:
            self._sum_sub(self.vecs[i])
            self.vecs[i] = v
            self._sum_add(v)
            if self.mu is not None:
                self.cnorm[i] = self._centered_norm(v)
            return
        self.slot[path] = len(self.paths)
        self.paths.append(path)
        self.vecs.append(v)
        self._sum_add(v)
        if self.mu is not None:
            self.cnorm.append(self._centered_norm(v))

    # -- :196-217
    def Delete(self, path: str):
        i = self.slot.get(path)
        if i is None:
            return
        self._sum_sub(self.vecs[i])
        last = len(self.paths) - 1
        if i != last:
            self.paths[i] = self.paths[last]
            self.vecs[i] = self.vecs[last]
            self.slot[self.paths[i]] = i
            if self.cnorm is not None:
                self.cnorm[i] = self.cnorm[last]
        self.paths.pop()
        self.vecs.pop()
        if self.cnorm is not None:
            self.cnorm.pop()
        del self.slot[path]

    def Len(self) -> int:  # :219
        return len(self.paths)

    # -- :222-228
    def _centered_norm(self, v) -> np.float32:
        if v.size != self.mu.size:  # Cosine returns 0 on a length mismatch
            n2 = max(0.0, 1.0 + self.muN2)
            return np.float32(np.sqrt(n2))
        return np.float32(O.lib().orc_centered_norm(v, self.mu, v.size, self.muN2))

    # -- :234-268
    def _maybe_recenter(self):
        if not self.centering:
            return
        n = len(self.paths)
        if n < MinCenterCount:
            self.mu, self.cnorm, self.nCentered = None, None, n
            return
        if self.mu is not None:
            drift = abs(n - self.nCentered)
            if drift <= self.nCentered // 10 + 32:
                return
        mu = np.empty(self.sum.size, np.float32)
        self.muN2 = O.lib().orc_mean_from_sum(self.sum, self.sum.size, n, mu)
        self.mu = mu
        self.cnorm = [self._centered_norm(v) for v in self.vecs]
        self.nCentered = n

    def _center_for(self, s):  # :272-277
        return None if s == ScorePlain else self.mu

    def _rows(self) -> np.ndarray:
        d = self.vecs[0].size
        rows = np.zeros((len(self.vecs), d), np.float32)
        for i, v in enumerate(self.vecs):
            if v.size == d:
                rows[i] = v
        return rows

    # -- :284-306 + :424-457
    def SearchScored(self, query, k: int, allow: Optional[Iterable[str]], s: int) -> Optional[List[SearchHit]]:
        self._maybe_recenter()
        slots = None
        if allow is not None:
            slots = self._collect_slots(allow)
            if len(slots) == 0:
                return None
        n = len(self.paths) if slots is None else len(slots)
        if n == 0 or k <= 0:
            return None
        q = O.normalize(query)
        mu = self._center_for(s)
        rows = self._rows()
        if rows.shape[1] != q.size:
            scores = np.zeros(n, np.float32)  # every Cosine hits the length-mismatch branch
        elif mu is None or q.size != mu.size:
            scores = O.scan_f32(rows, q, slots=slots)
        else:
            qc = np.empty_like(q)
            cq = O.lib().orc_center_query(q, mu, q.size, qc)
            scores = O.scan_f32(rows, qc, cnorm=np.asarray(self.cnorm, np.float32), cq=cq, slots=slots)
        return self._finish(scores, slots, k)

    def Search(self, query, k):  # :308-310
        return self.SearchScored(query, k, None, ScoreDefault)

    def SearchFiltered(self, query, k, allow):  # :314-316
        return self.SearchScored(query, k, allow, ScoreDefault)

    def SearchShared(self, spec: SharedSpec, k, allow):  # :334-336
        return self.SearchSharedScored(spec, k, allow, ScoreDefault)

    # -- :338-394
    def SearchSharedScored(self, spec: SharedSpec, k, allow, s):
        self._maybe_recenter()
        mu = self._center_for(s)

        def prep(vs):
            out = []
            for v in vs or []:
                n = O.normalize(v)
                if mu is not None and n.size == mu.size:
                    n = O.normalize(n - mu)
                out.append(n)
            return out

        sq = O.SharedQuery(prep(spec.Pos), spec.PosW, prep(spec.Neg), spec.NegW,
                           DefaultSharedBeta, DefaultSharedLambda)
        slots = None
        if allow is not None:
            slots = self._collect_slots(allow)
            if len(slots) == 0:
                return None
        n = len(self.paths) if slots is None else len(slots)
        if n == 0 or k <= 0:
            return None
        rows = self._rows()
        if mu is None:
            scores = sq.scan(rows, slots=slots)
        else:
            scores = sq.scan(rows, mu=mu, cnorm=np.asarray(self.cnorm, np.float32), slots=slots)
        return self._finish(scores, slots, k)

    # -- :398-419
    def _collect_slots(self, allow) -> List[int]:
        allow = set(allow)
        if len(self.paths) == 0 or len(allow) == 0:
            return []
        if len(allow) < len(self.paths):
            return [self.slot[p] for p in allow if p in self.slot]
        return [i for i, p in enumerate(self.paths) if p in allow]

    # -- :443-456 + :483-490
    def _finish(self, scores, slots, k) -> List[SearchHit]:
        n = scores.size
        k = min(k, n)
        top = O.topk_heap(scores, k)
        hits = []
        for j in top:
            sl = int(j) if slots is None else slots[int(j)]
            hits.append(SearchHit(self.paths[sl], np.float32(scores[int(j)])))
        hits.sort(key=_hit_key)
        return hits


def _hit_key(h: SearchHit):
    return (-float(h.Score), h.Path)


def New() -> ExactIndex:  # :144-146
    return ExactIndex(False)


def NewCentered() -> ExactIndex:  # :151-153
    return ExactIndex(True)
