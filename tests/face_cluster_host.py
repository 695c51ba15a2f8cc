"""Test mirror of the caller's side of the face-clustering sweeps (not part of the library: the
Go caller keeps this decision loop; here it exists so that the device kernels can be tested
through the same two functions the reference has).

``prescreenCandidates`` and ``scoreAgainstSeeds`` keep the names, argument meaning and
results of media-server/tasks/face_cluster.go:1189-1285 and :1315-1462.  The dense
arithmetic (every candidate against every seed, every face against every earlier face) runs
in the CUDA library; the sparse decision logic over the surviving pairs (vetoes,
cannot-links, corroboration, the mean guard) is restated here over Python dicts, exactly as
the reference keeps it in Go maps.

One point where the reference itself is not deterministic: when two people end with the same
effective score it keeps whichever its map iteration meets first
(media-server/tasks/face_cluster.go:1430-1452).  Here the lower person id wins.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence, Set

import numpy as np

from loki_b200 import _lib

# media-server/tasks/face_cluster.go:34-38, :47, :62
corroborationSlack = np.float32(0.06)
corroborationBonus = np.float32(0.02)
maxCorroborators = 3
userSeedWeight = 3
meanJoinSlack = np.float32(2) * corroborationSlack
maxFormCandidates = 256


@dataclass
class Face:  # the fields of media.Face these functions read
    ID: int
    Vec: np.ndarray
    Score: float = 0.0


@dataclass
class seed:  # media-server/tasks/face_cluster.go:372-377
    id: int
    vec: np.ndarray
    personID: int
    user: bool = False


@dataclass
class personAgg:  # media-server/tasks/face_cluster.go:389-394
    sum: np.ndarray
    n: np.float32 = np.float32(0)
    userSum: Optional[np.ndarray] = None
    userN: np.float32 = np.float32(0)


@dataclass
class personScore:  # media-server/tasks/face_cluster.go:65-68
    best: np.float32 = np.float32(0)
    count: int = 0


@dataclass
class prescreenResult:
    near: List[np.ndarray] = field(default_factory=list)
    overflow: np.ndarray = field(default_factory=lambda: np.zeros(0, bool))


def effectiveScore(s: personScore) -> np.float32:
    """media-server/tasks/face_cluster.go:71-80."""
    extra = min(max(s.count - 1, 0), maxCorroborators)
    return np.float32(s.best + np.float32(extra) * corroborationBonus)


def acceptJoin(s: personScore, threshold) -> bool:
    """media-server/tasks/face_cluster.go:86-88."""
    threshold = np.float32(threshold)
    return bool(effectiveScore(s) >= threshold and s.best >= np.float32(threshold - corroborationSlack))


def buildPersonAggs(seeds: Sequence[seed]) -> Dict[int, personAgg]:
    """media-server/tasks/face_cluster.go:401-426: float32 sums in seed order."""
    aggs: Dict[int, personAgg] = {}
    for s in seeds:
        v = np.asarray(s.vec, np.float32)
        a = aggs.get(s.personID)
        if a is None:
            a = aggs[s.personID] = personAgg(sum=np.zeros(v.size, np.float32))
        a.sum += v
        a.n = np.float32(a.n + np.float32(1))
        if s.user:
            if a.userSum is None:
                a.userSum = np.zeros(v.size, np.float32)
            a.userSum += v
            a.userN = np.float32(a.userN + np.float32(1))
    return aggs


def dot32(a, b) -> np.float32:
    """media-server/tasks/face_cluster.go:890-896: float64 accumulation in index order."""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    if a.size == 0:
        return np.float32(0)
    return np.float32(np.cumsum(a * b)[-1])  # cumsum adds left to right


def prescreenCandidates(faces: Sequence[Face], threshold, device: int = 0) -> prescreenResult:
    """media-server/tasks/face_cluster.go:1189-1285."""
    if len(faces) == 0:
        return prescreenResult()
    vecs = np.stack([np.asarray(f.Vec, np.float32) for f in faces])
    near, count, over = _lib.prescreen_pairs(vecs, float(np.float32(threshold)), device)
    return prescreenResult(near=[near[i, :count[i]].copy() for i in range(len(faces))], overflow=over)


def scoreAgainstSeeds(unassigned: Sequence[Face], seeds: Sequence[seed], aggs: Dict[int, personAgg], threshold,
                      vetoes: Dict[int, Iterable[int]], cannot: Dict[int, Iterable[int]], workers: int = 1,
                      device: int = 0) -> List[int]:
    """media-server/tasks/face_cluster.go:1315-1462: for every unassigned face the person it
    should join (0 = none).  `workers` is the reference's worker count for this call
    (clusterWorkerBudget capped by the number of faces): it decides which faces the reference
    scores four at a time and which one at a time, and so the last bit of their scores."""
    matches = [0] * len(unassigned)
    if len(unassigned) == 0 or len(seeds) == 0:
        return matches
    threshold = np.float32(threshold)
    userMeanFloor = np.float32(threshold - meanJoinSlack)
    autoMeanFloor = threshold
    floor_score = np.float32(threshold - corroborationSlack)
    w = max(1, min(int(workers), len(unassigned)))
    chunk = (len(unassigned) + w - 1) // w
    cand = np.stack([np.asarray(f.Vec, np.float32) for f in unassigned])
    svec = np.stack([np.asarray(s.vec, np.float32) for s in seeds])
    row_start, hit_seed, hit_score = _lib.seed_scores(cand, svec, float(floor_score), chunk, device)
    seed_index_by_id = {s.id: k for k, s in enumerate(seeds)}
    for i, f in enumerate(unassigned):
        forbidden: Set[int] = set(vetoes.get(f.ID, ()))
        for sid in cannot.get(f.ID, ()):  # a cannot-linked member takes its whole person off the table
            k = seed_index_by_id.get(sid)
            if k is not None:
                forbidden.add(seeds[k].personID)
        cl = set(cannot.get(f.ID, ()))
        scores: Dict[int, personScore] = {}
        for p in range(int(row_start[i]), int(row_start[i + 1])):
            s = seeds[int(hit_seed[p])]
            if s.id in cl or s.personID in forbidden:
                continue
            sc = np.float32(hit_score[p])
            ps = scores.setdefault(s.personID, personScore())
            if sc > ps.best:
                ps.best = sc
            ps.count += userSeedWeight if s.user else 1
        bestPerson, best = 0, personScore()
        for pid in sorted(scores):
            ps = scores[pid]
            if pid in forbidden or not acceptJoin(ps, threshold):
                continue
            a = aggs.get(pid)
            if a is None:
                continue
            mean = np.float32(dot32(f.Vec, a.sum) / a.n)
            floor = autoMeanFloor
            if a.userN > 0:
                mean = np.float32(dot32(f.Vec, a.userSum) / a.userN)
                floor = userMeanFloor
            if mean < floor:
                continue
            if bestPerson == 0 or effectiveScore(ps) > effectiveScore(best):
                bestPerson, best = pid, ps
        matches[i] = bestPerson
    return matches
