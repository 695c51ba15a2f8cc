"""CPU restatement of scoreAgainstSeeds and of the one-at-a-time version its own test pins it
to (media-server/tasks/face_cluster.go:1315-1462, media-server/tasks/face_score_kernel_test.go:17-78).

Test infrastructure only.  Scores come from the C restatement of dot4 / dotf; the decision
logic is restated here statement by statement.  Where the reference lets Go's map order pick
between people of equal effective score, the lower person id wins (stated in the tests).
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Sequence

import numpy as np

import oracle as O

corroborationSlack = np.float32(0.06)   # face_cluster.go:35
corroborationBonus = np.float32(0.02)   # :36
maxCorroborators = 3                    # :37
userSeedWeight = 3                      # :47
meanJoinSlack = np.float32(2) * corroborationSlack  # :62


def effective_score(best: np.float32, count: int) -> np.float32:  # :71-80
    extra = count - 1
    if extra < 0:
        extra = 0
    if extra > maxCorroborators:
        extra = maxCorroborators
    return np.float32(best + np.float32(extra) * corroborationBonus)


def accept_join(best: np.float32, count: int, threshold: np.float32) -> bool:  # :86-88
    return bool(effective_score(best, count) >= threshold and best >= np.float32(threshold - corroborationSlack))


def build_person_aggs(seed_vecs, seed_person: Sequence[int], seed_user: Sequence[bool]):  # :401-426
    aggs: Dict[int, dict] = {}
    for v, pid, user in zip(np.asarray(seed_vecs, np.float32), seed_person, seed_user):
        a = aggs.get(pid)
        if a is None:
            a = aggs[pid] = dict(sum=np.zeros(v.size, np.float32), n=np.float32(0), userSum=None, userN=np.float32(0))
        for k in range(v.size):
            a["sum"][k] = np.float32(a["sum"][k] + v[k])
        a["n"] = np.float32(a["n"] + np.float32(1))
        if user:
            if a["userSum"] is None:
                a["userSum"] = np.zeros(v.size, np.float32)
            for k in range(v.size):
                a["userSum"][k] = np.float32(a["userSum"][k] + v[k])
            a["userN"] = np.float32(a["userN"] + np.float32(1))
    return aggs


def score_against_seeds(cand_ids: Sequence[int], cand_vecs, seed_ids: Sequence[int], seed_vecs,
                        seed_person: Sequence[int], seed_user: Sequence[bool], aggs, threshold,
                        vetoes: Dict[int, Iterable[int]], cannot: Dict[int, Iterable[int]],
                        workers: int = 1, grouped: bool = True) -> List[int]:
    """grouped=True: scoreAgainstSeeds with `workers` worker chunks; False: the one-at-a-time
    version of the reference's test.  The decision part is the same text in both."""
    n = len(cand_ids)
    matches = [0] * n
    if n == 0 or len(seed_ids) == 0:
        return matches
    threshold = np.float32(threshold)
    user_mean_floor = np.float32(threshold - meanJoinSlack)
    auto_mean_floor = threshold
    w = max(1, min(int(workers), n))
    chunk = (n + w - 1) // w
    cand_vecs = np.asarray(cand_vecs, np.float32)
    dense = O.seed_scores(cand_vecs, seed_vecs, chunk, grouped)
    for i in range(n):
        scores: Dict[int, list] = {}
        forbidden = {pid: True for pid in vetoes.get(cand_ids[i], ())}
        cl = set(cannot.get(cand_ids[i], ()))
        for k in range(len(seed_ids)):
            pid = seed_person[k]
            if seed_ids[k] in cl:
                forbidden[pid] = True
                continue
            if forbidden.get(pid):
                continue
            sc = dense[i, k]
            if sc < np.float32(threshold - corroborationSlack):
                continue
            ps = scores.setdefault(pid, [np.float32(0), 0])
            if sc > ps[0]:
                ps[0] = sc
            ps[1] += userSeedWeight if seed_user[k] else 1
        best_person, best = 0, [np.float32(0), 0]
        for pid in sorted(scores):
            ps = scores[pid]
            if forbidden.get(pid) or not accept_join(ps[0], ps[1], threshold):
                continue
            a = aggs.get(pid)
            if a is None:
                continue
            mean = np.float32(O.dot32(cand_vecs[i], a["sum"]) / a["n"])
            floor = auto_mean_floor
            if a["userN"] > 0:
                mean = np.float32(O.dot32(cand_vecs[i], a["userSum"]) / a["userN"])
                floor = user_mean_floor
            if mean < floor:
                continue
            if best_person == 0 or effective_score(ps[0], ps[1]) > effective_score(best[0], best[1]):
                best_person, best = pid, ps
        matches[i] = best_person
    return matches
