"""GPU: candidate x seed scoring of face clustering against the oracle, bit for bit, and the
decisions of the mirrored scoreAgainstSeeds against the oracle's restatement."""
import numpy as np
import pytest

import oracle as O
from oracle import face_cluster as OF
from tests.synth import SEED_SCORING_CASES, seed_scoring_case

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n_cand,n_seed,dim,chunk", [(203, 517, 64, 0), (64, 257, 65, 0), (130, 300, 130, 50),
                                                     (3, 100, 32, 0), (1, 70, 7, 0), (517, 1030, 512, 173)])
def test_pair_lists_equal_the_oracle(lk, n_cand, n_seed, dim, chunk):
    rng = np.random.default_rng(n_cand * 7 + dim)
    centres = rng.standard_normal((9, dim)).astype(np.float32)
    def cloud(n):
        v = centres[rng.integers(0, 9, n)] + 0.4 * rng.standard_normal((n, dim)).astype(np.float32)
        return np.stack([O.normalize(x) for x in v])
    cands, seeds = cloud(n_cand), cloud(n_seed)
    floor = np.float32(0.5)
    row_start, hit_seed, hit_score = lk.seed_scores(cands, seeds, float(floor), chunk)
    dense = O.seed_scores(cands, seeds, chunk, True)
    assert row_start[-1] == len(hit_seed) == int((dense >= floor).sum()) > 0
    for i in range(n_cand):
        want = np.nonzero(dense[i] >= floor)[0]
        got = hit_seed[row_start[i]:row_start[i + 1]]
        assert np.array_equal(got, want)
        assert np.array_equal(hit_score[row_start[i]:row_start[i + 1]].view(np.uint32), dense[i, want].view(np.uint32))


def test_small_output_buffer_reports_the_needed_size(lk):
    import ctypes as C
    rng = np.random.default_rng(3)
    v = np.stack([O.normalize(x) for x in rng.standard_normal((40, 16)).astype(np.float32) + 2.0])
    row_start = np.zeros(41, np.int64)
    out_seed, out_score = np.zeros(8, np.int32), np.zeros(8, np.float32)
    total = C.c_int64(0)
    st = lk.lib.lk_seed_scores(lk.ptr(v), 40, lk.ptr(v), 40, 16, C.c_float(0.1), 0, 0, lk.ptr(row_start),
                               lk.ptr(out_seed), lk.ptr(out_score), 8, C.byref(total))
    assert st == lk.LK_ERANGE and total.value == 1600
    rs, hs, sc = lk.seed_scores(v, v, 0.1)
    assert rs[-1] == 1600 and np.array_equal(hs[:40], np.arange(40))


@pytest.mark.parametrize("case", SEED_SCORING_CASES, ids=lambda c: c[0])
def test_decisions_equal_the_oracle(lk, case):
    from tests import face_cluster_host as F
    name, n_cand, n_seed, people, dims, thr, vetoes, cannot, users = case
    sc = seed_scoring_case(n_cand, n_seed, people, dims, vetoes, cannot, users, seed=len(name) * 31)
    faces = [F.Face(ID=i, Vec=v) for i, v in zip(sc["cand_ids"], sc["cand_vecs"])]
    seeds = [F.seed(id=i, vec=v, personID=p, user=u)
             for i, v, p, u in zip(sc["seed_ids"], sc["seed_vecs"], sc["seed_person"], sc["seed_user"])]
    aggs = F.buildPersonAggs(seeds)
    oaggs = OF.build_person_aggs(sc["seed_vecs"], sc["seed_person"], sc["seed_user"])
    for pid, a in aggs.items():
        assert np.array_equal(a.sum, oaggs[pid]["sum"]) and a.n == oaggs[pid]["n"]
    for workers in (1, 3):
        got = F.scoreAgainstSeeds(faces, seeds, aggs, thr, sc["vetoes"], sc["cannot"], workers=workers)
        want = OF.score_against_seeds(sc["cand_ids"], sc["cand_vecs"], sc["seed_ids"], sc["seed_vecs"], sc["seed_person"],
                                      sc["seed_user"], oaggs, thr, sc["vetoes"], sc["cannot"], workers=workers)
        assert got == want
    assert any(m != 0 for m in want)


def test_prescreen_mirror_matches_the_oracle(lk):
    from tests import face_cluster_host as F
    rng = np.random.default_rng(42)
    v = rng.standard_normal((300, 64)).astype(np.float32)
    v[4::5] = v[3::5] + 0.05
    v = np.stack([O.normalize(x) for x in v])
    res = F.prescreenCandidates([F.Face(ID=i + 1, Vec=x) for i, x in enumerate(v)], 0.6)
    near, count, over = O.prescreen(v, 0.6, brute_force=True)
    for i in range(300):
        assert bool(res.overflow[i]) == bool(over[i])
        assert np.array_equal(res.near[i], near[i, :count[i]])
