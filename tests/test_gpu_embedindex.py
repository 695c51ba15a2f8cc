"""GPU: the reference's known-answer tests against the CUDA library through the
path-keyed interface, plus parity of centered / shared scoring with the oracle."""
import types

import numpy as np
import pytest

import oracle as O
from oracle import exact_index as OX
from tests import ref_cases
from tests.synth import gaussian_rows

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def impl(lk):
    from loki_b200 import embedindex as E
    return types.SimpleNamespace(New=E.New, NewCentered=E.NewCentered, SharedSpec=E.SharedSpec,
                                 ScoreDefault=E.ScoreDefault, ScorePlain=E.ScorePlain,
                                 MinCenterCount=E.MinCenterCount)


@pytest.mark.parametrize("case", ref_cases.ALL_CASES, ids=lambda f: f.__name__)
def test_reference_case_on_gpu(impl, case):
    case(impl)


def _common_rows(n, dim, seed):
    """Rows sharing a strong common component, like real image embeddings."""
    r = gaussian_rows(n, dim, seed)
    r[:, 0] += 6.0
    return r


def _assert_hits_close(got, want, rel=1e-5):
    assert len(got) == len(want)
    gs = np.array([h.Score for h in got], np.float32)
    ws = np.array([h.Score for h in want], np.float32)
    np.testing.assert_allclose(gs, ws, rtol=rel, atol=1e-6)
    for i, (g, w) in enumerate(zip(got, want)):
        if g.Path != w.Path:  # only tolerated between (nearly) tied neighbours
            assert abs(float(g.Score) - float(w.Score)) <= rel * max(abs(float(w.Score)), 1e-6)


@pytest.mark.parametrize("n,dim,k", [(64, 16, 10), (500, 96, 25), (3000, 768, 50)])
def test_centered_search_matches_oracle(impl, n, dim, k):
    rows = _common_rows(n, dim, 21)
    names = [f"img-{i:06d}" for i in range(n)]
    gi, oi = impl.NewCentered(), OX.NewCentered()
    gi.AddBatch(names, rows)
    for p, v in zip(names, rows):
        oi.Add(p, v)
    qs = _common_rows(3, dim, 22)
    for q in qs:
        _assert_hits_close(gi.Search(q, k), oi.Search(q, k))
        _assert_hits_close(gi.SearchScored(q, k, None, impl.ScorePlain), oi.SearchScored(q, k, None, OX.ScorePlain))
    allow = set(names[::7])
    _assert_hits_close(gi.SearchFiltered(qs[0], k, allow), oi.SearchFiltered(qs[0], k, allow))
    # churn: deletes (swap-remove), in-place updates, growth past the drift threshold
    for i in range(0, n, 5):
        gi.Delete(names[i]); oi.Delete(names[i])
    upd = _common_rows(4, dim, 23)
    for j, v in enumerate(upd):
        gi.Add(names[1 + 5 * j], v); oi.Add(names[1 + 5 * j], v)
    extra = _common_rows(n // 2, dim, 24)
    for j, v in enumerate(extra):
        gi.Add(f"new-{j:05d}", v); oi.Add(f"new-{j:05d}", v)
    assert gi.Len() == oi.Len()
    for q in qs:
        _assert_hits_close(gi.Search(q, k), oi.Search(q, k))


def test_centering_state_is_bit_identical_to_oracle(lk):
    """Column sum, mean and per-row centered norms against the oracle's bookkeeping."""
    n, dim = 400, 48
    rows = _common_rows(n, dim, 31)
    idx = lk.DeviceIndex(dim, lk.LK_F32, centered=True)
    idx.append(rows)
    oi = OX.NewCentered()
    for i, v in enumerate(rows):
        oi.Add(str(i), v)
    idx.search(rows[0], 1)          # triggers the first re-centre on both
    oi.Search(rows[0], 1)
    st = idx.center_state()
    assert st["live"] and st["n_centered"] == n
    assert np.array_equal(st["sum"], oi.sum), "float64 column sum must round like the row-by-row Add loop"
    assert np.array_equal(st["mu"], oi.mu)
    assert st["mu_n2"] == oi.muN2
    ocn = np.asarray(oi.cnorm, np.float32)
    # the per-row <v,mu> is reduced across lanes on the GPU: allow the last bit
    np.testing.assert_allclose(st["cnorm"], ocn, rtol=3e-7)
    assert (st["cnorm"] == ocn).mean() > 0.95


@pytest.mark.parametrize("centered", [False, True])
def test_shared_search_matches_oracle(impl, centered):
    n, dim, k = 1500, 128, 40
    rows = _common_rows(n, dim, 41)
    names = [f"m-{i:05d}" for i in range(n)]
    gi = impl.NewCentered() if centered else impl.New()
    oi = OX.NewCentered() if centered else OX.New()
    gi.AddBatch(names, rows)
    for p, v in zip(names, rows):
        oi.Add(p, v)
    pos = _common_rows(4, dim, 42)
    neg = _common_rows(2, dim, 43)
    for spec_kw in (dict(Pos=list(pos[:1])), dict(Pos=list(pos[:2])), dict(Pos=list(pos), PosW=[1, 2, 0.5, 1]),
                    dict(Pos=list(pos[:3]), Neg=list(neg), NegW=[0.5, -0.25]),
                    dict(Pos=[pos[0], pos[0], pos[1]])):
        g = gi.SearchShared(impl.SharedSpec(**spec_kw), k, None)
        w = oi.SearchShared(OX.SharedSpec(**spec_kw), k, None)
        _assert_hits_close(g, w, rel=2e-5)
    allow = set(names[::3])
    g = gi.SearchShared(impl.SharedSpec(Pos=list(pos[:3])), k, allow)
    w = oi.SearchShared(OX.SharedSpec(Pos=list(pos[:3])), k, allow)
    _assert_hits_close(g, w, rel=2e-5)


@pytest.mark.parametrize("npos,nneg", [(1, 0), (2, 0), (3, 1), (5, 2), (8, 0), (11, 3), (16, 1), (4, 0)])
def test_shared_search_large_index_matches_oracle(lk, npos, nneg):
    """Indexes of 8192 rows and more take the kernel that stages whole rows in shared
    memory; every term-count class of it, with a ragged last batch of rows."""
    _shared_large_case(lk, 9003, 200, 60, npos, nneg)


def test_shared_search_large_index_many_terms_wide_rows(lk):
    """31 query-side vectors of 768 floats do not fit in shared memory as float64: the
    kernel keeps them as float32 and widens them per batch of rows."""
    _shared_large_case(lk, 8210, 768, 25, 16, 0)


def _shared_large_case(lk, n, dim, k, npos, nneg):
    rows = np.stack([O.normalize(v) for v in _common_rows(n, dim, 51)])
    idx = lk.DeviceIndex(dim, lk.LK_F32)
    idx.append(rows)
    stored = idx.read_rows(0, n)
    pos = _common_rows(npos, dim, 52 + npos)
    neg = _common_rows(nneg, dim, 53 + npos) if nneg else None
    posw = list(np.linspace(0.5, 2.0, npos).astype(np.float32))
    negw = list(np.linspace(0.25, 0.5, nneg).astype(np.float32)) if nneg else None
    ids, scores = idx.search_shared(pos, posw=posw, neg=neg, negw=negw, k=k, scoring=lk.LK_SCORE_PLAIN)
    sq = O.SharedQuery([O.normalize(p) for p in pos], posw, None if neg is None else [O.normalize(v) for v in neg], negw)
    want = sq.scan(stored)
    order = np.lexsort((np.arange(n), -want.astype(np.float64)))[:k]
    assert len(ids) == k
    np.testing.assert_allclose(scores, want[order], rtol=2e-5, atol=1e-6)
    np.testing.assert_allclose(scores, want[ids], rtol=2e-5, atol=1e-6)   # each hit carries its own row's score
    assert np.all(np.diff(scores) <= 0)


@pytest.mark.parametrize("mislead", [False, True])
def test_shared_search_large_k_with_sampled_bound(lk, mislead):
    """k of 256 and more on a large index: a sample of the rows is scored first and bounds the scan from
    below.  With `mislead` every sampled row is a near-copy of the first positive and no other row is, so
    the bound lies above almost the whole index, too few rows pass, and the search must run again."""
    n, dim, k = 163_840, 128, 1000                # the sample of an index of this size: every 20th row
    rows = _common_rows(n, dim, 71)
    pos = _common_rows(2, dim, 72)
    if mislead:
        rng = np.random.default_rng(73)
        rows[::20] = pos[0] + 0.05 * rng.standard_normal((n // 20, dim)).astype(np.float32)
    rows = np.stack([O.normalize(v) for v in rows])
    idx = lk.DeviceIndex(dim, lk.LK_F32)
    idx.append(rows)
    stored = idx.read_rows(0, n)
    ids, scores = idx.search_shared(pos, k=k, scoring=lk.LK_SCORE_PLAIN)
    want = O.SharedQuery([O.normalize(p) for p in pos], None, None, None).scan(stored)
    order = np.lexsort((np.arange(n), -want.astype(np.float64)))[:k]
    assert len(ids) == k and len(set(ids.tolist())) == k
    np.testing.assert_allclose(scores, want[order], rtol=2e-5, atol=1e-6)
    np.testing.assert_allclose(scores, want[ids], rtol=2e-5, atol=1e-6)
    idx.close()


def test_shared_search_large_centered_index_matches_oracle(impl):
    n, dim, k = 8200, 64, 30
    rows = _common_rows(n, dim, 61)
    names = [f"c-{i:05d}" for i in range(n)]
    gi, oi = impl.NewCentered(), OX.NewCentered()
    gi.AddBatch(names, rows)
    for p, v in zip(names, rows):
        oi.Add(p, v)
    pos = _common_rows(6, dim, 62)
    neg = _common_rows(2, dim, 63)
    for spec_kw in (dict(Pos=list(pos[:2])), dict(Pos=list(pos), Neg=list(neg), NegW=[0.5, 0.25])):
        g = gi.SearchShared(impl.SharedSpec(**spec_kw), k, None)
        w = oi.SearchShared(OX.SharedSpec(**spec_kw), k, None)
        _assert_hits_close(g, w, rel=2e-5)


def test_shared_errors_match_reference(impl):
    idx = impl.New()
    idx.Add("a", [1, 0])
    for bad in (dict(Pos=[]), dict(Pos=[[1, 0]], PosW=[0]), dict(Pos=[[1, 0], [1, 0, 0]]),
                dict(Pos=[[1, 0]], Neg=[[1, 0]]), dict(Pos=[[1, 0]], PosW=[1, 2])):
        with pytest.raises(ValueError):
            idx.SearchShared(impl.SharedSpec(**bad), 5, None)


def test_shared_scorer_identities(lk):
    """media-server/embedvec/shared_test.go identities through the slot-level call
    (which takes beta and lambda): candidates are the stored rows."""
    cands = np.stack([O.normalize(v) for v in ([1, 0, 0], [0, 1, 0], [0.3, -0.7, 0.6], [1, 0.5, 0])])
    idx = lk.DeviceIndex(3, lk.LK_F32)
    idx.append(cands)
    q1, q2 = O.normalize([1, 0.5, 0]), O.normalize([1, -0.5, 0.2])
    ids, scores = idx.search_shared([q1, q2], k=4, beta=0.0, lam=1.0)   # :19-41, two examples -> min
    for i, s in zip(ids, scores):
        want = min(O.cosine(q1, cands[i]), O.cosine(q2, cands[i]))
        assert abs(float(s) - float(want)) <= 1e-5
    q = O.normalize([0.3, 0.7, 0.2])
    ids, scores = idx.search_shared([q], k=4)                            # :135-149, single positive -> cosine
    for i, s in zip(ids, scores):
        assert abs(float(s) - float(O.cosine(q, cands[i]))) <= 1e-5
    sq = O.SharedQuery([q1, q2], [1, 0.25], [cands[1]], [0.5], 0.6, 0.7)
    ids, scores = idx.search_shared([q1, q2], posw=[1, 0.25], neg=[cands[1]], negw=[0.5], k=4, beta=0.6, lam=0.7)
    for i, s in zip(ids, scores):
        assert abs(float(s) - float(sq.score(cands[i]))) <= 1e-6


def test_ties_are_ordered_by_path(impl):
    """Equal scores: the reference sorts by path (media-server/embedindex/embedindex.go:483-490)."""
    idx = impl.New()
    for p in ["zeta", "alpha", "mid", "beta"]:
        idx.Add(p, [1, 0, 0])
    idx.Add("other", [0, 1, 0])
    hits = idx.Search([1, 0, 0], 5)
    assert [h.Path for h in hits] == ["alpha", "beta", "mid", "zeta", "other"]


def test_wrong_length_vectors_score_zero(impl):
    """Cosine returns 0 on a length mismatch (media-server/embedvec/embedvec.go:114-116)."""
    idx = impl.New()
    idx.Add("a", [1, 0, 0])
    idx.Add("odd", [1, 0])          # stored, but can never match
    hits = idx.Search([1, 0, 0], 2)
    assert [h.Path for h in hits] == ["a", "odd"] and hits[1].Score == 0
    hits = idx.Search([1, 0], 2)    # a query of the wrong length scores 0 everywhere
    assert all(h.Score == 0 for h in hits)


def test_bulk_add_equals_row_by_row(impl):
    n, dim = 300, 40
    rows = gaussian_rows(n, dim, 51)
    names = [f"p{i % 250}" for i in range(n)]  # repeated paths: later Adds replace earlier ones
    a, b = impl.NewCentered(), impl.NewCentered()
    a.AddBatch(names, rows)
    for p, v in zip(names, rows):
        b.Add(p, v)
    assert a.Len() == b.Len() == 250
    q = gaussian_rows(1, dim, 52)[0]
    ha, hb = a.Search(q, 20), b.Search(q, 20)
    assert [(h.Path, h.Score) for h in ha] == [(h.Path, h.Score) for h in hb]
