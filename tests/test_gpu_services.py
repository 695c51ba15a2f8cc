"""GPU: the service layer's search functions (index branch and brute-force branch) with the
reference's own service-level cases, over in-memory rows in place of SQLite, and the CosineSim
entry point against the oracle.

Ported cases (literal vectors and expected orders are the reference's):
  media-server/tasks/embed_search_filtered_test.go:31-52   brute force ranks only within the allow set
  media-server/tasks/embed_search_filtered_test.go:54-76   the installed index honours the allow set
  media-server/tasks/embed_search_filtered_test.go:78-97   face search filtered by media path
  media-server/tasks/embed_similar_test.go:21-50           SimilarByPath ranks by cosine, self included
  media-server/swipe_similar_test.go:21-50, :88-104        b > orphan > c > d around the anchor
  media-server/tasks/face_index_test.go:48-113             face index build + search, brute-force fallback
"""
import numpy as np
import pytest

import oracle as O
from loki_b200 import embedindex as E
from loki_b200 import tasks as T
from tests.synth import gaussian_rows

pytestmark = pytest.mark.gpu


def _emb(*pairs):
    return [T.StoredEmbedding(p, np.asarray(v, np.float32)) for p, v in pairs]


def _filtered_db():
    return _emb(("nearest.jpg", O.normalize([1, 0])), ("mid.jpg", O.normalize([0.5, 0.5])), ("far.jpg", O.normalize([0, 1])))


def test_search_by_vector_within_brute_force(lk):
    db = _filtered_db()
    q = O.normalize([1, 0])
    hits = T.searchByVectorWithin(None, db, q, 10, {"mid.jpg", "far.jpg"})
    assert [h.Path for h in hits] == ["mid.jpg", "far.jpg"]
    allh = T.searchByVectorWithin(None, db, q, 10, None)
    assert len(allh) == 3 and allh[0].Path == "nearest.jpg"
    for h in allh:   # scores are CosineSim of the stored vectors
        want = O.cosine_sim(q, next(e.Vec for e in db if e.Path == h.Path))
        assert abs(h.Score - want) <= 1e-6


def test_search_by_vector_within_uses_index(lk):
    idx = E.New()
    idx.Add("nearest.jpg", O.normalize([1, 0]))
    idx.Add("mid.jpg", O.normalize([0.5, 0.5]))
    # far.jpg deliberately not indexed: the hits must come from the index alone
    hits = T.searchByVectorWithin(idx, _filtered_db(), O.normalize([1, 0]), 10, {"mid.jpg", "far.jpg"})
    assert [h.Path for h in hits] == ["mid.jpg"]
    idx.close()


def _faces():
    return [T.Face(1, "a.jpg", np.asarray([1, 0, 0], np.float32), "m1"),
            T.Face(2, "b.jpg", np.asarray([0.9, 0.1, 0], np.float32), "m1")]


def test_search_faces_within_filters_by_media_path(lk):
    faces = _faces()
    idx = E.New()
    for f in faces:
        idx.Add(str(f.ID), f.Vec)
    hits = T.searchFacesByVectorWithin(idx, faces, [1, 0, 0], 5, {"b.jpg"})
    assert len(hits) == 1 and hits[0].FaceID == 2 and hits[0].MediaPath == "b.jpg"
    assert abs(hits[0].Score - O.cosine_sim(np.float32([1, 0, 0]), faces[1].Vec)) <= 1e-6
    idx.close()


def test_similar_by_path_ranks_by_cosine(lk):
    db = _emb(("q.jpg", O.normalize([1, 0])), ("a.jpg", O.normalize([0.9, 0.1])), ("b.jpg", O.normalize([0, 1])),
              ("c.jpg", O.normalize([-1, 0])))
    for index in (None, "build"):
        idx = None
        if index:
            idx = E.New()
            for e in db:
                idx.Add(e.Path, e.Vec)
        hits = T.SimilarByPath(idx, db, "q.jpg", 10)
        assert len(hits) == 4                      # the query item itself is included
        assert hits[0].Path == "q.jpg" and hits[1].Path == "a.jpg" and hits[-1].Path == "c.jpg"
        if idx:
            idx.close()
    with pytest.raises(KeyError):
        T.SimilarByPath(None, db, "missing.jpg", 10)


def test_swipe_similar_order_around_the_anchor(lk):
    """Similarity to /lib/a.jpg ranks b > orphan > c > d (raw, un-normalised stored vectors);
    the handler then drops the anchor and rows without a media record."""
    vecs = {"/lib/a.jpg": [1, 0], "/lib/b.jpg": [0.99, 0.14], "/lib/orphan.jpg": [0.9, 0.44],
            "/lib/c.jpg": [0.7, 0.71], "/lib/d.jpg": [0, 1]}
    db = _emb(*vecs.items())
    hits = T.SimilarByPath(None, db, "/lib/a.jpg", 0)          # limit 0: every row, ranked
    assert [h.Path for h in hits] == ["/lib/a.jpg", "/lib/b.jpg", "/lib/orphan.jpg", "/lib/c.jpg", "/lib/d.jpg"]
    media = {"/lib/a.jpg", "/lib/b.jpg", "/lib/c.jpg", "/lib/d.jpg"}
    ranked = [h.Path for h in hits if h.Path != "/lib/a.jpg" and h.Path in media]
    assert ranked[:2] == ["/lib/b.jpg", "/lib/c.jpg"] and ranked[2:] == ["/lib/d.jpg"]   # page 1, then has_more


def test_face_index_build_and_search(lk):
    faces = [T.Face(11, "a.jpg", np.float32([1, 0, 0]), "m1"), T.Face(12, "a.jpg", np.float32([0, 1, 0]), "m1"),
             T.Face(13, "b.jpg", np.float32([0.9, 0.1, 0]), "m1")]
    idx = E.New()
    for f in faces:                                    # BuildFaceIndexFromDB: keyed by face id
        idx.Add(str(f.ID), f.Vec)
    assert idx.Len() == 3
    hits = T.SearchFacesByVector(idx, faces, [1, 0, 0], 2)
    assert len(hits) == 2
    assert hits[0].FaceID == 11 and hits[0].MediaPath == "a.jpg" and hits[1].FaceID == 13
    assert hits[0].Score >= 0.99 and hits[1].Score < hits[0].Score
    idx.close()


def test_face_search_brute_force_fallback(lk):
    faces = [T.Face(7, "a.jpg", np.float32([0, 0, 1]), "m1")]
    hits = T.SearchFacesByVector(None, faces, [0, 0, 1], 5)     # no index installed
    assert len(hits) == 1 and hits[0].FaceID == 7


def test_brute_force_equals_plain_index_order(lk):
    """sortSimilar's promise (embed_task.go:276-288): the fallback and a plain index return the
    same order, ties by path included."""
    rows = gaussian_rows(500, 24, 5)
    rows[100] = rows[7]
    rows[300] = 3.0 * rows[7]                        # same direction, other length: equal cosine
    paths = [f"p{(i * 37) % 500:04d}.jpg" for i in range(500)]
    db = [T.StoredEmbedding(p, r) for p, r in zip(paths, rows)]
    idx = E.New()
    idx.AddBatch(paths, rows)
    q = rows[7]
    a = T.SearchByVector(None, db, q, 40)
    b = T.SearchByVector(idx, db, q, 40)
    trio = {paths[7], paths[100], paths[300]}
    assert {h.Path for h in a[:3]} == trio and {h.Path for h in b[:3]} == trio
    for hits in (a, b):                              # the exact duplicates tie: path order decides
        pos = {h.Path: i for i, h in enumerate(hits)}
        lo, hi = sorted([paths[7], paths[100]])
        assert hits[pos[lo]].Score == hits[pos[hi]].Score and pos[lo] < pos[hi]
    for x, y in zip(a, b):
        assert abs(x.Score - y.Score) <= 2e-6
    assert [h.Path for h in a[3:]] == [h.Path for h in b[3:]]
    idx.close()


@pytest.mark.parametrize("n,dim,k", [(1, 3, 5), (33, 7, 10), (5000, 512, 50), (20000, 100, 3000), (3000, 768, 1)])
def test_cosine_sim_topk_matches_oracle(lk, n, dim, k):
    rng = np.random.default_rng(n + dim)
    rows = (rng.standard_normal((n, dim)) * rng.uniform(0.1, 30.0, (n, 1))).astype(np.float32)   # un-normalised
    if n > 10:
        rows[3] = 0.0                                 # a zero vector scores 0
        rows[5] = rows[9]                             # an exact tie: the lower row first
    q = rng.standard_normal(dim).astype(np.float32) * 5
    want = np.asarray([O.cosine_sim(q, r) for r in rows], np.float32)
    ids, scores = lk.cosine_sim_topk(rows, q, k)
    kk = min(k, n)
    assert ids.size == kk
    wid, wsc = O.topk_f32(want, k)
    np.testing.assert_allclose(scores, wsc, rtol=1e-5, atol=1e-7)
    for i in np.nonzero(ids != wid)[0]:              # only near-tied neighbours may swap
        assert abs(want[ids[i]] - wsc[i]) <= 1e-5 * max(abs(wsc[i]), 1e-7)
    if n > 10 and 5 in ids and 9 in ids:
        assert list(ids).index(5) + 1 == list(ids).index(9)
    # an allow list scores only those rows
    slots = rng.permutation(n)[:max(1, n // 3)].astype(np.int32)
    ids2, scores2 = lk.cosine_sim_topk(rows, q, k, allow_slots=slots)
    wid2, wsc2 = O.topk_f32(want[slots], k, ids=slots)
    np.testing.assert_allclose(scores2, wsc2, rtol=1e-5, atol=1e-7)
    assert set(ids2) <= set(slots.tolist())
    assert lk.cosine_sim_topk(rows, np.zeros(dim, np.float32), 3)[1].tolist() == [0.0] * min(3, n)


def test_shared_fallback_equals_installed_index(lk):
    rows = gaussian_rows(300, 32, 11)
    paths = [f"{i:04d}.jpg" for i in range(300)]
    db = [T.StoredEmbedding(p, r) for p, r in zip(paths, rows)]
    spec = E.SharedSpec(Pos=[rows[3], rows[50]], Neg=[rows[70]], NegW=[0.5])
    idx = E.NewCentered()
    idx.AddBatch(paths, rows)
    a = T.searchSharedWithin(None, db, spec, 20, None, E.ScoreDefault)
    b = T.searchSharedWithin(idx, db, spec, 20, None, E.ScoreDefault)
    assert [h.Path for h in a] == [h.Path for h in b]
    np.testing.assert_allclose([h.Score for h in a], [h.Score for h in b], rtol=1e-6)
    with pytest.raises(ValueError):
        T.searchSharedWithin(None, db, E.SharedSpec(Pos=[]), 5, None, E.ScoreDefault)
    idx.close()
