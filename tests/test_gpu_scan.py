"""GPU parity of the scan kernels against the CPU oracle, through the C ABI."""
import numpy as np
import pytest

import oracle as O
from tests.synth import clustered_rows, gaussian_rows

pytestmark = pytest.mark.gpu


def _oracle_i8(rows, queries, k, slots=None):
    codes, scales = O.build_i8(rows)
    out = []
    for q in queries:
        qc, qs = O.build_i8(q.reshape(1, -1))
        sc = O.scan_i8(codes, qc[0], slots=slots)
        ids, top = O.topk_i32(sc, k, ids=slots)
        dq = top.astype(np.float32) * (qs[0] * scales[ids])
        out.append((ids, top, dq))
    return codes, scales, out


@pytest.mark.parametrize("n,dim,k", [(1, 16, 1), (31, 16, 5), (32, 64, 10), (33, 100, 10), (1000, 768, 10),
                                     (5000, 768, 50), (4097, 1024, 100), (3000, 48, 7), (2000, 5, 3),
                                     (20000, 768, 1000), (700, 384, 700)])
def test_int8_scan_bit_exact(lk, n, dim, k):
    rows = gaussian_rows(n, dim, 100 + n)
    queries = gaussian_rows(4, dim, 200 + n)
    idx = lk.DeviceIndex(dim, lk.LK_I8)
    idx.append(rows)
    assert len(idx) == n
    codes, scales, want = _oracle_i8(rows, queries, k)
    got_codes, got_scales = idx.read_rows()
    assert np.array_equal(got_codes, codes[:, :dim]), "int8 codes differ from the oracle"
    assert np.array_equal(got_scales, scales), "int8 scales differ from the oracle"
    ids, scores, iscores, counts = idx.search(queries, k)
    for q, (wid, wsc, wdq) in enumerate(want):
        kk = min(k, n)
        assert counts[q] == kk
        assert np.array_equal(ids[q, :kk], wid), f"query {q}: ids differ"
        assert np.array_equal(iscores[q, :kk], wsc), f"query {q}: int32 scores differ"
        assert np.array_equal(scores[q, :kk], wdq), f"query {q}: de-quantised scores differ"
        assert np.all(ids[q, kk:] == -1)


def test_int8_scan_near_ties(lk):
    """Clustered rows make many equal int32 scores: ties must go to the lower slot."""
    n, dim, k = 6000, 768, 100
    rows = clustered_rows(n, dim, 7)
    rows[10] = rows[4000]
    rows[11] = rows[4000]  # exact duplicates -> exact ties
    queries = np.concatenate([gaussian_rows(2, dim, 8), rows[4000:4001], rows[1:2]])
    idx = lk.DeviceIndex(dim, lk.LK_I8)
    idx.append(rows)
    _, _, want = _oracle_i8(rows, queries, k)
    ids, scores, iscores, counts = idx.search(queries, k)
    for q, (wid, wsc, _) in enumerate(want):
        assert np.array_equal(ids[q], wid)
        assert np.array_equal(iscores[q], wsc)
    assert list(ids[2, :3]) == [10, 11, 4000]


@pytest.mark.parametrize("n,dim,k", [(1, 2, 1), (3, 2, 10), (300, 32, 50), (1000, 512, 10), (2049, 768, 50),
                                     (5000, 100, 20), (777, 1024, 777), (64, 3, 64)])
def test_f32_scan_matches_oracle(lk, n, dim, k):
    rows = gaussian_rows(n, dim, 300 + n)
    queries = gaussian_rows(3, dim, 400 + n)
    idx = lk.DeviceIndex(dim, lk.LK_F32)
    idx.append(rows)
    stored = idx.read_rows()
    want_rows = O.normalize_rows(rows)
    assert np.array_equal(stored, want_rows), "normalised rows differ from the oracle bit for bit"
    ids, scores, _, counts = idx.search(queries, k)
    kk = min(k, n)
    for q in range(queries.shape[0]):
        sc = O.scan_f32(want_rows, O.normalize(queries[q]))
        wid, wsc = O.topk_f32(sc, k)
        assert counts[q] == kk
        # tolerance from the task statement: 1e-5 relative on the cosine
        np.testing.assert_allclose(scores[q, :kk], wsc, rtol=1e-5, atol=1e-7)
        same = ids[q, :kk] == wid
        if not same.all():  # only allowed where neighbouring scores are (nearly) tied
            for i in np.nonzero(~same)[0]:
                assert abs(sc[ids[q, i]] - wsc[i]) <= 1e-5 * max(abs(wsc[i]), 1e-7)


def test_f32_self_query_ranks_first(lk):
    """Property from media-server/embedindex/embedindex_test.go:138-184 on this repo's own seeded data."""
    n, dim, k = 300, 32, 50
    rows = gaussian_rows(n, dim, 42)
    idx = lk.DeviceIndex(dim, lk.LK_F32)
    idx.append(rows)
    ids, scores, _, counts = idx.search(rows[123], k)
    assert counts[0] == k and ids[0, 0] == 123 and scores[0, 0] >= 0.999
    sc = O.scan_f32(O.normalize_rows(rows), O.normalize(rows[123]))
    wid, _ = O.topk_f32(sc, k)
    assert np.array_equal(ids[0], wid)


def test_allow_list_scan(lk):
    n, dim, k = 4000, 768, 10
    rows = gaussian_rows(n, dim, 5)
    q = gaussian_rows(1, dim, 6)
    rng = np.random.default_rng(9)
    for store in (lk.LK_I8, lk.LK_F32):
        idx = lk.DeviceIndex(dim, store)
        idx.append(rows)
        for m in (1, 33, 500, n):
            slots = rng.permutation(n)[:m].astype(np.int32)
            ids, scores, iscores, counts = idx.search(q, k, allow_slots=slots)
            kk = min(k, m)
            assert counts[0] == kk
            if store == lk.LK_I8:
                _, _, want = _oracle_i8(rows, q, k, slots=slots)
                assert np.array_equal(ids[0, :kk], want[0][0])
                assert np.array_equal(iscores[0, :kk], want[0][1])
            else:
                sc = O.scan_f32(O.normalize_rows(rows), O.normalize(q[0]), slots=slots)
                wid, wsc = O.topk_f32(sc, k, ids=slots)
                assert np.array_equal(ids[0, :kk], wid)
                np.testing.assert_allclose(scores[0, :kk], wsc, rtol=1e-5, atol=1e-7)
        ids, _, _, counts = idx.search(q, k, allow_slots=np.zeros(0, np.int32))
        assert counts[0] == 0 and np.all(ids == -1)


def test_k_beyond_single_pass(lk):
    """k above the per-pass limit (2048) runs several passes and still returns the exact ranking."""
    n, dim, k = 6000, 64, 5000
    rows = gaussian_rows(n, dim, 77)
    q = gaussian_rows(1, dim, 78)
    idx = lk.DeviceIndex(dim, lk.LK_I8)
    idx.append(rows)
    _, _, want = _oracle_i8(rows, q, k)
    ids, _, iscores, counts = idx.search(q, k)
    assert counts[0] == k
    assert np.array_equal(ids[0], want[0][0])
    assert np.array_equal(iscores[0], want[0][1])


def test_upsert_overwrite_and_swap_remove(lk):
    dim = 96
    rows = gaussian_rows(50, dim, 1)
    idx = lk.DeviceIndex(dim, lk.LK_F32)
    idx.append(rows)
    new = gaussian_rows(3, dim, 2)
    idx.upsert(10, new)  # in-place replacement of slots 10..12
    assert len(idx) == 50
    idx.swap_remove(5)   # last row moves into slot 5
    assert len(idx) == 49
    want = O.normalize_rows(rows)
    want[10:13] = O.normalize_rows(new)
    want[5] = want[49]
    want = want[:49]
    assert np.array_equal(idx.read_rows(), want)
    idx.swap_remove(48)
    assert np.array_equal(idx.read_rows(), want[:48])


def test_resident_queries_match_search(lk):
    n, dim, k = 3000, 768, 10
    rows = gaussian_rows(n, dim, 11)
    qs = gaussian_rows(16, dim, 12)
    idx = lk.DeviceIndex(dim, lk.LK_I8)
    idx.append(rows)
    ids, scores, iscores, counts = idx.search(qs, k)
    rq = idx.queries(qs)
    rq.enqueue(0, 16, k)
    ids2, scores2, iscores2, counts2 = rq.fetch(0, 16, k)
    assert np.array_equal(ids, ids2) and np.array_equal(iscores, iscores2)
    assert np.array_equal(scores, scores2) and np.array_equal(counts, counts2)


@pytest.mark.parametrize("n,dim,k", [(500, 64, 10), (20000, 768, 50), (3000, 100, 7), (9000, 1024, 20)])
def test_f16_scan_matches_oracle(lk, n, dim, k):
    """Half-precision storage (no counterpart in the reference: parity unpinned): rows are
    normalised like the reference, rounded to IEEE half (nearest even), and scored against
    the float32 query; the oracle accumulates the same values in float64."""
    rows = gaussian_rows(n, dim, 500 + n)
    queries = gaussian_rows(3, dim, 600 + n)
    idx = lk.DeviceIndex(dim, lk.LK_F16)
    idx.append(rows)
    stored = idx.read_rows()
    want_half = O.normalize_rows(rows).astype(np.float16)
    assert np.array_equal(stored.view(np.uint16), want_half.view(np.uint16)), "stored halves differ"
    deq = want_half.astype(np.float32)
    ids, scores, _, counts = idx.search(queries, k)
    kk = min(k, n)
    for q in range(queries.shape[0]):
        sc = O.scan_f32(deq, O.normalize(queries[q]))
        wid, wsc = O.topk_f32(sc, k)
        assert counts[q] == kk
        np.testing.assert_allclose(scores[q, :kk], wsc, rtol=1e-5, atol=2e-7)
        same = ids[q, :kk] == wid
        for i in np.nonzero(~same)[0]:  # float32 accumulation: neighbours within rounding may swap
            assert abs(sc[ids[q, i]] - wsc[i]) <= 1e-5 * max(abs(wsc[i]), 1e-6)
