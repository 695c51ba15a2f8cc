"""GPU: batches of queries on a float32 index (8 queries per pass on the float64
tensor-core path) against the single-query scans and against the oracle."""
import numpy as np
import pytest

import oracle as O
from tests.synth import gaussian_rows

pytestmark = pytest.mark.gpu


def _rows(n, dim, seed):
    r = gaussian_rows(n, dim, seed)
    r[:, 0] += 3.0   # a common component, like real embeddings: centering matters
    return r


def _same_hits(a, b, rel=2e-6):
    ids_a, sc_a, _, cnt_a = a
    ids_b, sc_b, _, cnt_b = b
    assert np.array_equal(cnt_a, cnt_b)
    np.testing.assert_allclose(sc_a, sc_b, rtol=rel, atol=1e-7)
    diff = ids_a != ids_b
    # different rows at the same rank only where their scores tie to the last bits
    assert np.all(np.abs(sc_a[diff] - sc_b[diff]) <= rel * np.maximum(np.abs(sc_b[diff]), 1e-6))
    return int(diff.sum())


@pytest.mark.parametrize("n,dim,centered", [(20011, 96, False), (9000, 200, True), (12345, 768, True), (8192, 64, False)])
@pytest.mark.parametrize("nq,k", [(3, 10), (8, 1), (13, 100), (64, 10)])
def test_batched_equals_single_scans(lk, n, dim, centered, nq, k):
    idx = lk.DeviceIndex(dim, lk.LK_F32, centered=centered)
    idx.append(_rows(n, dim, 7))
    qs = _rows(nq, dim, 8)
    for scoring in ((lk.LK_SCORE_DEFAULT, lk.LK_SCORE_PLAIN) if centered else (lk.LK_SCORE_DEFAULT,)):
        idx.set_batch_mode(True)
        before = idx.stats()
        batched = idx.search(qs, k, scoring=scoring)
        after = idx.stats()
        assert after["scan_launches"] == before["scan_launches"]                       # no single-query scan ran,
        assert after["aux_launches"] >= before["aux_launches"] + (nq + 7) // 8 + 1      # the batched kernels did
        idx.set_batch_mode(False)
        single = idx.search(qs, k, scoring=scoring)
        swapped = _same_hits(batched, single)
        assert swapped <= max(2, nq * k // 50)
        assert np.all(batched[3] == min(k, n))


def test_batched_matches_oracle(lk):
    n, dim, nq, k = 10007, 128, 9, 25
    rows = np.stack([O.normalize(v) for v in _rows(n, dim, 17)])
    idx = lk.DeviceIndex(dim, lk.LK_F32)
    idx.append(rows)
    stored = idx.read_rows(0, n)
    qs = _rows(nq, dim, 18)
    ids, scores, _, counts = idx.search(qs, k)
    for q in range(nq):
        want = np.array([O.cosine(O.normalize(qs[q]), stored[i]) for i in ids[q]], np.float32)
        np.testing.assert_array_equal(scores[q], want)   # float64 accumulation, one rounding: the same float32
        full = stored.astype(np.float64) @ O.normalize(qs[q]).astype(np.float64)
        order = np.lexsort((np.arange(n), -full.astype(np.float32)))[:k]
        assert len(set(ids[q]) ^ set(order)) <= 2
        assert counts[q] == k


def test_small_batches_and_small_indexes_keep_the_scan_path(lk):
    idx = lk.DeviceIndex(32, lk.LK_F32)
    idx.append(_rows(500, 32, 1))
    scans = idx.stats()["scan_launches"]
    idx.search(_rows(16, 32, 2), 5)
    assert idx.stats()["scan_launches"] == scans + 16
