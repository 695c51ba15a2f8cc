"""GPU: the face-clustering neighbour prescreen against the oracle's restatement of
prescreenCandidates / dotf (media-server/tasks/face_cluster.go:908-925, :1189-1285)."""
import numpy as np
import pytest

import oracle as O

pytestmark = pytest.mark.gpu


def clustered_unit(n, dim, seed, centres=30, noise=0.45):
    rng = np.random.default_rng(seed)
    c = rng.standard_normal((centres, dim)).astype(np.float32)
    v = c[rng.integers(0, centres, n)] + np.float32(noise) * rng.standard_normal((n, dim)).astype(np.float32)
    return O.normalize_rows(v)


@pytest.mark.parametrize("n,dim,thr", [(1, 8, 0.5), (63, 16, 0.5), (900, 64, 0.6), (2000, 512, 0.47), (700, 130, 0.55),
                                       (1500, 6, 0.9)])
def test_prescreen_equals_dotf_definition(lk, n, dim, thr):
    """Bit-exact against 'every j < i with dotf >= threshold', the definition the reference's
    own test uses (media-server/tasks/face_cluster_perf_test.go:52-81)."""
    v = clustered_unit(n, dim, 70 + n)
    near, count, over = lk.prescreen_pairs(v, thr)
    wnear, wcount, wover = O.prescreen(v, thr, brute_force=True)
    assert np.array_equal(over, wover)
    assert np.array_equal(count, wcount)
    for i in range(n):
        assert np.array_equal(near[i, :count[i]], wnear[i, :wcount[i]]), i


def test_prescreen_matches_reference_tiling_up_to_last_bit(lk):
    """Against the literal restatement (four rows at a time through dot4 off the diagonal):
    lists may differ only for pairs whose dot sits within rounding of the threshold."""
    n, dim, thr = 1200, 128, 0.6
    v = clustered_unit(n, dim, 5)
    near, count, over = lk.prescreen_pairs(v, thr)
    wnear, wcount, wover = O.prescreen(v, thr)
    assert np.array_equal(over, wover)
    for i in range(n):
        a, b = set(near[i, :count[i]].tolist()), set(wnear[i, :wcount[i]].tolist())
        for j in a ^ b:
            assert abs(float(O.dotf(v[i], v[j])) - thr) <= 1e-6


def test_prescreen_overflow_rule(lk):
    """A vector with more than 256 earlier neighbours is flagged and its list dropped."""
    dim = 32
    base = O.normalize(np.ones(dim, np.float32))
    v = np.tile(base, (400, 1))
    v[::7] = O.normalize(np.arange(dim, dtype=np.float32) - 16)  # a few strangers
    near, count, over = lk.prescreen_pairs(v, 0.9)
    wnear, wcount, wover = O.prescreen(v, 0.9, brute_force=True)
    assert over.any() and np.array_equal(over, wover) and np.array_equal(count, wcount)
    assert np.all(count[over] == 0)
