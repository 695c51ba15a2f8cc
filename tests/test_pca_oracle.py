"""CPU: the oracle's ProjectPCA3 against the properties the reference's tests state
(media-server/embedvec/pca_test.go), over this repo's seeded generator."""
import numpy as np
import pytest

import oracle as O


def planted_cloud(n=200, d=32, seed=7):
    """pca_test.go:13-40: a 3-D cloud (std 3, 2, 1) rotated into d dimensions plus 0.01 noise."""
    rng = np.random.default_rng(seed)
    basis, _ = np.linalg.qr(rng.standard_normal((d, 3)))
    latent = rng.standard_normal((n, 3)) * np.array([3.0, 2.0, 1.0])
    return latent, (latent @ basis.T + 0.01 * rng.standard_normal((n, d))).astype(np.float32)


def check_planted(latent, coords, variance, rng):
    assert coords.shape == (len(latent), 3)
    assert variance.sum() >= 0.99 and variance[0] >= variance[1] >= variance[2]
    checked = 0
    for _ in range(500):   # distance order on clear-cut triples, pca_test.go:57-83
        a, b, c = rng.integers(0, len(latent), 3)
        db, dc = np.linalg.norm(latent[a] - latent[b]), np.linalg.norm(latent[a] - latent[c])
        if db * 2 >= dc:
            continue
        checked += 1
        pa, pb, pc = coords[a].astype(np.float64), coords[b].astype(np.float64), coords[c].astype(np.float64)
        assert np.linalg.norm(pa - pb) < np.linalg.norm(pa - pc)
    assert checked >= 50


@pytest.mark.parametrize("workers", [1, 8])
def test_planted_structure_is_recovered(workers):
    latent, vecs = planted_cloud()
    coords, variance = O.pca3(vecs, workers)
    check_planted(latent, coords, variance, np.random.default_rng(1))


def test_deterministic_bounded_and_degenerate():
    rng = np.random.default_rng(3)
    vecs = rng.standard_normal((100, 16)).astype(np.float32)
    c1, v1 = O.pca3(vecs, 4)
    c2, v2 = O.pca3(vecs, 4)
    assert np.array_equal(c1, c2) and np.array_equal(v1, v2)            # pca_test.go:88-107
    big = (rng.standard_normal((50, 8)) * 100).astype(np.float32)        # pca_test.go:111-135
    c, _ = O.pca3(big, 4)
    assert np.abs(c).max() <= 1 + 1e-6 and np.abs(c).max() >= 0.999
    c, v = O.pca3(np.zeros((0, 8), np.float32), 4)                       # pca_test.go: degenerate inputs
    assert c.shape == (0, 3) and not v.any()
    same = np.tile(rng.standard_normal((1, 8)).astype(np.float32), (20, 1))
    c, v = O.pca3(same, 4)
    assert not c.any() and not v.any()
    line = np.outer(np.linspace(-1, 1, 30), np.ones(6)).astype(np.float32)   # rank 1: one component only
    c, v = O.pca3(line, 4)
    assert v[0] > 0.999 and v[1] == 0 and v[2] == 0 and not c[:, 1:].any()


def test_worker_count_changes_only_the_last_bits():
    _, vecs = planted_cloud(300, 24, seed=9)
    c1, v1 = O.pca3(vecs, 1)
    c7, v7 = O.pca3(vecs, 7)
    np.testing.assert_allclose(c1, c7, atol=1e-5)
    np.testing.assert_allclose(v1, v7, rtol=1e-9)
