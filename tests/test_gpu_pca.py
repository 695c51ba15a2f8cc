"""GPU: lk_pca3 against the oracle (coords bit for bit for the same worker count) and the
reference's property tests through the mirrored embedvec.ProjectPCA3."""
import numpy as np
import pytest

import oracle as O
from tests.test_pca_oracle import check_planted, planted_cloud

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,d,workers", [(200, 32, 1), (200, 32, 8), (1000, 96, 5), (333, 7, 64), (50, 8, 100), (4000, 768, 16)])
def test_coords_equal_the_oracle_bit_for_bit(lk, n, d, workers):
    rng = np.random.default_rng(n + d)
    centres = rng.standard_normal((5, d)).astype(np.float32) * 2
    vecs = (centres[rng.integers(0, 5, n)] + rng.standard_normal((n, d)).astype(np.float32)).astype(np.float32)
    coords, variance = lk.pca3(vecs, workers)
    want_c, want_v = O.pca3(vecs, workers)
    assert np.array_equal(coords.view(np.uint32), want_c.view(np.uint32))
    np.testing.assert_allclose(variance, want_v, rtol=1e-11)


def test_reference_properties(lk):
    from loki_b200 import embedvec as V
    latent, vecs = planted_cloud()
    coords, variance = V.ProjectPCA3(list(vecs), workers=8)
    check_planted(latent, coords, variance, np.random.default_rng(1))
    again_c, again_v = V.ProjectPCA3(list(vecs), workers=8)
    assert np.array_equal(coords, again_c) and np.array_equal(variance, again_v)
    rng = np.random.default_rng(11)
    c, _ = V.ProjectPCA3(list((rng.standard_normal((50, 8)) * 100).astype(np.float32)), workers=8)
    assert np.abs(c).max() <= 1 + 1e-6 and np.abs(c).max() >= 0.999
    c, v = V.ProjectPCA3([], workers=8)
    assert c.shape == (0, 3) and not v.any()
    same = np.tile(rng.standard_normal((1, 8)).astype(np.float32), (20, 1))
    c, v = V.ProjectPCA3(list(same), workers=8)
    assert not c.any() and not v.any()
    line = np.outer(np.linspace(-1, 1, 30), np.ones(6)).astype(np.float32)
    c, v = lk.pca3(line, 4)
    want_c, want_v = O.pca3(line, 4)
    assert np.array_equal(c, want_c) and v[1] == 0 and v[2] == 0
    np.testing.assert_allclose(v, want_v, rtol=1e-11)
