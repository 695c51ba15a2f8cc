"""GPU: 64-bit Hamming kernels against the oracle (parity unpinned by the reference:
it has no perceptual-hash code; the definition is this project's)."""
import numpy as np
import pytest

import oracle as O
from tests.synth import phash_set

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [0, 1, 2, 1023, 1024, 1025, 5000])
def test_hamming_pairs_match_oracle(lk, n):
    h = phash_set(n, 100 + n) if n else np.zeros(0, np.uint64)
    want, total = O.hamming_pairs(h, 6) if n else (np.zeros((0, 2), np.uint32), 0)
    got, cnt = lk.hamming_pairs(h, 6)
    assert cnt == total
    assert np.array_equal(got, want)


def test_hamming_pairs_radius_and_duplicates(lk):
    h = phash_set(3000, 7)
    h[17] = h[2900]  # exact duplicate, distance 0
    for r in (0, 1, 6, 10):
        want, total = O.hamming_pairs(h, r)
        got, cnt = lk.hamming_pairs(h, r)
        assert cnt == total and np.array_equal(got, want)
    assert [17, 2900] in lk.hamming_pairs(h, 0)[0].tolist()


def test_hamming_pairs_partitioned_union(lk):
    """Splitting the upper triangle over 4 callers (one per GPU) gives the same pair set."""
    h = phash_set(6000, 9)
    want, total = O.hamming_pairs(h, 6)
    parts = [lk.hamming_pairs(h, 6, part=p, parts=4) for p in range(4)]
    assert sum(c for _, c in parts) == total
    allp = np.concatenate([p for p, _ in parts])
    packed = np.sort(allp[:, 0].astype(np.uint64) << np.uint64(32) | allp[:, 1].astype(np.uint64))
    wpacked = want[:, 0].astype(np.uint64) << np.uint64(32) | want[:, 1].astype(np.uint64)
    assert np.array_equal(packed, wpacked)


def _pack(pairs):
    return pairs[:, 0].astype(np.uint64) << np.uint64(32) | pairs[:, 1].astype(np.uint64)


def _union(parts):
    return np.sort(_pack(np.concatenate([p for p, _ in parts])))


@pytest.fixture(scope="module")
def big_set():
    """200,000 hashes: buckets of the bit-field tables hold 400 (radius 6) to 3,000 (radius 9)
    hashes, i.e. several 256-wide tiles each, the case where a split over callers depends on
    every caller seeing the same bucket layout."""
    h = phash_set(200_000, 77, max_flips=9)
    return h, {r: O.hamming_pairs_threaded(h, r, cap=1 << 22) for r in (6, 9)}


@pytest.mark.parametrize("radius", [6, 9])
@pytest.mark.parametrize("parts", [2, 3, 8])
def test_hamming_pairs_split_is_a_partition(lk, big_set, radius, parts):
    h, want = big_set
    wpairs, wtotal = want[radius]
    single, cnt = lk.hamming_pairs(h, radius)
    assert cnt == wtotal and np.array_equal(single, wpairs)
    shares = [lk.hamming_pairs(h, radius, part=p, parts=parts) for p in range(parts)]
    assert sum(c for _, c in shares) == wtotal
    assert np.array_equal(_union(shares), _pack(wpairs))     # disjoint and complete
    again = lk.hamming_pairs(h, radius, part=parts - 1, parts=parts)
    assert np.array_equal(again[0], shares[-1][0])            # a share is the same on every call


def test_hamming_pairs_split_repeats(lk, big_set):
    """Twenty runs of the 3-way split at radius 9 (the case that used to lose or repeat a pair)."""
    h, want = big_set
    wpairs, wtotal = want[9]
    for _ in range(20):
        shares = [lk.hamming_pairs(h, 9, part=p, parts=3) for p in range(3)]
        assert sum(c for _, c in shares) == wtotal
        assert np.array_equal(_union(shares), _pack(wpairs))


def test_hamming_pairs_cap(lk):
    h = phash_set(3000, 5)
    _, total = O.hamming_pairs(h, 6)
    got, cnt = lk.hamming_pairs(h, 6, cap=10)
    assert cnt == total and got.shape[0] == 10


def test_hamming_scan(lk):
    h = phash_set(20000, 3)
    q = int(h[77])
    d = O.hamming_scan(h, q)
    ids, dist, cnt = lk.hamming_scan(h, q, 8)
    want = np.nonzero(d <= 8)[0]
    assert cnt == want.size and np.array_equal(ids, want.astype(np.uint32)) and np.array_equal(dist, d[want])


def test_hamming_full_size_properties(lk):
    """2,000,000 hashes (the benchmark's size): too many pairs for the CPU oracle, so check
    properties: every planted near-duplicate pair is found, every reported pair really is
    within the radius, pairs are sorted and unique."""
    n = 2_000_000
    rng = np.random.default_rng(1004)
    base = rng.integers(0, 2**64, size=n - 200_000, dtype=np.uint64)
    src = rng.integers(0, base.size, size=200_000)
    flips = rng.integers(0, 7, size=200_000)
    dup = base[src].copy()
    for f in range(1, 7):  # flip f distinct bits where flips >= f
        sel = np.nonzero(flips >= f)[0]
        bits = np.stack([rng.permutation(64)[:6] for _ in range(64)])[rng.integers(0, 64, sel.size), f - 1]
        dup[sel] ^= np.uint64(1) << bits.astype(np.uint64)
    h = np.concatenate([base, dup])
    perm = rng.permutation(n)
    h = h[perm]
    inv = np.empty(n, np.int64)
    inv[perm] = np.arange(n)
    pairs, cnt = lk.hamming_pairs(h, 6, cap=1 << 22)
    assert cnt == pairs.shape[0] >= 200_000
    x = h[pairs[:, 0]] ^ h[pairs[:, 1]]
    pop = np.zeros(x.size, np.int32)
    for b in range(64):
        pop += ((x >> np.uint64(b)) & np.uint64(1)).astype(np.int32)
    assert pop.max() <= 6 and np.all(pairs[:, 0] < pairs[:, 1])
    packed = pairs[:, 0].astype(np.uint64) << np.uint64(32) | pairs[:, 1].astype(np.uint64)
    assert np.all(np.diff(packed.astype(np.int64)) > 0)
    a, b = inv[src], inv[base.size + np.arange(200_000)]
    lo, hi = np.minimum(a, b), np.maximum(a, b)
    planted = lo.astype(np.uint64) << np.uint64(32) | hi.astype(np.uint64)
    assert np.isin(planted, packed).all()
    # the 8-way split (one share per GPU of a box) is a partition of that list
    shares = [lk.hamming_pairs(h, 6, part=p, parts=8, cap=1 << 22) for p in range(8)]
    assert sum(c for _, c in shares) == cnt
    assert np.array_equal(_union(shares), packed)


@pytest.mark.parametrize("radius", [0, 2, 3, 6, 9, 12, 20])
def test_hamming_pairs_indexed_and_swept_paths(lk, radius):
    """20,000 hashes: small radii take the multi-index path (buckets per bit field), large
    radii the plain sweep; both must equal the oracle's all-pairs loop."""
    h = phash_set(20000, 55, max_flips=12)
    h[5] = h[19000]           # exact duplicates
    h[6] = h[19000]
    want, total = O.hamming_pairs(h, radius, cap=1 << 22)
    got, cnt = lk.hamming_pairs(h, radius, cap=1 << 22)
    assert cnt == total
    assert np.array_equal(got, want)
    parts = [lk.hamming_pairs(h, radius, part=p, parts=3, cap=1 << 22) for p in range(3)]
    assert sum(c for _, c in parts) == total
    assert np.array_equal(_union(parts), _pack(want))


def test_hamming_pairs_skewed_buckets(lk):
    """Many hashes sharing whole bit fields (one huge bucket in some tables) stay exact."""
    rng = np.random.default_rng(3)
    h = rng.integers(0, 2**64, size=12000, dtype=np.uint64)
    h[:6000] &= np.uint64(0xFFFFFFFF00000000)       # low 32 bits all zero
    h[3000:9000] |= np.uint64(0xFFFF000000000000)   # top 16 bits all one
    want, total = O.hamming_pairs(h, 6, cap=1 << 22)
    got, cnt = lk.hamming_pairs(h, 6, cap=1 << 22)
    assert cnt == total and np.array_equal(got, want)
