"""CPU tests (no GPU): the oracle against the reference's known-answer tests, and the
int8 / Hamming oracle against an independent numpy restatement."""
import types

import numpy as np
import pytest

import oracle as O
from oracle import exact_index as OX
from tests import ref_cases
from tests.synth import gaussian_rows, phash_set

oracle_impl = types.SimpleNamespace(
    New=OX.New, NewCentered=OX.NewCentered, SharedSpec=OX.SharedSpec, ScoreDefault=OX.ScoreDefault,
    ScorePlain=OX.ScorePlain, MinCenterCount=OX.MinCenterCount)


@pytest.mark.parametrize("case", ref_cases.ALL_CASES, ids=lambda f: f.__name__)
def test_reference_case_on_oracle(case):
    case(oracle_impl)


# ---- media-server/embedvec/embedvec_test.go ----------------------------------------

def test_encode_decode_round_trip():  # :8-22
    v = np.array([0.5, -0.25, 1.0, 0.0], np.float32)
    out = O.decode(O.encode(v))
    assert out.dtype == np.float32 and np.array_equal(out, v)
    assert O.encode(np.array([1.0], np.float32)) == b"\x00\x00\x80\x3f"  # little endian


def test_decode_rejects_ragged():  # :24-28
    with pytest.raises(ValueError):
        O.decode(bytes([1, 2, 3]))


def test_normalize_unit_length():  # :30-39
    v = O.normalize([3, 4])
    assert abs(float(np.sum(v.astype(np.float64) ** 2)) - 1.0) <= 1e-6
    assert np.array_equal(v, np.array([0.6, 0.8], np.float32))


def test_cosine_identical():  # :41-46
    a = O.normalize([1, 2, 3])
    assert abs(float(O.cosine(a, a)) - 1.0) <= 1e-6


def test_cosine_length_mismatch():  # :48-52
    assert O.cosine([1, 0], [1, 0, 0]) == 0


def test_normalize_zero_vector():  # :167-174
    assert np.all(O.normalize([0, 0, 0]) == 0)


def test_cosine_sim_unnormalised():
    assert abs(float(O.cosine_sim([10, 0], [3, 0])) - 1.0) <= 1e-6
    assert O.cosine_sim([0, 0], [1, 0]) == 0


# ---- media-server/embedvec/shared_test.go -------------------------------------------

def test_shared_two_examples_is_min():  # :19-41
    q1, q2 = O.normalize([1, 0.5, 0]), O.normalize([1, -0.5, 0.2])
    sq = O.SharedQuery([q1, q2], None, None, None, 0, 1)
    for cand in (O.normalize([1, 0, 0]), O.normalize([0, 1, 0]), O.normalize([0.3, -0.7, 0.6]), q1):
        want = min(O.cosine(q1, cand), O.cosine(q2, cand))
        assert abs(float(sq.score(cand)) - float(want)) <= 1e-5


def test_shared_full_projection_collapses_variation():  # :47-64
    q1, q2 = O.normalize([1, 1, 0]), O.normalize([1, -1, 0])
    sq = O.SharedQuery([q1, q2], None, None, None, 1, 1)
    assert abs(float(sq.score([1, 0, 0])) - 1) <= 1e-5
    assert abs(float(sq.score(q1)) - 1) <= 1e-5
    assert abs(float(sq.score([0, 0, 1]))) <= 1e-5


def test_shared_football_scenario():  # :70-88
    q1, q2, q3 = O.normalize([1, 1, 0, 0]), O.normalize([1, 0, 1, 0]), O.normalize([1, 0, 0, 1])
    sq = O.SharedQuery([q1, q2, q3], None, None, None, 0.25, 1.0)
    football, one, scenery = sq.score([1, 0, 0, 0]), sq.score(q1), sq.score([0, 1, 0, 0])
    assert football > one > scenery


def test_shared_negative_penalty():  # :93-111
    pos, neg = [O.normalize([1, 0, 0])], [O.normalize([0, 1, 0])]
    sq = O.SharedQuery(pos, None, neg, [0.5], 0, 1)
    clean, tainted = O.normalize([1, 0, 0.3]), O.normalize([1, 0.3, 0])
    assert sq.score(clean) > sq.score(tainted)
    v = O.normalize([1, 1, 0])
    want = O.cosine(pos[0], v) - np.float32(0.5) * O.cosine(neg[0], v)
    assert abs(float(sq.score(v)) - float(want)) <= 1e-5


def test_shared_weights():  # :115-131
    q1, q2 = O.normalize([1, 0, 0]), O.normalize([0, 1, 0])
    heavy = O.SharedQuery([q1, q2], [1, 0.25], None, None, 0, 0)
    even = O.SharedQuery([q1, q2], None, None, None, 0, 0)
    assert heavy.score(q1) > even.score(q1)


def test_shared_single_positive_is_cosine():  # :135-149
    q = O.normalize([0.3, 0.7, 0.2])
    sq = O.SharedQuery([q], None, None, None, 0.25, 1.0)
    for cand in (O.normalize([1, 0, 0]), O.normalize([-0.2, 0.5, 0.9])):
        assert abs(float(sq.score(cand)) - float(O.cosine(q, cand))) <= 1e-5


def test_shared_duplicate_examples():  # :154-164
    q = O.normalize([1, 2, 3])
    sq = O.SharedQuery([q, q, q], None, None, None, 0.25, 1.0)
    got = float(sq.score(q))
    assert not np.isnan(got) and abs(got - 1) <= 1e-4
    assert sq.rank == 0


def test_shared_errors():  # :167-181
    with pytest.raises(ValueError):
        O.SharedQuery([], None, None, None, 0.5, 1)
    v = [1, 0]
    with pytest.raises(ValueError):
        O.SharedQuery([v], [0], None, None, 0.5, 1)
    with pytest.raises(ValueError):
        O.SharedQuery([v, [1, 0, 0]], None, None, None, 0.5, 1)
    with pytest.raises(ValueError):
        O.SharedQuery([v], None, [[1, 0]], None, 0.5, 1)


# ---- heap top-k (media-server/embedindex/embedindex.go:495-534) vs a plain sort -----

def test_heap_topk_equals_sorted_topk_without_boundary_ties():
    rng = np.random.default_rng(3)
    for n, k in [(1, 1), (10, 3), (1000, 50), (1000, 1000), (5000, 1)]:
        sc = rng.standard_normal(n).astype(np.float32)
        h = O.topk_heap(sc, k)
        ids, _ = O.topk_f32(sc, k)
        assert sorted(h.tolist()) == sorted(ids.tolist())
        assert h.size == min(k, n)


def test_heap_keeps_earlier_of_equal_scores():
    sc = np.array([1, 1, 1, 1, 1], np.float32)
    assert sorted(O.topk_heap(sc, 2).tolist()) == [0, 1]  # later equal scores never displace


# ---- int8 / Hamming oracle vs an independent numpy restatement (parity unpinned) ----

def _np_build_i8(rows):
    x = rows.astype(np.float64)
    nrm = np.sqrt((x * x).sum(axis=1, keepdims=True))
    y = np.where(nrm > 0, x / np.where(nrm > 0, nrm, 1), x).astype(np.float32)
    amax = np.abs(y).max(axis=1)
    scale = (amax / np.float32(127)).astype(np.float32)
    safe = np.where(scale > 0, scale, np.float32(1))
    q = np.rint((y / safe[:, None]).astype(np.float32))  # numpy rint: half to even
    q = np.clip(q, -127, 127).astype(np.int8)
    q[scale == 0] = 0
    return q, scale


@pytest.mark.parametrize("n,dim", [(50, 16), (200, 768), (64, 100), (10, 1)])
def test_int8_oracle_matches_numpy(n, dim):
    rows = gaussian_rows(n, dim, 5 + n)
    rows[0] = 0  # zero row
    codes, scales = O.build_i8(rows)
    ncodes, nscales = _np_build_i8(rows)
    # numpy sums squares pairwise, the oracle in index order: the norm can differ in the last
    # bit, which can move a code that sits exactly on a rounding boundary by one.
    assert np.array_equal(scales == 0, nscales == 0)
    np.testing.assert_allclose(scales, nscales, rtol=2e-7)
    assert np.abs(codes.astype(np.int32) - ncodes.astype(np.int32)).max() <= 1
    assert (codes != ncodes).mean() < 1e-3
    assert np.all(codes[0] == 0) and scales[0] == 0
    assert np.abs(codes).max() == 127
    q = codes[1 % n]
    want = codes.astype(np.int32) @ q.astype(np.int32)
    assert np.array_equal(O.scan_i8(codes, q), want)
    ids, sc = O.topk_i32(want, 7)
    order = np.lexsort((np.arange(n), -want.astype(np.int64)))[:7]
    assert np.array_equal(ids, order) and np.array_equal(sc, want[order])


def test_quantise_rounding_rule():
    # scale = 1/127 exactly representable inputs: x/scale = 63.5 -> 64 (even), 62.5 -> 62 (even)
    x = np.array([1.0, 0.5, 62.5 / 127, -0.5, 0.0], np.float32)
    q = np.zeros(5, np.int8)
    import ctypes as C
    s = C.c_float(0)
    O.lib().orc_quantize_i8(x, 5, q, C.byref(s))
    assert abs(s.value - 1 / 127) < 1e-9
    assert q[0] == 127 and q[4] == 0 and q[3] == -q[1]
    assert q[1] in (63, 64)


def test_hamming_oracle_matches_numpy():
    h = phash_set(1500, 11)
    pairs, total = O.hamming_pairs(h, 6)
    x = h[:, None] ^ h[None, :]
    pop = np.zeros(x.shape, np.int32)
    for b in range(64):
        pop += ((x >> np.uint64(b)) & np.uint64(1)).astype(np.int32)
    ii, jj = np.nonzero(np.triu(pop <= 6, k=1))
    assert total == ii.size
    assert np.array_equal(pairs[:, 0], ii.astype(np.uint32)) and np.array_equal(pairs[:, 1], jj.astype(np.uint32))
    assert total > 100  # the generator plants near-duplicates
    d = O.hamming_scan(h, int(h[3]))
    assert np.array_equal(d, pop[3])


def test_multithreaded_scan_equals_serial():
    rows = O.normalize_rows(gaussian_rows(1000, 64, 1))
    q = O.normalize(gaussian_rows(1, 64, 2)[0])
    a = O.scan_f32(rows, q, workers=1)
    b = O.scan_f32(rows, q, workers=7)
    assert np.array_equal(a, b)
