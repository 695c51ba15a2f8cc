"""CPU: the oracle's restatement of the face-clustering scorers against the properties the
reference's own tests state for them."""
import numpy as np
import pytest

import oracle as O
from oracle import face_cluster as OF
from tests.synth import SEED_SCORING_CASES, seed_scoring_case


@pytest.mark.parametrize("case", SEED_SCORING_CASES, ids=lambda c: c[0])
def test_grouped_scoring_decides_like_one_at_a_time(case):
    """media-server/tasks/face_score_kernel_test.go:80-166: the grouped scorer must pick the same
    person for every candidate as the one-at-a-time version, and somebody must join."""
    name, n_cand, n_seed, people, dims, thr, vetoes, cannot, users = case
    sc = seed_scoring_case(n_cand, n_seed, people, dims, vetoes, cannot, users, seed=len(name) * 31)
    aggs = OF.build_person_aggs(sc["seed_vecs"], sc["seed_person"], sc["seed_user"])
    args = (sc["cand_ids"], sc["cand_vecs"], sc["seed_ids"], sc["seed_vecs"], sc["seed_person"], sc["seed_user"],
            aggs, thr, sc["vetoes"], sc["cannot"])
    want = OF.score_against_seeds(*args, grouped=False)
    for workers in (1, 3):
        assert OF.score_against_seeds(*args, workers=workers, grouped=True) == want
    assert any(m != 0 for m in want), "no candidate joined anything: the case proves nothing"
    for cid, m in zip(sc["cand_ids"], want):  # a vetoed person is never the answer
        assert m == 0 or m not in sc["vetoes"].get(cid, ())


def test_dot4_agrees_with_dotf_to_rounding():
    """media-server/tasks/face_score_kernel_test.go:170-190."""
    rng = np.random.default_rng(17)
    for dims in (1, 2, 3, 7, 8, 63, 64, 512):
        b = rng.standard_normal((1, dims)).astype(np.float32)
        b /= np.linalg.norm(b)
        a = rng.standard_normal((4, dims)).astype(np.float32)
        a /= np.linalg.norm(a, axis=1, keepdims=True)
        grouped = O.seed_scores(a, b, 0, True)[:, 0]
        single = O.seed_scores(a, b, 0, False)[:, 0]
        assert np.all(np.abs(grouped - single) <= 1e-5)
        for r in range(4):
            assert single[r] == O.dotf(a[r], b[0])


def test_chunking_decides_which_candidates_are_grouped():
    rng = np.random.default_rng(5)
    c = rng.standard_normal((11, 33)).astype(np.float32)
    s = rng.standard_normal((7, 33)).astype(np.float32)
    single = O.seed_scores(c, s, 0, False)
    one_chunk = O.seed_scores(c, s, 0, True)
    assert np.array_equal(one_chunk[8:], single[8:])          # 11 = 4 + 4 + 3 one at a time
    chunks_of_6 = O.seed_scores(c, s, 6, True)                 # [0,6): 4 + 2; [6,11): 4 + 1
    assert np.array_equal(chunks_of_6[4:6], single[4:6]) and np.array_equal(chunks_of_6[10:], single[10:])
    assert np.array_equal(chunks_of_6[:4], one_chunk[:4])
    assert np.allclose(one_chunk, single, atol=1e-5)
