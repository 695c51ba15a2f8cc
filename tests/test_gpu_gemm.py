"""GPU: the batched int8 search on tensor cores (tcgen05.mma kind::i8 with the top-k fused
into the epilogue) must return exactly what query-by-query scans return, and what the
CPU oracle returns (parity unpinned by the reference: it has no int8 path)."""
import numpy as np
import pytest

import oracle as O
from tests.synth import clustered_rows, gaussian_rows

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,dim,nq,k", [(5000, 768, 64, 10), (20011, 768, 200, 100), (9000, 100, 40, 33),
                                        (30000, 1024, 129, 50), (4096, 128, 32, 256)])
def test_batched_tensor_core_search_equals_single_query_scans(lk, n, dim, nq, k):
    rows = clustered_rows(n, dim, 60 + n)   # half the rows cluster: many equal int32 scores
    queries = np.concatenate([gaussian_rows(nq - 3, dim, 61 + n), rows[1:4]])
    idx = lk.DeviceIndex(dim, lk.LK_I8)
    idx.append(rows)
    idx.set_batch_mode(False)
    ids0, sc0, isc0, cnt0 = idx.search(queries, k)
    launches0 = idx.stats()["scan_launches"]
    idx.set_batch_mode(True)
    ids1, sc1, isc1, cnt1 = idx.search(queries, k)
    assert idx.stats()["scan_launches"] == launches0, "batch mode must not fall back to single-query scans"
    assert np.array_equal(cnt0, cnt1)
    assert np.array_equal(isc0, isc1), "int32 scores differ"
    assert np.array_equal(ids0, ids1), "ids differ"
    assert np.array_equal(sc0, sc1), "de-quantised scores differ"
    # and against the oracle for a few of the queries
    codes, scales = O.build_i8(rows)
    for q in (0, nq // 2, nq - 1):
        qc, _ = O.build_i8(queries[q:q + 1])
        wid, wsc = O.topk_i32(O.scan_i8(codes, qc[0]), k)
        assert np.array_equal(ids1[q], wid) and np.array_equal(isc1[q], wsc)
