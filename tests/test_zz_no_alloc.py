"""GPU: the allocation-free scan entry point (lk_scan_i8_prealloc) against lk_search.

The entry point exists for hosts that may not allocate device memory while serving
(a fixed GPU budget handed out at start-up, a latency path that cannot take the
device-wide stall of cudaMalloc, a plug-in inside someone else's memory arena).  Here
the test owns all buffers (torch tensors) and checks that two calls in a row, which
share the library's built-in scratch array, each reproduce the regular search bit for
bit: ids, raw int32 dots and de-quantised float scores, and that the calls leave the amount
of free device memory where it was.
"""
import ctypes as C

import numpy as np
import pytest

from tests.synth import gaussian_rows

pytestmark = pytest.mark.gpu


def _prepared_query(lk, q, dim):
    """int8 codes + scale of a query, produced by the library itself (a query is
    normalised and quantised exactly like a row)."""
    tmp = lk.DeviceIndex(dim, lk.LK_I8)
    tmp.append(q.reshape(1, -1))
    codes, scales = tmp.read_rows()
    tmp.close()
    return codes[0], float(scales[0])


@pytest.mark.parametrize("n,dim,k", [(40_000, 768, 10), (3_000, 100, 128), (40_000, 1024, 50)])
def test_prealloc_scan_matches_search_twice(lk, n, dim, k):
    import torch

    rows = gaussian_rows(n, dim, 900 + dim)
    queries = gaussian_rows(2, dim, 901 + dim)
    idx = lk.DeviceIndex(dim, lk.LK_I8)
    idx.append(rows)
    want_ids, want_scores, want_iscores, want_counts = idx.search(queries, k)

    codes, scales = idx.read_rows()
    ld = (dim + 15) // 16 * 16
    padded = np.zeros((n, ld), np.int8)
    padded[:, :dim] = codes
    dev = torch.device("cuda", 0)
    d_codes = torch.from_numpy(padded).to(dev)
    d_scales = torch.from_numpy(scales).to(dev)
    d_ids = torch.empty(k, dtype=torch.int64, device=dev)
    d_scores = torch.empty(k, dtype=torch.float32, device=dev)
    d_iscores = torch.empty(k, dtype=torch.int32, device=dev)
    d_count = torch.empty(1, dtype=torch.int32, device=dev)
    torch.cuda.synchronize()

    prepared = [_prepared_query(lk, queries[qi], dim) for qi in range(2)]
    d_queries = []
    for qcodes, _ in prepared:
        qpad = np.zeros(ld, np.int8)
        qpad[:dim] = qcodes
        d_queries.append(torch.from_numpy(qpad).to(dev))
    torch.cuda.synchronize()
    free_before = None
    for qi in range(2):  # two calls in a row share the built-in scratch array
        qscale = prepared[qi][1]
        d_query = d_queries[qi]
        if qi == 1:      # the first call has set the entry point up; from here on nothing may be allocated
            free_before = torch.cuda.mem_get_info(dev)[0]
        st = lk.lib.lk_scan_i8_prealloc(0, C.c_void_p(d_codes.data_ptr()), n, dim, ld, C.c_void_p(d_scales.data_ptr()),
                                        C.c_void_p(d_query.data_ptr()), C.c_float(qscale), k,
                                        C.c_void_p(d_ids.data_ptr()), C.c_void_p(d_scores.data_ptr()),
                                        C.c_void_p(d_iscores.data_ptr()), C.c_void_p(d_count.data_ptr()), None)
        lk.check(st)
        torch.cuda.synchronize()
        if qi == 1:
            assert torch.cuda.mem_get_info(dev)[0] == free_before, "the call changed the free device memory"
        assert int(d_count.item()) == want_counts[qi] == k
        assert np.array_equal(d_ids.cpu().numpy(), want_ids[qi])
        assert np.array_equal(d_iscores.cpu().numpy(), want_iscores[qi])
        assert np.array_equal(d_scores.cpu().numpy(), want_scores[qi])


def test_prealloc_scan_rejects_sizes_beyond_its_scratch(lk):
    import torch

    dev = torch.device("cuda", 0)
    buf = torch.zeros(4096, dtype=torch.int8, device=dev)
    f = torch.zeros(64, dtype=torch.float32, device=dev)
    out = torch.zeros(4096, dtype=torch.int64, device=dev)
    p = lambda t: C.c_void_p(t.data_ptr())
    st = lk.lib.lk_scan_i8_prealloc(0, p(buf), 16, 16, 16, p(f), p(buf), C.c_float(1.0), lk.LK_PREALLOC_MAX_K + 1,
                                    p(out), p(f), None, p(out), None)
    assert st == lk.LK_ERANGE
    assert b"LK_PREALLOC_MAX_K" in lk.lib.lk_last_error()
    st = lk.lib.lk_scan_i8_prealloc(0, p(buf), 16, 16, 24, p(f), p(buf), C.c_float(1.0), 4, p(out), p(f), None, p(out), None)
    assert st == lk.LK_EINVAL  # ld not a multiple of 16
