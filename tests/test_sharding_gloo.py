"""CPU, two processes over gloo: the sharded search (per-shard top-k, all-gather of the
ranked keys, merge) gives the same result as one scan of the whole corpus."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle as O
from loki_b200 import sharding as S
from tests.synth import clustered_rows, gaussian_rows


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n, dim, k, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rows = clustered_rows(n, dim, 5)      # every rank can generate every row: take its own range
        queries = gaussian_rows(3, dim, 6)
        base, cnt = S.shard_bounds(n, world)[rank]
        codes, _ = O.build_i8(rows[base:base + cnt])
        results = []
        for q in queries:
            qc, _ = O.build_i8(q.reshape(1, -1))
            ids, sc = O.topk_i32(O.scan_i8(codes, qc[0]), k)       # shard-local ids
            keys = np.zeros(k, np.uint64)
            keys[:ids.size] = S.pack_keys_i32(sc, ids)
            mine = torch.from_numpy(keys.view(np.int64).copy())
            gathered = [torch.zeros(k, dtype=torch.int64) for _ in range(world)]
            dist.all_gather(gathered, mine)
            bases = [b for b, _ in S.shard_bounds(n, world)]
            merged = S.merge_ranked([g.numpy().view(np.uint64) for g in gathered], bases, k)
            results.append(merged)
        np.save(os.path.join(out_dir, f"rank{rank}.npy"), np.stack(results))
    finally:
        dist.destroy_process_group()


def test_sharded_topk_equals_global_topk(tmp_path):
    n, dim, k, world = 3001, 96, 25, 2
    mp.spawn(_worker, args=(world, _free_port(), n, dim, k, str(tmp_path)), nprocs=world, join=True)
    rows = clustered_rows(n, dim, 5)
    queries = gaussian_rows(3, dim, 6)
    codes, _ = O.build_i8(rows)
    got = [np.load(tmp_path / f"rank{r}.npy") for r in range(world)]
    assert np.array_equal(got[0], got[1]), "every rank must hold the same merged result"
    for i, q in enumerate(queries):
        qc, _ = O.build_i8(q.reshape(1, -1))
        ids, sc = O.topk_i32(O.scan_i8(codes, qc[0]), k)
        assert np.array_equal(S.key_ids(got[0][i]), ids.astype(np.int64))
        assert np.array_equal(S.key_scores_i32(got[0][i]), sc)


def test_shard_bounds_cover_everything():
    for n, w in [(0, 1), (1, 8), (10, 3), (16_000_000, 8), (7, 8)]:
        b = S.shard_bounds(n, w)
        assert len(b) == w and sum(c for _, c in b) == n
        pos = 0
        for base, cnt in b:
            assert base == pos or cnt == 0
            pos += cnt


def test_key_packing_orders_like_the_index():
    rng = np.random.default_rng(0)
    sc = rng.integers(-5, 6, size=200).astype(np.int32)
    ids = rng.permutation(200).astype(np.int32)
    keys = S.pack_keys_i32(sc, ids)
    order = np.argsort(keys)[::-1]
    want = np.lexsort((ids, -sc.astype(np.int64)))
    assert np.array_equal(order, want)
    assert np.array_equal(S.key_ids(keys), ids) and np.array_equal(S.key_scores_i32(keys), sc)
    f = np.array([0.0, -0.0, 1.5, -2.0, 3e-9, -1e-30], np.float32)
    fk = S.pack_keys_f32(f, np.arange(6, dtype=np.int32))
    assert fk[0] > fk[1] and (fk[0] >> np.uint64(32)) == (fk[1] >> np.uint64(32))  # -0 ties with +0, lower id first
    assert np.array_equal(np.argsort(fk)[::-1], np.array([2, 4, 0, 1, 5, 3]))
    assert np.array_equal(S.key_scores_f32(fk)[2:], f[2:])
