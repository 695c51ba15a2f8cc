"""Timed runs of the library's entry points on seeded synthetic inputs.

    python -m loki_b200.workloads scan   [--rows 1000000 --dim 768 --store i8|f32|f16 --k 10 --centered]
    python -m loki_b200.workloads gemm   [--rows 2000000 --dim 768 --queries 4096 --k 100]
    python -m loki_b200.workloads multi  [--rows 1000000 --dim 768 --queries 64 --k 10 --centered]
    python -m loki_b200.workloads shared [--rows 1000000 --dim 768 --positives 1,2,4,8,16 --k 50]
    python -m loki_b200.workloads hamming [--rows 2000000 --radius 6]
    python -m loki_b200.workloads faces  [--rows 20000 --seeds 50000 --dim 512]
    python -m loki_b200.workloads pca    [--rows 20000 --dim 768 --workers 8]
    python -m loki_b200.workloads cache  [--rows 1000000 --dim 768 --store i8]
    python -m loki_b200.workloads i8peak [--rows 8192]      the int8 tensor rate the batched search is measured against

The benchmark of the headline workload is `bench.py`; these are the other configurations,
each printing what it ran and how long it took.  They are also the commands the profiler is
pointed at (one entry point per run keeps a capture small).  Inputs are seeded N(0,1) vectors
with a common component (like real embeddings) unless stated; corpora are generated on the
device when PyTorch is available, so that building a large index takes milliseconds.
"""
from __future__ import annotations

import argparse
import os
import tempfile
import time

import numpy as np

from . import _lib as lk

STORES = {"f32": lk.LK_F32, "f16": lk.LK_F16, "i8": lk.LK_I8}


def build_index(rows: int, dim: int, store: int, centered: bool = False, seed: int = 1000) -> "lk.DeviceIndex":
    idx = lk.DeviceIndex(dim, store, centered=centered)
    idx.reserve(rows)
    step = 50_000
    try:
        import torch
        g = torch.Generator(device="cuda")
        for c, lo in enumerate(range(0, rows, step)):
            m = min(step, rows - lo)
            g.manual_seed(seed * 7919 + c)
            b = torch.randn((m, dim), generator=g, device="cuda")
            b[:, 0] += 3.0
            idx.upsert_device(lo, m, b.data_ptr())
            del b
        torch.cuda.synchronize()
    except ImportError:
        rng = np.random.default_rng(seed)
        for lo in range(0, rows, step):
            m = min(step, rows - lo)
            b = rng.standard_normal((m, dim), dtype=np.float32)
            b[:, 0] += 3.0
            idx.upsert(lo, b)
    return idx


def queries(n: int, dim: int, seed: int = 2000) -> np.ndarray:
    q = np.random.default_rng(seed).standard_normal((n, dim), dtype=np.float32)
    q[:, 0] += 3.0
    return q


def unit_cloud(n: int, dim: int, rng, centres: int = 200, spread: float = 0.6) -> np.ndarray:
    c = rng.standard_normal((centres, dim)).astype(np.float32)
    v = c[rng.integers(0, centres, n)] + spread * rng.standard_normal((n, dim)).astype(np.float32)
    v /= np.linalg.norm(v.astype(np.float64), axis=1, keepdims=True)
    return v.astype(np.float32)


def run_scan(a):
    store = STORES[a.store]
    idx = build_index(a.rows, a.dim, store, a.centered)
    qs = queries(72, a.dim)
    elem = {lk.LK_F32: 4, lk.LK_F16: 2, lk.LK_I8: 1}[store]
    rq = idx.queries(qs, lk.LK_SCORE_DEFAULT)
    rq.enqueue(0, 8, a.k)
    idx.sync()
    idx.timer_start()
    rq.enqueue(8, 64, a.k)
    ms = idx.timer_stop() / 64
    print(f"scan {a.rows} x {a.dim} {a.store} centered={a.centered} k={a.k}: {ms * 1e3:.1f} us/query queued back to back, "
          f"{a.rows * a.dim * elem / (ms * 1e-3) / 1e9:.0f} GB/s of rows")
    t0 = time.perf_counter()
    for i in range(32):
        idx.search(qs[i], a.k)
    print(f"  one synchronous call per query: {(time.perf_counter() - t0) / 32 * 1e6:.1f} us")


def run_gemm(a):
    idx = build_index(a.rows, a.dim, lk.LK_I8, seed=1003)
    qs = queries(a.queries, a.dim, 2003)
    idx.search(qs[:256], a.k)
    for _ in range(a.reps):
        idx.timer_start()
        t0 = time.perf_counter()
        idx.search(qs, a.k)
        wall = time.perf_counter() - t0
        ms = idx.timer_stop()
        print(f"gemm {a.queries} queries x {a.rows} x {a.dim} int8 k={a.k}: call {wall * 1e3:.2f} ms ({a.queries / wall:.0f} queries/s), "
              f"{ms:.2f} ms between stream events, {2.0 * a.queries * a.rows * a.dim / wall / 1e12:.0f} Tops/s over the call")


def run_i8peak(a):
    """The denominator for the batched int8 search: a plain int8 x int8 -> int32 matrix product of
    the vendor library (torch._int_mm, rows^3), measured like the bf16 peak of this machine: the best
    of ten single products (burst) and a back-to-back loop of about three seconds (sustained, under
    the power cap).  The corpus-sized product of the batched search runs for milliseconds, in bursts
    between host work: it is held against the burst figure."""
    import torch
    n = a.rows if a.rows and a.rows <= 16384 else 8192
    dev = torch.device("cuda")
    x = torch.randint(-127, 128, (n, n), dtype=torch.int8, device=dev)
    y = torch.randint(-127, 128, (n, n), dtype=torch.int8, device=dev).t()   # column-major right operand
    ops = 2.0 * n * n * n
    for _ in range(3):
        torch._int_mm(x, y)
    torch.cuda.synchronize()
    best = 1e9
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(10):
        e0.record()
        torch._int_mm(x, y)
        e1.record()
        e1.synchronize()
        best = min(best, e0.elapsed_time(e1))
    reps = max(10, int(3000.0 / best))
    e0.record()
    for _ in range(reps):
        torch._int_mm(x, y)
    e1.record()
    e1.synchronize()
    sustained = e0.elapsed_time(e1) / reps
    print(f"i8peak {n}^3 int8 -> int32 (torch._int_mm): burst {best:.3f} ms = {ops / best / 1e9:.0f} Tops/s; "
          f"sustained over {reps} products {sustained:.3f} ms = {ops / sustained / 1e9:.0f} Tops/s")


def run_multi(a):
    idx = build_index(a.rows, a.dim, lk.LK_F32, a.centered)
    qs = queries(a.queries, a.dim)
    for mode in (True, False):
        idx.set_batch_mode(mode)
        idx.search(qs, a.k)
        t0 = time.perf_counter()
        for _ in range(a.reps):
            idx.search(qs, a.k)
        dt = (time.perf_counter() - t0) / a.reps
        print(f"multi {a.queries} queries x {a.rows} x {a.dim} float32 centered={a.centered} k={a.k} "
              f"{'8 per pass' if mode else 'single scans'}: {dt * 1e3:.2f} ms per call, {dt / a.queries * 1e6:.1f} us/query")


def run_shared(a):
    idx = build_index(a.rows, a.dim, lk.LK_F32, True)
    qs = queries(64, a.dim)
    for p in [int(x) for x in a.positives.split(",")]:
        idx.search_shared(qs[:p], k=a.k)
        t0 = time.perf_counter()
        for _ in range(a.reps):
            idx.search_shared(qs[:p], k=a.k)
        dt = (time.perf_counter() - t0) / a.reps
        print(f"shared {p} positives x {a.rows} x {a.dim} float32 centered k={a.k}: {dt * 1e6:.0f} us per call, "
              f"{a.rows * a.dim * 4 / dt / 1e9:.0f} GB/s of rows")


def run_hamming(a):
    rng = np.random.default_rng(1004)
    n_dup = a.rows // 10
    base = rng.integers(0, 2 ** 64, size=a.rows - n_dup, dtype=np.uint64)
    dup = base[rng.integers(0, base.size, size=n_dup)].copy()
    flips = rng.integers(0, 7, size=n_dup)
    for f in range(1, 7):      # near-duplicates: 0..6 distinct bits flipped
        sel = np.nonzero(flips >= f)[0]
        bits = rng.integers(0, 64, size=sel.size).astype(np.uint64)
        dup[sel] ^= np.uint64(1) << bits
    h = np.concatenate([base, dup])
    rng.shuffle(h)
    lk.hamming_pairs(h[:1000], a.radius)
    for _ in range(a.reps):
        t0 = time.perf_counter()
        pairs, cnt = lk.hamming_pairs(h, a.radius, cap=1 << 22)
        dt = time.perf_counter() - t0
        print(f"hamming {a.rows} hashes radius {a.radius}: {cnt} pairs in {dt * 1e3:.1f} ms")


def run_faces(a):
    rng = np.random.default_rng(1)
    faces = unit_cloud(a.rows, a.dim, rng)
    seeds = unit_cloud(a.seeds, a.dim, rng)
    lk.prescreen_pairs(faces[:2000], 0.6)
    lk.seed_scores(faces[:512], seeds[:512], 0.5)
    for _ in range(a.reps):
        t0 = time.perf_counter()
        near, count, over = lk.prescreen_pairs(faces, 0.6)
        dt = time.perf_counter() - t0
        print(f"prescreen {a.rows} x {a.dim}: {dt * 1e3:.1f} ms, {int(count.sum())} neighbours, {int(over.sum())} overflows")
        t0 = time.perf_counter()
        rs, hs, sc = lk.seed_scores(faces, seeds, 0.5)
        dt = time.perf_counter() - t0
        print(f"seed scores {a.rows} x {a.seeds} x {a.dim}: {dt * 1e3:.1f} ms, {hs.size} pairs at or above the floor")


def run_pca(a):
    rng = np.random.default_rng(0)
    centres = rng.standard_normal((30, a.dim)).astype(np.float32) * 2
    x = (centres[rng.integers(0, 30, a.rows)] + rng.standard_normal((a.rows, a.dim)).astype(np.float32)).astype(np.float32)
    lk.pca3(x[:500], a.workers)
    for _ in range(a.reps):
        t0 = time.perf_counter()
        coords, variance = lk.pca3(x, a.workers)
        print(f"pca3 {a.rows} x {a.dim} workers={a.workers}: {(time.perf_counter() - t0) * 1e3:.1f} ms, variance {variance}")


def run_cache(a):
    store = STORES[a.store]
    rows = np.random.default_rng(0).standard_normal((a.rows, a.dim), dtype=np.float32)
    t0 = time.perf_counter()
    idx = lk.DeviceIndex(a.dim, store)
    idx.reserve(a.rows)
    idx.upsert(0, rows)
    t1 = time.perf_counter()
    d = tempfile.mkdtemp(dir="/dev/shm" if os.path.isdir("/dev/shm") else None)
    path = os.path.join(d, "index.lkidx")
    idx.save(path, tag=a.rows)
    t2 = time.perf_counter()
    back = lk.DeviceIndex.load(path, tag=a.rows)
    t3 = time.perf_counter()
    size = os.path.getsize(path)
    same = all(np.array_equal(x, y) for x, y in zip(idx.search(rows[:4], 10), back.search(rows[:4], 10)))
    print(f"cache {a.rows} x {a.dim} {a.store}: build from host float32 {1e3 * (t1 - t0):.0f} ms, save {1e3 * (t2 - t1):.0f} ms "
          f"({size / 1e6:.0f} MB), load {1e3 * (t3 - t2):.0f} ms ({size / (t3 - t2) / 1e9:.2f} GB/s), same results: {same}")
    os.remove(path)
    os.rmdir(d)


def main(argv=None):
    ap = argparse.ArgumentParser(prog="python -m loki_b200.workloads", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("workload", choices=["scan", "gemm", "multi", "shared", "hamming", "faces", "pca", "cache", "i8peak"])
    ap.add_argument("--rows", type=int)
    ap.add_argument("--dim", type=int)
    ap.add_argument("--store", default="i8", choices=sorted(STORES))
    ap.add_argument("--k", type=int)
    ap.add_argument("--centered", action="store_true")
    ap.add_argument("--queries", type=int)
    ap.add_argument("--positives", default="1,2,4,8,16")
    ap.add_argument("--radius", type=int, default=6)
    ap.add_argument("--seeds", type=int, default=50_000)
    ap.add_argument("--workers", type=int, default=8)
    ap.add_argument("--reps", type=int, default=3)
    a = ap.parse_args(argv)
    defaults = {"scan": (1_000_000, 768, 10, 0), "gemm": (2_000_000, 768, 100, 4096), "multi": (1_000_000, 768, 10, 64),
                "shared": (1_000_000, 768, 50, 0), "hamming": (2_000_000, 0, 0, 0), "faces": (20_000, 512, 0, 0),
                "pca": (20_000, 768, 0, 0), "cache": (1_000_000, 768, 0, 0), "i8peak": (8192, 0, 0, 0)}[a.workload]
    a.rows = a.rows or defaults[0]
    a.dim = a.dim or defaults[1]
    a.k = a.k or defaults[2]
    a.queries = a.queries or defaults[3]
    {"scan": run_scan, "gemm": run_gemm, "multi": run_multi, "shared": run_shared, "hamming": run_hamming,
     "faces": run_faces, "pca": run_pca, "cache": run_cache, "i8peak": run_i8peak}[a.workload](a)


if __name__ == "__main__":
    main()
