#!/usr/bin/env python
"""Benchmark of the int8 top-10 single-query scan (1,000,000 x 768 rows per GPU).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is ONE query: one launch of the fused scan + top-k kernel over the GPU's
whole shard (768 MB, larger than the 126 MB L2, so every step streams from HBM).
Prints one JSON line (rank 0).

* ``value``      queries/s with the prepared queries already in HBM, K launches
                 queued back to back, timed with CUDA events on the library's stream.
                 At N GPUs every GPU holds its own 1M-row shard (weak scaling: the
                 corpus is N x 1M rows), each query is scanned by all shards and the
                 per-shard top-10 lists are exchanged and merged on every rank; the value
                 counts 1M-row shard scans per second over all GPUs (= global
                 queries/s x N), ``config.global_queries_per_s`` is the plain figure.
* ``e2e``        the same through ``lk_search`` with host buffers, one synchronous
                 call per query (host prep, H2D, scan, [exchange, merge,] D2H).
* ``roofline``   algorithmic bytes of one launch (rows x 768) / average launch time.
* ``parity``     after the timed region: complete hit lists of several of the timed queries
                 against the CPU oracle run over the codes the index stores (at N > 1 the
                 oracle's per-shard lists are merged by the host statement of the merge rule).
* ``cpu_baseline`` the reference's algorithm (float32 rows, float64 accumulate,
                 per-core row chunks, serial heap top-k) restated in C (the Go
                 toolchain is absent), timed on this host's cores.
* ``other_workloads`` the sharded shapes the task names beside the headline (10,000,000 x 768
                 and 16,000,000 x 1,024 rows split over the N GPUs, 100,000 x 512 float32),
                 each with its own HBM fraction and oracle check.

``--impl reference`` times that CPU restatement alone, on the same metric and configuration.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

ROWS_PER_GPU = 1_000_000
DIM = 768
TOPK = 10
METRIC = "queries/sec, int8 top-10 scan of 1M x 768 rows per GPU shard"
WORKLOAD = ("1,000,000 x 768 int8 rows per GPU (per-row scale after L2 normalisation), "
            "single queries issued one at a time, int32 dot, top-10")
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the scan kernel on this workload
# (one ncu capture on one GPU; the kernel reads every row once and writes k keys per CTA)
NCU_TRAFFIC_BYTES_PER_LAUNCH = 771.9e6
CHUNK = 62_500  # rows generated per torch call (192 MB of float32)


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed regions run."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                power.append(float(r[3]))
            except ValueError:
                continue
            for name, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        # "under load": the samples drawn while the GPU was busy (power above the idle half)
        busy = [s for s, p in zip(sm, power) if power and p >= 0.5 * max(power)] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "samples_under_load": len(busy), "reasons": sorted(reasons)}


def make_queries(n: int, seed: int, dim: int = DIM) -> np.ndarray:
    return np.random.default_rng(seed).standard_normal((n, dim), dtype=np.float32)


# ---------------------------------------------------------------------------------------------
# CPU legs: the reference's scan restated in C (oracle/), all host cores
# ---------------------------------------------------------------------------------------------

def _reference_shaped_corpus(n: int, dim: int, seed: int, per_row: bool):
    """Normalised float32 rows as the reference holds them: one separately allocated vector per
    row (media-server/embedindex/embedindex.go:124), or one contiguous arena."""
    import ctypes as C

    import oracle as O

    rows = O.normalize_rows(np.random.default_rng(seed).standard_normal((n, dim), dtype=np.float32))
    if not per_row:
        return rows, None, None
    keep = [rows[i].copy() for i in range(n)]
    rowp = (C.c_void_p * n)(*[a.ctypes.data for a in keep])
    return rows, np.frombuffer(rowp, dtype=np.uint64), (keep, rowp)


def cpu_scan_timed(rows, rowp, queries, k: int, warmup: int):
    """Seconds per query of scan + serial heap top-k + ordering (scanTopK, embedindex.go:424-457)."""
    import oracle as O

    cores = os.cpu_count() or 1
    used = []
    for i in range(queries.shape[0]):
        q = O.normalize(queries[i])
        t0 = time.perf_counter()
        sc = O.scan_f32(rows, q, workers=cores, rowp=rowp)
        h = O.topk_heap(sc, k)
        hits = sorted(((-float(sc[j]), int(j)) for j in h))
        dt = time.perf_counter() - t0
        assert len(hits) == min(k, rows.shape[0])
        if i >= warmup:
            used.append(dt)
    return sum(used) / len(used)


def cpu_reference_arm(steps: int, warmup: int):
    """The reference arm's figure: every step is one query over the reference's own storage, on a
    250,000-row sample of the shard, its time scaled linearly to the 1,000,000 rows (the scan is
    linear in rows; the sample, 768 MB of float32, is far larger than the host's caches)."""
    cores = os.cpu_count() or 1
    n = 250_000
    rows, rowp, keep = _reference_shaped_corpus(n, DIM, 1002, per_row=True)
    per_q = cpu_scan_timed(rows, rowp, make_queries(steps + warmup, 2002), TOPK, warmup)
    del keep
    scale = ROWS_PER_GPU / n
    desc = (f"{steps} timed queries (+{warmup} warm-up) over {n} rows x {DIM} float32, one allocation per row "
            f"(the reference's storage)" + ("" if n == ROWS_PER_GPU else f", time scaled x{scale:g} to {ROWS_PER_GPU} rows")
            + f"; C restatement of the Go scan, {cores} threads")
    return 1.0 / (per_q * scale), cores, desc, per_q * scale


def cpu_baseline_leg():
    """Bounded CPU baselines for the GPU arm's line (about 20 s): the headline shape on a 250,000-row
    sample in both storage layouts, and the reference's own benchmark shapes at full size."""
    cores = os.cpu_count() or 1
    n = 250_000
    scale = ROWS_PER_GPU / n
    qs = make_queries(10, 2002)
    rows, rowp, keep = _reference_shaped_corpus(n, DIM, 1002, per_row=True)
    per_row = cpu_scan_timed(rows, rowp, qs, TOPK, 2) * scale
    contiguous = cpu_scan_timed(rows, None, qs, TOPK, 2) * scale
    del keep, rowp
    # the reference's own benchmark shape (media-server/embedindex/embedindex_test.go:189-208)
    c0 = cpu_scan_timed(rows[:50_000], None, qs, 50, 2)
    del rows
    rows1, _, _ = _reference_shaped_corpus(100_000, 512, 1001, per_row=False)
    c1 = cpu_scan_timed(rows1, None, make_queries(64, 2001, 512), 10, 4)
    return {
        "value": 1.0 / per_row, "unit": "queries/s", "cores": cores, "kind": "port",
        "sample": (f"8 queries over the first {n} rows x {DIM} float32, one allocation per row (the reference's "
                   f"storage), time scaled x{scale:g} to {ROWS_PER_GPU} rows; C restatement of the Go scan, {cores} threads"),
        "variants": {
            "contiguous_arena_queries_per_s": 1.0 / contiguous,
            "ref_bench_shape_50000x768_f32_k50_queries_per_s": 1.0 / c0,
            "config1_100000x512_f32_k10_queries_per_s": 1.0 / c1,
        },
    }


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    qps, cores, desc, per_q = cpu_reference_arm(args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": METRIC,
        "value": qps, "unit": "queries/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": per_q * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "note": "the reference has no int8 path: its scan stores float32 rows and accumulates in float64; "
                           "CPU only, no GPU used; unit = scans of one 1M-row shard per second, the same unit as the "
                           "GPU arm at any N"},
        "cpu_baseline": {"value": qps, "unit": "queries/s", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": qps, "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------

class Ranks:
    """The process group of the run (one process per GPU), or a single process."""

    def __init__(self):
        import torch
        self.torch = torch
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            import torch.distributed as dist
            self.dist = dist
            dist.init_process_group("nccl", device_id=self.dev)

    def barrier(self, idx=None):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()
        if idx is not None:
            idx.sync()

    def max_over_ranks(self, x: float) -> float:
        if self.world == 1:
            return x
        t = self.torch.tensor([x], device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def gather_objects(self, obj):
        if self.world == 1:
            return [obj]
        out = [None] * self.world
        self.dist.all_gather_object(out, obj)
        return out

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def build_shard(lk, R: Ranks, rows: int, dim: int, store: int, seed: int, shard: int):
    """This rank's shard, generated on the device (seeded N(0,1)), normalised and stored by the library."""
    torch = R.torch
    idx = lk.DeviceIndex(dim, store, device=R.local)
    idx.reserve(rows)
    gen = torch.Generator(device=R.dev)
    for c0 in range(0, rows, CHUNK):
        m = min(CHUNK, rows - c0)
        gen.manual_seed(seed * 1_000_003 + shard * 4096 + c0 // CHUNK)
        block = torch.randn((m, dim), generator=gen, device=R.dev, dtype=torch.float32)
        idx.upsert_device(c0, m, block.data_ptr())
        del block
    torch.cuda.synchronize()
    assert len(idx) == rows
    return idx


def make_comm(lk, R: Ranks, peer: bool):
    uid = [lk.Comm.unique_id() if R.rank == 0 else None]
    R.dist.broadcast_object_list(uid, src=0)
    comm = lk.Comm(R.world, R.rank, R.local, uid[0])
    if peer:  # exchange the per-shard top-k inside the scan kernel, over peer memory
        handles = [None] * R.world
        R.dist.all_gather_object(handles, comm.peer_export())
        comm.peer_attach(handles)
    return comm


def oracle_check(lk, R: Ranks, idx, base: int, queries: np.ndarray, k: int, got_ids, got_scores, store: int):
    """Complete hit lists against the CPU oracle: every rank scores its own shard's stored rows with the
    oracle, rank 0 merges the per-shard lists with the host statement of the merge rule and compares."""
    import oracle as O
    from loki_b200 import sharding as S

    cores = max(1, (os.cpu_count() or 1) // max(1, R.world))
    lists = []
    if store == lk.LK_I8:
        codes, _ = idx.read_rows()
        for q in queries:
            qc, _ = O.build_i8(q.reshape(1, -1))
            ids, sc = O.topk_i32(O.scan_i8(codes, qc[0], workers=cores), k)
            lists.append(S.pack_keys_i32(sc, ids))
    else:
        rows = idx.read_rows()
        for q in queries:
            ids, sc = O.topk_f32(O.scan_f32(rows, O.normalize(q), workers=cores), k)
            lists.append(S.pack_keys_f32(sc, ids))
    allr = R.gather_objects((base, lists))
    if R.rank != 0:
        return None
    ok = True
    for qi in range(len(queries)):
        merged = S.merge_ranked([lst[qi] for _, lst in allr], [b for b, _ in allr], k)
        ids = S.key_ids(merged)
        if store == lk.LK_I8:   # bit-exact: ids and int32 scores
            ok &= bool(np.array_equal(ids, got_ids[qi]) and np.array_equal(S.key_scores_i32(merged), got_scores[qi]))
        else:                   # float32: 1e-5 relative on the score; ids may swap only between near-tied neighbours
            want = S.key_scores_f32(merged)
            ok &= bool(np.allclose(got_scores[qi], want, rtol=1e-5, atol=1e-7))
            ok &= bool(np.all((ids == got_ids[qi]) | (np.abs(got_scores[qi] - want) <= 1e-5 * np.abs(want))))
    return {"checked": len(queries), "ok": ok,
            "against": "CPU oracle over the stored rows" + ("" if R.world == 1 else ", per-shard lists merged on the host")}


def timed_scans(R: Ranks, idx, rq, warm: int, steps: int, k: int):
    """`steps` queued scans timed on the device (max over ranks); `warm` untimed ones first, the last
    two of them after the barrier so that the ranks' streams are aligned when the clock starts."""
    pre = max(0, warm - 2)
    if pre:
        rq.enqueue(0, pre, k)
    R.barrier(idx)
    if warm - pre:
        rq.enqueue(pre, warm - pre, k)
    idx.timer_start()
    rq.enqueue(warm, steps, k)
    ms = idx.timer_stop()
    R.barrier(idx)
    return R.max_over_ranks(ms)


# int8 x int8 -> int32 tensor rate of this pool's B200 (python -m loki_b200.workloads i8peak: the vendor
# library's 8192^3 product, best of ten): the denominator for the batched search
I8_TENSOR_PEAK_TOPS = 3072.0


def other_workload(lk, R: Ranks, comm, name: str, total_rows: int, dim: int, store: int, k: int, steps: int, seed: int,
                   peak: float, batch: int = 0):
    """One more shape of the path, its rows split over the ranks (strong scaling of a fixed corpus).
    With `batch`, that many queries also go through one lk_search call (host buffers in and out):
    on an int8 index one tensor-core matrix product per shard and one all-gather for the batch."""
    rows = total_rows // R.world
    base = R.rank * rows
    idx = build_shard(lk, R, rows, dim, store, seed, R.rank)
    if comm is not None:
        idx.attach_comm(comm, base)
    warm = 6
    queries = make_queries(warm + steps, seed + 1000, dim)
    rq = idx.queries(queries)
    ms = timed_scans(R, idx, rq, warm, steps, k)
    picks = [warm, warm + steps - 1]
    ids, fsc, isc, _ = rq.fetch(0, warm + steps, k)
    par = oracle_check(lk, R, idx, base, queries[picks], k, ids[picks], (isc if store == lk.LK_I8 else fsc)[picks], store)
    elem = 1 if store == lk.LK_I8 else 4
    per_q = ms * 1e-3 / steps
    out = {"rows_total": total_rows, "rows_per_gpu": rows, "dim": dim, "k": k, "dtype": "int8" if elem == 1 else "f32",
           "queries": steps, "ms_per_query": per_q * 1e3, "queries_per_s": 1.0 / per_q,
           "hbm_gbs_per_gpu": rows * dim * elem / per_q / 1e9, "hbm_frac_per_gpu": rows * dim * elem / per_q / 1e9 / peak,
           "parity": par}
    if batch:
        bq = make_queries(batch, seed + 2000, dim)
        idx.search(bq[:max(64, batch // 8)], k)          # warm-up: scratch of the batched path
        R.barrier(idx)
        best = None
        for _ in range(3):
            t0 = time.perf_counter()
            got = idx.search(bq, k)
            dt = R.max_over_ranks(time.perf_counter() - t0)
            best = dt if best is None else min(best, dt)
            R.barrier(idx)
        idx.set_batch_mode(False)                         # the same queries one at a time: must agree bit for bit
        same = True
        for qi in (0, batch // 2, batch - 1):
            one = idx.search_one(bq[qi], k)
            same &= bool(np.array_equal(one[0][0], got[0][qi]) and np.array_equal(one[2][0], got[2][qi]))
        idx.set_batch_mode(True)
        ops = 2.0 * batch * rows * dim
        out["batch"] = {"queries": batch, "ms_per_call": best * 1e3, "queries_per_s": batch / best,
                        "int8_tops_per_gpu": ops / best / 1e12, "tensor_frac_per_gpu": ops / best / 1e12 / I8_TENSOR_PEAK_TOPS,
                        "tensor_peak": f"{I8_TENSOR_PEAK_TOPS:.0f} Tops/s, measured (vendor int8 product, burst)",
                        "hbm_gbs_per_gpu": rows * dim / best / 1e9, "hbm_frac_per_gpu": rows * dim / best / 1e9 / peak,
                        "equals_single_scans": same,
                        "note": "whole call: raw float queries up, quantised on the device, product + fused top-k"
                                + (", all-gather + merge" if R.world > 1 else "") + ", hits down"}
    rq.close()
    idx.close()
    return name, out


def run_ours(args):
    from loki_b200 import _lib as lk

    R = Ranks()
    world, rank = R.world, R.rank
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one process per GPU)")
    assert lk.device_count() > R.local, "bench.py needs a CUDA device (there is no CPU path)"

    sampler = ClockSampler(R.local)
    if rank == 0:
        sampler.start()  # long before the timed regions: nothing rank-specific sits next to them

    idx = build_shard(lk, R, ROWS_PER_GPU, DIM, lk.LK_I8, 1002, rank)
    comm = None
    if world > 1:
        comm = make_comm(lk, R, peer=not args.nccl_merge)
        idx.attach_comm(comm, rank * ROWS_PER_GPU)

    K, W = args.steps, args.warmup
    queries = make_queries(K + W, 2002)  # identical on every rank: the query is broadcast by construction
    rq = idx.queries(queries)

    # ---- device-resident throughput: K launches queued back to back
    launches0 = idx.stats()
    ms = timed_scans(R, idx, rq, W, K, TOPK)
    launches1 = idx.stats()
    scan_launches = launches1["scan_launches"] - launches0["scan_launches"]
    aux_launches = launches1["aux_launches"] - launches0["aux_launches"]

    # ---- end to end: one synchronous lk_search per query, host buffers in and out
    E = min(K, 256)
    for i in range(min(W, 8)):
        idx.search_one(queries[i], TOPK)
    R.barrier(idx)
    t0 = time.perf_counter()
    for i in range(E):
        last = idx.search_one(queries[W + i], TOPK)
    e2e_s = time.perf_counter() - t0
    last = [a.copy() for a in last]
    R.barrier(idx)
    e2e_s = R.max_over_ranks(e2e_s)

    # ---- the queued and the synchronous path agree; several timed queries equal the oracle's lists
    ids_r, _, isc_r, _ = rq.fetch(0, W + K, TOPK)
    assert np.array_equal(ids_r[W + E - 1], last[0][0]) and np.array_equal(isc_r[W + E - 1], last[2][0]), "queued != synchronous result"
    picks = sorted({W, W + 1, W + K // 2, W + K - 1})
    parity = oracle_check(lk, R, idx, rank * ROWS_PER_GPU, queries[picks], TOPK, ids_r[picks], isc_r[picks], lk.LK_I8)
    clocks = sampler.stop() if rank == 0 else None

    rq.close()
    idx.close()
    peak, peak_kind = load_peaks()
    others = {}
    if not args.no_extras:
        for spec in (("10,000,000 x 768 int8 over the GPUs of the run, top-10", 10_000_000, 768, lk.LK_I8, 10, 48, 1010, 0),
                     ("16,000,000 x 1,024 int8 over the GPUs of the run, top-50; 512 queries also as one batch",
                      16_000_000, 1024, lk.LK_I8, 50, 32, 1005, 512),
                     ("2,000,000 x 768 int8 over the GPUs of the run, top-100; 4,096 queries also as one batch",
                      2_000_000, 768, lk.LK_I8, 100, 16, 1003, 4096),
                     ("100,000 x 512 float32 over the GPUs of the run, top-10", 100_000, 512, lk.LK_F32, 10, 64, 1001, 0)):
            name, out = other_workload(lk, R, comm, spec[0], spec[1], spec[2], spec[3], spec[4], spec[5], spec[6], peak,
                                       batch=spec[7])
            others[name] = out

    if rank == 0:
        per_launch_s = ms * 1e-3 / K
        algo_bytes = ROWS_PER_GPU * DIM
        achieved = algo_bytes / per_launch_s / 1e9
        line = {
            "metric": METRIC,
            "value": world * K / (ms * 1e-3), "unit": "queries/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8", "data": "synthetic",
            "config": {"workload": WORKLOAD,
                       "rows_per_gpu": ROWS_PER_GPU, "global_rows": ROWS_PER_GPU * world, "dim": DIM, "k": TOPK,
                       "global_queries_per_s": K / (ms * 1e-3),
                       "l2": "shard is 768 MB, larger than the 126 MB L2: every step streams from HBM",
                       "merge": "none" if world == 1 else (
                           "NCCL all-gather of per-shard top-10 + merge kernel per query" if args.nccl_merge else
                           "inside the scan kernel: each shard's top-10 stored into every rank's inbox over NVLink "
                           "(peer memory); queued scans merge three queries behind, synchronous calls at once")},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": f"of {peak_kind}", "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH,
                         "traffic_unit": "bytes per launch", "traffic_source": "constant: one ncu capture of this kernel on "
                         "this workload (1 GPU), not measured in this run", "algorithmic_bytes": algo_bytes,
                         "note": "achieved = rows x 768 B / (timed region / K): launch gaps"
                                 + (", exchange and merge" if world > 1 else "") + " are inside the denominator"},
            "e2e": {"value": world * E / e2e_s, "unit": "queries/s", "steps": E,
                    "h2d_bytes_per_step": DIM, "d2h_bytes_per_step": (TOPK * 16 + 4 + 15) // 16 * 16,
                    "global_queries_per_s": E / e2e_s, "ms_per_query": e2e_s / E * 1e3},
            "gpu_launches": int(scan_launches + aux_launches),
            "parity": parity,
            "clocks": clocks,
        }
        if others:
            line["other_workloads"] = others
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline_leg()
        print(json.dumps(line), flush=True)
    if comm is not None:
        comm.close()
    R.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1024)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extras", action="store_true", help="skip the other workloads (10M x 768, 16M x 1024, 100k x 512)")
    ap.add_argument("--nccl-merge", action="store_true",
                    help="N>1: merge through ncclAllGather + a merge kernel instead of the in-kernel peer exchange")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
