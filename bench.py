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
                 per-shard top-10 lists are merged after an NCCL all-gather; the value
                 counts 1M-row shard scans per second over all GPUs (= global
                 queries/s x N), ``config.global_queries_per_s`` is the plain figure.
* ``e2e``        the same through ``lk_search`` with host buffers, one synchronous
                 call per query (host prep, H2D, scan, [all-gather, merge,] D2H).
* ``roofline``   algorithmic bytes of one launch (rows x 768) / average launch time.
* ``cpu_baseline`` the reference's algorithm (float32 rows, float64 accumulate,
                 per-core row chunks, serial heap top-k) restated in C (the Go
                 toolchain is absent), timed on this host's cores on a row sample.
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
# dram__bytes_read.sum + dram__bytes_write.sum of one k_scan_bulk launch on this workload,
# from the ncu capture summarised in profiles/k_scan_bulk_int8_1Mx768_k10.md
NCU_TRAFFIC_BYTES_PER_LAUNCH = 771.8e6
CHUNK = 62_500  # rows generated per torch call (192 MB of float32)


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

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
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
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
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def make_queries(n: int, seed: int) -> np.ndarray:
    return np.random.default_rng(seed).standard_normal((n, DIM), dtype=np.float32)


def cpu_reference_scan(steps: int, warmup: int, sample_rows: int = 100_000):
    """The reference's scan (float32 rows, one heap slice per row, float64 accumulate,
    NumCPU contiguous chunks, serial min-heap) on `sample_rows` rows; returns
    (queries/s scaled to ROWS_PER_GPU rows, cores, description, seconds per query on the sample)."""
    import ctypes as C

    import oracle as O

    cores = os.cpu_count() or 1
    rng = np.random.default_rng(1002)
    rows = O.normalize_rows(rng.standard_normal((sample_rows, DIM), dtype=np.float32))
    # one separately allocated vector per row, like the reference's [][]float32
    # (media-server/embedindex/embedindex.go:124)
    keep = [rows[i].copy() for i in range(sample_rows)]
    rowp = (C.c_void_p * sample_rows)(*[a.ctypes.data for a in keep])
    rowp_arr = np.frombuffer(rowp, dtype=np.uint64)
    qs = make_queries(steps + warmup, 2002)
    t_used = []
    for i in range(steps + warmup):
        q = O.normalize(qs[i])
        t0 = time.perf_counter()
        sc = O.scan_f32(rows, q, workers=cores, rowp=rowp_arr)
        h = O.topk_heap(sc, TOPK)
        hits = sorted(((-float(sc[j]), int(j)) for j in h))
        dt = time.perf_counter() - t0
        if i >= warmup:
            t_used.append(dt)
        assert len(hits) == TOPK
    per_q = sum(t_used) / len(t_used)
    scaled_qps = 1.0 / (per_q * ROWS_PER_GPU / sample_rows)
    desc = (f"{len(t_used)} queries over the first {sample_rows} rows x {DIM} float32 (reference's storage), "
            f"time scaled linearly to {ROWS_PER_GPU} rows; C restatement of the Go scan, {cores} threads")
    return scaled_qps, cores, desc, per_q


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = min(args.steps, 16)
    qps, cores, desc, per_q = cpu_reference_scan(steps, min(args.warmup, 3))
    line = {
        "impl": "reference", "metric": "queries/sec, top-10 scan of 1M x 768 rows per GPU shard",
        "value": qps, "unit": "queries/s", "n_gpus": args.gpus, "steps": steps, "warmup": min(args.warmup, 3),
        "ms_per_step": per_q * 1e3 * ROWS_PER_GPU / 100_000, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": "1,000,000 x 768 rows, single queries, top-10 (reference stores float32, accumulates float64)",
                   "note": "CPU path, no GPU used; unit = scans of one 1M-row shard per second, the same unit as the GPU arm at any N"},
        "cpu_baseline": {"value": qps, "unit": "queries/s", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": qps, "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args):
    import torch
    import torch.distributed as dist

    from loki_b200 import _lib as lk

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one process per GPU)")
    assert lk.device_count() > local, "bench.py needs a CUDA device (there is no CPU path)"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    # ---- build this rank's shard on the device (synthetic N(0,1), normalised + quantised by the library)
    idx = lk.DeviceIndex(DIM, lk.LK_I8, device=local)
    idx.reserve(ROWS_PER_GPU)
    gen = torch.Generator(device=dev)
    for c in range(ROWS_PER_GPU // CHUNK):
        gen.manual_seed(1002 * 1_000_003 + rank * 4096 + c)
        block = torch.randn((CHUNK, DIM), generator=gen, device=dev, dtype=torch.float32)
        idx.upsert_device(c * CHUNK, CHUNK, block.data_ptr())
        del block
    torch.cuda.synchronize()
    assert len(idx) == ROWS_PER_GPU

    comm = None
    if world > 1:
        uid = [lk.Comm.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        comm = lk.Comm(world, rank, local, uid[0])
        if not args.nccl_merge:  # exchange the per-shard top-k inside the scan kernel, over peer memory
            handles = [None] * world
            dist.all_gather_object(handles, comm.peer_export())
            comm.peer_attach(handles)
        idx.attach_comm(comm, rank * ROWS_PER_GPU)

    K, W = args.steps, args.warmup
    queries = make_queries(K + W, 2002)  # identical on every rank: the query is broadcast by construction
    rq = idx.queries(queries)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        idx.sync()

    # ---- device-resident throughput: K launches queued back to back
    rq.enqueue(0, W, TOPK)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = idx.stats()
    idx.timer_start()
    rq.enqueue(W, K, TOPK)
    ms = idx.timer_stop()
    barrier()
    launches1 = idx.stats()
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    scan_launches = launches1["scan_launches"] - launches0["scan_launches"]
    aux_launches = launches1["aux_launches"] - launches0["aux_launches"]

    # ---- end to end: one synchronous lk_search per query, host buffers in and out
    E = min(K, 256)
    for i in range(min(W, 8)):
        idx.search(queries[i], TOPK)
    barrier()
    t0 = time.perf_counter()
    last = None
    for i in range(E):
        last = idx.search(queries[W + i], TOPK)
    barrier()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())

    # ---- sanity: resident and synchronous paths agree on the last query
    ids_r, _, isc_r, _ = rq.fetch(W + E - 1, 1, TOPK)
    assert np.array_equal(ids_r[0], last[0][0]) and np.array_equal(isc_r[0], last[2][0]), "resident != e2e result"

    if rank == 0:
        peak, peak_kind = load_peaks()
        per_launch_s = ms * 1e-3 / K
        algo_bytes = ROWS_PER_GPU * DIM
        achieved = algo_bytes / per_launch_s / 1e9
        line = {
            "metric": "queries/sec, int8 top-10 scan of 1M x 768 rows per GPU shard",
            "value": world * K / (ms * 1e-3), "unit": "queries/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8", "data": "synthetic",
            "config": {"workload": "1,000,000 x 768 int8 rows per GPU (per-row scale after L2 normalisation), "
                                   "single queries issued one at a time, int32 dot, top-10",
                       "rows_per_gpu": ROWS_PER_GPU, "global_rows": ROWS_PER_GPU * world, "dim": DIM, "k": TOPK,
                       "global_queries_per_s": K / (ms * 1e-3),
                       "l2": "shard is 768 MB, larger than the 126 MB L2: every step streams from HBM",
                       "merge": "none" if world == 1 else (
                           "NCCL all-gather of per-shard top-10 + merge kernel per query" if args.nccl_merge else
                           "inside the scan kernel: each shard's top-10 stored into every rank's inbox over NVLink "
                           "(peer memory), merged by the last CTA")},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": f"of {peak_kind}", "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH,
                         "traffic_unit": "bytes per launch (ncu, 1 GPU)", "algorithmic_bytes": algo_bytes,
                         "note": "achieved = rows x 768 B / (timed region / K): launch gaps"
                                 + (", exchange and merge" if world > 1 else "") + " are inside the denominator"},
            "e2e": {"value": world * E / e2e_s, "unit": "queries/s", "steps": E,
                    "h2d_bytes_per_step": DIM, "d2h_bytes_per_step": (TOPK * 16 + 4 + 15) // 16 * 16,
                    "global_queries_per_s": E / e2e_s, "ms_per_query": e2e_s / E * 1e3},
            "gpu_launches": int(scan_launches + aux_launches),
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu:
            qps, cores, desc, _ = cpu_reference_scan(8, 2)
            line["cpu_baseline"] = {"value": qps, "unit": "queries/s", "cores": cores, "kind": "port", "sample": desc}
        print(json.dumps(line), flush=True)
    rq.close()
    idx.close()
    if comm is not None:
        comm.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1024)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
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
