"""GPU, 2 ranks (one process per GPU): the sharded search over NCCL gives the same
result as one index holding every row.  Skipped when fewer than 2 GPUs are visible."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys
sys.path.insert(0, os.environ["LK_ROOT"])
import numpy as np
import torch
import torch.distributed as dist
from loki_b200 import _lib as lk
from loki_b200 import sharding as S
from tests.synth import clustered_rows, gaussian_rows

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
n, dim, k = 20011, 768, 50
rows = clustered_rows(n, dim, 5)
queries = gaussian_rows(5, dim, 6)
uid = [lk.Comm.unique_id() if rank == 0 else None]
dist.broadcast_object_list(uid, src=0)
comm = lk.Comm(world, rank, rank, uid[0])
out = {}
for mode in ("nccl", "peer"):
    if mode == "peer":  # switch the same communicator to the in-kernel exchange over peer memory
        handles = [None] * world
        dist.all_gather_object(handles, comm.peer_export())
        comm.peer_attach(handles)
    for name, store in (("i8", lk.LK_I8), ("f32", lk.LK_F32)):
        base, cnt = S.shard_bounds(n, world)[rank]
        idx = lk.DeviceIndex(dim, store, device=rank)
        idx.append(rows[base:base + cnt])
        idx.attach_comm(comm, base)
        ids, scores, iscores, counts = idx.search(queries, k)
        rq = idx.queries(queries)
        rq.enqueue(0, 5, k)
        ids2, scores2, iscores2, counts2 = rq.fetch(0, 5, k)
        assert np.array_equal(ids, ids2) and np.array_equal(scores, scores2) and np.array_equal(iscores, iscores2)
        out[f"{mode}_{name}_ids"], out[f"{mode}_{name}_scores"], out[f"{mode}_{name}_iscores"] = ids, scores, iscores
        # a batch: int8 runs as one tensor-core product per shard + one all-gather, float32 as queued scans
        qb = gaussian_rows(70, dim, 8)
        bi, bs, bisc, _ = idx.search(qb, k)
        out[f"{mode}_{name}_batch_ids"], out[f"{mode}_{name}_batch_scores"], out[f"{mode}_{name}_batch_iscores"] = bi, bs, bisc
        if mode == "peer":  # k above the peer path's limit falls back to the all-gather
            big = idx.search(queries[:1], 300)
            out[f"big_{name}_ids"] = big[0]
        rq.close(); idx.close()
# duplicate detection split over the ranks: every rank ends up with the complete sorted list
from tests.synth import phash_set
h = phash_set(60000, 21, max_flips=9)
for r in (6, 9):
    out[f"ham{r}_pairs"], cnt = comm.hamming_pairs(h, r)
    out[f"ham{r}_total"] = np.int64(cnt)
np.savez(os.path.join(os.environ["LK_OUT"], f"rank{rank}.npz"), **out)
dist.barrier()
comm.close()
dist.destroy_process_group()
'''


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_sharded_search_over_nccl_equals_single_index(lk, tmp_path):
    if lk.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from tests.synth import clustered_rows, gaussian_rows
    world = 2
    port = _free_port()
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), LK_ROOT=ROOT, LK_OUT=str(tmp_path), NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=600)[0] for p in procs]
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o[-3000:]
    n, dim, k = 20011, 768, 50
    rows = clustered_rows(n, dim, 5)
    queries = gaussian_rows(5, dim, 6)
    got = [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]
    for name, store in (("i8", lk.LK_I8), ("f32", lk.LK_F32)):
        idx = lk.DeviceIndex(dim, store)
        idx.append(rows)
        ids, scores, iscores, _ = idx.search(queries, k)
        big = idx.search(queries[:1], 300)[0]
        idx.set_batch_mode(False)
        bids, bscores, biscores, _ = idx.search(gaussian_rows(70, dim, 8), k)
        for g in got:
            for mode in ("nccl", "peer"):
                assert np.array_equal(g[f"{mode}_{name}_ids"], ids), (mode, name)
                assert np.array_equal(g[f"{mode}_{name}_scores"], scores), (mode, name)
                assert np.array_equal(g[f"{mode}_{name}_iscores"], iscores), (mode, name)
                assert np.array_equal(g[f"{mode}_{name}_batch_ids"], bids), (mode, name, "batch")
                assert np.array_equal(g[f"{mode}_{name}_batch_scores"], bscores), (mode, name, "batch")
                assert np.array_equal(g[f"{mode}_{name}_batch_iscores"], biscores), (mode, name, "batch")
            assert np.array_equal(g[f"big_{name}_ids"], big), name
    from tests.synth import phash_set
    h = phash_set(60000, 21, max_flips=9)
    for r in (6, 9):
        pairs, total = lk.hamming_pairs(h, r)
        for g in got:
            assert int(g[f"ham{r}_total"]) == total
            assert np.array_equal(g[f"ham{r}_pairs"], pairs)


TIMEOUT_WORKER = r'''
import os, sys, time
sys.path.insert(0, os.environ["LK_ROOT"])
import numpy as np
import torch
import torch.distributed as dist
from loki_b200 import _lib as lk
from tests.synth import gaussian_rows

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
uid = [lk.Comm.unique_id() if rank == 0 else None]
dist.broadcast_object_list(uid, src=0)
comm = lk.Comm(world, rank, rank, uid[0])
handles = [None] * world
dist.all_gather_object(handles, comm.peer_export())
comm.peer_attach(handles)
idx = lk.DeviceIndex(64, lk.LK_I8, device=rank)
idx.append(gaussian_rows(5000, 64, 10 + rank))
idx.attach_comm(comm, 5000 * rank)
q = gaussian_rows(1, 64, 3)
ids, _, _, counts = idx.search(q, 10)          # both ranks take part: a normal exchange
assert counts[0] == 10
dist.barrier()
status = "no error"
if rank == 0:
    t0 = time.time()
    try:                                        # rank 1 stays away: the wait inside the kernel must run out
        idx.search(q, 10)
    except lk.LokiError as e:
        status = f"{e.status} after {time.time() - t0:.1f} s"
else:
    time.sleep(6.0)                             # between steps, nothing of this rank in flight
with open(os.path.join(os.environ["LK_OUT"], f"timeout{rank}.txt"), "w") as f:
    f.write(status)
dist.barrier()
idx.close()
comm.close()
dist.destroy_process_group()
'''


def test_a_rank_that_stays_away_ends_the_exchange_with_a_timeout(lk, tmp_path):
    """The exchange inside the scan kernel waits for the other shards' lists with a 2-second
    bound; when a rank does not take part the call returns LK_ETIMEOUT and the GPU stays usable."""
    if lk.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world = 2
    port = _free_port()
    script = tmp_path / "timeout_worker.py"
    script.write_text(TIMEOUT_WORKER)
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), LK_ROOT=ROOT, LK_OUT=str(tmp_path), NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=300)[0] for p in procs]
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o[-3000:]
    status = (tmp_path / "timeout0.txt").read_text()
    assert status.startswith(f"{lk.LK_ETIMEOUT} after"), status
    assert float(status.split()[2]) < 5.0
    # the device that timed out still answers
    idx = lk.DeviceIndex(64, lk.LK_I8)
    from tests.synth import gaussian_rows
    idx.append(gaussian_rows(1000, 64, 1))
    assert idx.search(gaussian_rows(1, 64, 2), 5)[3][0] == 5
