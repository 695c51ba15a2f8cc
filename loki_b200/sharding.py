"""Row sharding of one corpus over the GPUs of a box, and the rule by which per-shard
candidate lists merge into the global result.

The corpus is split into contiguous row ranges, one per rank, exactly as the
reference splits rows over CPU workers (``parallelChunks``,
media-server/embedindex/embedindex.go:460-479), one level up.  Every rank scans its
own shard and produces a ranked list of k 64-bit keys with shard-local row numbers;
the lists are all-gathered (k x 8 bytes per rank and query) and merged on every rank.
The exact global top-k is always contained in the union of the per-shard top-k lists.

The functions here state the key format and the merge rule in numpy.  The GPU does
the same in ``k_merge_lists`` (csrc/scan_kernels.cu); this host-side statement is what
the multi-process CPU tests exercise over gloo, and what a caller can use to merge
lists gathered by its own transport.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import numpy as np


def shard_bounds(n_total: int, world: int) -> List[Tuple[int, int]]:
    """(base, count) of every rank: contiguous, sizes differing by at most one chunk."""
    chunk = (n_total + world - 1) // world if world > 0 else 0
    out = []
    for r in range(world):
        lo = min(r * chunk, n_total)
        hi = min(lo + chunk, n_total)
        out.append((lo, hi - lo))
    return out


def pack_keys_i32(scores: np.ndarray, ids: np.ndarray) -> np.ndarray:
    """key = (score ^ 0x80000000) << 32 | ~id : larger key = higher score, then lower id."""
    o = (scores.astype(np.int64) + (1 << 31)).astype(np.uint64)
    return (o << np.uint64(32)) | (~ids.astype(np.uint32)).astype(np.uint64)


def pack_keys_f32(scores: np.ndarray, ids: np.ndarray) -> np.ndarray:
    s = scores.astype(np.float32) + np.float32(0.0)  # -0 -> +0
    b = s.view(np.uint32)
    o = np.where(b & np.uint32(0x80000000), ~b, b | np.uint32(0x80000000)).astype(np.uint64)
    return (o << np.uint64(32)) | (~ids.astype(np.uint32)).astype(np.uint64)


def key_ids(keys: np.ndarray) -> np.ndarray:
    return (~(keys & np.uint64(0xFFFFFFFF)).astype(np.uint32)).astype(np.int64)


def key_scores_i32(keys: np.ndarray) -> np.ndarray:
    return ((keys >> np.uint64(32)).astype(np.int64) - (1 << 31)).astype(np.int32)


def key_scores_f32(keys: np.ndarray) -> np.ndarray:
    o = (keys >> np.uint64(32)).astype(np.uint32)
    b = np.where(o & np.uint32(0x80000000), o & np.uint32(0x7FFFFFFF), ~o).astype(np.uint32)
    return b.view(np.float32)


def merge_ranked(lists: Sequence[np.ndarray], bases: Sequence[int], k: int) -> np.ndarray:
    """Merge per-shard ranked key lists (0 = empty entry, ids shard-local) into the global
    top-k keys with GLOBAL ids.  The low word holds ~id, so subtracting a shard's base
    from a key adds it to the id."""
    allk = []
    for keys, base in zip(lists, bases):
        keys = np.asarray(keys, np.uint64)
        keys = keys[keys != 0]
        allk.append(keys - np.uint64(base))
    allk = np.concatenate(allk) if allk else np.zeros(0, np.uint64)
    return np.sort(allk)[::-1][:k]
