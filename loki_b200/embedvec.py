"""The BLOB codec of ``media-server/embedvec`` for callers that feed this library.

Vectors are stored by the server as little-endian float32 BLOBs
(``media-server/embedvec/embedvec.go:12-31``; tables ``media_embedding.vector`` and
``face.vector``).  ``decode_rows`` turns a batch of BLOBs into the row matrix that
``VectorIndex.AddBatch`` / ``lk_index_upsert_f32`` take.  Scoring itself never runs
here: it runs on the GPU.
"""
from __future__ import annotations

from typing import Iterable

import numpy as np


def Encode(v) -> bytes:
    """media-server/embedvec/embedvec.go:13-19."""
    return np.ascontiguousarray(v, dtype=np.float32).astype("<f4").tobytes()


def Decode(b: bytes) -> np.ndarray:
    """media-server/embedvec/embedvec.go:22-31: rejects lengths that are not a multiple of 4."""
    if len(b) % 4 != 0:
        raise ValueError(f"embedvec: byte length {len(b)} is not a multiple of 4")
    return np.frombuffer(b, dtype="<f4").astype(np.float32)


def decode_rows(blobs: Iterable[bytes], dim: int) -> np.ndarray:
    """Decode BLOBs into an (n, dim) float32 matrix; a BLOB of another length becomes
    a zero row (it can never match: Cosine returns 0 on a length mismatch)."""
    blobs = list(blobs)
    out = np.zeros((len(blobs), dim), np.float32)
    for i, b in enumerate(blobs):
        if len(b) == dim * 4:
            out[i] = np.frombuffer(b, dtype="<f4")
    return out


def ProjectPCA3(vecs, workers: int | None = None, device: int = 0):
    """media-server/embedvec/pca.go:22-128: -> (coords, variance): one [x, y, z] per input,
    uniformly scaled into [-1, 1]^3, and the variance fraction of each component.

    `workers` is the reference's runtime.NumCPU(): it fixes the order in which the reference
    adds its per-chunk partial sums, and with it the last bits of the result (default: this
    machine's CPU count, like the reference running here)."""
    import os

    from . import _lib
    rows = [np.asarray(v, np.float32) for v in vecs]
    if len(rows) == 0 or rows[0].size == 0:
        return np.zeros((len(rows), 3), np.float32), np.zeros(3, np.float64)
    x = np.stack(rows)
    return _lib.pca3(x, workers if workers else (os.cpu_count() or 1), device)
