"""The search functions of the reference's service layer, over an installed index or by brute force.

Mirrors the part of ``media-server/tasks`` that sits directly on the scan: ``SearchByVector``,
``searchByVectorWithin``, ``searchByVectorCrossModal``, ``searchByVectorScored``
(embed_task.go:222-272), ``searchSharedWithin`` (embed_task.go:320-386), ``SimilarByPath``
(embed_task.go:394-403), ``SearchFacesByVector`` / ``searchFacesByVectorWithin``
(face_search.go:190-249).  In the reference each of them asks the installed index first and, when
there is none for the model (or, for faces, when an allow set is given), loops over every stored
vector on one thread with ``embedvec.CosineSim``.  Here both branches run on the GPU: the index
branch is :mod:`loki_b200.embedindex`, the fallback is ``lk_cosine_sim_topk`` (the same CosineSim
over the raw rows, fused with the top-k).

The database stays with the caller: where the reference takes ``db`` and loads rows from SQLite,
these functions take the loaded rows (``StoredEmbedding`` / ``Face`` records).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence

import numpy as np

from . import _lib
from . import embedindex
from .embedindex import ScoreDefault, ScorePlain, SharedSpec, VectorIndex


@dataclass
class StoredEmbedding:  # media-server/media/embedding.go: StoredEmbedding{Path, Vec}
    Path: str
    Vec: np.ndarray


@dataclass
class SimilarHit:  # media-server/tasks/embed_task.go: SimilarHit{Path, Score}
    Path: str
    Score: np.float32


@dataclass
class Face:  # the fields of media.Face the search uses
    ID: int
    MediaPath: str
    Vec: np.ndarray
    Model: str = ""


@dataclass
class FaceHit:  # media-server/tasks/face_search.go: FaceHit (id, media path, score)
    FaceID: int
    MediaPath: str
    Score: np.float32


PathSet = Optional[Iterable[str]]  # None = whole library (Go's nil map)


def _rows_by_path(all_rows: Sequence[StoredEmbedding], allow: PathSet):
    """Rows in path order (so that the device's lower-row-first rule among equal scores is the
    reference's path order, sortSimilar, embed_task.go:279-288) and the allowed row numbers."""
    order = sorted(range(len(all_rows)), key=lambda i: all_rows[i].Path)
    paths = [all_rows[i].Path for i in order]
    dim = max((np.asarray(all_rows[i].Vec).size for i in order), default=0)
    rows = np.zeros((len(order), max(dim, 1)), np.float32)
    same_len = np.ones(len(order), bool)
    for r, i in enumerate(order):
        v = np.asarray(all_rows[i].Vec, np.float32).reshape(-1)
        rows[r, :v.size] = v
        same_len[r] = v.size == dim
    slots = None
    if allow is not None:
        allowed = set(allow)
        slots = np.asarray([r for r, p in enumerate(paths) if p in allowed], np.int32)
    return paths, rows, slots, same_len


def searchByVectorScored(index: Optional[VectorIndex], all_rows: Sequence[StoredEmbedding], query, limit: int,
                         allow: PathSet, s: int, device: int = 0) -> List[SimilarHit]:
    """embed_task.go:241-273.  `index` is the index installed for the model, or None."""
    if index is not None:
        raw = index.SearchScored(query, limit, allow, s)
        return [SimilarHit(h.Path, h.Score) for h in (raw or [])]
    q = np.asarray(query, np.float32).reshape(-1)
    paths, rows, slots, same_len = _rows_by_path(all_rows, allow)
    n_cand = len(paths) if slots is None else slots.size
    if n_cand == 0:
        return []
    if rows.shape[1] != q.size or not same_len.all():
        # CosineSim is 0 for vectors of another length (embedvec.go:128-130): give such rows a zero vector
        fixed = np.zeros((rows.shape[0], q.size), np.float32)
        if rows.shape[1] == q.size:
            fixed[same_len] = rows[same_len]
        rows = fixed
    k = n_cand if limit <= 0 else min(limit, n_cand)
    ids, scores = _lib.cosine_sim_topk(rows, q, k, allow_slots=slots, device=device)
    return [SimilarHit(paths[int(i)], np.float32(sc)) for i, sc in zip(ids, scores)]


def searchByVectorWithin(index, all_rows, query, limit: int, allow: PathSet, device: int = 0):
    """embed_task.go:228-230"""
    return searchByVectorScored(index, all_rows, query, limit, allow, ScoreDefault, device)


def searchByVectorCrossModal(index, all_rows, query, limit: int, allow: PathSet, device: int = 0):
    """embed_task.go:237-239"""
    return searchByVectorScored(index, all_rows, query, limit, allow, ScorePlain, device)


def SearchByVector(index, all_rows, query, limit: int, device: int = 0):
    """embed_task.go:222-224"""
    return searchByVectorWithin(index, all_rows, query, limit, None, device)


def SimilarByPath(index, all_rows: Sequence[StoredEmbedding], path: str, limit: int, device: int = 0):
    """embed_task.go:394-403: the query item itself is included (cosine 1.0 ranks it first)."""
    for e in all_rows:
        if e.Path == path:
            return SearchByVector(index, all_rows, e.Vec, limit, device)
    raise KeyError(f"no embedding for {path!r}")


def searchSharedWithin(index: Optional[VectorIndex], all_rows: Sequence[StoredEmbedding], spec: SharedSpec, limit: int,
                       allow: PathSet, s: int, device: int = 0) -> List[SimilarHit]:
    """embed_task.go:320-386.  Without an installed index the reference normalises every stored
    vector, centres when the library has at least MinCenterCount of them and the query is not
    cross-modal, and scores with the shared query: that is a (centered) index built on the spot."""
    if index is not None:
        raw = index.SearchSharedScored(spec, limit, allow, s)
        return [SimilarHit(h.Path, h.Score) for h in (raw or [])]
    if not all_rows:
        if not spec.Pos:
            raise ValueError("embedvec: shared query has no positive terms")
        return []
    tmp = embedindex.NewCentered(device) if s != ScorePlain else embedindex.New(device=device)
    try:
        tmp.AddBatch([e.Path for e in all_rows], np.stack([np.asarray(e.Vec, np.float32) for e in all_rows]))
        k = len(all_rows) if limit <= 0 else limit
        raw = tmp.SearchSharedScored(spec, k, allow, s)
        return [SimilarHit(h.Path, h.Score) for h in (raw or [])]
    finally:
        tmp.close()


def searchFacesByVectorWithin(face_index: Optional[VectorIndex], faces: Sequence[Face], query, limit: int,
                              allow: PathSet, device: int = 0) -> List[FaceHit]:
    """face_search.go:198-249.  The face index is keyed by face id and cannot see media paths, so a
    search restricted to media paths, like a search without an index, scores every stored face."""
    by_id: Dict[int, Face] = {f.ID: f for f in faces}
    if allow is None and face_index is not None:
        hits = []
        for h in face_index.Search(query, limit) or []:
            try:
                fid = int(h.Path)
            except ValueError:
                continue  # foreign key in the index; skipped like the reference does
            if fid in by_id:
                hits.append(FaceHit(fid, by_id[fid].MediaPath, h.Score))
        return hits
    q = np.asarray(query, np.float32).reshape(-1)
    order = sorted(range(len(faces)), key=lambda i: faces[i].ID)
    if not order:
        return []
    rows = np.zeros((len(order), q.size), np.float32)
    for r, i in enumerate(order):
        v = np.asarray(faces[i].Vec, np.float32).reshape(-1)
        if v.size == q.size:
            rows[r] = v
    slots = None
    if allow is not None:
        allowed = set(allow)
        slots = np.asarray([r for r, i in enumerate(order) if faces[i].MediaPath in allowed], np.int32)
        if slots.size == 0:
            return []
    n_cand = len(order) if slots is None else slots.size
    k = n_cand if limit <= 0 else min(limit, n_cand)
    ids, scores = _lib.cosine_sim_topk(rows, q, k, allow_slots=slots, device=device)
    return [FaceHit(faces[order[int(i)]].ID, faces[order[int(i)]].MediaPath, np.float32(sc)) for i, sc in zip(ids, scores)]


def SearchFacesByVector(face_index, faces, query, limit: int, device: int = 0):
    """face_search.go:190-192"""
    return searchFacesByVectorWithin(face_index, faces, query, limit, None, device)
