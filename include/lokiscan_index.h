/*
 * Path-keyed exact index with the interface of the reference's Go VectorIndex
 * (media-server/embedindex/embedindex.go:93-117), for hosts that are not Go.
 *
 * A Go server keeps its own `paths []string` + `slot map[string]int` and binds the
 * slot-level API in lokiscan.h directly.  This header exposes the same bookkeeping
 * implemented in C++ inside the library (path table, slot map, swap-remove delete,
 * allow-set resolution, tie order by path), so that C, C++ or Python callers get
 * New / NewCentered / Add / Delete / Search* / Len with the reference's argument
 * meaning and error behaviour.  All scoring runs on the GPU through lokiscan.h.
 *
 * Threading: like the reference (media-server/embedindex/embedindex.go:90-92), one
 * call at a time per index.
 */
#ifndef LOKISCAN_INDEX_H
#define LOKISCAN_INDEX_H

#include "lokiscan.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct lkx_index lkx_index;
typedef struct lkx_hits lkx_hits;

/* embedindex.New() (centered = 0) / NewCentered() (centered = 1):
 * media-server/embedindex/embedindex.go:144-153.  The vector length is fixed by the
 * first Add.  store is an lk_dtype; centered needs LK_F32. */
LK_API int lkx_new(int centered, int store, int device, lkx_index **out);
LK_API int lkx_free(lkx_index *x);

/* Add (media-server/embedindex/embedindex.go:176-194): insert or replace the vector of
 * `path`; raw model output is fine, it is L2-normalised on the way in.  A vector
 * whose length differs from the index's is stored as a zero row: like the
 * reference's length check in Cosine (media-server/embedvec/embedvec.go:114-116) it
 * then scores 0 against every query. */
LK_API int lkx_add(lkx_index *x, const char *path, const float *vec, int len);
/* n Adds in order (the bulk build of media-server/tasks/embed_task.go:189-210);
 * rows is n*len floats.  New paths are uploaded in large batches. */
LK_API int lkx_add_batch(lkx_index *x, const char *const *paths, const float *rows, int64_t n, int len);
/* Delete (media-server/embedindex/embedindex.go:196-217): no-op when absent. */
LK_API int lkx_delete(lkx_index *x, const char *path);
/* Len (media-server/embedindex/embedindex.go:219). */
LK_API int64_t lkx_len(const lkx_index *x);

/* On-disk cache of the built index: lk_index_save's file plus `<path>.paths` with the paths in
 * slot order.  Replaces BuildIndexFromDB's rebuild at start (media-server/tasks/embed_task.go:189-210)
 * whenever the caller's tag (model + row count) still matches. */
LK_API int lkx_save(lkx_index *x, const char *path, uint64_t tag);
LK_API int lkx_load(const char *path, uint64_t tag, int device, lkx_index **out);

/* Search / SearchFiltered / SearchScored (media-server/embedindex/embedindex.go:308-328).
 * has_allow = 0 is Go's nil allow set (no restriction); has_allow = 1 restricts to
 * the n_allow paths in `allow` (unknown paths are skipped; an empty or fully
 * unknown set yields no hits).  *out is NULL when the reference would return nil,
 * else a hit list ordered by score descending, path ascending on equal scores
 * (media-server/embedindex/embedindex.go:483-490). */
LK_API int lkx_search_scored(lkx_index *x, const float *query, int len, int k, int has_allow,
                             const char *const *allow, int64_t n_allow, int scoring, lkx_hits **out);

/* SearchShared / SearchSharedScored (media-server/embedindex/embedindex.go:334-394).
 * pos[i] has pos_len[i] floats; n_posw is 0 (Go's nil: equal weights) or the number
 * of weights given.  Returns LK_EINVAL with the reference's message for its
 * constructor errors (no positives, weight/term count mismatch, length mismatch,
 * non-positive weight: media-server/embedvec/shared.go:62-70, :89-99, :107-109). */
LK_API int lkx_search_shared_scored(lkx_index *x, const float *const *pos, const int *pos_len, int npos,
                                    const float *posw, int n_posw, const float *const *neg,
                                    const int *neg_len, int nneg, const float *negw, int n_negw, int k,
                                    int has_allow, const char *const *allow, int64_t n_allow, int scoring,
                                    lkx_hits **out);

LK_API int64_t lkx_hits_len(const lkx_hits *h);
LK_API const char *lkx_hits_path(const lkx_hits *h, int64_t i);
LK_API float lkx_hits_score(const lkx_hits *h, int64_t i);
LK_API void lkx_hits_free(lkx_hits *h);

/* The slot-level handle behind a path-keyed index (NULL before the first Add). */
LK_API lk_index *lkx_device_index(lkx_index *x);
/* Slot of a path, or -1. */
LK_API int64_t lkx_slot_of(const lkx_index *x, const char *path);

#ifdef __cplusplus
}
#endif
#endif /* LOKISCAN_INDEX_H */
