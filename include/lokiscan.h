/*
 * lokiscan: B200-native exact vector scan behind the API of Lowkey Media Server's
 * media-server/embedindex + media-server/embedvec packages.
 *
 * The reference is pure Go with no FFI, so this header is the boundary a cgo
 * binding would call.  Strings never cross it: the caller keeps the path <-> slot
 * map (media-server/embedindex/embedindex.go:122-126) and this library sees slot
 * numbers only.  Every function returns an lk_status (0 = success) unless noted;
 * lk_last_error() gives the message for the calling thread's last failure.
 *
 * Threading contract (same as media-server/embedindex/embedindex.go:90-92): calls
 * on one handle must be serialised by the caller; distinct handles may be used
 * concurrently.  All pointers are host pointers borrowed for the duration of the
 * call unless a parameter is documented as a device pointer.
 *
 * There is no CPU fallback: every entry point that computes needs a CUDA device
 * and fails with LK_ECUDA without one.
 */
#ifndef LOKISCAN_H
#define LOKISCAN_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LK_API __attribute__((visibility("default")))

typedef enum {
    LK_OK = 0,
    LK_EINVAL = 1,   /* bad argument */
    LK_EDIM = 2,     /* vector length does not match the index */
    LK_ENOMEM = 3,   /* host or device allocation failed */
    LK_ECUDA = 4,    /* CUDA runtime error (message in lk_last_error) */
    LK_ENCCL = 5,    /* NCCL error or NCCL not loadable */
    LK_ETIMEOUT = 6, /* a bounded device-side or host-side wait ran out */
    LK_ERANGE = 7    /* size beyond a documented limit */
} lk_status;

/* Storage type of the corpus rows (what the scan streams from HBM). */
typedef enum {
    LK_F32 = 0, /* L2-normalised float32: the reference's own representation */
    LK_F16 = 1, /* L2-normalised, rounded to IEEE half */
    LK_I8 = 2   /* L2-normalised, per-row symmetric int8 codes + float32 scale */
} lk_dtype;

/* Scoring mode of a query: media-server/embedindex/embedindex.go:64-77. */
typedef enum {
    LK_SCORE_DEFAULT = 0, /* centered cosine on a centered index, else plain */
    LK_SCORE_PLAIN = 1    /* always plain cosine (cross-modal queries) */
} lk_scoring;

#define LK_MIN_CENTER_COUNT 64 /* media-server/embedindex/embedindex.go:55 */
#define LK_MAX_DIM 8192
#define LK_SHARED_MAX_TERMS 32 /* positives + basis + negatives of one shared query */

typedef struct lk_index lk_index;
typedef struct lk_queries lk_queries;
typedef struct lk_comm lk_comm;

/* ---- library ------------------------------------------------------------ */

/* Message of the calling thread's most recent failed call ("" if none). */
LK_API const char *lk_last_error(void);
/* Number of CUDA devices visible (0 when there is no driver or no GPU). */
LK_API int lk_device_count(void);
/* Library version, e.g. "0.1.0". */
LK_API const char *lk_version(void);

/* ---- index life cycle --------------------------------------------------- */

/* Replaces embedindex.New() / NewCentered() (media-server/embedindex/embedindex.go:144-153).
 * dim: vector length (1..LK_MAX_DIM).  store: lk_dtype.  centered != 0 enables
 * mean-centering (float32 storage only).  device: CUDA ordinal. */
LK_API int lk_index_create(int dim, int store, int centered, int device, lk_index **out);
LK_API int lk_index_destroy(lk_index *idx);
/* Pre-size device storage for n rows (growth is otherwise geometric). */
LK_API int lk_index_reserve(lk_index *idx, int64_t n);
/* Replaces Len() (media-server/embedindex/embedindex.go:219). */
LK_API int64_t lk_index_len(const lk_index *idx);
LK_API int lk_index_dim(const lk_index *idx);
/* Storage type (LK_F32 / LK_F16 / LK_I8) and whether the index was created centered. */
LK_API int lk_index_kind(const lk_index *idx, int *store, int *centered);

/* Replaces Add (media-server/embedindex/embedindex.go:176-194) for n rows at once:
 * rows[i] (dim floats each, raw model output) is L2-normalised on the device
 * (float64 sum of squares in index order, like embedvec.Normalize,
 * media-server/embedvec/embedvec.go:34-50), converted to the storage type and
 * written to slot first_slot+i.  first_slot <= len; slots below len are
 * overwritten in place, slots from len on are appended.  A centered index keeps
 * its float64 column sum and, once centering is live, its per-row centered norm
 * up to date exactly as Add does. */
LK_API int lk_index_upsert_f32(lk_index *idx, int64_t first_slot, int64_t n, const float *rows);
/* Same, rows being a DEVICE pointer on the index's device (row stride = dim). */
LK_API int lk_index_upsert_f32_device(lk_index *idx, int64_t first_slot, int64_t n,
                                      const float *d_rows);
/* Replaces the storage half of Delete (media-server/embedindex/embedindex.go:196-217):
 * the last row moves into `slot` and the length drops by one.  The caller
 * mirrors the move in its own path table. */
LK_API int lk_index_swap_remove(lk_index *idx, int64_t slot);

/* Read back stored rows [first, first+n): `out` receives n*dim elements of the
 * storage type (float, uint16 half bits or int8), padding stripped; `scales`
 * (may be NULL) receives the n int8 scales.  For tests and for callers that
 * need a stored vector (Delete's column-sum bookkeeping is done internally). */
LK_API int lk_index_read_rows(lk_index *idx, int64_t first, int64_t n, void *out, float *scales);

/* Centering state (media-server/embedindex/embedindex.go:127-139): *live is 1 when a
 * mean is in use; mu (dim floats), sum (dim doubles), cnorm (len floats) may
 * each be NULL.  Does not trigger a re-centre. */
LK_API int lk_index_center_state(lk_index *idx, int *live, int64_t *n_centered, double *mu_n2,
                                 float *mu, double *sum, float *cnorm);

/* ---- search ------------------------------------------------------------- */

/* Replaces Search / SearchFiltered / SearchScored
 * (media-server/embedindex/embedindex.go:308-328) for nq independent queries.
 *   queries      nq*dim floats, raw (normalised internally, like the reference)
 *   k            hits wanted per query; k' = min(k, candidates) are returned
 *   scoring      lk_scoring
 *   allow_slots  NULL = every row; else n_allow DISTINCT slot numbers to score
 *                (the resolved allow set, media-server/embedindex/embedindex.go:398-419);
 *                n_allow == 0 returns no hits
 *   out_ids      nq*k slot numbers (plus the shard base when one is set), rank order
 *   out_scores   nq*k float scores (cosine; for LK_I8 the de-quantised dot
 *                int_score * scale_query * scale_row)
 *   out_iscores  NULL or nq*k raw int32 dots (LK_I8 only; zero otherwise)
 *   out_counts   nq hit counts
 * Rank order is score descending, slot ascending on equal scores (for LK_I8 the
 * key is the raw int32 dot).  A centered index re-centres first when it has
 * drifted (media-server/embedindex/embedindex.go:234-268), so this call may mutate.
 * With a communicator attached (lk_index_attach_comm) every rank must call with
 * the same queries and k and receives the merged global result.
 * For k of 256 and more on an unsharded, unfiltered index of 64k+ rows the call scans a
 * sample of the rows first and uses its result as a lower bound for the scan; a query for
 * which that bound lets fewer than k rows through is scanned again without it, so the hits
 * are the exact top k in every case (lk_search_shared does the same). */
LK_API int lk_search(lk_index *idx, const float *queries, int nq, int k, int scoring,
                     const int32_t *allow_slots, int64_t n_allow,
                     int64_t *out_ids, float *out_scores, int32_t *out_iscores,
                     int32_t *out_counts);

/* Replaces SearchShared / SearchSharedScored
 * (media-server/embedindex/embedindex.go:334-394, media-server/embedvec/shared.go:61-220).
 * pos: npos*dim floats, posw: NULL (equal) or npos weights > 0; neg/negw: nneg
 * steer-away terms.  beta/lambda as embedvec.NewSharedQuery (defaults 0.25 / 1.0).
 * float32 storage only.  LK_EINVAL mirrors the reference's constructor errors. */
LK_API int lk_search_shared(lk_index *idx, const float *pos, const float *posw, int npos,
                            const float *neg, const float *negw, int nneg,
                            float beta, float lambda, int k, int scoring,
                            const int32_t *allow_slots, int64_t n_allow,
                            int64_t *out_ids, float *out_scores, int32_t *out_count);

/* Replaces the brute-force loops of the service layer, which run when no index is installed for a
 * model or a face search is restricted to a set of media paths
 * (media-server/tasks/embed_task.go:249-272, media-server/tasks/face_search.go:199-216, :235-248):
 * embedvec.CosineSim (media-server/embedvec/embedvec.go:127-141) of one query against n RAW rows
 * (host memory, n*dim floats, as the database holds them: not normalised), exact top-k.
 * score = float32(dot / (sqrt(|q|^2) * sqrt(|v|^2))) in float64, 0 when either vector is all
 * zero.  allow_slots as in lk_search.  Rank order: score descending, row number ascending on
 * equal scores (pass the rows sorted by path to get the reference's path order among ties).
 * Any k: more than 2,048 hits are selected in passes over the uploaded rows. */
LK_API int lk_cosine_sim_topk(const float *rows, int64_t n, int dim, const float *query, int k,
                              const int32_t *allow_slots, int64_t n_allow, int device,
                              int64_t *out_ids, float *out_scores, int32_t *out_count);

/* On-disk cache of a built index, replacing the rebuild from SQLite BLOBs at every start
 * (media-server/tasks/embed_task.go:189-210: LoadAllEmbeddings, then one Add per row).  The file
 * holds the index as it sits in device memory (normalised or quantised rows, scales, the
 * centering state a search would see) behind a 128-byte header with a checksum.  `tag` is the
 * caller's key, e.g. a hash of model name and row count: lk_index_load refuses a file written
 * under another tag (LK_EINVAL), as it does a truncated, extended or damaged one.  Slot order
 * is preserved; the caller keeps its own path list in the same order. */
LK_API int lk_index_save(lk_index *idx, const char *path, uint64_t tag);
LK_API int lk_index_load(const char *path, uint64_t tag, int device, lk_index **out);

/* How lk_search runs a batch of queries (no allow-list, k <= 256).
 * mode 1 (default): 32 or more queries on an LK_I8 index as one int8 tensor-core matrix
 * product with the top-k fused into its epilogue (on a sharded index: one such product per
 * shard, then ONE all-gather of the shards' nq x k ranked hits and a merge on every rank);
 * 3 or more queries on an unsharded LK_F32 index of 8,192+ rows eight to a pass over the corpus
 * on the float64 tensor-core path.
 * mode 0: consecutive single-query scans.  int8 results are identical.  float32 scores come
 * from the same arithmetic (exact products, float64 accumulation, one rounding) summed in a
 * different order, so hit lists can differ only between rows whose scores tie to the last bits. */
LK_API int lk_index_set_batch_mode(lk_index *idx, int mode);

/* ---- device-resident queries (throughput measurement, pipelined callers) -- */

/* Prepare nq queries (normalise, centre/quantise as the index requires) and keep
 * them on the device. */
LK_API int lk_queries_create(lk_index *idx, const float *queries, int nq, int scoring,
                             lk_queries **out);
LK_API int lk_queries_destroy(lk_queries *q);
/* Enqueue one scan per query [first, first+count) on the index's stream, no host
 * synchronisation; results stay on the device until lk_queries_fetch.  With k of 256 and
 * more on a large index every query is first scanned over a sample of the rows, whose result
 * bounds the real scan from below (the sample scans of up to 64 queries are issued together,
 * ahead of their scans). */
LK_API int lk_search_resident(lk_index *idx, lk_queries *q, int first, int count, int k);
/* Wait for the stream and copy the results of queries [first, first+count) out.  A query
 * whose sampled bound let fewer than k rows through is scanned again here, without the bound,
 * before its result is returned: results are exact either way. */
LK_API int lk_queries_fetch(lk_index *idx, lk_queries *q, int first, int count, int k,
                            int64_t *out_ids, float *out_scores, int32_t *out_iscores,
                            int32_t *out_counts);
/* CUDA-event stopwatch on the index's stream. */
LK_API int lk_timer_start(lk_index *idx);
LK_API int lk_timer_stop(lk_index *idx, float *elapsed_ms);
LK_API int lk_index_sync(lk_index *idx);

/* ---- multi-GPU: row shards + one all-gather of candidates ---------------- */

/* 128-byte NCCL unique id, created on one rank and passed to the others by the caller. */
LK_API int lk_comm_unique_id(void *out128);
LK_API int lk_comm_create(int world, int rank, int device, const void *id128, lk_comm **out);
LK_API int lk_comm_destroy(lk_comm *c);
/* Optional fast path for the GPUs of one box: instead of an NCCL all-gather per search,
 * the scan kernel itself stores each shard's k results into every rank's inbox over
 * NVLink (peer memory) and merges as soon as all have landed.  Every rank calls
 * lk_comm_peer_export, the caller passes the LK_PEER_HANDLE_BYTES of each rank to all
 * ranks (rank order), every rank calls lk_comm_peer_attach, then lk_index_attach_comm.
 * One process per GPU (CUDA IPC).  Used for k <= 128; larger k takes the NCCL path.
 * One sharded search at a time per communicator; a rank that does not deliver within
 * 2 s makes the others return LK_ETIMEOUT. */
#define LK_PEER_HANDLE_BYTES 64
LK_API int lk_comm_peer_export(lk_comm *c, void *out_handle);
LK_API int lk_comm_peer_attach(lk_comm *c, const void *handles /* world x LK_PEER_HANDLE_BYTES */);
/* This index holds global rows [shard_base, shard_base+len). */
LK_API int lk_index_attach_comm(lk_index *idx, lk_comm *c, int64_t shard_base);
LK_API int lk_index_set_shard_base(lk_index *idx, int64_t shard_base);

/* ---- 64-bit Hamming (no counterpart in the reference) --------------------- */

/* All pairs i<j of hashes[0..n) with popcount(a^b) <= radius, written to `pairs`
 * as (i,j) uint32 couples in lexicographic order, at most cap couples;
 * *count = total found (may exceed cap; which cap pairs are kept is then unspecified).
 * part/parts split the work across callers (0/1 = everything): the shares are disjoint and
 * their union is the complete result for any parts. */
LK_API int lk_hamming_pairs(const uint64_t *hashes, int64_t n, int radius, int part, int parts,
                            int device, uint32_t *pairs, int64_t cap, int64_t *count);
/* The same search spread over the GPUs of a communicator (every rank passes the same hashes:
 * 2,000,000 of them are 16 MB): rank r tests share r of world, the per-GPU pair lists are
 * all-gathered (NCCL: counts, then lists padded to the longest) and sorted on every GPU, and
 * every rank receives the complete ordered list.  Structure of the reference's tiled all-pairs
 * sweep with per-worker lists merged in order (media-server/tasks/face_cluster.go:1189-1285). */
LK_API int lk_hamming_pairs_sharded(lk_comm *c, const uint64_t *hashes, int64_t n, int radius,
                                    uint32_t *pairs, int64_t cap, int64_t *count);
/* One hash against n: ids (ascending) and distances of those within radius. */
LK_API int lk_hamming_scan(const uint64_t *hashes, int64_t n, uint64_t query, int radius,
                           int device, uint32_t *out_ids, int32_t *out_dist, int64_t cap,
                           int64_t *count);

/* ---- scan without any allocation (no counterpart in the reference) ---------- */

/* For callers that are not allowed to allocate device memory while they run: a server
 * whose GPU budget is handed out once at start-up, a request path that cannot afford
 * the device-wide stall of cudaMalloc / cudaFree, a plug-in inside another framework's
 * memory arena.  One int8 top-k scan (same kernel, same ranking as lk_search on an
 * LK_I8 index); every buffer is a DEVICE pointer owned by the caller, and the kernel's
 * scratch is a fixed array inside the library image, LK_PREALLOC_SCRATCH_BYTES per GPU
 * that loads the library, held until the process exits.  The call makes no cudaMalloc,
 * cudaFree or other allocating call; it enqueues on `stream` (a cudaStream_t, NULL =
 * default stream) and returns without waiting.  The caller's current device is the same after
 * the call as before it.
 *   d_codes   n rows of int8 codes, ld bytes apart (ld a multiple of 16, padding zero),
 *             16-byte aligned: the layout lk_index_read_rows describes, kept on device
 *   d_scales  n per-row float scales (score = int dot * query_scale * row scale)
 *   d_query   ld bytes: the query's int8 codes, zero padded; query_scale its scale
 *   k         1..LK_PREALLOC_MAX_K; larger k is refused with LK_ERANGE
 *   outputs   k ids (row numbers, -1 padded), k float scores, k raw int32 dots (may be
 *             NULL), one count (-1 if a bounded wait inside the kernel ran out)
 * The first call on a device looks up the scratch array's address; make that call
 * once per device before starting any stream capture.  All calls on a device share the
 * one array, which keeps the previous call's contents (the call clears the few words
 * that must start at zero): calls that overlap on the GPU, e.g. on two streams, race. */
#define LK_PREALLOC_MAX_K 128
#define LK_PREALLOC_MAX_CTAS 1024
#define LK_PREALLOC_SCRATCH_BYTES (256 + LK_PREALLOC_MAX_K * 8 + LK_PREALLOC_MAX_CTAS * LK_PREALLOC_MAX_K * 8)
LK_API int lk_scan_i8_prealloc(int device, const int8_t *d_codes, int64_t n, int dim, int64_t ld,
                               const float *d_scales, const int8_t *d_query, float query_scale, int k,
                               int64_t *d_out_ids, float *d_out_scores, int32_t *d_out_iscores,
                               int32_t *d_out_count, void *stream);

/* ---- face-clustering neighbour prescreen ------------------------------------ */

/* Replaces prescreenCandidates (media-server/tasks/face_cluster.go:1189-1285): for every
 * vector i (n unit vectors of dim floats, row-major, in processing order) the earlier
 * vectors j < i with dotf(v_i, v_j) >= threshold (media-server/tasks/face_cluster.go:908-925:
 * float32, four interleaved accumulators), ascending.
 *   near      n x LK_PRESCREEN_MAX int32: row i holds count[i] neighbour positions
 *   count     n int32
 *   overflow  n bytes: 1 = more than LK_PRESCREEN_MAX neighbours, list dropped (count 0),
 *             exactly the reference's overflow rule */
#define LK_PRESCREEN_MAX 256
LK_API int lk_prescreen_pairs(const float *vecs, int64_t n, int dim, float threshold, int device,
                              int32_t *near, int32_t *count, uint8_t *overflow);

/* ---- face-clustering candidate x seed scores ---------------------------------- */

/* Replaces the dot products of scoreAgainstSeeds (media-server/tasks/face_cluster.go:1315-1462):
 * for every candidate (n_cand unit vectors of dim floats, row-major) the seeds (n_seeds unit
 * vectors) whose float32 dot with it is >= min_score, in ascending seed order, with the
 * scores.  The caller passes min_score = threshold - corroborationSlack (:1417) and runs the
 * reference's decision logic over the lists.
 * Arithmetic follows the reference bit for bit: candidates are scored four at a time with
 * dot4 (:939-967), the last 1-3 candidates of each worker chunk with dotf (:908-925).
 *   chunk      candidates per worker chunk of the reference, (n + workers - 1) / workers
 *              (:1349-1350); 0 = all candidates in one chunk
 *   row_start  n_cand + 1 offsets: candidate i's pairs are out_seed/out_score[row_start[i] .. row_start[i+1])
 *   cap        pairs out_seed / out_score can hold
 *   out_total  pairs that reach the floor; when it exceeds cap nothing is written, the
 *              call returns LK_ERANGE and can be repeated with room for out_total pairs */
LK_API int lk_seed_scores(const float *cands, int64_t n_cand, const float *seeds, int64_t n_seeds, int dim,
                          float min_score, int64_t chunk, int device, int64_t *row_start, int32_t *out_seed,
                          float *out_score, int64_t cap, int64_t *out_total);

/* ---- PCA projection for the embedding-space view ----------------------------- */

/* Replaces embedvec.ProjectPCA3 (media-server/embedvec/pca.go:22-128): n vectors of dim floats
 * (row-major) -> coords n x 3 float32, uniformly scaled into [-1, 1]^3, and the fraction of the
 * total variance each component explains (zeros for components that do not exist).
 *   workers   runtime.NumCPU() of the machine the reference would run on (its row chunks'
 *             partial sums are merged in chunk order, pca.go:137-177): coords are bit-identical
 *             to the reference's for that count.  The variance fractions agree to ~1e-13
 *             relative (the reference sums the total variance as one long chain). */
LK_API int lk_pca3(const float *vecs, int64_t n, int dim, int workers, int device, float *coords, double *variance);

/* ---- statistics ----------------------------------------------------------- */

typedef struct {
    int64_t len;
    int64_t capacity;
    int64_t bytes_resident;    /* device bytes held by this index */
    int64_t scan_launches;     /* scan kernels launched so far */
    int64_t aux_launches;      /* other kernels launched so far */
    float last_search_ms;      /* wall time of the last lk_search call */
    int grid;                  /* CTAs per scan launch */
    int sm_count;
} lk_stats_t;
LK_API int lk_stats(lk_index *idx, lk_stats_t *out);

#ifdef __cplusplus
}
#endif
#endif /* LOKISCAN_H */
