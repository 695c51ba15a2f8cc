// Host-visible interface of the scoring-scan kernels (scan_kernels.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace lk {

// Direct exchange of per-shard results between the GPUs of one box (peer memory over
// NVLink): every rank owns an inbox that all ranks can write.
constexpr int kPeerSlots = 8;    // queries in flight before an inbox slot is reused (>= 2 * kPeerDefer + 2)
constexpr int kPeerDefer = 3;    // queued scans: a launch merges the query issued this many launches earlier
constexpr int kPeerMaxWorld = 16;
constexpr int kPeerMaxK = 128;   // larger k goes through the NCCL all-gather
struct PeerInbox {
    unsigned int flags[kPeerSlots][kPeerMaxWorld];                    // tag of the list present (peer_tag)
    unsigned int pad[64];
    unsigned long long keys[kPeerSlots][kPeerMaxWorld][kPeerMaxK];    // ranked keys, GLOBAL row ids
    float payload[kPeerSlots][kPeerMaxWorld][kPeerMaxK];              // finished float score of int8 hits
};
struct PeerTable {                    // lives in device memory of each rank
    int world, rank;
    long long base;                   // first global row of this rank's shard
    PeerInbox *inbox[kPeerMaxWorld];  // every rank's inbox as mapped into this process
};

constexpr int kInlineQueryBytes = 3072;  // int8 rows up to 3072 B, float32 up to 768 elements

// One scan = one query against n candidate rows, fused with top-k selection.
struct ScanArgs {
    const unsigned char *rows;  // corpus base (device)
    long long ld;               // row stride in bytes, a multiple of 16
    int chunks;                 // 16-byte chunks per row (= ld / 16)
    long long n;                // number of candidates (rows, or entries of slots)
    const int *slots;           // nullptr = rows 0..n-1; else n slot numbers to score
    const unsigned char *query; // prepared query (device): int8 codes, or float32, padded to the row width
    const float *cnorm;         // nullptr = plain cosine; else per-slot centered norm
    float cq;                   // <qc, mu> of the centered query
    int k;                      // 1..kMaxK
    const unsigned long long *bound;  // nullptr, or exclusive upper bound on accepted keys
    // nullptr, or an exclusive LOWER bound: keys at or below *floor are not candidates.  For large k the
    // caller first scans a sample of the rows and takes a key that, with a wide margin, at least k rows
    // of the whole corpus exceed: each CTA then keeps a few dozen candidates instead of its own best k.
    // Should fewer than k hits come out after all, the caller repeats the scan without a floor.
    const unsigned long long *floor;
    // 1 when the launch that wrote *floor may still be running as this one starts (it is the one just
    // before on the stream): the kernel then waits for it before its first row.  0 when a launch in
    // plain stream order lies between the two (a batch's sample scans are all issued first).
    int floor_wait;
    unsigned long long *part;   // scratch [grid][k]: per-CTA candidate lists
    int *part_cnt;              // scratch [grid]: keys in each of them (nullptr: not recorded; the merge then searches)
    unsigned int *ticket;       // scratch: CTAs finished so far (self-resetting)
    unsigned int *next_batch;   // scratch: next 32-row batch to hand out (TMA-staged kernel; self-resetting)
    int *error;                 // scratch: raised by a CTA whose bounded wait ran out (self-resetting)
    unsigned long long *out_keys;  // [k] ranked keys, zero padded
    long long *out_ids;         // [k] shard_base + slot, -1 padded
    float *out_scores;          // [k]
    int *out_iscores;           // [k] or nullptr (int8: raw dots)
    int *out_count;             // hits written; -1 when a bounded device-side wait ran out
    const float *scales;        // int8: per-slot scale
    float qscale;               // int8: scale of the query
    long long shard_base;
    const PeerTable *peer;      // nullptr, or: exchange the result with the other shards inside the kernel
    unsigned int seq;           // sequence number of this query, the same on every rank
    // Which query this launch merges once its own list is published.  defer == 0: its own, i.e. it
    // waits until every shard's list for this query has arrived (a caller that needs the answer
    // now).  defer == kPeerDefer (queued scans): the query issued that many launches earlier, whose
    // outputs are d_out_* (nullptr: none, the first launches of a batch); a rank then stalls only
    // when another rank is more than kPeerDefer queries behind, and peer_drain_launch merges the
    // last queries of the batch.
    int defer;
    long long *d_out_ids;
    float *d_out_scores;
    int *d_out_iscores;
    int *d_out_count;
    // Low-latency single query: outputs may point into mapped pinned host memory; after they
    // are written the kernel releases *done_flag = done_value for a host that is polling it.
    unsigned int *done_flag;    // nullptr = none
    unsigned int done_value;
    // query == nullptr: the prepared query travels in the launch parameters instead
    alignas(16) unsigned char query_inline[kInlineQueryBytes];
};

enum ScanType { SCAN_F32 = 0, SCAN_F16 = 1, SCAN_I8 = 2 };

// Bytes of one prepared query as it sits in global memory.
int scan_query_bytes(int type, long long ld);
// Lane-group width used for rows of this many 16-byte chunks.
int scan_group_width(int chunks);

// Launch configuration of both scan kernels for one (storage type, row width, k).
struct ScanPlan {
    // register-staged kernel (any input, allow-lists)
    int g = 32;            // lane-group width
    int grid = 1;          // CTAs resident at once
    size_t smem = 0;
    // TMA-staged kernel (whole contiguous rows)
    bool bulk_ok = false;
    int bulk_g = 32;
    int bulk_grid = 1;     // one CTA per SM
    int slab_bytes = 0;    // bytes of each row held per stage
    int n_slabs = 1;       // stages per 32-row batch
    int fixed_chunks = 0;  // > 0: slab width (in 16-byte chunks) has a compile-time kernel
    size_t bulk_smem = 0;
    int bulk_per_sm = 1;   // CTAs of the TMA-staged kernel one SM can hold (narrow rows: several)
    // TMA-staged kernel for wide rows (ld a multiple of 512 B, >= 1 KB): whole-row batches
    bool wide_ok = false;
    int wide_nj = 0;       // 512-byte units per row
    int wide_rows = 0;     // rows per batch
    int wide_warps = 0;
    int wide_run = 1;      // consecutive batches handed out per counter access
    size_t wide_smem = 0;
    int wide_per_sm = 1;
};
int scan_plan(int type, int chunks, int k, int device, ScanPlan *plan);
int scan_max_grid(const ScanPlan &plan);   // CTAs to size the per-CTA list scratch for
// Consecutive launches of the TMA-staged kernels overlap at their edges (programmatic dependent
// launch) and rotate over kScanOverlap batch counters and error words.  One SM holds one CTA of
// the usual shapes, which limits the overlap to two launches by itself; where several CTAs fit
// on an SM (narrow rows) the launch that reuses slot 0 is issued with plain stream order
// (`overlap` false), so that never more than kScanOverlap launches are in flight.
constexpr int kScanOverlap = 4;
bool scan_may_overlap(const ScanPlan &plan, long long launch_index);
int scan_launch(int type, const ScanArgs &a, const ScanPlan &plan, cudaStream_t stream, bool overlap = true);

// Brute-force CosineSim scan over raw float rows (scan_kernels.cu).  With a.part == nullptr
// only *grid_out is computed (to size the per-CTA list scratch: grid x k keys).
int cosine_sim_launch(const ScanArgs &a, int dim, double q_n2, int sm_count, cudaStream_t stream, int *grid_out);

// After a batch of queued sharded scans: merge queries seq_first .. seq_first+count-1 (count <=
// kPeerDefer) from this rank's inbox into out_*[i*k], one CTA, plain stream order.
struct DrainArgs {
    const PeerTable *peer;
    unsigned int seq_first;
    int count, k, type;
    long long *out_ids;
    float *out_scores;
    int *out_iscores;
    int *out_count;
};
int peer_drain_launch(const DrainArgs &a, cudaStream_t stream);

// Merge, for each of nq queries, `lists` ranked key lists of k entries each (global
// memory, zero padded) into one ranked result of k entries at out_*[q*k];
// used after the all-gather of per-shard candidates.
struct MergeArgs {
    const unsigned long long *keys;  // [lists][nq][k] ranked descending, ids local to each list
    const float *payload;            // [lists][nq][k] finished float score of each int8 hit, else nullptr
    const float *qscales;            // int8 without payload: per-query scale ...
    const float *scales;             // ... and per-row scale (rows local to this GPU), to finish the float score here
    unsigned long long *scratch;     // [nq][lists*k] work space
    const long long *list_base;      // [lists] ascending id offset of each list (device)
    int lists;
    int nq;                          // one CTA per query
    int k;
    int type;                        // ScanType: how to decode the score bits
    long long *out_ids;
    float *out_scores;
    int *out_iscores;
    int *out_count;
    unsigned long long *out_keys;    // nullptr, or [nq][k]: the ranked keys themselves (what a further merge takes)
};
int merge_launch(const MergeArgs &a, cudaStream_t stream);

}  // namespace lk
