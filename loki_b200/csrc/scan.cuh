// Host-visible interface of the scoring-scan kernels (scan_kernels.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace lk {

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
    unsigned long long *part;   // scratch [grid][k]: per-CTA candidate lists
    unsigned int *ticket;       // scratch: CTAs finished so far (self-resetting)
    unsigned long long *out_keys;  // [k] ranked keys, zero padded
    long long *out_ids;         // [k] shard_base + slot, -1 padded
    float *out_scores;          // [k]
    int *out_iscores;           // [k] or nullptr (int8: raw dots)
    int *out_count;             // hits written
    const float *scales;        // int8: per-slot scale
    float qscale;               // int8: scale of the query
    long long shard_base;
};

enum ScanType { SCAN_F32 = 0, SCAN_F16 = 1, SCAN_I8 = 2 };

// Bytes of prepared-query data per 16-byte corpus chunk as it sits in global memory.
int scan_query_bytes(int type, long long ld);
// Lane-group width the launcher will use for this row width.
int scan_group_width(int chunks);
// CTAs that fit on the device at once for this configuration (grid size to launch).
int scan_resident_grid(int type, int chunks, int k, int device, int *err);
int scan_launch(int type, const ScanArgs &a, int grid, cudaStream_t stream);

// Merge, for each of nq queries, `lists` ranked key lists of k entries each (global
// memory, zero padded) into one ranked result of k entries at out_*[q*k];
// used after the all-gather of per-shard candidates.
struct MergeArgs {
    const unsigned long long *keys;  // [lists][nq][k] ranked descending, ids local to each list
    const float *payload;            // [lists][nq][k] finished float score of each int8 hit, else nullptr
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
};
int merge_launch(const MergeArgs &a, cudaStream_t stream);

}  // namespace lk
