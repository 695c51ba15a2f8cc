// Multi-GPU exchange: row shards on every GPU, one all-gather of each shard's
// ranked candidates per search, merged on every rank.  NCCL is loaded at run time
// (dlopen) the first time a communicator is created, so a single-GPU user of the
// library never needs it.
#pragma once
#include <cuda_runtime.h>

#include <functional>

#include "../../include/lokiscan.h"

namespace lk {

struct ResultArena;

// After the per-shard scans of queries [q_first, q_first+nq) are enqueued on idx's
// stream with results in `res`: gather all ranks' [nq][k] ranked keys (+ float
// scores for int8), merge per query and overwrite those queries' entries of `res`
// with the global result (ids are global row numbers).
int comm_gather_merge(lk_comm *c, lk_index *idx, const ResultArena &res, int q_first, int nq, int k);

// Device table for the in-kernel exchange over peer memory, or nullptr when it has not
// been set up (or k is above its limit): the caller then uses comm_gather_merge.
struct PeerTable;
const PeerTable *comm_peer_table(lk_comm *c, int k);
// Sequence number of the next sharded query (every rank issues the same queries in the same order).
unsigned int comm_next_seq(lk_comm *c);

// All-gather of `bytes` from every rank into recv (rank order), enqueued on `st`; returns an lk_status.
using HamAllGather = std::function<int(const void *send, void *recv, size_t bytes, cudaStream_t st)>;
// Hamming all-pairs (hamming.cu): share `part` of `parts`; with `gather`, parts = world and the
// shares are united and sorted on every rank.
int ham_pairs(const uint64_t *hashes, int64_t n, int radius, int part, int parts, int device, uint32_t *pairs, int64_t cap,
              int64_t *count, const HamAllGather *gather);

}  // namespace lk
