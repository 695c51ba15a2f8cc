// Multi-GPU exchange: row shards on every GPU, one all-gather of each shard's
// ranked candidates per search, merged on every rank.  NCCL is loaded at run time
// (dlopen) the first time a communicator is created, so a single-GPU user of the
// library never needs it.
#pragma once
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

}  // namespace lk
