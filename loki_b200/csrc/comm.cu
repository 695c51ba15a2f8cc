// NCCL plumbing for the sharded index (see comm.hpp).
#include <dlfcn.h>
#include <nccl.h>  // types and enums only; every function is resolved with dlsym

#include <mutex>
#include <string>
#include <vector>

#include "comm.hpp"
#include "index_internal.cuh"
#include "scan.cuh"

namespace lk {

struct NcclApi {
    void *handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    std::string why;
};

static NcclApi *nccl_api() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        // If the process already holds an NCCL (e.g. the one bundled with PyTorch),
        // dlopen by soname returns that same copy.
        for (const char *name : {"libnccl.so.2", "libnccl.so"}) {
            api.handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
            if (api.handle) break;
        }
        if (!api.handle) {
            api.why = std::string("cannot load libnccl: ") + dlerror();
            return;
        }
#define LK_SYM(field, sym)                                              \
    api.field = reinterpret_cast<decltype(api.field)>(dlsym(api.handle, sym)); \
    if (!api.field) { api.why = std::string("libnccl lacks ") + sym; return; }
        LK_SYM(GetUniqueId, "ncclGetUniqueId")
        LK_SYM(CommInitRank, "ncclCommInitRank")
        LK_SYM(CommDestroy, "ncclCommDestroy")
        LK_SYM(AllGather, "ncclAllGather")
        LK_SYM(GroupStart, "ncclGroupStart")
        LK_SYM(GroupEnd, "ncclGroupEnd")
        LK_SYM(GetErrorString, "ncclGetErrorString")
#undef LK_SYM
    });
    return api.why.empty() ? &api : nullptr;
}

static int nccl_unavailable() {
    static NcclApi *probe = nullptr;
    (void)probe;
    return fail(LK_ENCCL, "NCCL is not available: libnccl.so.2 could not be loaded or lacks a needed symbol");
}

#define LK_NCCL(api, expr)                                                                      \
    do {                                                                                        \
        ncclResult_t _r = (expr);                                                               \
        if (_r != ncclSuccess) return fail(LK_ENCCL, std::string(#expr) + ": " + (api)->GetErrorString(_r)); \
    } while (0)

}  // namespace lk

using namespace lk;

struct lk_comm {
    int world = 1, rank = 0, device = 0;
    ncclComm_t comm = nullptr;
    long long *d_bases = nullptr;  // [world] shard base of every rank (device)
    bool bases_valid = false;
    // direct exchange over peer memory (optional, see lk_comm_peer_export / _attach)
    PeerInbox *inbox = nullptr;               // this rank's inbox (cudaMalloc)
    PeerInbox *peer_inbox[kPeerMaxWorld] = {};  // every rank's inbox as mapped here
    PeerTable *d_table = nullptr;             // device copy handed to the kernels
    bool peer_ready = false;
    unsigned int seq = 0;                     // sharded queries issued so far (same on every rank)
};

namespace lk {

int comm_gather_merge(lk_comm *c, lk_index *idx, const ResultArena &res, int q_first, int nq, int k) {
    NcclApi *api = nccl_api();
    if (!api) return nccl_unavailable();
    const size_t e = (size_t)nq * k;
    const bool i8 = idx->type == SCAN_I8;
    // receive: keys [world][nq][k] | scores [world][nq][k] | merge scratch [nq][world*k]
    const size_t keys_bytes = (size_t)c->world * e * 8;
    const size_t pay_bytes = i8 ? (size_t)c->world * e * 4 : 0;
    const size_t pay_off = keys_bytes;
    const size_t scr_off = (size_t)round_up((int64_t)(pay_off + pay_bytes), 16);
    LK_TRY(idx->gather.reserve(scr_off + keys_bytes));
    unsigned char *g = (unsigned char *)idx->gather.p;
    LK_NCCL(api, api->GroupStart());
    const size_t o = (size_t)q_first * k;
    LK_NCCL(api, api->AllGather(res.d_keys() + o, g, e, ncclUint64, c->comm, idx->stream));
    if (i8) LK_NCCL(api, api->AllGather(res.d_scores() + o, g + pay_off, e, ncclFloat32, c->comm, idx->stream));
    LK_NCCL(api, api->GroupEnd());
    MergeArgs m;
    m.keys = (const unsigned long long *)g;
    m.payload = i8 ? (const float *)(g + pay_off) : nullptr;
    m.qscales = nullptr;
    m.scales = nullptr;
    m.scratch = (unsigned long long *)(g + scr_off);
    m.list_base = c->d_bases;
    m.lists = c->world;
    m.nq = nq;
    m.k = k;
    m.type = idx->type;
    m.out_ids = res.d_ids() + o;
    m.out_scores = res.d_scores() + o;
    m.out_iscores = res.d_iscores() + o;
    m.out_count = res.d_counts() + q_first;
    m.out_keys = nullptr;
    LK_TRY(merge_launch(m, idx->stream));
    idx->aux_launches++;
    return 0;
}

const PeerTable *comm_peer_table(lk_comm *c, int k) {
    return (c && c->peer_ready && c->d_table && k <= kPeerMaxK) ? c->d_table : nullptr;
}
unsigned int comm_next_seq(lk_comm *c) { return c->seq++; }

}  // namespace lk

extern "C" {

int lk_comm_unique_id(void *out128) {
    if (!out128) return fail(LK_EINVAL, "lk_comm_unique_id: out is NULL");
    NcclApi *api = nccl_api();
    if (!api) return nccl_unavailable();
    ncclUniqueId id;
    LK_NCCL(api, api->GetUniqueId(&id));
    memcpy(out128, id.internal, NCCL_UNIQUE_ID_BYTES);
    return LK_OK;
}

int lk_comm_create(int world, int rank, int device, const void *id128, lk_comm **out) {
    if (!out || !id128 || world < 1 || rank < 0 || rank >= world) return fail(LK_EINVAL, "lk_comm_create: bad argument");
    *out = nullptr;
    NcclApi *api = nccl_api();
    if (!api) return nccl_unavailable();
    LK_CUDA(cudaSetDevice(device));
    lk_comm *c = new (std::nothrow) lk_comm();
    if (!c) return fail(LK_ENOMEM, "lk_comm_create: out of host memory");
    c->world = world;
    c->rank = rank;
    c->device = device;
    ncclUniqueId id;
    memcpy(id.internal, id128, NCCL_UNIQUE_ID_BYTES);
    ncclResult_t r = api->CommInitRank(&c->comm, world, id, rank);
    if (r != ncclSuccess) {
        delete c;
        return fail(LK_ENCCL, std::string("ncclCommInitRank: ") + api->GetErrorString(r));
    }
    cudaError_t e = cudaMalloc((void **)&c->d_bases, sizeof(long long) * (size_t)world);
    if (e != cudaSuccess) {
        api->CommDestroy(c->comm);
        delete c;
        return fail(LK_ENOMEM, std::string("lk_comm_create: ") + cudaGetErrorString(e));
    }
    *out = c;
    return LK_OK;
}

int lk_comm_peer_export(lk_comm *c, void *out64) {
    if (!c || !out64) return fail(LK_EINVAL, "lk_comm_peer_export: bad argument");
    if (c->world > kPeerMaxWorld) return fail(LK_ERANGE, "lk_comm_peer_export: more than 16 ranks");
    LK_CUDA(cudaSetDevice(c->device));
    if (!c->inbox) {
        LK_CUDA(cudaMalloc((void **)&c->inbox, sizeof(PeerInbox)));
        LK_CUDA(cudaMemset(c->inbox, 0, sizeof(PeerInbox)));
    }
    cudaIpcMemHandle_t h;
    LK_CUDA(cudaIpcGetMemHandle(&h, c->inbox));
    static_assert(sizeof(h) == LK_PEER_HANDLE_BYTES, "CUDA IPC handle size");
    memcpy(out64, &h, sizeof(h));
    return LK_OK;
}

int lk_comm_peer_attach(lk_comm *c, const void *handles) {
    if (!c || !handles) return fail(LK_EINVAL, "lk_comm_peer_attach: bad argument");
    if (!c->inbox) return fail(LK_EINVAL, "lk_comm_peer_attach: call lk_comm_peer_export first");
    LK_CUDA(cudaSetDevice(c->device));
    for (int r = 0; r < c->world; ++r) {
        if (r == c->rank) {
            c->peer_inbox[r] = c->inbox;
            continue;
        }
        cudaIpcMemHandle_t h;
        memcpy(&h, (const char *)handles + (size_t)r * LK_PEER_HANDLE_BYTES, sizeof(h));
        void *p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return fail(LK_ECUDA, std::string("cudaIpcOpenMemHandle(rank ") + std::to_string(r) + "): " + cudaGetErrorString(e));
        }
        c->peer_inbox[r] = static_cast<PeerInbox *>(p);
    }
    if (!c->d_table) LK_CUDA(cudaMalloc((void **)&c->d_table, sizeof(PeerTable)));
    c->peer_ready = true;
    return LK_OK;
}

int lk_hamming_pairs_sharded(lk_comm *c, const uint64_t *hashes, int64_t n, int radius, uint32_t *pairs, int64_t cap,
                             int64_t *count) {
    if (!c || n < 0 || (n > 0 && !hashes) || radius < 0 || radius > 64 || cap < 0 || (cap > 0 && !pairs) || !count)
        return fail(LK_EINVAL, "lk_hamming_pairs_sharded: bad argument");
    if (n > 0xffffffffll) return fail(LK_ERANGE, "lk_hamming_pairs_sharded: more than 2^32 hashes");
    *count = 0;
    if (n < 2) return LK_OK;
    NcclApi *api = nccl_api();
    if (!api) return nccl_unavailable();
    const HamAllGather gather = [api, c](const void *send, void *recv, size_t bytes, cudaStream_t st) -> int {
        LK_NCCL(api, api->AllGather(send, recv, bytes, ncclUint8, c->comm, st));
        return LK_OK;
    };
    return ham_pairs(hashes, n, radius, c->rank, c->world, c->device, pairs, cap, count, &gather);
}

int lk_comm_destroy(lk_comm *c) {
    if (!c) return LK_OK;
    NcclApi *api = nccl_api();
    cudaSetDevice(c->device);
    for (int r = 0; r < c->world && r < kPeerMaxWorld; ++r)
        if (r != c->rank && c->peer_inbox[r]) cudaIpcCloseMemHandle(c->peer_inbox[r]);
    if (c->inbox) cudaFree(c->inbox);
    if (c->d_table) cudaFree(c->d_table);
    if (c->d_bases) cudaFree(c->d_bases);
    if (api && c->comm) api->CommDestroy(c->comm);
    delete c;
    return LK_OK;
}

int lk_index_attach_comm(lk_index *idx, lk_comm *c, int64_t shard_base) {
    if (!idx || shard_base < 0) return fail(LK_EINVAL, "lk_index_attach_comm: bad argument");
    if (!c) {
        idx->comm = nullptr;
        idx->shard_base = shard_base;
        return LK_OK;
    }
    if (c->device != idx->device) return fail(LK_EINVAL, "lk_index_attach_comm: communicator and index are on different devices");
    NcclApi *api = nccl_api();
    if (!api) return nccl_unavailable();
    LK_CUDA(cudaSetDevice(idx->device));
    // The scan emits shard-local ids; the merge adds each rank's base.  Share the bases once.
    long long *d_mine = nullptr;
    LK_CUDA(cudaMalloc((void **)&d_mine, sizeof(long long)));
    const long long base = shard_base;
    LK_CUDA(cudaMemcpyAsync(d_mine, &base, sizeof(long long), cudaMemcpyHostToDevice, idx->stream));
    ncclResult_t r = api->AllGather(d_mine, c->d_bases, 1, ncclUint64, c->comm, idx->stream);
    cudaError_t e = cudaStreamSynchronize(idx->stream);
    cudaFree(d_mine);
    if (r != ncclSuccess) return fail(LK_ENCCL, std::string("ncclAllGather(bases): ") + api->GetErrorString(r));
    if (e != cudaSuccess) return fail(LK_ECUDA, std::string("lk_index_attach_comm: ") + cudaGetErrorString(e));
    c->bases_valid = true;
    if (c->peer_ready) {
        PeerTable t = {};
        t.world = c->world;
        t.rank = c->rank;
        t.base = shard_base;
        for (int r2 = 0; r2 < c->world; ++r2) t.inbox[r2] = c->peer_inbox[r2];
        LK_CUDA(cudaMemcpy(c->d_table, &t, sizeof(t), cudaMemcpyHostToDevice));
    }
    idx->comm = c;
    idx->shard_base = 0;  // ids stay local until the merge re-bases them
    return LK_OK;
}

}  // extern "C"
