// lk_scan_i8_prealloc: the int8 top-k scan for callers that must not allocate.
//
// Some hosts of this library may not create or release device memory once they are
// running: a media server that hands its whole GPU budget to its pools at start-up
// and treats any later cudaMalloc as a bug; a request path where cudaMalloc or
// cudaFree would stall every other stream of the process while the driver updates
// its tables; a plug-in that lives inside another framework's memory arena.  The
// regular entry points grow their scratch on demand, so they are off limits there.
//
// This entry point takes every input and output as a device pointer owned by the
// caller and keeps the kernel's own scratch (one ranked list of k keys per CTA, the
// merged key list, and a few control words) in a fixed array that is part of the
// library image.  Loading the library on a GPU therefore costs
// LK_PREALLOC_SCRATCH_BYTES of its memory until the process exits, used or not.
#include <mutex>

#include "../../include/lokiscan.h"
#include "lk_common.cuh"
#include "scan.cuh"
#include "topk.cuh"

namespace lk {

// control block (256 B: ticket, error flag, batch counters) | merged keys | per-CTA lists
constexpr size_t kPreCtrlBytes = 256;
constexpr size_t kPreKeysBytes = (size_t)LK_PREALLOC_MAX_K * 8;
constexpr size_t kPreListBytes = (size_t)LK_PREALLOC_MAX_CTAS * LK_PREALLOC_MAX_K * 8;
static_assert(kPreCtrlBytes + kPreKeysBytes + kPreListBytes == LK_PREALLOC_SCRATCH_BYTES,
              "the header must state the real size of the scratch array");

// In host code this name is only a handle for the runtime, not a device address:
// the address comes from cudaGetSymbolAddress, per device, below.
static __device__ __align__(256) unsigned char g_prealloc_scratch[LK_PREALLOC_SCRATCH_BYTES];

constexpr int kPreMaxDevices = 64;
static std::mutex g_pre_mutex;
static unsigned char *g_pre_ptr[kPreMaxDevices];  // device address of the array on each GPU, once known

// First use on a device: look the array's address up with that device current.
static int prealloc_scratch(int device, unsigned char **out) {
    std::lock_guard<std::mutex> lock(g_pre_mutex);
    if (g_pre_ptr[device] == nullptr) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_prealloc_scratch);
        if (e != cudaSuccess) return fail(LK_ECUDA, std::string("cudaGetSymbolAddress(scratch): ") + cudaGetErrorString(e));
        g_pre_ptr[device] = static_cast<unsigned char *>(p);
    }
    *out = g_pre_ptr[device];
    return 0;
}

// The hosts this entry point is for live inside someone else's runtime: put the caller's
// current device back when the call ends.
struct DeviceRestore {
    int prev = -1;
    ~DeviceRestore() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

}  // namespace lk

using namespace lk;

extern "C" int lk_scan_i8_prealloc(int device, const int8_t *d_codes, int64_t n, int dim, int64_t ld,
                                   const float *d_scales, const int8_t *d_query, float query_scale, int k,
                                   int64_t *d_out_ids, float *d_out_scores, int32_t *d_out_iscores,
                                   int32_t *d_out_count, void *stream) {
    if (!d_codes || !d_scales || !d_query || !d_out_ids || !d_out_scores || !d_out_count || n < 0 || dim < 1)
        return fail(LK_EINVAL, "lk_scan_i8_prealloc: NULL pointer or bad size");
    if (ld < dim || ld % 16 != 0 || ld > LK_MAX_DIM)
        return fail(LK_EINVAL, "lk_scan_i8_prealloc: ld must be a multiple of 16, at least dim and at most LK_MAX_DIM");
    if ((reinterpret_cast<uintptr_t>(d_codes) | reinterpret_cast<uintptr_t>(d_query)) & 15)
        return fail(LK_EINVAL, "lk_scan_i8_prealloc: d_codes and d_query must be 16-byte aligned");
    if (k < 1 || k > LK_PREALLOC_MAX_K)
        return fail(LK_ERANGE, "lk_scan_i8_prealloc: k is limited to LK_PREALLOC_MAX_K (128): the scratch array is fixed");
    if (n > 0xfffffff0ll) return fail(LK_ERANGE, "lk_scan_i8_prealloc: more than 2^32-16 rows");
    if (device < 0 || device >= kPreMaxDevices || device >= lk_device_count())
        return fail(LK_ECUDA, "lk_scan_i8_prealloc: no such CUDA device (this library has no CPU path)");
    DeviceRestore restore;
    if (cudaGetDevice(&restore.prev) != cudaSuccess) restore.prev = -1;
    if (restore.prev == device) restore.prev = -1;  // nothing to put back
    else LK_CUDA(cudaSetDevice(device));
    unsigned char *scratch = nullptr;
    LK_TRY(prealloc_scratch(device, &scratch));
    ScanPlan plan;
    LK_TRY(scan_plan(SCAN_I8, (int)(ld / 16), k, device, &plan));
    if (scan_max_grid(plan) > LK_PREALLOC_MAX_CTAS)
        return fail(LK_ERANGE, "lk_scan_i8_prealloc: this GPU runs more CTAs at once than LK_PREALLOC_MAX_CTAS (1024)");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // The array keeps whatever the last call left.  The control words must start at
    // zero (a failed call may have left them set); the lists are rewritten in full.
    LK_CUDA(cudaMemsetAsync(scratch, 0, kPreCtrlBytes, st));
    ScanArgs a = {};
    a.rows = reinterpret_cast<const unsigned char *>(d_codes);
    a.ld = ld;
    a.chunks = (int)(ld / 16);
    a.n = n;
    a.slots = nullptr;
    a.query = reinterpret_cast<const unsigned char *>(d_query);
    a.cnorm = nullptr;
    a.cq = 0.0f;
    a.k = k;
    a.bound = nullptr;
    a.ticket = reinterpret_cast<unsigned int *>(scratch);
    a.error = reinterpret_cast<int *>(scratch) + 1;
    a.next_batch = reinterpret_cast<unsigned int *>(scratch) + 2;
    a.out_keys = reinterpret_cast<unsigned long long *>(scratch + kPreCtrlBytes);
    a.part = reinterpret_cast<unsigned long long *>(scratch + kPreCtrlBytes + kPreKeysBytes);
    a.out_ids = reinterpret_cast<long long *>(d_out_ids);
    a.out_scores = d_out_scores;
    a.out_iscores = d_out_iscores;
    a.out_count = d_out_count;
    a.scales = d_scales;
    a.qscale = query_scale;
    a.shard_base = 0;
    a.peer = nullptr;
    a.seq = 0;
    a.done_flag = nullptr;
    a.done_value = 0;
    return scan_launch(SCAN_I8, a, plan, st);
}
