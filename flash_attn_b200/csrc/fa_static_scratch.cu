// fa_fwd_static_scratch: the split-KV forward for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc on the path that launches
// attention: a serving loop that has handed the whole device to its own memory
// pool, a plugin loaded into a process whose allocator is owned by someone else,
// or a real-time path where an allocation (and the implicit synchronisation it
// can bring) is not acceptable.  fa_fwd already takes a caller-provided
// workspace; this entry point is for callers that cannot even provide that.  The
// split partials (un-merged O and log-sum-exp of every KV split) live in a
// fixed array in device global memory that is part of the loaded module.
#include <mutex>
#include <cuda_runtime.h>
#include "../../include/fa_b200.h"

namespace {

// Every GPU that loads the library holds this array until the process exits.
static __device__ __align__(256) unsigned char g_split_scratch[FA_STATIC_SCRATCH_BYTES];

std::mutex g_mutex;
void* g_scratch_addr[64] = {};  // device address of g_split_scratch, per device ordinal

// In host code the name g_split_scratch is only a handle for the runtime, not a
// device address; the address a kernel can use comes from cudaGetSymbolAddress,
// asked once per device with that device current.
int scratch_for_current_device(void** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return FA_ERR_CUDA;
    if (dev < 0 || dev >= 64) return FA_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_scratch_addr[dev] == nullptr) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_split_scratch) != cudaSuccess || ptr == nullptr) return FA_ERR_CUDA;
        g_scratch_addr[dev] = ptr;
    }
    *out = g_scratch_addr[dev];
    return FA_OK;
}

}  // namespace

extern "C" {

size_t fa_static_scratch_bytes(void) { return FA_STATIC_SCRATCH_BYTES; }

int fa_fwd_static_scratch(const fa_fwd_params* p) {
    if (!p) return FA_ERR_INVALID_ARG;
    fa_fwd_params q = *p;
    q.workspace = nullptr;
    q.workspace_bytes = 0;
    const int splits = fa_fwd_resolve_splits(&q);
    if (splits < 0) return splits;
    const size_t need = fa_fwd_workspace_bytes(&q);
    if (need > FA_STATIC_SCRATCH_BYTES) return FA_ERR_TOO_LARGE;
    void* scratch = nullptr;
    const int rc = scratch_for_current_device(&scratch);
    if (rc != FA_OK) return rc;
    // Nothing in the scratch has to start at zero: the split kernel writes the
    // partial O and log-sum-exp of every (unit, split, row) it is launched for,
    // empty splits included, and the combine kernel reads only those.
    q.num_splits = splits;
    q.workspace = scratch;
    q.workspace_bytes = FA_STATIC_SCRATCH_BYTES;
    return fa_fwd(&q);
}

}  // extern "C"
