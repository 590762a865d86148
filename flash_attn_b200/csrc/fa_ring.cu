// Ring attention behind the C ABI: the sequence-sharded forward of one rank of an
// NCCL communicator (include/fa_b200.h, fa_ring_fwd).
//
// The reference has no multi-GPU path.  What is generalised here is the algebra of its
// split-KV combine (src/flash_forward_splitkv.h:359-397): a query row's result over a key
// sequence that arrives block by block is the log-sum-exp merge of the blocks' results.
// The sequence is cut into 2*P chunks; rank r owns chunks r and 2P-1-r ("zig-zag": equal
// causal work on every rank).  Q and O stay put; the rank's K/V chunks travel round the
// ring as one message per step (ncclSend to rank+1, ncclRecv from rank-1, grouped, on a
// communication stream) into the other of two caller-owned message buffers, while the
// compute stream runs one forward launch per visible (query chunk, key chunk) pair of the
// message at hand, with global positions, each merging into the rank's running fp32
// (O, LSE) pair in its own epilogue; the launch of a query chunk's last visible block also
// writes the 16-bit output.  Events order the two streams; remote K/V always lands in
// this GPU's own memory before a TMA load reads it.
//
// NCCL is resolved at run time (dlopen of libnccl.so.2: the copy the process has already
// loaded, e.g. the one a framework brought, else the system's), so that the library keeps
// linking against the CUDA runtime only.
#include <dlfcn.h>
#include <cstring>
#include <mutex>
#include <cuda_runtime.h>
#include <nccl.h>
#include "../../include/fa_b200.h"

namespace {

struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*);
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*GroupStart)();
    ncclResult_t (*GroupEnd)();
    ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*);
    bool ok = false;
};

const NcclApi& nccl() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
        if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) return;
        bool all = true;
        auto sym = [&](const char* name) {
            void* p = dlsym(h, name);
            if (!p) all = false;
            return p;
        };
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
        api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(sym("ncclGroupStart"));
        api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(sym("ncclGroupEnd"));
        api.Send = reinterpret_cast<decltype(api.Send)>(sym("ncclSend"));
        api.Recv = reinterpret_cast<decltype(api.Recv)>(sym("ncclRecv"));
        api.CommGetAsyncError = reinterpret_cast<decltype(api.CommGetAsyncError)>(sym("ncclCommGetAsyncError"));
        api.ok = all;
    });
    return api;
}

size_t elem_bytes(int dtype) { return dtype == FA_DTYPE_FP32 ? 4 : 2; }

// Can any query of chunk a attend to any key of chunk b?  (Blocks that cannot are not launched.)
bool block_visible(long long a, long long b, long long chunk, int causal, int wl, int wr) {
    const long long q_lo = a * chunk, q_hi = (a + 1) * chunk - 1;
    const long long k_lo = b * chunk, k_hi = (b + 1) * chunk - 1;
    if ((causal || wr == 0) && k_lo > q_hi) return false;
    if (wr > 0 && k_lo > q_hi + wr) return false;
    if (wl >= 0 && k_hi < q_lo - wl) return false;
    return true;
}

}  // namespace

extern "C" {

size_t fa_ring_message_bytes(const fa_ring_params* p) {
    if (!p || p->batch < 1 || p->heads < 1 || p->chunk_rows < 1 || p->head_dim < 1) return 0;
    const int hk = p->heads_k > 0 ? p->heads_k : p->heads;
    // K and V of the rank's two chunks
    return static_cast<size_t>(4) * p->batch * hk * p->chunk_rows * p->head_dim * elem_bytes(p->dtype);
}

int fa_ring_unique_id(void* id_out, size_t bytes) {
    if (!id_out || bytes < sizeof(ncclUniqueId)) return FA_ERR_INVALID_ARG;
    if (!nccl().ok) return FA_ERR_UNSUPPORTED;
    ncclUniqueId id;
    if (nccl().GetUniqueId(&id) != ncclSuccess) return FA_ERR_CUDA;
    std::memcpy(id_out, &id, sizeof(id));
    return FA_OK;
}

int fa_ring_comm_create(void** comm_out, int world, int rank, const void* id, size_t bytes) {
    if (!comm_out || !id || bytes < sizeof(ncclUniqueId) || world < 1 || rank < 0 || rank >= world) return FA_ERR_INVALID_ARG;
    if (!nccl().ok) return FA_ERR_UNSUPPORTED;
    ncclUniqueId uid;
    std::memcpy(&uid, id, sizeof(uid));
    ncclComm_t c = nullptr;
    if (nccl().CommInitRank(&c, world, uid, rank) != ncclSuccess) return FA_ERR_CUDA;
    *comm_out = c;
    return FA_OK;
}

int fa_ring_comm_destroy(void* comm) {
    if (!comm) return FA_OK;
    if (!nccl().ok) return FA_ERR_UNSUPPORTED;
    return nccl().CommDestroy(static_cast<ncclComm_t>(comm)) == ncclSuccess ? FA_OK : FA_ERR_CUDA;
}

int fa_ring_fwd(const fa_ring_params* p) {
    if (!p) return FA_ERR_INVALID_ARG;
    const int world = p->world, rank = p->rank;
    if (world < 1 || rank < 0 || rank >= world) return FA_ERR_INVALID_ARG;
    if (world > 1 && (!p->comm || !p->message[1])) return FA_ERR_INVALID_ARG;
    if (!p->message[0]) return FA_ERR_INVALID_ARG;
    for (int i = 0; i < 2; ++i)
        if (!p->q[i] || !p->k[i] || !p->v[i] || !p->o[i] || !p->accum_o[i] || !p->accum_lse[i]) return FA_ERR_INVALID_ARG;
    if (p->p_dropout != 0.0f) return FA_ERR_UNSUPPORTED;  // the reference's dropout streams are keyed on the tile grid of
                                                          // one whole-sequence launch, which a shard does not have
    if (world > 1 && !nccl().ok) return FA_ERR_UNSUPPORTED;
    const size_t msg = fa_ring_message_bytes(p);
    if (msg == 0) return FA_ERR_INVALID_ARG;
    const int hk = p->heads_k > 0 ? p->heads_k : p->heads;
    const size_t chunk_bytes = msg / 4;  // one of K0, K1, V0, V1
    const long long C = p->chunk_rows;
    cudaStream_t compute = static_cast<cudaStream_t>(p->compute_stream);
    cudaStream_t comm_stream = static_cast<cudaStream_t>(p->comm_stream);
    if (world > 1 && comm_stream == compute) return FA_ERR_INVALID_ARG;  // the exchange must be able to overlap

    // schedule of this rank: for every ring step the visible (query chunk, key chunk) pairs
    const long long mine[2] = {rank, 2LL * world - 1 - rank};
    int total[2] = {0, 0}, done[2] = {0, 0};
    for (int step = 0; step < world; ++step) {
        const int src = ((rank - step) % world + world) % world;
        const long long theirs[2] = {src, 2LL * world - 1 - src};
        for (int qi = 0; qi < 2; ++qi)
            for (int ki = 0; ki < 2; ++ki)
                if (block_visible(mine[qi], theirs[ki], C, p->is_causal, p->window_left, p->window_right)) ++total[qi];
    }

    // message layout: K chunk 0 | K chunk 1 | V chunk 0 | V chunk 1
    char* buf[2] = {static_cast<char*>(p->message[0]), static_cast<char*>(p->message[1])};
    bool ok = cudaMemcpyAsync(buf[0], p->k[0], chunk_bytes, cudaMemcpyDeviceToDevice, compute) == cudaSuccess &&
              cudaMemcpyAsync(buf[0] + chunk_bytes, p->k[1], chunk_bytes, cudaMemcpyDeviceToDevice, compute) == cudaSuccess &&
              cudaMemcpyAsync(buf[0] + 2 * chunk_bytes, p->v[0], chunk_bytes, cudaMemcpyDeviceToDevice, compute) == cudaSuccess &&
              cudaMemcpyAsync(buf[0] + 3 * chunk_bytes, p->v[1], chunk_bytes, cudaMemcpyDeviceToDevice, compute) == cudaSuccess;
    if (!ok) return FA_ERR_CUDA;

    cudaEvent_t ev_ready = nullptr, ev_received = nullptr, ev_computed = nullptr;  // re-recorded every step
    if (world > 1) {
        if (cudaEventCreateWithFlags(&ev_ready, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&ev_received, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&ev_computed, cudaEventDisableTiming) != cudaSuccess)
            return FA_ERR_CUDA;
        // the first message is complete once the copies above are
        if (cudaEventRecord(ev_ready, compute) != cudaSuccess || cudaStreamWaitEvent(comm_stream, ev_ready, 0) != cudaSuccess)
            return FA_ERR_CUDA;
    }
    int rc = FA_OK;
    const int nxt = (rank + 1) % world, prv = (rank - 1 + world) % world;
    for (int step = 0; step < world && rc == FA_OK; ++step) {
        char* cur = buf[step & 1];
        if (step + 1 < world) {
            // post the exchange first: it runs on the communication stream while the launches below compute.
            // The buffer it receives into was read by the launches of the step before.
            if (step > 0 && cudaStreamWaitEvent(comm_stream, ev_computed, 0) != cudaSuccess) { rc = FA_ERR_CUDA; break; }
            ncclComm_t c = static_cast<ncclComm_t>(p->comm);
            if (nccl().GroupStart() != ncclSuccess ||
                nccl().Send(cur, msg, ncclInt8, nxt, c, comm_stream) != ncclSuccess ||
                nccl().Recv(buf[(step + 1) & 1], msg, ncclInt8, prv, c, comm_stream) != ncclSuccess ||
                nccl().GroupEnd() != ncclSuccess) { rc = FA_ERR_CUDA; break; }
            if (cudaEventRecord(ev_received, comm_stream) != cudaSuccess) { rc = FA_ERR_CUDA; break; }
        }
        const int src = ((rank - step) % world + world) % world;
        const long long theirs[2] = {src, 2LL * world - 1 - src};
        for (int qi = 0; qi < 2 && rc == FA_OK; ++qi) {
            for (int ki = 0; ki < 2 && rc == FA_OK; ++ki) {
                const long long a = mine[qi], b = theirs[ki];
                if (!block_visible(a, b, C, p->is_causal, p->window_left, p->window_right)) continue;
                fa_fwd_params f;
                std::memset(&f, 0, sizeof(f));
                f.q = p->q[qi];
                f.k = cur + ki * chunk_bytes;
                f.v = cur + (2 + ki) * chunk_bytes;
                f.dtype = p->dtype;
                f.o_dtype = p->dtype;
                f.batch = p->batch; f.heads = p->heads; f.heads_k = hk;
                f.seqlen_q = f.seqlen_k = p->chunk_rows;
                f.head_dim = p->head_dim;
                f.softmax_scale = p->softmax_scale;
                // blocks that lie wholly before the query chunk need no causal test
                f.is_causal = (p->is_causal && a == b) ? 1 : 0;
                f.window_left = p->window_left; f.window_right = p->window_right;
                f.alibi_slopes = p->alibi_slopes;
                f.num_splits = 1;
                f.q_pos0 = a * C; f.k_pos0 = b * C;
                f.status = p->status;
                f.stream = p->compute_stream;
                f.accum_o = p->accum_o[qi]; f.accum_lse = p->accum_lse[qi];
                const bool first = done[qi] == 0, final = done[qi] + 1 == total[qi];
                f.accum_flags = (first ? FA_ACCUM_FIRST : 0) | (final ? FA_ACCUM_FINAL : 0);
                if (final) { f.o = p->o[qi]; f.lse = p->lse[qi]; }
                ++done[qi];
                rc = fa_fwd(&f);
            }
        }
        if (step + 1 < world && rc == FA_OK) {
            // the next step's launches read the buffer the exchange fills; the next exchange overwrites this one
            if (cudaEventRecord(ev_computed, compute) != cudaSuccess || cudaStreamWaitEvent(compute, ev_received, 0) != cudaSuccess)
                rc = FA_ERR_CUDA;
        }
    }
    // (every query chunk sees at least its own key chunk, so both outputs have been written)
    if (ev_ready) cudaEventDestroy(ev_ready);      // (destruction is deferred by the runtime until the work recorded has completed)
    if (ev_received) cudaEventDestroy(ev_received);
    if (ev_computed) cudaEventDestroy(ev_computed);
    if (rc == FA_OK && world > 1 && p->comm) {
        ncclResult_t async = ncclSuccess;
        if (nccl().CommGetAsyncError(static_cast<ncclComm_t>(p->comm), &async) == ncclSuccess && async != ncclSuccess) rc = FA_ERR_CUDA;
    }
    return rc;
}

}  // extern "C"
