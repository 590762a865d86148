// C-ABI entry points (include/fa_b200.h): argument checks, split policy, TMA
// tensor maps and kernel dispatch.  This is the successor of the launcher block
// of the reference's main() (src/main.cu:109-205) with every compile-time switch
// (src/main.cu:39-49) turned into a run-time parameter.
#include <atomic>
#include <cmath>
#include <cstring>
#include <mutex>
#include <vector>
#include <algorithm>
#include <cuda.h>
#include <cuda_runtime.h>
#include "../../include/fa_b200.h"
#include "fa_internal.h"

namespace {

using namespace fa;

typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is fetched through the runtime, so the library links
// against libcudart only.
encode_tiled_fn get_encode_tiled() {
    static encode_tiled_fn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<encode_tiled_fn>(p);
    }();
    return fn;
}

// [units, rows, d] 16-bit tensor, box = 64 elements x 128 rows x 1 unit, 128-byte
// swizzle; out-of-range rows and columns read as zero, which replaces the
// reference's hand-written zero padding (include/utils.h:67-114).
int make_tensor_map(CUtensorMap* m, bool bf16, const void* base, int d, long long rows, long long units,
                    int box_rows = kTile) {
    // A tensor map is a pure function of these arguments, so the last few are kept per host thread:
    // a caller that runs the same buffers again (every layer of every step) skips the driver call.
    struct Entry {
        const void* base;
        long long rows, units;
        int d, box_rows, bf16, valid;
        CUtensorMap map;
    };
    constexpr int kEntries = 8;
    thread_local Entry cache[kEntries] = {};
    thread_local int next_victim = 0;
    for (int i = 0; i < kEntries; ++i) {
        const Entry& e = cache[i];
        if (e.valid && e.base == base && e.rows == rows && e.units == units && e.d == d && e.box_rows == box_rows &&
            e.bf16 == static_cast<int>(bf16)) {
            *m = e.map;
            return FA_OK;
        }
    }
    encode_tiled_fn enc = get_encode_tiled();
    if (!enc) return FA_ERR_CUDA;
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(d), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(units)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(d) * 2, static_cast<cuuint64_t>(rows) * d * 2};
    cuuint32_t box[3] = {64, static_cast<cuuint32_t>(box_rows), 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(m, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                     const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return FA_ERR_CUDA;
    Entry& e = cache[next_victim];
    next_victim = (next_victim + 1) % kEntries;
    e.base = base; e.rows = rows; e.units = units; e.d = d; e.box_rows = box_rows; e.bf16 = bf16; e.map = *m; e.valid = 1;
    return FA_OK;
}

// curand_uniform's map of a raw draw to (0,1]: x*2^-32 + 2^-33 in fp32.
float uniform_of(uint32_t x) {
    volatile float f = static_cast<float>(x);
    volatile float r = f * 2.3283064365386963e-10f;
    r = r + 1.1641532182693481e-10f;
    return r;
}
// Smallest raw draw that is kept: the reference drops when uniform < p
// (src/flash_forward.h:230) and uniform_of is monotone, so the dropped draws are [0, T).
unsigned long long keep_threshold(float p) {
    if (!(uniform_of(0u) < p)) return 0ull;
    if (uniform_of(0xFFFFFFFFu) < p) return 1ull << 32;
    unsigned long long lo = 0, hi = 0xFFFFFFFFull;  // lo dropped, hi kept
    while (hi - lo > 1) {
        const unsigned long long mid = lo + (hi - lo) / 2;
        if (uniform_of(static_cast<uint32_t>(mid)) < p) lo = mid; else hi = mid;
    }
    return hi;
}

int sm_count_of_current_device(int* sms, int* major) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return FA_ERR_CUDA;
    // (SM count << 8 | major) per device ordinal, 0 = not asked yet; concurrent first calls store the same value
    static std::atomic<int> cached[64];
    if (dev >= 0 && dev < 64) {
        const int c = cached[dev].load(std::memory_order_relaxed);
        if (c > 0) {
            *sms = c >> 8;
            *major = c & 0xff;
            return FA_OK;
        }
    }
    if (cudaDeviceGetAttribute(sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return FA_ERR_CUDA;
    if (cudaDeviceGetAttribute(major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return FA_ERR_CUDA;
    if (dev >= 0 && dev < 64) cached[dev].store((*sms << 8) | (*major & 0xff), std::memory_order_relaxed);
    return FA_OK;
}

int validate(const fa_fwd_params* p) {
    if (!p || !p->q || !p->k || !p->v) return FA_ERR_INVALID_ARG;
    // the output may be left out only by a launch that merges into a running result and is not its last
    const bool accum_only = p->accum_o != nullptr && !(p->accum_flags & FA_ACCUM_FINAL);
    if (!p->o && !accum_only) return FA_ERR_INVALID_ARG;
    if (p->accum_o != nullptr && (!p->accum_lse || (reinterpret_cast<uintptr_t>(p->accum_o) & 15u))) return FA_ERR_INVALID_ARG;
    if (p->batch < 1 || p->heads < 1 || p->seqlen_q < 1 || p->seqlen_k < 1 || p->head_dim < 1) return FA_ERR_INVALID_ARG;
    if (p->heads_k < 0 || (p->heads_k > 0 && p->heads % p->heads_k != 0)) return FA_ERR_INVALID_ARG;
    if (p->dtype != FA_DTYPE_FP16 && p->dtype != FA_DTYPE_BF16) return FA_ERR_UNSUPPORTED;
    if (p->o_dtype != p->dtype && p->o_dtype != FA_DTYPE_FP32) return FA_ERR_UNSUPPORTED;
    if (p->head_dim > 128) return FA_ERR_UNSUPPORTED;
    if (!(p->softmax_scale > 0.0f) || !std::isfinite(p->softmax_scale)) return FA_ERR_INVALID_ARG;
    if (!(p->p_dropout >= 0.0f) || !(p->p_dropout < 1.0f)) return FA_ERR_INVALID_ARG;
    if (p->window_left < -1 || p->window_right < -1 || p->num_splits < 0) return FA_ERR_INVALID_ARG;
    // rows are 16-byte multiples when head_dim % 8 == 0 (TMA reads them in place); otherwise the
    // tensors are copied to a padded pitch first and only element alignment is needed
    const uintptr_t align_mask = (p->head_dim % 8 == 0) ? 15u : 3u;
    if ((reinterpret_cast<uintptr_t>(p->q) | reinterpret_cast<uintptr_t>(p->k) | reinterpret_cast<uintptr_t>(p->v) |
         reinterpret_cast<uintptr_t>(p->o)) & align_mask)
        return FA_ERR_INVALID_ARG;
    const long long units = static_cast<long long>(p->batch) * p->heads;
    const long long tr = (p->seqlen_q + kTile - 1) / kTile;
    if (units * tr > 0x3fffffffLL) return FA_ERR_TOO_LARGE;
    return FA_OK;
}

// K/V heads of the call (heads_k = 0 means one K/V head per query head).
int kv_heads(const fa_fwd_params* p) { return p->heads_k > 0 ? p->heads_k : p->heads; }

int resolve_splits(const fa_fwd_params* p, int sms) {
    const int tr = (p->seqlen_q + kTile - 1) / kTile;
    const int tc = (p->seqlen_k + kTile - 1) / kTile;
    int s = p->num_splits;
    if (s == 0) {
        const long long blocks = static_cast<long long>(p->batch) * p->heads * tr;
        // argument shape of the reference's call, src/main.cu:125
        s = fa_num_splits_heuristic(static_cast<int>(std::min<long long>(blocks, 1 << 30)), sms, tc, tc, tc * kTile);
    }
    return std::max(1, std::min(s, tc));
}

void fill_args(const fa_fwd_params* p, int splits, FwdArgs* a) {
    std::memset(a, 0, sizeof(*a));
    a->o = p->o;
    a->lse = p->lse;
    a->alibi_slopes = p->alibi_slopes;
    a->status = p->status;
    a->heads = p->heads;
    a->units = p->batch * p->heads;
    a->kv_group = p->heads / kv_heads(p);
    // query blocks of very different cost (causal, no left window): heaviest-first over groups of
    // 16 units; otherwise unit-major, which keeps neighbouring CTAs on the same K/V tiles in L2
    a->unit_group = (p->is_causal && p->window_left < 0) ? 16 : 1;
    a->seqlen_q = p->seqlen_q;
    a->seqlen_k = p->seqlen_k;
    a->head_dim = p->head_dim;
    a->tr = (p->seqlen_q + kTile - 1) / kTile;
    a->tc = (p->seqlen_k + kTile - 1) / kTile;
    a->num_splits = splits;
    a->tiles_per_split = (a->tc + splits - 1) / splits;
    a->scale_log2 = p->softmax_scale * 1.4426950408889634f;
    a->is_causal = p->is_causal ? 1 : 0;
    a->window_left = p->window_left;
    a->window_right = p->window_right;
    a->q_pos0 = p->q_pos0;
    a->k_pos0 = p->k_pos0;
    a->o_is_fp32 = p->o_dtype == FA_DTYPE_FP32;
    a->accum_o = p->accum_o;
    a->accum_lse = p->accum_lse;
    a->accum_first = (p->accum_flags & FA_ACCUM_FIRST) ? 1 : 0;
    a->accum_final = (p->accum_flags & FA_ACCUM_FINAL) ? 1 : 0;
    a->drop.seed_lo = static_cast<uint32_t>(p->seed);
    a->drop.seed_hi = static_cast<uint32_t>(p->seed >> 32);
    a->drop.offset = p->offset;
    a->drop.launch_index = p->launch_index;
    a->drop.unit0 = p->unit0;
    a->drop.threshold = p->p_dropout > 0.0f ? keep_threshold(p->p_dropout) : 0ull;
    a->drop.inv_keep = p->p_dropout > 0.0f ? 1.0f / (1.0f - p->p_dropout) : 1.0f;
}

size_t partial_bytes(const fa_fwd_params* p, int splits, size_t* lse_off) {
    const size_t rows = static_cast<size_t>(p->batch) * p->heads * splits * p->seqlen_q;
    const size_t o_bytes = (rows * p->head_dim * sizeof(float) + 255) & ~static_cast<size_t>(255);
    if (lse_off) *lse_off = o_bytes;
    return o_bytes + ((rows * sizeof(float) + 255) & ~static_cast<size_t>(255));
}

// head_dim that is not a multiple of 8: Q/K/V are copied to a pitch of d8 = ceil8(head_dim)
// elements (zero columns), the kernels run on the padded problem, O is copied back.
struct PadPlan {
    int d8;
    size_t q_bytes, kv_bytes, o_bytes, total;
};
PadPlan pad_plan(const fa_fwd_params* p) {
    PadPlan pl;
    auto up = [](size_t x) { return (x + 255) & ~static_cast<size_t>(255); };
    pl.d8 = (p->head_dim + 7) / 8 * 8;
    const size_t units = static_cast<size_t>(p->batch) * p->heads;
    pl.q_bytes = up(units * p->seqlen_q * pl.d8 * 2);
    pl.kv_bytes = up(static_cast<size_t>(p->batch) * kv_heads(p) * p->seqlen_k * pl.d8 * 2);
    pl.o_bytes = up(units * p->seqlen_q * pl.d8 * (p->o_dtype == FA_DTYPE_FP32 ? 4 : 2));
    pl.total = pl.q_bytes + 2 * pl.kv_bytes + pl.o_bytes;
    return pl;
}

}  // namespace

extern "C" {

int fa_version(void) { return FA_B200_VERSION; }

const char* fa_strerror(int code) {
    switch (code) {
        case FA_OK: return "success";
        case FA_ERR_INVALID_ARG: return "invalid argument";
        case FA_ERR_UNSUPPORTED: return "unsupported dtype or head_dim (need fp16/bf16 inputs, head_dim <= 128)";
        case FA_ERR_WORKSPACE: return "workspace missing or too small (see fa_fwd_workspace_bytes)";
        case FA_ERR_CUDA: return "CUDA call failed";
        case FA_ERR_DEVICE_TIMEOUT: return "a device-side wait timed out";
        case FA_ERR_NOT_SM100: return "device is not compute capability 10.x";
        case FA_ERR_TOO_LARGE: return "size beyond the limit of this entry point";
        default: return "unknown error";
    }
}

int fa_num_splits_heuristic(int batch_nheads_mblocks, int num_sms, int num_n_blocks, int max_splits, int seq_len) {
    // Same policy as the reference (src/main.cu:391-422): no split once there are
    // four waves of CTAs; otherwise the smallest eligible split whose wave
    // efficiency is within 85 % of the best one.
    if (static_cast<float>(batch_nheads_mblocks) >= 4.0f * static_cast<float>(num_sms)) return 1;
    max_splits = std::min(max_splits, std::min(num_sms, num_n_blocks));
    auto tiles = [&](int s) { return (num_n_blocks + s - 1) / s; };
    auto eligible = [&](int s) {
        return seq_len % (kTile * s) == 0 && (s == 1 || tiles(s) != tiles(s - 1));
    };
    auto efficiency = [&](int s) {
        const float waves = static_cast<float>(batch_nheads_mblocks * s) / static_cast<float>(num_sms);
        return waves / std::ceil(waves);
    };
    float best = 0.0f;
    for (int s = 1; s <= max_splits; ++s)
        if (eligible(s)) best = std::max(best, efficiency(s));
    for (int s = 1; s <= max_splits; ++s)
        if (eligible(s) && efficiency(s) >= 0.85 * best) return s;
    return 1;
}

int fa_fwd_resolve_splits(const fa_fwd_params* p) {
    int rc = validate(p);
    if (rc != FA_OK) return rc;
    int sms = 148, major = 10;
    if (p->num_splits == 0 && sm_count_of_current_device(&sms, &major) != FA_OK) return FA_ERR_CUDA;
    return resolve_splits(p, sms);
}

size_t fa_fwd_workspace_bytes(const fa_fwd_params* p) {
    const int s = fa_fwd_resolve_splits(p);
    if (s < 1) return 0;
    size_t bytes = 0;
    if (p->head_dim % 8 != 0) {
        fa_fwd_params q = *p;
        q.head_dim = pad_plan(p).d8;
        bytes = pad_plan(p).total + (s > 1 ? partial_bytes(&q, s, nullptr) : 0);
    } else if (s > 1) {
        bytes = partial_bytes(p, s, nullptr);
    }
    return bytes;
}

int fa_fwd(const fa_fwd_params* p) {
    int rc = validate(p);
    if (rc != FA_OK) return rc;
    int sms = 0, major = 0;
    rc = sm_count_of_current_device(&sms, &major);
    if (rc != FA_OK) return rc;
    if (major != 10) return FA_ERR_NOT_SM100;
    const int splits = resolve_splits(p, sms);
    if (p->accum_o != nullptr && (splits > 1 || p->head_dim % 8 != 0)) return FA_ERR_UNSUPPORTED;
    const int units = p->batch * p->heads;
    cudaStream_t stream = static_cast<cudaStream_t>(p->stream);
    if (p->head_dim % 8 != 0) {
        // padded pitch: re-pitch Q, K, V into the workspace, run on head_dim = d8, re-pitch O back
        const PadPlan pl = pad_plan(p);
        fa_fwd_params q = *p;
        q.head_dim = pl.d8;
        const size_t part = splits > 1 ? partial_bytes(&q, splits, nullptr) : 0;
        if (!p->workspace || p->workspace_bytes < pl.total + part) return FA_ERR_WORKSPACE;
        if (reinterpret_cast<uintptr_t>(p->workspace) & 255u) return FA_ERR_INVALID_ARG;
        char* ws = static_cast<char*>(p->workspace);
        char* qp = ws; char* kp = qp + pl.q_bytes; char* vp = kp + pl.kv_bytes; char* op = vp + pl.kv_bytes;
        const long long rq = static_cast<long long>(units) * p->seqlen_q;
        const long long rk = static_cast<long long>(p->batch) * kv_heads(p) * p->seqlen_k;
        if (launch_repitch(p->q, qp, 2, rq, p->head_dim, pl.d8, stream) != cudaSuccess ||
            launch_repitch(p->k, kp, 2, rk, p->head_dim, pl.d8, stream) != cudaSuccess ||
            launch_repitch(p->v, vp, 2, rk, p->head_dim, pl.d8, stream) != cudaSuccess)
            return FA_ERR_CUDA;
        q.q = qp; q.k = kp; q.v = vp; q.o = op;
        q.num_splits = splits;
        q.workspace = part ? op + pl.o_bytes : nullptr;
        q.workspace_bytes = part;
        rc = fa_fwd(&q);
        if (rc != FA_OK) return rc;
        if (launch_repitch(op, p->o, p->o_dtype == FA_DTYPE_FP32 ? 4 : 2, rq, pl.d8, p->head_dim, stream) != cudaSuccess)
            return FA_ERR_CUDA;
        return FA_OK;
    }
    FwdArgs a;
    fill_args(p, splits, &a);
    if (splits > 1) {
        size_t lse_off = 0;
        const size_t need = partial_bytes(p, splits, &lse_off);
        if (!p->workspace || p->workspace_bytes < need) return FA_ERR_WORKSPACE;
        if (reinterpret_cast<uintptr_t>(p->workspace) & 15u) return FA_ERR_INVALID_ARG;
        a.o_partial = static_cast<float*>(p->workspace);
        a.lse_partial = reinterpret_cast<float*>(static_cast<char*>(p->workspace) + lse_off);
    }
    const bool bf16 = p->dtype == FA_DTYPE_BF16;
    CUtensorMap tq, tk, tv;
    if ((rc = make_tensor_map(&tq, bf16, p->q, p->head_dim, p->seqlen_q, units)) != FA_OK) return rc;
    const int units_k = p->batch * kv_heads(p);
    if ((rc = make_tensor_map(&tk, bf16, p->k, p->head_dim, p->seqlen_k, units_k)) != FA_OK) return rc;
    if ((rc = make_tensor_map(&tv, bf16, p->v, p->head_dim, p->seqlen_k, units_k)) != FA_OK) return rc;
    // 16-bit output of an unsplit launch is written by TMA stores, one 32-row box per warp
    CUtensorMap to = tq;
    a.o_tma = (splits == 1 && p->o_dtype != FA_DTYPE_FP32 && p->accum_o == nullptr) ? 1 : 0;
    if (a.o_tma && (rc = make_tensor_map(&to, bf16, p->o, p->head_dim, p->seqlen_q, units, 32)) != FA_OK) return rc;
    if (p->seqlen_q <= 8 && p->accum_o == nullptr) {
        // one to eight query rows per unit: the streaming kernel with keys on the tensor-memory lanes
        DecodeArgs d;
        std::memset(&d, 0, sizeof(d));
        d.q = p->q; d.o = p->o; d.lse = p->lse;
        d.o_partial = a.o_partial; d.lse_partial = a.lse_partial;
        d.alibi_slopes = p->alibi_slopes; d.status = p->status;
        d.heads = p->heads; d.kv_group = a.kv_group; d.seqlen_q = p->seqlen_q; d.seqlen_k = p->seqlen_k; d.head_dim = p->head_dim; d.tc = a.tc;
        d.num_splits = splits; d.tiles_per_split = a.tiles_per_split; d.scale_log2 = a.scale_log2;
        d.is_causal = a.is_causal; d.window_left = a.window_left; d.window_right = a.window_right;
        d.q_pos0 = a.q_pos0; d.k_pos0 = a.k_pos0; d.o_is_fp32 = a.o_is_fp32; d.drop = a.drop;
        if (launch_decode(d, tk, tv, units, bf16, stream) != cudaSuccess) return FA_ERR_CUDA;
    } else if (launch_fwd_tiled(a, tq, tk, tv, to, units, bf16, p->p_dropout > 0.0f, stream) != cudaSuccess) {
        return FA_ERR_CUDA;
    }
    if (splits > 1) {
        CombineArgs c;
        c.o_partial = a.o_partial;
        c.lse_partial = a.lse_partial;
        c.o = p->o;
        c.lse = p->lse;
        c.rows_per_unit = p->seqlen_q;
        c.num_splits = splits;
        c.head_dim = p->head_dim;
        c.o_dtype = p->o_dtype;
        if (launch_combine(c, units, stream) != cudaSuccess) return FA_ERR_CUDA;
    }
    return FA_OK;
}

int fa_dropout_mask(const fa_fwd_params* p, uint8_t* keep) {
    int rc = validate(p);
    if (rc != FA_OK) return rc;
    if (!keep) return FA_ERR_INVALID_ARG;
    int sms = 148, major = 10;
    if (p->num_splits == 0 && (rc = sm_count_of_current_device(&sms, &major)) != FA_OK) return rc;
    FwdArgs a;
    fill_args(p, resolve_splits(p, sms), &a);
    if (!(p->p_dropout > 0.0f)) a.drop.threshold = 0ull;
    if (launch_dropout_mask(a, keep, static_cast<long long>(p->batch) * p->heads,
                            static_cast<cudaStream_t>(p->stream)) != cudaSuccess)
        return FA_ERR_CUDA;
    return FA_OK;
}

int fa_merge_partial(float* o_acc, float* lse_acc, const void* o_part, const float* lse_part, int part_dtype,
                     int64_t rows, int head_dim, void* stream) {
    if (!o_acc || !lse_acc || !o_part || !lse_part || rows < 0 || head_dim < 1) return FA_ERR_INVALID_ARG;
    if (part_dtype != FA_DTYPE_FP16 && part_dtype != FA_DTYPE_BF16 && part_dtype != FA_DTYPE_FP32) return FA_ERR_UNSUPPORTED;
    return launch_merge(o_acc, lse_acc, o_part, lse_part, part_dtype, rows, head_dim,
                        static_cast<cudaStream_t>(stream)) == cudaSuccess ? FA_OK : FA_ERR_CUDA;
}

int fa_cast_output(const float* o_acc, void* o, int o_dtype, int64_t elems, void* stream) {
    if (!o_acc || !o || elems < 0) return FA_ERR_INVALID_ARG;
    if (o_dtype != FA_DTYPE_FP16 && o_dtype != FA_DTYPE_BF16 && o_dtype != FA_DTYPE_FP32) return FA_ERR_UNSUPPORTED;
    return launch_cast(o_acc, o, o_dtype, elems, static_cast<cudaStream_t>(stream)) == cudaSuccess ? FA_OK : FA_ERR_CUDA;
}

}  // extern "C"

// ------------------------------------------------------------------ host-buffer path
namespace {

struct HostStage {
    void* buf = nullptr;
    size_t bytes = 0;
    cudaStream_t streams[2] = {nullptr, nullptr};
    void* shim_ws = nullptr;   // workspace of fa_launch_reference_params
    size_t shim_bytes = 0;
};
// one lock per device ordinal: calls for different devices (one host thread per GPU) do not wait for
// one another; calls for the same device share its staging buffers and are serialised
std::mutex g_stage_mutex[64];
HostStage g_stage[64];

}  // namespace

extern "C" {

void fa_fwd_host_release(void) {
    int prev = 0;
    cudaGetDevice(&prev);
    for (int d = 0; d < 64; ++d) {
        std::lock_guard<std::mutex> lock(g_stage_mutex[d]);
        HostStage& st = g_stage[d];
        if (!st.buf && !st.streams[0] && !st.shim_ws) continue;
        cudaSetDevice(d);
        if (st.buf) cudaFree(st.buf);
        if (st.shim_ws) cudaFree(st.shim_ws);
        for (auto& s : st.streams) if (s) { cudaStreamDestroy(s); s = nullptr; }
        st.buf = nullptr;
        st.bytes = 0;
        st.shim_ws = nullptr;
        st.shim_bytes = 0;
    }
    cudaSetDevice(prev);
}

int fa_launch_reference_params(const fa_ref_kernel_params* param, int heads, int batch, int is_dropout,
                               int is_causal, int is_local, int has_alibi, unsigned long long dropout_seed,
                               void* stream) {
    if (!param) return FA_ERR_INVALID_ARG;
    fa_fwd_params p;
    std::memset(&p, 0, sizeof(p));
    p.q = param->Q; p.k = param->K; p.v = param->V; p.o = param->O;
    p.dtype = FA_DTYPE_FP16;
    p.o_dtype = FA_DTYPE_FP32;
    p.batch = batch; p.heads = heads;
    p.seqlen_q = p.seqlen_k = param->N;
    p.head_dim = param->d;
    p.softmax_scale = param->softmax_scale;
    p.is_causal = is_causal ? 1 : 0;
    p.window_left = is_local ? param->window_size_left : -1;
    p.window_right = is_local ? param->window_size_right : -1;
    p.alibi_slopes = has_alibi ? param->alibi_slopes_ptr : nullptr;
    p.p_dropout = is_dropout ? param->dropout_prob : 0.0f;
    p.seed = dropout_seed;
    p.num_splits = param->split_num > 0 ? param->split_num : 1;
    p.stream = stream;
    const size_t need = fa_fwd_workspace_bytes(&p);
    if (need) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FA_ERR_CUDA;
        std::lock_guard<std::mutex> lock(g_stage_mutex[dev]);
        HostStage& st = g_stage[dev];
        if (st.shim_bytes < need) {
            // the old buffer may still be in use by an earlier launch on another stream
            if (st.shim_ws) { cudaDeviceSynchronize(); cudaFree(st.shim_ws); st.shim_ws = nullptr; st.shim_bytes = 0; }
            if (cudaMalloc(&st.shim_ws, need) != cudaSuccess) return FA_ERR_CUDA;
            st.shim_bytes = need;
        }
        p.workspace = st.shim_ws;
        p.workspace_bytes = st.shim_bytes;
    }
    return fa_fwd(&p);
}

int fa_fwd_host(const fa_fwd_params* p) {
    // Pointer alignment is a device-side requirement; check the rest on a copy
    // whose pointers are known to be fine.
    if (!p || !p->q || !p->k || !p->v || !p->o) return FA_ERR_INVALID_ARG;
    fa_fwd_params chk = *p;
    chk.q = chk.k = chk.v = reinterpret_cast<const void*>(256);
    chk.o = reinterpret_cast<void*>(256);
    int rc = validate(&chk);
    if (rc != FA_OK) return rc;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FA_ERR_CUDA;
    std::lock_guard<std::mutex> lock(g_stage_mutex[dev]);
    HostStage& st = g_stage[dev];
    for (auto& s : st.streams)
        if (!s && cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess) return FA_ERR_CUDA;

    const long long units = static_cast<long long>(p->batch) * p->heads;
    const long long group = p->heads / kv_heads(p);  // query units per K/V unit; slices hold whole groups
    const long long kunits = units / group;
    const size_t esz = 2, osz = p->o_dtype == FA_DTYPE_FP32 ? 4 : 2;
    const size_t q_unit = static_cast<size_t>(p->seqlen_q) * p->head_dim * esz;
    const size_t kv_unit = static_cast<size_t>(p->seqlen_k) * p->head_dim * esz;
    const size_t o_unit = static_cast<size_t>(p->seqlen_q) * p->head_dim * osz;
    const size_t lse_unit = static_cast<size_t>(p->seqlen_q) * sizeof(float);
    // slices of units, double-buffered so copies in one stream overlap work in the other.  The count follows
    // the transfer size: about 32 MB of host-to-device traffic per slice (long enough to run the link at its
    // rate, short enough that the first kernel starts early and the last copy back is short), 2 to 16 slices.
    const size_t h2d_total = static_cast<size_t>(units) * q_unit + 2 * static_cast<size_t>(kunits) * kv_unit;
    const long long by_size = static_cast<long long>(h2d_total / (32u << 20));
    const long long slices = std::min<long long>(kunits, std::max<long long>(2, std::min<long long>(16, by_size)));
    const long long per_k = (kunits + slices - 1) / slices;
    const long long per = per_k * group;
    auto align = [](size_t x) { return (x + 255) & ~static_cast<size_t>(255); };
    fa_fwd_params probe = chk;
    probe.batch = 1;
    probe.heads = static_cast<int>(per);
    probe.heads_k = static_cast<int>(per_k);
    const int splits = fa_fwd_resolve_splits(&probe);
    if (splits < 1) return splits;
    const size_t ws_bytes = fa_fwd_workspace_bytes(&probe);
    const size_t slot = align(q_unit * per) + 2 * align(kv_unit * per_k) + align(o_unit * per) + align(lse_unit * per) +
                        align(sizeof(float) * per) + align(ws_bytes) + align(sizeof(int));
    if (st.bytes < 2 * slot) {
        if (st.buf) cudaFree(st.buf);
        st.buf = nullptr;
        st.bytes = 0;
        if (cudaMalloc(&st.buf, 2 * slot) != cudaSuccess) return FA_ERR_CUDA;
        st.bytes = 2 * slot;
    }
    std::vector<float> slopes_by_unit;
    if (p->alibi_slopes) {
        slopes_by_unit.resize(units);
        for (long long u = 0; u < units; ++u) slopes_by_unit[u] = p->alibi_slopes[u % p->heads];
    }
    int result = FA_OK;
    for (long long s = 0, u0 = 0; u0 < units; ++s, u0 += per) {
        const long long n = std::min(per, units - u0);
        cudaStream_t stream = st.streams[s & 1];
        char* base = static_cast<char*>(st.buf) + (s & 1) * slot;
        char* dq = base;
        char* dk = dq + align(q_unit * per);
        char* dv = dk + align(kv_unit * per_k);
        char* dout = dv + align(kv_unit * per_k);
        char* dlse = dout + align(o_unit * per);
        char* dslopes = dlse + align(lse_unit * per);
        char* dws = dslopes + align(sizeof(float) * per);
        int* dstatus = reinterpret_cast<int*>(dws + align(ws_bytes));
        // the word the kernels set when one of their bounded waits gives up: cleared once per slot, read
        // back after the streams have drained (a slice that timed out leaves it set for the rest of the call)
        bool ok = s >= 2 || cudaMemsetAsync(dstatus, 0, sizeof(int), stream) == cudaSuccess;
        ok = ok && cudaMemcpyAsync(dq, static_cast<const char*>(p->q) + u0 * q_unit, n * q_unit, cudaMemcpyHostToDevice, stream) == cudaSuccess;
        ok = ok && cudaMemcpyAsync(dk, static_cast<const char*>(p->k) + (u0 / group) * kv_unit, (n / group) * kv_unit, cudaMemcpyHostToDevice, stream) == cudaSuccess;
        ok = ok && cudaMemcpyAsync(dv, static_cast<const char*>(p->v) + (u0 / group) * kv_unit, (n / group) * kv_unit, cudaMemcpyHostToDevice, stream) == cudaSuccess;
        if (ok && p->alibi_slopes)
            ok = cudaMemcpyAsync(dslopes, slopes_by_unit.data() + u0, n * sizeof(float), cudaMemcpyHostToDevice, stream) == cudaSuccess;
        if (!ok) { result = FA_ERR_CUDA; break; }
        fa_fwd_params q = *p;
        q.q = dq; q.k = dk; q.v = dv; q.o = dout;
        q.lse = p->lse ? reinterpret_cast<float*>(dlse) : nullptr;
        q.batch = 1;
        q.heads = static_cast<int>(n);
        q.heads_k = static_cast<int>(n / group);
        q.alibi_slopes = p->alibi_slopes ? reinterpret_cast<const float*>(dslopes) : nullptr;
        q.unit0 = p->unit0 + static_cast<uint64_t>(u0);
        q.num_splits = splits;
        q.workspace = ws_bytes ? dws : nullptr;
        q.workspace_bytes = ws_bytes;
        q.status = dstatus;
        q.accum_o = nullptr;  // (a running result lives in device memory: not a host-buffer feature)
        q.accum_lse = nullptr;
        q.accum_flags = 0;
        q.stream = stream;
        result = fa_fwd(&q);
        if (result != FA_OK) break;
        ok = cudaMemcpyAsync(static_cast<char*>(p->o) + u0 * o_unit, dout, n * o_unit, cudaMemcpyDeviceToHost, stream) == cudaSuccess;
        if (ok && p->lse)
            ok = cudaMemcpyAsync(reinterpret_cast<char*>(p->lse) + u0 * lse_unit, dlse, n * lse_unit, cudaMemcpyDeviceToHost, stream) == cudaSuccess;
        if (!ok) { result = FA_ERR_CUDA; break; }
    }
    for (auto& s : st.streams)
        if (cudaStreamSynchronize(s) != cudaSuccess && result == FA_OK) result = FA_ERR_CUDA;
    if (result == FA_OK) {
        const long long n_slices = (units + per - 1) / per;
        for (int b = 0; b < 2 && b < n_slices; ++b) {
            int hs = 0;
            const char* slot_base = static_cast<const char*>(st.buf) + b * slot;
            const char* word = slot_base + (slot - align(sizeof(int)));
            if (cudaMemcpy(&hs, word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return FA_ERR_CUDA;
            if (hs != 0) result = FA_ERR_DEVICE_TIMEOUT;
        }
    }
    return result;
}

}  // extern "C"
