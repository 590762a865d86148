// Memory-bound helper kernels: the split combine (replaces
// forward_kernel_splitkv_combine, src/flash_forward_splitkv.h:347-399), the
// partial-result merge used when a sequence is sharded across GPUs, the output
// cast, and the dropout keep-mask dump.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "../../include/fa_b200.h"
#include "fa_internal.h"
#include "sm100_ptx.cuh"

namespace fa {

namespace {

__device__ __forceinline__ void store_out(void* o, int o_dtype, long long idx, float v) {
    if (o_dtype == FA_DTYPE_FP32) static_cast<float*>(o)[idx] = v;
    else if (o_dtype == FA_DTYPE_BF16) static_cast<__nv_bfloat16*>(o)[idx] = __float2bfloat16_rn(v);
    else static_cast<__half*>(o)[idx] = __float2half_rn(v);
}

// One warp per output row; lanes stride over head_dim, so every partial row is
// read with coalesced 128-byte requests (the reference reads one row per thread,
// src/flash_forward_splitkv.h:390).  lse = log sum_j exp(lse_j);
// O = sum_j exp(lse_j - lse) O_j, the reference's (M, L) algebra with
// lse_j = M_j + log L_j folded into one number per split.
__global__ void combine_kernel(const CombineArgs a, long long total_rows) {
    // launched with programmatic stream serialization behind the kernel that writes the partials:
    // the CTAs are resident and waiting when that kernel ends
    grid_dep_wait();
    const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= total_rows) return;
    const long long unit = row / a.rows_per_unit;
    const long long r = row - unit * a.rows_per_unit;
    const float* lp = a.lse_partial + unit * a.num_splits * a.rows_per_unit + r;
    float m = -INFINITY;
    for (int j = 0; j < a.num_splits; ++j) m = fmaxf(m, lp[j * a.rows_per_unit]);
    float l = 0.0f;
    if (m != -INFINITY)
        for (int j = 0; j < a.num_splits; ++j) l += __expf(lp[j * a.rows_per_unit] - m);
    const float lse = (m == -INFINITY) ? -INFINITY : m + __logf(l);
    if (lane == 0 && a.lse != nullptr) a.lse[row] = lse;
    for (int c = lane; c < a.head_dim; c += 32) {
        float acc = 0.0f;
        if (m != -INFINITY) {
            for (int j = 0; j < a.num_splits; ++j) {
                const float w = __expf(lp[j * a.rows_per_unit] - lse);
                const long long prow = (unit * a.num_splits + j) * a.rows_per_unit + r;
                acc += w * a.o_partial[prow * a.head_dim + c];
            }
        }
        store_out(a.o, a.o_dtype, row * a.head_dim + c, acc);
    }
}

__global__ void merge_kernel(float* o_acc, float* lse_acc, const void* o_part, const float* lse_part,
                             int part_dtype, long long rows, int d) {
    const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float la = lse_acc[row], lb = lse_part[row];
    const float m = fmaxf(la, lb);
    float wa = 0.0f, wb = 0.0f, lse = -INFINITY;
    if (m != -INFINITY) {
        const float ea = __expf(la - m), eb = __expf(lb - m);
        const float s = ea + eb;
        wa = ea / s;
        wb = eb / s;
        lse = m + __logf(s);
    }
    for (int c = lane; c < d; c += 32) {
        const long long i = row * d + c;
        float pv;
        if (part_dtype == FA_DTYPE_FP32) pv = static_cast<const float*>(o_part)[i];
        else if (part_dtype == FA_DTYPE_BF16) pv = __bfloat162float(static_cast<const __nv_bfloat16*>(o_part)[i]);
        else pv = __half2float(static_cast<const __half*>(o_part)[i]);
        // a weight of zero must also silence whatever the other side holds
        const float a_term = (wa == 0.0f) ? 0.0f : wa * o_acc[i];
        const float b_term = (wb == 0.0f) ? 0.0f : wb * pv;
        o_acc[i] = a_term + b_term;
    }
    __syncwarp();
    if (lane == 0) lse_acc[row] = lse;
}

__global__ void cast_kernel(const float* src, void* dst, int o_dtype, long long n) {
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) store_out(dst, o_dtype, i, src[i]);
}

// Row-pitch change for head dims that are not a multiple of 8 (TMA needs 16-byte row
// strides): [rows, d_src] -> [rows, d_dst], zero-filling new columns / dropping extra ones.
// This replaces the reference's scalar zero-padding loader (include/utils.h:85-114) by a
// separate memory-bound pass.
template <typename T>
__global__ void repitch_kernel(const T* src, T* dst, long long rows, int d_src, int d_dst) {
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= rows * d_dst) return;
    const long long r = i / d_dst;
    const int c = static_cast<int>(i - r * d_dst);
    dst[i] = c < d_src ? src[r * d_src + c] : T(0);
}

// keep[unit, row, col] for the geometry in `a` (same map as the tiled kernel).
__global__ void dropout_mask_kernel(const FwdArgs a, uint8_t* keep, long long total) {
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const long long per_unit = static_cast<long long>(a.seqlen_q) * a.seqlen_k;
    const long long unit = idx / per_unit;
    const long long rem = idx - unit * per_unit;
    const int row = static_cast<int>(rem / a.seqlen_k);
    const int col = static_cast<int>(rem - static_cast<long long>(row) * a.seqlen_k);
    const int rb = row / kTile, cb = col / kTile;
    int split = 0, lo = 0;
    if (a.num_splits > 1) {
        split = cb / a.tiles_per_split;
        lo = a.tiles_per_split * split;
    }
    int hi = a.num_splits > 1 ? min(lo + a.tiles_per_split, a.tc) : a.tc;
    const long long q0 = a.q_pos0 + static_cast<long long>(rb) * kTile;
    if (a.window_left >= 0) {
        const long long w = (q0 - a.window_left - a.k_pos0) / kTile;
        lo = max(lo, static_cast<int>(max(0LL, min(w, static_cast<long long>(a.tc)))));
    }
    // upper end of the CTA's tile range (src/flash_forward.h:42-48): it decides how far a later launch
    // of a loop has advanced the stream
    if (a.window_right >= 0) {
        const long long last = q0 + kTile - 1 + a.window_right - a.k_pos0;
        hi = min(hi, last < 0 ? 0 : static_cast<int>(min(last / kTile + 1, static_cast<long long>(a.tc))));
    }
    if (a.is_causal) {
        const long long last = q0 + kTile - 1 - a.k_pos0;
        hi = min(hi, last < 0 ? 0 : static_cast<int>(min(last / kTile + 1, static_cast<long long>(a.tc))));
    }
    const unsigned long long subseq =
        (a.drop.unit0 + unit) * static_cast<unsigned long long>(a.tr * a.num_splits) +
        static_cast<unsigned long long>(rb * a.num_splits + split);
    const int cc = col % kTile, rr = row % kTile;
    const int i = cc / 16;
    const int half = (rr % 16) / 8;
    const int w = 2 * ((cc % 16) / 8) + (cc % 2);
    uint8_t k = 1;
    if (cb >= lo) {
        const uint32_t bits = philox_keep4(a.drop, subseq, continuation(a.drop, hi - lo) + 64ull * (cb - lo) + 8ull * i + 4ull * half);
        k = (bits >> w) & 1u;
    }
    keep[idx] = k;
}

}  // namespace

cudaError_t launch_combine(const CombineArgs& a, long long units, cudaStream_t stream) {
    const long long rows = units * a.rows_per_unit;
    if (rows <= 0) return cudaSuccess;
    const int threads = 256;
    const long long blocks = (rows * 32 + threads - 1) / threads;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(blocks));
    cfg.blockDim = dim3(threads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, combine_kernel, a, rows);
}

cudaError_t launch_merge(float* o_acc, float* lse_acc, const void* o_part, const float* lse_part, int part_dtype,
                         long long rows, int d, cudaStream_t stream) {
    if (rows <= 0) return cudaSuccess;
    const int threads = 256;
    const long long blocks = (rows * 32 + threads - 1) / threads;
    merge_kernel<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(o_acc, lse_acc, o_part, lse_part, part_dtype, rows, d);
    return cudaGetLastError();
}

cudaError_t launch_cast(const float* src, void* dst, int o_dtype, long long n, cudaStream_t stream) {
    if (n <= 0) return cudaSuccess;
    const int threads = 256;
    cast_kernel<<<static_cast<unsigned>((n + threads - 1) / threads), threads, 0, stream>>>(src, dst, o_dtype, n);
    return cudaGetLastError();
}

cudaError_t launch_repitch(const void* src, void* dst, int elem_bytes, long long rows, int d_src, int d_dst,
                           cudaStream_t stream) {
    const long long total = rows * d_dst;
    if (total <= 0) return cudaSuccess;
    const int threads = 256;
    const unsigned blocks = static_cast<unsigned>((total + threads - 1) / threads);
    if (elem_bytes == 2)
        repitch_kernel<uint16_t><<<blocks, threads, 0, stream>>>(static_cast<const uint16_t*>(src), static_cast<uint16_t*>(dst), rows, d_src, d_dst);
    else
        repitch_kernel<uint32_t><<<blocks, threads, 0, stream>>>(static_cast<const uint32_t*>(src), static_cast<uint32_t*>(dst), rows, d_src, d_dst);
    return cudaGetLastError();
}

cudaError_t launch_dropout_mask(const FwdArgs& a, uint8_t* keep, long long units, cudaStream_t stream) {
    const long long total = units * a.seqlen_q * a.seqlen_k;
    if (total <= 0) return cudaSuccess;
    const int threads = 256;
    dropout_mask_kernel<<<static_cast<unsigned>((total + threads - 1) / threads), threads, 0, stream>>>(a, keep, total);
    return cudaGetLastError();
}

}  // namespace fa
