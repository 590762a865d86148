// Internal declarations shared by the C-ABI translation unit and the kernels.
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>
#include "philox.cuh"

namespace fa {

constexpr int kTile = 128;  // Br = Bc = 128, as the reference fixes them (src/main.cu:116-117)

// Division by a launch-constant divisor without the hardware's slow integer divide: the
// quotient is mulhi(x, m) with m = floor(2^32 / d) + 1, which is floor(x / d) or one more.
struct FastDiv {
    uint32_t d, m;
};
inline FastDiv make_fastdiv(uint32_t d) {
    FastDiv f;
    f.d = d < 1 ? 1 : d;
    f.m = f.d == 1 ? 0u : static_cast<uint32_t>((1ull << 32) / f.d) + 1u;
    return f;
}

// Device-side argument block of the tiled forward kernel (the successor of
// mykernelParamType, include/utils.h:21-44).  Q/K/V travel as TMA tensor maps.
struct FwdArgs {
    void* o;                // [units, Nq, d] in o dtype (non-split)
    float* lse;             // [units, Nq] or null
    float* o_partial;       // [units, splits, Nq, d] fp32 (split)
    float* lse_partial;     // [units, splits, Nq]
    const float* alibi_slopes;
    int* status;
    int heads;
    int units;              // batch * heads of this launch
    int unit_group;         // units whose CTAs are interleaved in launch order (1 = unit-major)
    int kv_group;           // query units per K/V unit (grouped-query attention); K/V unit = unit / kv_group
    int seqlen_q, seqlen_k, head_dim;
    int tr, tc;             // query / key tiles
    int num_splits, tiles_per_split;
    float scale_log2;       // softmax_scale * log2(e)
    int is_causal, window_left, window_right;
    long long q_pos0, k_pos0;
    int o_is_fp32;
    int o_tma;              // O leaves through the TMA store map (16-bit output, unsplit launch)
    float* accum_o;         // running fp32 result [units, Nq, d] merged in the epilogue, or null
    float* accum_lse;       // running log-sum-exp [units, Nq]
    int accum_first;        // nothing is carried yet: the running pair is only written
    int accum_final;        // last block: o / lse receive the merged result (the running O is then left as it is)
    // launch order of the CTAs (filled by launch_fwd_tiled): divisors of the block index
    FastDiv div_group_ctas, div_gsize, div_last_gsize, div_splits, div_kv_group;
    DropoutParams drop;
};

// Launchers implemented in the .cu files; all return a cudaError_t.  `to` is the store map of O
// (32-row boxes); it is read only when a.o_tma is set.
cudaError_t launch_fwd_tiled(const FwdArgs& a, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                             const CUtensorMap& to, int units, bool bf16, bool dropout, cudaStream_t stream);

// Device-side argument block of the decode kernel (seqlen_q = 1).
struct DecodeArgs {
    const void* q;          // [units, d]
    void* o;                // [units, d] (non-split)
    float* lse;             // [units] or null
    float* o_partial;       // [units, splits, d] fp32 (split)
    float* lse_partial;     // [units, splits]
    const float* alibi_slopes;
    int* status;
    int heads;
    int kv_group;           // query units per K/V unit; K/V unit = unit / kv_group
    int subgroups;          // CTAs (of up to eight query columns) per K/V unit on the packed path; set by launch_decode
    int seqlen_q;           // query rows per unit, 1..8
    int seqlen_k, head_dim;
    int tc;
    int num_splits, tiles_per_split;
    float scale_log2;
    int is_causal, window_left, window_right;
    long long q_pos0, k_pos0;
    int o_is_fp32;
    DropoutParams drop;
};
cudaError_t launch_decode(const DecodeArgs& a, const CUtensorMap& tk, const CUtensorMap& tv, int units, bool bf16,
                          cudaStream_t stream);

struct CombineArgs {
    const float* o_partial; const float* lse_partial;
    void* o; float* lse;
    long long rows_per_unit;   // Nq
    int num_splits, head_dim;
    int o_dtype;               // FA_DTYPE_*
};
cudaError_t launch_combine(const CombineArgs& a, long long units, cudaStream_t stream);
cudaError_t launch_merge(float* o_acc, float* lse_acc, const void* o_part, const float* lse_part, int part_dtype,
                         long long rows, int d, cudaStream_t stream);
cudaError_t launch_cast(const float* src, void* dst, int o_dtype, long long n, cudaStream_t stream);
cudaError_t launch_repitch(const void* src, void* dst, int elem_bytes, long long rows, int d_src, int d_dst,
                           cudaStream_t stream);
cudaError_t launch_dropout_mask(const FwdArgs& a, uint8_t* keep, long long units, cudaStream_t stream);

}  // namespace fa
