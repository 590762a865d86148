// Tiled flash-attention forward for sm_100a.  Replaces the reference's
// forward_kernel (src/flash_forward.h:13-306) and forward_kernel_splitkv
// (src/flash_forward_splitkv.h:14-344).
//
// One CTA owns one 128-row query tile of one (batch, head) unit, optionally one
// KV split of it, exactly the reference's work decomposition (grid
// (Tr*splits, H, B), src/main.cu:142-158).  Inside the CTA the roles are split by warp:
//   warps 0-3  softmax: thread r owns query row r.  S is read from tensor memory
//              (tcgen05.ld), masked / biased / exponentiated in registers, the
//              16-bit P is written back to tensor memory over S (tcgen05.st), and
//              the running (max, sum) and the lazy rescale of O live here.
//   warp 4     TMA producer: streams the Q tile once and K/V tiles through an
//              mbarrier ring (cp.async.bulk.tensor, 128-byte swizzle).
//   warp 5     MMA issuer: one thread issues tcgen05.mma for S = Q K^T (both
//              operands in shared memory) and O += P V (P in tensor memory, V in
//              shared memory, MN-major), with accumulators in tensor memory.
// The reference keeps O in shared memory and renormalises it every tile
// (src/flash_forward.h:248-290); here O stays un-normalised in tensor memory and
// is divided by the row sum once, in the epilogue.  Two CTAs are resident per SM
// (256 TMEM columns, <= 97 KB shared memory each) so that one CTA's softmax
// overlaps the other's tensor-core work.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "fa_internal.h"
#include "sm100_ptx.cuh"

namespace fa {

namespace {

constexpr int kThreads = 192;
constexpr int kSoftmaxThreads = 128;
constexpr float kRescaleThreshold = 8.0f;  // log2 units: rescale O only when the max grew by > 2^8

template <int D>
struct Cfg {
    static constexpr int kStages = (D == 64) ? 2 : 1;
    static constexpr int kBoxes = D / 64;              // 64-element (128-byte) column blocks per tile
    static constexpr int kTileBytes = kTile * D * 2;   // one Q, K or V tile
    static constexpr int kTmemCols = 256;              // S: [0,128)  (P aliases [0,64));  O: [128,128+D)
    static constexpr int kSmemQ = 0;
    static constexpr int kSmemK = kTileBytes;
    static constexpr int kSmemV = kSmemK + kStages * kTileBytes;
    static constexpr int kSmemBar = kSmemV + kStages * kTileBytes;
    static constexpr int kNumBars = 4 + 4 * kStages;
    static constexpr int kSmemBytes = kSmemBar + 8 * kNumBars + 16 + 1024;  // + alignment slack
};

struct TileRange {
    int lo, hi;  // KV tiles [lo, hi)
};

__device__ __forceinline__ TileRange kv_tile_range(const FwdArgs& a, int rb, int split) {
    const long long q0 = a.q_pos0 + static_cast<long long>(rb) * kTile;
    int lo = 0, hi = a.tc;
    if (a.num_splits > 1) {  // src/flash_forward_splitkv.h:40-43
        lo = a.tiles_per_split * split;
        hi = min(lo + a.tiles_per_split, a.tc);
    }
    if (a.window_left >= 0) {  // src/flash_forward.h:39
        const long long w = (q0 - a.window_left - a.k_pos0) / kTile;  // truncating, like the reference
        lo = max(lo, static_cast<int>(max(0LL, min(w, static_cast<long long>(a.tc)))));
    }
    if (a.window_right >= 0) {  // src/flash_forward.h:42-44
        const long long last = q0 + kTile - 1 + a.window_right - a.k_pos0;
        hi = min(hi, last < 0 ? 0 : static_cast<int>(min(last / kTile + 1, static_cast<long long>(a.tc))));
    }
    if (a.is_causal) {  // src/flash_forward.h:46-48
        const long long last = q0 + kTile - 1 - a.k_pos0;
        hi = min(hi, last < 0 ? 0 : static_cast<int>(min(last / kTile + 1, static_cast<long long>(a.tc))));
    }
    return {lo, hi};
}

template <bool kBf16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    if constexpr (kBf16) {
        __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&t);
    } else {
        __half2 t = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&t);
    }
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int D, bool kBf16, bool kAlibi, bool kDropout>
__global__ void __launch_bounds__(kThreads, 2)
fwd_tiled_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const FwdArgs a) {
    using C = Cfg<D>;
    extern __shared__ uint8_t smem_raw[];
    // 128-byte-swizzled tiles need a 1024-byte aligned base
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t sQ = smem_base + C::kSmemQ;
    const uint32_t sK = smem_base + C::kSmemK;
    const uint32_t sV = smem_base + C::kSmemV;
    const uint32_t bar0 = smem_base + C::kSmemBar;
    // barrier map
    const uint32_t bar_q_full = bar0;
    const uint32_t bar_s_full = bar0 + 8;
    const uint32_t bar_p_full = bar0 + 16;
    const uint32_t bar_o_full = bar0 + 24;
    const uint32_t bar_k_full = bar0 + 32;                      // [kStages]
    const uint32_t bar_k_empty = bar_k_full + 8 * C::kStages;   // [kStages]
    const uint32_t bar_v_full = bar_k_empty + 8 * C::kStages;   // [kStages]
    const uint32_t bar_v_empty = bar_v_full + 8 * C::kStages;   // [kStages]
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + C::kSmemBar + 8 * C::kNumBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + C::kSmemBar + 8 * C::kNumBars + 4);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // ---- which tile is this CTA ------------------------------------------------
    const int per_unit = a.tr * a.num_splits;
    const int unit = blockIdx.x / per_unit;
    const int bx = blockIdx.x - unit * per_unit;
    const int split = bx % a.num_splits;
    int rb = bx / a.num_splits;
    if (a.is_causal) rb = a.tr - 1 - rb;  // heaviest query tiles first
    const TileRange range = kv_tile_range(a, rb, split);
    const int n_tiles = range.hi - range.lo;

    // ---- set-up ----------------------------------------------------------------
    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(bar_q_full, 1);
        mbar_init(bar_s_full, 1);
        mbar_init(bar_p_full, kSoftmaxThreads);
        mbar_init(bar_o_full, 1);
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(bar_k_full + 8 * s, 1);
            mbar_init(bar_k_empty + 8 * s, 1);
            mbar_init(bar_v_full + 8 * s, 1);
            mbar_init(bar_v_empty + 8 * s, 1);
        }
        mbar_fence_init();
    }
    if (warp == 5 && n_tiles > 0) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), C::kTmemCols);
        tmem_relinquish();
    }
    if (warp == 4 && lane == 0) {
        tma_prefetch_desc(&tmap_q);
        tma_prefetch_desc(&tmap_k);
        tma_prefetch_desc(&tmap_v);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = (n_tiles > 0) ? *tmem_slot : 0u;
    const uint32_t tmem_s = tmem_base;          // S accumulator, 128 fp32 columns
    const uint32_t tmem_p = tmem_base;          // P (16-bit, two per column) over S[0,64)
    const uint32_t tmem_o = tmem_base + kTile;  // O accumulator, D fp32 columns

    int fail = 0;

    if (n_tiles > 0 && warp == 4) {
        // ======================= TMA producer ===================================
        if (lane == 0) {
            mbar_expect_tx(bar_q_full, C::kTileBytes);
#pragma unroll
            for (int b = 0; b < C::kBoxes; ++b)
                tma_load_3d(sQ + b * (kTile * 128), &tmap_q, bar_q_full, b * 64, rb * kTile, unit);
            for (int j = 0; j < n_tiles; ++j) {
                const int st = j % C::kStages;
                const uint32_t ph = (j / C::kStages) & 1;
                const int row = (range.lo + j) * kTile;
                if (!mbar_wait(bar_k_empty + 8 * st, ph ^ 1, abort_flag)) { fail = 1; break; }
                mbar_expect_tx(bar_k_full + 8 * st, C::kTileBytes);
#pragma unroll
                for (int b = 0; b < C::kBoxes; ++b)
                    tma_load_3d(sK + st * C::kTileBytes + b * (kTile * 128), &tmap_k, bar_k_full + 8 * st, b * 64, row, unit);
                if (!mbar_wait(bar_v_empty + 8 * st, ph ^ 1, abort_flag)) { fail = 2; break; }
                mbar_expect_tx(bar_v_full + 8 * st, C::kTileBytes);
#pragma unroll
                for (int b = 0; b < C::kBoxes; ++b)
                    tma_load_3d(sV + st * C::kTileBytes + b * (kTile * 128), &tmap_v, bar_v_full + 8 * st, b * 64, row, unit);
            }
        }
    } else if (n_tiles > 0 && warp == 5) {
        // ======================= MMA issuer =====================================
        if (lane == 0) {
            constexpr uint32_t idesc_qk = make_idesc_f16(kTile, kTile, kBf16, false);
            constexpr uint32_t idesc_pv = make_idesc_f16(kTile, D, kBf16, true);
            auto issue_qk = [&](int st) {
                // S = Q K^T: K-dimension = head_dim, 16 elements (32 bytes) per instruction
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t off = (ks / 4) * (kTile * 128) + (ks % 4) * 32;
                    umma_ss(tmem_s, make_smem_desc(sQ + off, 0, 1024),
                            make_smem_desc(sK + st * C::kTileBytes + off, 0, 1024), idesc_qk, ks > 0);
                }
            };
            do {
                if (!mbar_wait(bar_q_full, 0, abort_flag)) { fail = 3; break; }
                if (!mbar_wait(bar_k_full, 0, abort_flag)) { fail = 4; break; }
                tc_fence_after_sync();
                issue_qk(0);
                umma_commit(bar_k_empty);
                umma_commit(bar_s_full);
                for (int j = 0; j < n_tiles; ++j) {
                    const int st = j % C::kStages;
                    const uint32_t ph = (j / C::kStages) & 1;
                    if (!mbar_wait(bar_p_full, j & 1, abort_flag)) { fail = 5; break; }
                    if (!mbar_wait(bar_v_full + 8 * st, ph, abort_flag)) { fail = 6; break; }
                    tc_fence_after_sync();
                    // O += P V: K-dimension = 128 keys, 16 per instruction = 8 TMEM columns of P and
                    // 16 rows (2048 bytes) of V; the two 64-wide halves of V are 16 KB apart.
#pragma unroll
                    for (int ks = 0; ks < kTile / 16; ++ks)
                        umma_ts(tmem_o, tmem_p + ks * 8,
                                make_smem_desc(sV + st * C::kTileBytes + ks * 2048, kTile * 128, 1024), idesc_pv,
                                (j > 0 || ks > 0) ? 1u : 0u);
                    umma_commit(bar_v_empty + 8 * st);
                    if (j + 1 < n_tiles) {
                        const int st1 = (j + 1) % C::kStages;
                        const uint32_t ph1 = ((j + 1) / C::kStages) & 1;
                        if (!mbar_wait(bar_k_full + 8 * st1, ph1, abort_flag)) { fail = 7; break; }
                        tc_fence_after_sync();
                        issue_qk(st1);
                        umma_commit(bar_k_empty + 8 * st1);
                        umma_commit(bar_s_full);
                    } else {
                        umma_commit(bar_o_full);
                    }
                }
            } while (false);
        }
    } else if (warp < 4) {
        // ======================= softmax / epilogue =============================
        const int r = threadIdx.x;                       // row inside the tile
        const int row = rb * kTile + r;                  // row inside the unit
        const long long qpos = a.q_pos0 + row;
        const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
        float m_ref = -INFINITY;  // running max in log2 units (scaled, biased)
        float l_sum = 0.0f;
        float slope2 = 0.0f;
        if constexpr (kAlibi) slope2 = a.alibi_slopes[unit % a.heads] * 1.4426950408889634f;
        unsigned long long subseq = 0;
        if constexpr (kDropout)
            subseq = (a.drop.unit0 + unit) * static_cast<unsigned long long>(per_unit) +
                     static_cast<unsigned long long>(rb * a.num_splits + split);

        for (int j = 0; j < n_tiles; ++j) {
            const int cb = range.lo + j;
            const long long kbase = a.k_pos0 + static_cast<long long>(cb) * kTile;
            // the TMEM loads below are warp-collective: decide as a warp
            if (!__all_sync(0xffffffffu, mbar_wait(bar_s_full, j & 1, abort_flag))) { fail = 8; break; }
            tc_fence_after_sync();

            uint32_t sr[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld32(tmem_s + lane_base + c * 32, sr[c]);
            tmem_wait_ld();

            // columns this row may attend to inside the tile: [c_lo, c_hi]
            int c_lo = 0, c_hi = min(kTile - 1, a.seqlen_k - 1 - cb * kTile);
            if (a.is_causal) c_hi = static_cast<int>(min(static_cast<long long>(c_hi), qpos - kbase));
            if (a.window_right >= 0) c_hi = static_cast<int>(min(static_cast<long long>(c_hi), qpos + a.window_right - kbase));
            if (a.window_left >= 0) c_lo = static_cast<int>(max(0LL, min(qpos - a.window_left - kbase, 128LL)));
            const bool need_mask = __any_sync(0xffffffffu, c_lo > 0 || c_hi < kTile - 1);

            // scaled (and biased) scores in log2 units, and the tile max
            float m_tile = -INFINITY;
            const float dist0 = static_cast<float>(qpos - kbase);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    float s = __uint_as_float(sr[c][i]) * a.scale_log2;
                    if constexpr (kAlibi) s = fmaf(-slope2, fabsf(dist0 - static_cast<float>(c * 32 + i)), s);
                    if (need_mask) {
                        const int col = c * 32 + i;
                        if (col < c_lo || col > c_hi) s = -INFINITY;
                    }
                    sr[c][i] = __float_as_uint(s);
                    m_tile = fmaxf(m_tile, s);
                }
            }

            // lazy rescale: keep the old reference max unless the new one is much larger
            float m_new = m_ref;
            float factor = 1.0f;
            if (m_tile > m_ref + kRescaleThreshold || m_ref == -INFINITY) {
                m_new = fmaxf(m_ref, m_tile);
                factor = (m_ref == -INFINITY) ? 0.0f : fast_exp2(m_ref - m_new);
            }
            const bool rescale = (j > 0) && (m_new != m_ref);
            if (__any_sync(0xffffffffu, rescale)) {
                // PV of the previous tile has completed (its commit precedes s_full), so O is stable.
                const float f = rescale ? factor : 1.0f;
#pragma unroll
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t orow[32];
                    tmem_ld32(tmem_o + lane_base + c * 32, orow);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) orow[i] = __float_as_uint(__uint_as_float(orow[i]) * f);
                    tmem_st32(tmem_o + lane_base + c * 32, orow);
                }
            }
            l_sum *= (m_new != m_ref) ? factor : 1.0f;
            m_ref = m_new;
            const float m_use = (m_ref == -INFINITY) ? 0.0f : m_ref;

            // dropout keep bits of this row for the tile: bit 4*i + w <-> 16-column block i,
            // w = 2*((col%16)/8) + col%2
            uint32_t keep_bits = 0xffffffffu;
            if constexpr (kDropout) {
                const unsigned long long tile_first = 64ull * static_cast<unsigned long long>(j);
                uint32_t mine = 0;
                if (lane < 16)  // lane = 2*i + row-half: draws 8*i + 4*half + {0..3}
                    mine = philox_keep4(a.drop, subseq, tile_first + 4ull * lane);
                const int half = (lane >> 3) & 1;
                keep_bits = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i) keep_bits |= __shfl_sync(0xffffffffu, mine, 2 * i + half) << (4 * i);
            }

            // P = exp2(s - m), row sum over the undropped P (src/flash_forward.h:198-213, 221-237)
            float acc = 0.0f;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t pr[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int col = c * 64 + 2 * i;
                    const float p0 = fast_exp2(__uint_as_float(sr[col / 32][col % 32]) - m_use);
                    const float p1 = fast_exp2(__uint_as_float(sr[(col + 1) / 32][(col + 1) % 32]) - m_use);
                    acc += p0 + p1;
                    uint32_t packed = pack2<kBf16>(p0, p1);
                    if constexpr (kDropout) {
                        const uint32_t nib = keep_bits >> (4 * (col / 16) + 2 * ((col % 16) / 8));
                        const uint32_t msk = ((nib & 1u) ? 0x0000ffffu : 0u) | ((nib & 2u) ? 0xffff0000u : 0u);
                        packed &= msk;
                    }
                    pr[i] = packed;
                }
                tmem_st32(tmem_p + lane_base + c * 32, pr);
            }
            l_sum += acc;
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(bar_p_full);
        }

        // ---- epilogue: normalise and write O, LSE --------------------------------
        bool have_o = false;
        if (n_tiles > 0 && fail == 0) {
            if (__all_sync(0xffffffffu, mbar_wait(bar_o_full, 0, abort_flag))) { tc_fence_after_sync(); have_o = true; }
            else fail = 9;
        }
        float inv = 0.0f;
        if (l_sum > 0.0f) inv = (kDropout ? a.drop.inv_keep : 1.0f) / l_sum;
        const bool row_ok = row < a.seqlen_q;
        const float lse_val = (l_sum > 0.0f) ? (m_ref * 0.6931471805599453f + __logf(l_sum)) : -INFINITY;
        const long long unit_ll = unit;
        if (a.num_splits > 1) {
            const long long prow = (unit_ll * a.num_splits + split) * a.seqlen_q + row;
            if (row_ok) a.lse_partial[prow] = lse_val;
        } else if (a.lse != nullptr && row_ok) {
            a.lse[unit_ll * a.seqlen_q + row] = lse_val;
        }
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
            uint32_t orow[32];
            if (have_o) {
                tmem_ld32(tmem_o + lane_base + c * 32, orow);
                tmem_wait_ld();
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) orow[i] = 0u;
            }
            if (!row_ok) continue;
            const int col0 = c * 32;
            if (a.num_splits > 1 || a.o_is_fp32) {
                float* dst = (a.num_splits > 1)
                                 ? a.o_partial + ((unit_ll * a.num_splits + split) * a.seqlen_q + row) * a.head_dim
                                 : static_cast<float*>(a.o) + (unit_ll * a.seqlen_q + row) * a.head_dim;
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    if (col0 + i < a.head_dim) {
                        float4 v4 = make_float4(__uint_as_float(orow[i]) * inv, __uint_as_float(orow[i + 1]) * inv,
                                                __uint_as_float(orow[i + 2]) * inv, __uint_as_float(orow[i + 3]) * inv);
                        *reinterpret_cast<float4*>(dst + col0 + i) = v4;
                    }
                }
            } else {
                uint16_t* dst = static_cast<uint16_t*>(a.o) + (unit_ll * a.seqlen_q + row) * a.head_dim;
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    if (col0 + i < a.head_dim) {
                        uint4 v4;
                        v4.x = pack2<kBf16>(__uint_as_float(orow[i]) * inv, __uint_as_float(orow[i + 1]) * inv);
                        v4.y = pack2<kBf16>(__uint_as_float(orow[i + 2]) * inv, __uint_as_float(orow[i + 3]) * inv);
                        v4.z = pack2<kBf16>(__uint_as_float(orow[i + 4]) * inv, __uint_as_float(orow[i + 5]) * inv);
                        v4.w = pack2<kBf16>(__uint_as_float(orow[i + 6]) * inv, __uint_as_float(orow[i + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + col0 + i) = v4;
                    }
                }
            }
        }
    }

    // ---- teardown ------------------------------------------------------------------
    if (fail != 0) {
        *abort_flag = 1;
        if (a.status != nullptr) atomicExch(a.status, 100 + fail);
        // give copies that are still in flight time to land before the CTA's memory is reused
        const long long t0 = clock64();
        while (clock64() - t0 < 200000) { }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 5 && n_tiles > 0) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

template <int D, bool kBf16, bool kAlibi, bool kDropout>
cudaError_t launch_one(const FwdArgs& a, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                       int units, cudaStream_t stream) {
    auto kern = fwd_tiled_kernel<D, kBf16, kAlibi, kDropout>;
    constexpr int smem = Cfg<D>::kSmemBytes;
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    const long long ctas = static_cast<long long>(units) * a.tr * a.num_splits;
    if (ctas <= 0 || ctas > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    kern<<<static_cast<unsigned>(ctas), kThreads, smem, stream>>>(tq, tk, tv, a);
    return cudaGetLastError();
}

template <int D, bool kBf16>
cudaError_t launch_flags(const FwdArgs& a, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                         int units, bool alibi, bool dropout, cudaStream_t stream) {
    if (alibi) {
        return dropout ? launch_one<D, kBf16, true, true>(a, tq, tk, tv, units, stream)
                       : launch_one<D, kBf16, true, false>(a, tq, tk, tv, units, stream);
    }
    return dropout ? launch_one<D, kBf16, false, true>(a, tq, tk, tv, units, stream)
                   : launch_one<D, kBf16, false, false>(a, tq, tk, tv, units, stream);
}

}  // namespace

cudaError_t launch_fwd_tiled(const FwdArgs& a, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                             int units, bool bf16, bool dropout, cudaStream_t stream) {
    const bool alibi = a.alibi_slopes != nullptr;
    if (a.head_dim <= 64) {
        return bf16 ? launch_flags<64, true>(a, tq, tk, tv, units, alibi, dropout, stream)
                    : launch_flags<64, false>(a, tq, tk, tv, units, alibi, dropout, stream);
    }
    return bf16 ? launch_flags<128, true>(a, tq, tk, tv, units, alibi, dropout, stream)
                : launch_flags<128, false>(a, tq, tk, tv, units, alibi, dropout, stream);
}

}  // namespace fa
