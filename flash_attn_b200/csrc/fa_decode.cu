// Split-KV decode for sm_100a: one query row per (batch, head) unit against a long
// K/V.  Replaces the reference's forward_kernel_splitkv (src/flash_forward_splitkv.h:14-344)
// for seqlen_q = 1, where the work is a pure stream of K and V through the SM: every byte
// is used once, so the kernel is built around the TMA ring and nothing else may stall it.
//
// One CTA = one (unit, split).  The operands are swapped so that the 128 lanes of tensor
// memory hold KEYS, not queries:
//     S^T[128 keys x 16] = K_tile[128 x d] * Qpad^T[d x 16]      (tcgen05.mma, M=128, N=16)
//     O^T[d x 16]       += V_tile^T[d x 128 keys] * P[128 keys x 16]
// Column 0 of S^T / O^T belongs to the query; columns 1-15 are padding whose inputs (rows
// 1-15 of the Q and P operand tiles) are never initialised and whose results are never
// read -- an operand row only influences its own output column.  Thread r of the four
// softmax warps owns key r of every tile, so masking, ALiBi, exp and dropout are spread over
// 128 threads; one CTA-wide max per chunk of four tiles keeps them on a common scale.
// The MMAs are tiny (N = 16): the tensor pipe is a convenient dot-product engine that
// reads K/V straight from the swizzled TMA tiles, and the kernel stays HBM-bound.
//
// Stream order of the TMA ring: K(0), K(1), V(0), K(2), V(1), ... (chunks of four tiles), so
// the scores of chunk c+1 are computed while the softmax of chunk c runs.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "fa_internal.h"
#include "sm100_ptx.cuh"

namespace fa {

namespace {

constexpr int kDThreads = 192;
constexpr int kChunkTiles = 4;             // KV tiles per softmax chunk
constexpr int kDStages = 3;                // ring slots of one K or V tile
constexpr int kDTileBytes = kTile * 128 * 2;  // 32 KB: [128 keys x 128 columns], two 64-column boxes
constexpr int kPTileBytes = 2048;          // P operand of one tile: two 1 KB atoms, row 0 = 64 keys each
constexpr int kDSmemRing = 0;
constexpr int kDSmemP = kDStages * kDTileBytes;                  // 8 KB + 2 KB that garbage rows may touch
constexpr int kDSmemQ = kDSmemP + kChunkTiles * kPTileBytes + 2048;  // 2 KB + 2 KB slack
constexpr int kDSmemBar = kDSmemQ + 4096;
constexpr int kDNumBars = 2 * kDStages + 2 + 2 + 3;
constexpr int kDSmemRed = kDSmemBar + 8 * kDNumBars;             // float[2][4] + float[4]
constexpr int kDSmemMisc = kDSmemRed + 64;
constexpr int kDSmemBytes = kDSmemMisc + 16 + 1024;
constexpr int kDTmemCols = 256;            // S^T: 2 buffers x 4 tiles x 16 columns; O^T: 16 columns at 128

constexpr float kDLog2e = 1.4426950408889634f;
constexpr float kDLn2 = 0.6931471805599453f;

__host__ __device__ constexpr uint32_t make_idesc_swapped(bool is_bf16, bool a_mn_major) {
    return (1u << 4) | ((is_bf16 ? 1u : 0u) << 7) | ((is_bf16 ? 1u : 0u) << 10) |
           ((a_mn_major ? 1u : 0u) << 15) | (0u << 16) | (static_cast<uint32_t>(16 >> 3) << 17) |
           (static_cast<uint32_t>(kTile >> 4) << 24);
}

__device__ __forceinline__ float ex2f(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t tmem_ld1(uint32_t taddr) {
    uint32_t r;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r) : "r"(taddr) : "memory");
    return r;
}
__device__ __forceinline__ void tmem_st1(uint32_t taddr, uint32_t v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(taddr), "r"(v) : "memory");
}
__device__ __forceinline__ bool mbar_wait_warp_ok(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag) ? 1 : 0) != 0;
}
__device__ __forceinline__ void named_barrier_128() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <bool kBf16>
__global__ void __launch_bounds__(kDThreads, 2)
decode_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v, const DecodeArgs a) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t sRing = smem_base + kDSmemRing;
    const uint32_t sP = smem_base + kDSmemP;
    const uint32_t sQ = smem_base + kDSmemQ;
    const uint32_t bar0 = smem_base + kDSmemBar;
    const uint32_t bar_full = bar0;                          // [kDStages]
    const uint32_t bar_empty = bar_full + 8 * kDStages;      // [kDStages]
    const uint32_t bar_s_full = bar_empty + 8 * kDStages;    // [2]
    const uint32_t bar_s_free = bar_s_full + 16;             // [2]
    const uint32_t bar_p_full = bar_s_free + 16;
    const uint32_t bar_p_free = bar_p_full + 8;
    const uint32_t bar_o_done = bar_p_free + 8;
    float* red = reinterpret_cast<float*>(smem_gen + kDSmemRed);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + kDSmemMisc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + kDSmemMisc + 4);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.x / a.num_splits;
    const int split = blockIdx.x - unit * a.num_splits;
    const int kv_unit = a.kv_group > 1 ? unit / a.kv_group : unit;  // grouped-query attention: K/V head of this unit

    // KV tiles of this split, clipped by the masks at tile granularity (as kv_tile_range
    // of the tiled kernel, for the single query row at position q_pos0)
    int lo = a.tiles_per_split * split, hi = min(lo + a.tiles_per_split, a.tc);
    if (a.window_left >= 0) {
        const long long w = (a.q_pos0 - a.window_left - a.k_pos0) / kTile;
        lo = max(lo, static_cast<int>(max(0LL, min(w, static_cast<long long>(a.tc)))));
    }
    if (a.window_right >= 0) {
        const long long last = a.q_pos0 + a.window_right - a.k_pos0;
        hi = min(hi, last < 0 ? 0 : static_cast<int>(min(last / kTile + 1, static_cast<long long>(a.tc))));
    }
    if (a.is_causal) {
        const long long last = a.q_pos0 - a.k_pos0;
        hi = min(hi, last < 0 ? 0 : static_cast<int>(min(last / kTile + 1, static_cast<long long>(a.tc))));
    }
    const int n_tiles = hi > lo ? hi - lo : 0;
    const int n_chunks = (n_tiles + kChunkTiles - 1) / kChunkTiles;
    auto chunk_tiles = [&](int c) { return min(kChunkTiles, n_tiles - c * kChunkTiles); };

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < kDStages; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_s_full + 8 * i, 1);
            mbar_init(bar_s_free + 8 * i, 4);
        }
        mbar_init(bar_p_full, 4);
        mbar_init(bar_p_free, 1);
        mbar_init(bar_o_done, 1);
        mbar_fence_init();
    }
    if (warp == 5 && n_tiles > 0) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kDTmemCols);
        tmem_relinquish();
    }
    if (threadIdx.x < 16 && n_tiles > 0) {
        // the query row goes to row 0 of the two Q atoms (16-byte unit u -> atom u/8, unit u%8)
        const int u = threadIdx.x;
        uint4 val = make_uint4(0u, 0u, 0u, 0u);
        if (u * 8 < a.head_dim)
            val = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(a.q) + static_cast<long long>(unit) * a.head_dim + u * 8);
        *reinterpret_cast<uint4*>(smem_gen + kDSmemQ + (u >> 3) * 1024 + (u & 7) * 16) = val;
        fence_proxy_async_smem();
    }
    if (warp == 4 && lane == 0) {
        tma_prefetch_desc(&tmap_k);
        tma_prefetch_desc(&tmap_v);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = (n_tiles > 0) ? *tmem_slot : 0u;
    const uint32_t tmem_o = tmem_base + 128;

    int fail = 0;

    if (n_tiles > 0 && warp == 4) {
        // ======================= TMA producer ===================================
        if (lane == 0) {
            int slot = 0;  // running count of tiles pushed into the ring
            auto push = [&](const CUtensorMap* map, int tile) -> bool {
                const int st = slot % kDStages;
                const uint32_t ph = (slot / kDStages) & 1;
                if (!mbar_wait(bar_empty + 8 * st, ph ^ 1, abort_flag)) return false;
                mbar_expect_tx(bar_full + 8 * st, kDTileBytes);
                tma_load_3d(sRing + st * kDTileBytes, map, bar_full + 8 * st, 0, tile * kTile, kv_unit);
                tma_load_3d(sRing + st * kDTileBytes + kTile * 128, map, bar_full + 8 * st, 64, tile * kTile, kv_unit);
                ++slot;
                return true;
            };
            auto push_chunk = [&](const CUtensorMap* map, int c) -> bool {
                for (int t = 0; t < chunk_tiles(c); ++t)
                    if (!push(map, lo + c * kChunkTiles + t)) return false;
                return true;
            };
            bool ok = push_chunk(&tmap_k, 0);
            for (int c = 0; ok && c < n_chunks; ++c) {
                if (c + 1 < n_chunks) ok = push_chunk(&tmap_k, c + 1);
                if (ok) ok = push_chunk(&tmap_v, c);
            }
            if (!ok) fail = 1;
        }
    } else if (n_tiles > 0 && warp == 5) {
        // ======================= MMA issuer =====================================
        if (lane == 0) {
            constexpr uint32_t idesc_qk = make_idesc_swapped(kBf16, false);
            constexpr uint32_t idesc_pv = make_idesc_swapped(kBf16, true);
            int slot = 0;
            auto qk_chunk = [&](int c) -> bool {
                const int buf = c & 1;
                if (c >= 2 && !mbar_wait(bar_s_free + 8 * buf, ((c >> 1) - 1) & 1, abort_flag)) return false;
                tc_fence_after_sync();
                for (int t = 0; t < chunk_tiles(c); ++t) {
                    const int st = slot % kDStages;
                    if (!mbar_wait(bar_full + 8 * st, (slot / kDStages) & 1, abort_flag)) return false;
                    tc_fence_after_sync();
                    const uint32_t kt = sRing + st * kDTileBytes;
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks) {
                        const uint32_t off = (ks / 4) * (kTile * 128) + (ks % 4) * 32;
                        const uint32_t qoff = (ks / 4) * 1024 + (ks % 4) * 32;
                        umma_ss(tmem_base + buf * 64 + t * 16, make_smem_desc(kt + off, 0, 1024),
                                make_smem_desc(sQ + qoff, 0, 1024), idesc_qk, ks > 0 ? 1u : 0u);
                    }
                    umma_commit(bar_empty + 8 * st);
                    ++slot;
                }
                umma_commit(bar_s_full + 8 * buf);
                return true;
            };
            auto pv_chunk = [&](int c) -> bool {
                if (!mbar_wait(bar_p_full, c & 1, abort_flag)) return false;
                tc_fence_after_sync();
                for (int t = 0; t < chunk_tiles(c); ++t) {
                    const int st = slot % kDStages;
                    if (!mbar_wait(bar_full + 8 * st, (slot / kDStages) & 1, abort_flag)) return false;
                    tc_fence_after_sync();
                    const uint32_t vt = sRing + st * kDTileBytes;
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks) {
                        // A = V^T: 16 keys (2048 bytes) per step, the two 64-column halves 16 KB apart
                        const uint32_t poff = t * kPTileBytes + (ks / 4) * 1024 + (ks % 4) * 32;
                        umma_ss(tmem_o, make_smem_desc(vt + ks * 2048, kTile * 128, 1024),
                                make_smem_desc(sP + poff, 0, 1024), idesc_pv, (c > 0 || t > 0 || ks > 0) ? 1u : 0u);
                    }
                    umma_commit(bar_empty + 8 * st);
                    ++slot;
                }
                umma_commit(bar_p_free);
                return true;
            };
            bool ok = qk_chunk(0);
            for (int c = 0; ok && c < n_chunks; ++c) {
                if (c + 1 < n_chunks) ok = qk_chunk(c + 1);
                if (ok) ok = pv_chunk(c);
            }
            if (ok) umma_commit(bar_o_done);
            else fail = 2;
        }
    } else if (warp < 4) {
        // ======================= softmax over keys / epilogue ===================
        const int r = threadIdx.x;  // key inside a tile; output column in the epilogue
        const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
        const float scale2 = a.scale_log2;
        float slope2 = 0.0f;
        if (a.alibi_slopes != nullptr) slope2 = a.alibi_slopes[unit % a.heads] * kDLog2e;
        const bool dropout = a.drop.threshold != 0ull;
        const unsigned long long subseq =
            (a.drop.unit0 + unit) * static_cast<unsigned long long>(a.num_splits) + static_cast<unsigned long long>(split);
        float m_ref = -INFINITY;  // CTA-wide running max, log2 units
        float l_part = 0.0f;      // this thread's share of the row sum

        for (int c = 0; c < n_chunks; ++c) {
            const int buf = c & 1;
            const int nt = chunk_tiles(c);
            bool ok = mbar_wait_warp_ok(bar_s_full + 8 * buf, (c >> 1) & 1, abort_flag);
            if (!ok) fail = 3;
            tc_fence_after_sync();
            float v[kChunkTiles];
#pragma unroll
            for (int t = 0; t < kChunkTiles; ++t) {
                uint32_t raw = 0;
                if (t < nt) raw = tmem_ld1(tmem_base + lane_base + buf * 64 + t * 16);
                v[t] = __uint_as_float(raw);
            }
            tmem_wait_ld();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_s_free + 8 * buf);

            float m_thr = -INFINITY;
#pragma unroll
            for (int t = 0; t < kChunkTiles; ++t) {
                const int tile = lo + c * kChunkTiles + t;
                const long long key = static_cast<long long>(tile) * kTile + r;
                const long long kpos = a.k_pos0 + key;
                bool keep = t < nt && key < a.seqlen_k;
                if (a.is_causal && kpos > a.q_pos0) keep = false;
                if (a.window_left >= 0 && a.q_pos0 - kpos > a.window_left) keep = false;
                if (a.window_right >= 0 && kpos - a.q_pos0 > a.window_right) keep = false;
                float s = v[t] * scale2;
                if (slope2 != 0.0f) s = fmaf(-slope2, fabsf(static_cast<float>(a.q_pos0 - kpos)), s);
                v[t] = keep ? s : -INFINITY;
                m_thr = fmaxf(m_thr, v[t]);
            }
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) m_thr = fmaxf(m_thr, __shfl_xor_sync(0xffffffffu, m_thr, o));
            if (lane == 0) red[buf * 4 + warp] = m_thr;
            named_barrier_128();
            const float m_chunk = fmaxf(fmaxf(red[buf * 4], red[buf * 4 + 1]), fmaxf(red[buf * 4 + 2], red[buf * 4 + 3]));

            // the previous chunk's P V must be done before P is overwritten or O rescaled
            if (c > 0) {
                if (!mbar_wait_warp_ok(bar_p_free, (c - 1) & 1, abort_flag)) fail = 4;
                tc_fence_after_sync();
            }
            float m_new = m_ref, factor = 1.0f;
            if (m_chunk > m_ref + 8.0f || m_ref == -INFINITY) {
                m_new = fmaxf(m_ref, m_chunk);
                factor = (m_ref == -INFINITY) ? 0.0f : ex2f(m_ref - m_new);
            }
            if (c > 0 && m_new != m_ref) {  // CTA-uniform: every thread sees the same maxima
                const uint32_t ov = tmem_ld1(tmem_o + lane_base);
                tmem_wait_ld();
                tmem_st1(tmem_o + lane_base, __float_as_uint(__uint_as_float(ov) * factor));
                tmem_wait_st();
            }
            if (m_new != m_ref) l_part *= factor;
            m_ref = m_new;
            const float m_use = (m_ref == -INFINITY) ? 0.0f : m_ref;

#pragma unroll
            for (int t = 0; t < kChunkTiles; ++t) {
                if (t < nt) {
                    const float p = ex2f(v[t] - m_use);
                    l_part += p;
                    bool kept = true;
                    if (dropout) {
                        // reference draw order for query row 0: draw 64*tile_index + 8*(col/16) + 2*((col%16)/8) + col%2
                        const unsigned long long first = 64ull * static_cast<unsigned long long>(c * kChunkTiles + t) +
                                                         8ull * (r >> 4);
                        const uint32_t bits = philox_keep4(a.drop, subseq, first);
                        kept = (bits >> (2 * ((r >> 3) & 1) + (r & 1))) & 1u;
                    }
                    const float pk = kept ? p : 0.0f;
                    uint16_t h;
                    if constexpr (kBf16) h = __bfloat16_as_ushort(__float2bfloat16_rn(pk));
                    else h = __half_as_ushort(__float2half_rn(pk));
                    *reinterpret_cast<uint16_t*>(smem_gen + kDSmemP + t * kPTileBytes + (r >> 6) * 1024 + (r & 63) * 2) = h;
                }
            }
            fence_proxy_async_smem();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_p_full);
        }

        // ---- epilogue ----------------------------------------------------------------
        float l_warp = l_part;
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) l_warp += __shfl_xor_sync(0xffffffffu, l_warp, o);
        if (lane == 0) red[8 + warp] = l_warp;
        named_barrier_128();
        const float l_sum = (red[8] + red[9]) + (red[10] + red[11]);
        float o_val = 0.0f;
        if (n_tiles > 0 && fail == 0) {
            if (mbar_wait_warp_ok(bar_o_done, 0, abort_flag)) {
                tc_fence_after_sync();
                o_val = __uint_as_float(tmem_ld1(tmem_o + lane_base));
                tmem_wait_ld();
            } else {
                fail = 5;
            }
        }
        const float inv = l_sum > 0.0f ? a.drop.inv_keep / l_sum : 0.0f;
        const float lse_val = l_sum > 0.0f ? m_ref * kDLn2 + __logf(l_sum) : -INFINITY;
        o_val *= inv;
        const long long out_row = (a.num_splits > 1) ? static_cast<long long>(unit) * a.num_splits + split : unit;
        if (r < a.head_dim) {
            if (a.num_splits > 1) a.o_partial[out_row * a.head_dim + r] = o_val;
            else if (a.o_is_fp32) static_cast<float*>(a.o)[out_row * a.head_dim + r] = o_val;
            else if (kBf16) static_cast<__nv_bfloat16*>(a.o)[out_row * a.head_dim + r] = __float2bfloat16_rn(o_val);
            else static_cast<__half*>(a.o)[out_row * a.head_dim + r] = __float2half_rn(o_val);
        }
        if (r == 0) {
            if (a.num_splits > 1) a.lse_partial[out_row] = lse_val;
            else if (a.lse != nullptr) a.lse[out_row] = lse_val;
        }
    }

    if (fail != 0) {
        *abort_flag = 1;
        if (a.status != nullptr) atomicExch(a.status, 200 + fail);
        const long long t0 = clock64();
        while (clock64() - t0 < 200000) { }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 5 && n_tiles > 0) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kDTmemCols);
    }
}

}  // namespace

cudaError_t launch_decode(const DecodeArgs& a, const CUtensorMap& tk, const CUtensorMap& tv, int units, bool bf16,
                          cudaStream_t stream) {
    static bool configured[2][64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const long long ctas = static_cast<long long>(units) * a.num_splits;
    if (ctas <= 0 || ctas > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    auto run = [&](auto kern, int which) -> cudaError_t {
        if (dev < 0 || dev >= 64 || !configured[which][dev]) {
            cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kDSmemBytes);
            if (err != cudaSuccess) return err;
            if (dev >= 0 && dev < 64) configured[which][dev] = true;
        }
        kern<<<static_cast<unsigned>(ctas), kDThreads, kDSmemBytes, stream>>>(tk, tv, a);
        return cudaGetLastError();
    };
    return bf16 ? run(decode_kernel<true>, 0) : run(decode_kernel<false>, 1);
}

}  // namespace fa
