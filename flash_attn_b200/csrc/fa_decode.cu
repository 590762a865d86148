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
// Grouped-query attention and short query blocks (kH = 8): the query heads that share one K/V
// head, and the seqlen_q <= 8 query rows of each, ride in columns 0..7 of the same MMAs (rows
// 0..7 of the Q and P operand tiles; column = head * seqlen_q + row), so a CTA streams its K/V
// split once for up to eight queries; every per-query quantity (position, masks, max, sum, ALiBi
// slope, dropout stream, LSE) becomes an array over the columns.  Groups that need more than
// eight columns are cut into sub-groups of whole heads, one CTA each.
//
// Stream order of the TMA ring: K(0), K(1), V(0), K(2), V(1), ... (chunks of four tiles), so
// the scores of chunk c+1 are computed while the softmax of chunk c runs.
#include <atomic>
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
constexpr int kDSmemRed = kDSmemBar + 8 * kDNumBars;             // float[2][4][8] maxima + float[4][8] sums
constexpr int kDSmemMisc = kDSmemRed + 384;
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
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
// kH columns of one TMEM lane (kH = 1 or 8)
template <int kH>
__device__ __forceinline__ void tmem_ld_heads(uint32_t taddr, uint32_t (&r)[kH]) {
    if constexpr (kH == 1) r[0] = tmem_ld1(taddr);
    else tmem_ld8(taddr, r);
}
template <int kH>
__device__ __forceinline__ void tmem_st_heads(uint32_t taddr, const uint32_t (&r)[kH]) {
    if constexpr (kH == 1) tmem_st1(taddr, r[0]);
    else tmem_st8(taddr, r);
}
__device__ __forceinline__ bool mbar_wait_warp_ok(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag) ? 1 : 0) != 0;
}
__device__ __forceinline__ void named_barrier_128() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <bool kBf16, int kH>
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
    // the combine kernel behind a split launch may take its place on the SMs as they free up
    // (it waits for this grid's completion before reading the partials)
    grid_dep_launch_dependents();
    // kH = 1: one CTA per (query unit, split).  kH = 8: one CTA per (K/V unit, sub-group of up to
    // eight of its query heads, split); `unit` is then the first query unit of the sub-group.
    const int cta_unit = blockIdx.x / a.num_splits;
    const int split = blockIdx.x - cta_unit * a.num_splits;
    int unit, kv_unit, gh = 1;
    const int sq = (kH == 1) ? 1 : a.seqlen_q;  // query rows per head (columns per head)
    if constexpr (kH == 1) {
        unit = cta_unit;
        kv_unit = a.kv_group > 1 ? unit / a.kv_group : unit;
    } else {
        const int heads_per_cta = kH / sq;
        kv_unit = cta_unit / a.subgroups;
        const int sub = cta_unit - kv_unit * a.subgroups;
        unit = kv_unit * a.kv_group + sub * heads_per_cta;
        gh = min(heads_per_cta, a.kv_group - sub * heads_per_cta);  // query heads of this CTA
    }
    const int nc = gh * sq;  // columns in use: column n = head n / sq, query row n % sq

    // KV tiles of this split, clipped by the masks at tile granularity (as kv_tile_range
    // of the tiled kernel, for the query rows at positions q_pos0 .. q_pos0 + sq - 1)
    int lo = a.tiles_per_split * split, hi = min(lo + a.tiles_per_split, a.tc);
    if (a.window_left >= 0) {
        const long long w = (a.q_pos0 - a.window_left - a.k_pos0) / kTile;
        lo = max(lo, static_cast<int>(max(0LL, min(w, static_cast<long long>(a.tc)))));
    }
    if (a.window_right >= 0) {
        const long long last = a.q_pos0 + (sq - 1) + a.window_right - a.k_pos0;
        hi = min(hi, last < 0 ? 0 : static_cast<int>(min(last / kTile + 1, static_cast<long long>(a.tc))));
    }
    if (a.is_causal) {
        const long long last = a.q_pos0 + (sq - 1) - a.k_pos0;
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
    if (threadIdx.x < 16 * kH && n_tiles > 0) {
        // query n (head n / sq, row n % sq: consecutive rows of Q) goes to row n of the two Q atoms
        // (16-byte unit u -> atom u/8, unit (u%8) ^ n: the 128-byte swizzle of row n)
        const int u = threadIdx.x & 15, n = threadIdx.x >> 4;
        uint4 val = make_uint4(0u, 0u, 0u, 0u);
        if (n < nc && u * 8 < a.head_dim)
            val = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(a.q) +
                                                  (static_cast<long long>(unit) * sq + n) * a.head_dim + u * 8);
        *reinterpret_cast<uint4*>(smem_gen + kDSmemQ + (u >> 3) * 1024 + n * 128 + (((u & 7) ^ n) << 4)) = val;
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
        float slope2[kH];
        int qrow[kH];  // each column's query row; its global position is q_pos0 + qrow
#pragma unroll
        for (int n = 0; n < kH; ++n) {
            slope2[n] = (a.alibi_slopes != nullptr && n < nc) ? a.alibi_slopes[(unit + n / sq) % a.heads] * kDLog2e : 0.0f;
            qrow[n] = (kH == 1) ? 0 : n % sq;
        }
        const bool dropout = a.drop.threshold != 0ull;
        float m_ref[kH];   // CTA-wide running max per head, log2 units
        float l_part[kH];  // this thread's share of each head's row sum
#pragma unroll
        for (int n = 0; n < kH; ++n) {
            m_ref[n] = -INFINITY;
            l_part[n] = 0.0f;
        }

        for (int c = 0; c < n_chunks; ++c) {
            const int buf = c & 1;
            const int nt = chunk_tiles(c);
            bool ok = mbar_wait_warp_ok(bar_s_full + 8 * buf, (c >> 1) & 1, abort_flag);
            if (!ok) fail = 3;
            tc_fence_after_sync();
            float v[kChunkTiles][kH];
#pragma unroll
            for (int t = 0; t < kChunkTiles; ++t) {
                uint32_t raw[kH];
#pragma unroll
                for (int n = 0; n < kH; ++n) raw[n] = 0u;
                if (t < nt) tmem_ld_heads<kH>(tmem_base + lane_base + buf * 64 + t * 16, raw);
#pragma unroll
                for (int n = 0; n < kH; ++n) v[t][n] = __uint_as_float(raw[n]);
            }
            tmem_wait_ld();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_s_free + 8 * buf);

            float m_thr[kH];
#pragma unroll
            for (int n = 0; n < kH; ++n) m_thr[n] = -INFINITY;
#pragma unroll
            for (int t = 0; t < kChunkTiles; ++t) {
                const int tile = lo + c * kChunkTiles + t;
                const long long key = static_cast<long long>(tile) * kTile + r;
                const long long kpos = a.k_pos0 + key;
                const bool in_range = t < nt && key < a.seqlen_k;
                // key position relative to query row 0, saturated far outside any window
                const long long rel64 = kpos - a.q_pos0;
                const int rel = static_cast<int>(max(-0x40000000LL, min(rel64, 0x40000000LL)));
#pragma unroll
                for (int n = 0; n < kH; ++n) {
                    const int ahead = rel - qrow[n];  // > 0: the key lies after the query
                    bool keep = in_range;
                    if (a.is_causal && ahead > 0) keep = false;
                    if (a.window_left >= 0 && -ahead > a.window_left) keep = false;
                    if (a.window_right >= 0 && ahead > a.window_right) keep = false;
                    float sc = v[t][n] * scale2;
                    if (slope2[n] != 0.0f) sc = fmaf(-slope2[n], fabsf(static_cast<float>(ahead)), sc);
                    v[t][n] = keep ? sc : -INFINITY;
                    m_thr[n] = fmaxf(m_thr[n], v[t][n]);
                }
            }
#pragma unroll
            for (int n = 0; n < kH; ++n) {
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1) m_thr[n] = fmaxf(m_thr[n], __shfl_xor_sync(0xffffffffu, m_thr[n], o));
                if (lane == 0) red[(buf * 4 + warp) * 8 + n] = m_thr[n];
            }
            named_barrier_128();

            // the previous chunk's P V must be done before P is overwritten or O rescaled
            if (c > 0) {
                if (!mbar_wait_warp_ok(bar_p_free, (c - 1) & 1, abort_flag)) fail = 4;
                tc_fence_after_sync();
            }
            float m_use[kH], factor[kH];
            bool any_rescale = false;
#pragma unroll
            for (int n = 0; n < kH; ++n) {
                const float m_chunk = fmaxf(fmaxf(red[(buf * 4) * 8 + n], red[(buf * 4 + 1) * 8 + n]),
                                            fmaxf(red[(buf * 4 + 2) * 8 + n], red[(buf * 4 + 3) * 8 + n]));
                float m_new = m_ref[n];
                factor[n] = 1.0f;
                if (m_chunk > m_ref[n] + 8.0f || m_ref[n] == -INFINITY) {
                    m_new = fmaxf(m_ref[n], m_chunk);
                    factor[n] = (m_ref[n] == -INFINITY) ? 0.0f : ex2f(m_ref[n] - m_new);
                }
                if (m_new != m_ref[n]) {
                    any_rescale = true;
                    l_part[n] *= factor[n];
                }
                m_ref[n] = m_new;
                m_use[n] = (m_new == -INFINITY) ? 0.0f : m_new;
            }
            if (c > 0 && any_rescale) {  // CTA-uniform: every thread sees the same maxima
                uint32_t ov[kH];
                tmem_ld_heads<kH>(tmem_o + lane_base, ov);
                tmem_wait_ld();
#pragma unroll
                for (int n = 0; n < kH; ++n) ov[n] = __float_as_uint(__uint_as_float(ov[n]) * factor[n]);
                tmem_st_heads<kH>(tmem_o + lane_base, ov);
                tmem_wait_st();
            }

#pragma unroll
            for (int t = 0; t < kChunkTiles; ++t) {
                if (t < nt) {
#pragma unroll
                    for (int n = 0; n < kH; ++n) {
                        const float p = ex2f(v[t][n] - m_use[n]);
                        l_part[n] += p;
                        bool kept = true;
                        if (dropout && n < nc) {
                            // reference draw order for query rows 0..7 (one 8-row group shares its draws):
                            // draw 64*tile_index + 8*(col/16) + 2*((col%16)/8) + col%2
                            const unsigned long long subseq =
                                (a.drop.unit0 + unit + n / sq) * static_cast<unsigned long long>(a.num_splits) +
                                static_cast<unsigned long long>(split);
                            const unsigned long long first = continuation(a.drop, n_tiles) +
                                                             64ull * static_cast<unsigned long long>(c * kChunkTiles + t) +
                                                             8ull * (r >> 4);
                            const uint32_t bits = philox_keep4(a.drop, subseq, first);
                            kept = (bits >> (2 * ((r >> 3) & 1) + (r & 1))) & 1u;
                        }
                        const float pk = kept ? p : 0.0f;
                        uint16_t h;
                        if constexpr (kBf16) h = __bfloat16_as_ushort(__float2bfloat16_rn(pk));
                        else h = __half_as_ushort(__float2half_rn(pk));
                        // P operand row n (head n), 128-byte swizzled like the Q rows
                        *reinterpret_cast<uint16_t*>(smem_gen + kDSmemP + t * kPTileBytes + (r >> 6) * 1024 + n * 128 +
                                                     (((((r & 63) >> 3) ^ n) & 7) << 4) + (r & 7) * 2) = h;
                    }
                }
            }
            fence_proxy_async_smem();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_p_full);
        }

        // ---- epilogue ----------------------------------------------------------------
#pragma unroll
        for (int n = 0; n < kH; ++n) {
            float l_warp = l_part[n];
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) l_warp += __shfl_xor_sync(0xffffffffu, l_warp, o);
            if (lane == 0) red[64 + warp * 8 + n] = l_warp;
        }
        named_barrier_128();
        uint32_t o_raw[kH];
#pragma unroll
        for (int n = 0; n < kH; ++n) o_raw[n] = 0u;
        if (n_tiles > 0 && fail == 0) {
            if (mbar_wait_warp_ok(bar_o_done, 0, abort_flag)) {
                tc_fence_after_sync();
                tmem_ld_heads<kH>(tmem_o + lane_base, o_raw);
                tmem_wait_ld();
            } else {
                fail = 5;
            }
        }
#pragma unroll
        for (int n = 0; n < kH; ++n) {
            if (n >= nc) continue;
            const float l_sum = (red[64 + n] + red[64 + 8 + n]) + (red[64 + 16 + n] + red[64 + 24 + n]);
            const float inv = l_sum > 0.0f ? a.drop.inv_keep / l_sum : 0.0f;
            const float lse_val = l_sum > 0.0f ? m_ref[n] * kDLn2 + __logf(l_sum) : -INFINITY;
            const float o_val = __uint_as_float(o_raw[n]) * inv;
            // non-split: row (unit + head, query row) of O; split: the same row of this split's partial
            const long long head_n = unit + n / sq;
            const long long out_row = (a.num_splits > 1) ? (head_n * a.num_splits + split) * sq + n % sq : head_n * sq + n % sq;
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

cudaError_t launch_decode(const DecodeArgs& a_in, const CUtensorMap& tk, const CUtensorMap& tv, int units, bool bf16,
                          cudaStream_t stream) {
    static std::atomic<bool> configured[4][64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    DecodeArgs a = a_in;
    // query heads that share a K/V head are packed into one CTA, eight at a time
    if (a.seqlen_q < 1 || a.seqlen_q > 8) return cudaErrorInvalidValue;
    const bool packed = a.kv_group > 1 || a.seqlen_q > 1;
    const int heads_per_cta = 8 / a.seqlen_q;  // whole heads whose query rows fit the eight columns
    a.subgroups = packed ? (a.kv_group + heads_per_cta - 1) / heads_per_cta : 1;
    const long long cta_units = packed ? static_cast<long long>(units / a.kv_group) * a.subgroups : units;
    const long long ctas = cta_units * a.num_splits;
    if (ctas <= 0 || ctas > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    auto run = [&](auto kern, int which) -> cudaError_t {
        if (dev < 0 || dev >= 64 || !configured[which][dev].load(std::memory_order_acquire)) {
            cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kDSmemBytes);
            if (err != cudaSuccess) return err;
            if (dev >= 0 && dev < 64) configured[which][dev].store(true, std::memory_order_release);
        }
        kern<<<static_cast<unsigned>(ctas), kDThreads, kDSmemBytes, stream>>>(tk, tv, a);
        return cudaGetLastError();
    };
    if (packed) return bf16 ? run(decode_kernel<true, 8>, 2) : run(decode_kernel<false, 8>, 3);
    return bf16 ? run(decode_kernel<true, 1>, 0) : run(decode_kernel<false, 1>, 1);
}

}  // namespace fa
