// Tiled flash-attention forward for sm_100a.  Replaces the reference's
// forward_kernel (src/flash_forward.h:13-306) and forward_kernel_splitkv
// (src/flash_forward_splitkv.h:14-344).
//
// A CTA owns NQ (1 or 2) consecutive 128-row query tiles of one (batch, head)
// unit, optionally one KV split of them; each query tile is exactly one CTA of
// the reference's decomposition (grid (Tr*splits, H, B), src/main.cu:142-158),
// which is what the dropout streams are keyed on.  Roles by warp:
//   softmax groups (4 warps per query tile): thread r owns query row r.  S is read
//       from tensor memory (tcgen05.ld), masked / biased / exponentiated in
//       registers, the 16-bit P is written back to tensor memory over S
//       (tcgen05.st); the running (max, sum) and the lazy rescale of O live here.
//   TMA producer warp: streams the Q tiles once and K/V tiles through an mbarrier
//       ring (cp.async.bulk.tensor, 128-byte swizzle).
//   MMA issuer warp: one thread issues tcgen05.mma for S_i = Q_i K^T (operands in
//       shared memory) and O_i += P_i V (P in tensor memory, V in shared memory,
//       MN-major), accumulators in tensor memory.  With NQ = 2 the two query tiles
//       alternate on the tensor pipe, so the softmax of one overlaps the MMAs of
//       the other while both share every K/V tile brought in by TMA.
// KV tiles are visited from the last to the first (the softmax is order-independent and the
// dropout draw of an element is a function of its position): with a causal mask the second
// query tile of a CTA owns one KV tile more than the first, the diagonal one, and walking
// backwards puts that solo tile at the start, where it overlaps the first tile of the other
// query tile, instead of at the end, where the other warpgroup would idle.
// The reference keeps O in shared memory and renormalises it every tile
// (src/flash_forward.h:248-290); here O stays un-normalised in tensor memory and
// is divided by the row sum once, in the epilogue.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <algorithm>
#include <atomic>
#include <type_traits>
#include "fa_internal.h"
#include "sm100_ptx.cuh"

// Optional timeline tracing for kernel development (compiled out unless FA_TRACE is
// defined): lane 0 of every warp of CTA FA_TRACE_CTA records (event, clock) pairs.
#ifdef FA_TRACE
#ifndef FA_TRACE_CTA
#define FA_TRACE_CTA 0
#endif
__device__ long long fa_trace_buf[16 * 512];
extern "C" int fa_trace_read(long long* host_out) {
    return static_cast<int>(cudaMemcpyFromSymbol(host_out, fa_trace_buf, sizeof(long long) * 16 * 512));
}
#define FA_TR(ev)                                                                              \
    do {                                                                                       \
        if (blockIdx.x == FA_TRACE_CTA && (threadIdx.x & 31) == 0 && tr_n < 255) {                        \
            fa_trace_buf[(threadIdx.x >> 5) * 512 + 2 * tr_n] = (ev);                          \
            fa_trace_buf[(threadIdx.x >> 5) * 512 + 2 * tr_n + 1] = clock64();                 \
            ++tr_n;                                                                            \
        }                                                                                      \
    } while (0)
#else
#define FA_TR(ev) do { } while (0)
#endif

// Test build only (-DFA_TEST_SHORT_WAIT): the producer can be told to leave out the loads of one KV
// tile, so that a consumer's bounded wait runs out and the give-up path (status word, drain, TMEM
// release, clean exit) can be checked on a GPU without faulting or hanging anything.
#ifdef FA_TEST_SHORT_WAIT
__device__ int fa_test_skip_tile = -1;
extern "C" int fa_test_skip_kv_tile(int t) {
    return static_cast<int>(cudaMemcpyToSymbol(fa_test_skip_tile, &t, sizeof(int)));
}
#define FA_TEST_SKIPS(t) (fa_test_skip_tile == (t))
#else
#define FA_TEST_SKIPS(t) false
#endif

namespace fa {

namespace {

constexpr float kRescaleThreshold = 8.0f;  // log2 units: rescale O only when the max grew by > 2^8
// Which column pairs take the polynomial exp2: one pair of every four (a quarter of the elements), bit
// 4*(g%2) + q = pair q of an even / odd group of eight columns.  The position decides how the cubic's FMAs
// interleave with the MUFU results around them; measured over all sixteen placements, pair 0 everywhere is
// the fastest without dropout and pairs 0 / 1 of even / odd groups with it (up to 2 % between placements).
constexpr uint32_t kPolyMaskPlain = 0x11u;
constexpr uint32_t kPolyMaskDropout = 0x21u;
constexpr int kKeepChunk = 2;              // KV tiles whose dropout keep bits are handed over at a time (one Philox pass)
constexpr int kKeepRing = 2 * kKeepChunk;  // tiles the keep-bit table holds
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

template <int D, int NQ>
struct Cfg {
    // The helper warps (producer, MMA issuer) are rounded up to a full warpgroup so that registers
    // can be moved from it to the softmax warpgroups (setmaxnreg works on whole warpgroups).
    static constexpr int kThreads = NQ == 2 ? 384 : 256;
    // Register hand-over (setmaxnreg): the CTA owns kThreads * kRegsLaunch registers from launch on
    // and nothing more; an increase that asks for more than the helpers released would block
    // forever, hence the static_assert.
    // ptxas allots 168 registers per thread under __launch_bounds__(384, 1) and 128 under (256, 2)
    static constexpr int kRegsLaunch = NQ == 2 ? 168 : 128;
    static constexpr int kRegsHelper = NQ == 2 ? 56 : 48;     // producer / MMA warpgroup after the hand-over
    static constexpr int kRegsSoftmax = NQ == 2 ? 224 : 208;  // softmax warpgroups after the hand-over
    static_assert(NQ * 128 * kRegsSoftmax + 128 * kRegsHelper <= kThreads * kRegsLaunch,
                  "register hand-over exceeds the CTA's allocation");
    static constexpr int kProducerWarp = NQ * 4;
    static constexpr int kMmaWarp = NQ * 4 + 1;
    static constexpr int kStages = (D == 64) ? (NQ == 2 ? 3 : 2) : (NQ == 2 ? 2 : 1);
    static constexpr int kBoxes = D / 64;             // 64-element (128-byte) column blocks per tile
    static constexpr int kTileBytes = kTile * D * 2;  // one Q, K or V tile
    // TMEM columns: S_i at i*128 (P_i aliases S_i[0,64)); O_i after the S blocks.
    static constexpr int kTmemCols = NQ == 2 ? 512 : 256;
    static constexpr int kTmemO = NQ * kTile;
    static constexpr int kSmemQ = 0;
    static constexpr int kSmemK = NQ * kTileBytes;
    static constexpr int kSmemV = kSmemK + kStages * kTileBytes;
    static constexpr int kSmemBar = kSmemV + kStages * kTileBytes;
    static constexpr int kNumBars = 1 + 2 * NQ + 4 * kStages;
    // dropout keep bits, written by a helper warp per query tile: [NQ][2 row halves][kKeepRing tiles] words
    static constexpr int kSmemKeep = kSmemBar + 8 * kNumBars + 16;
    static constexpr int kSmemBytes = kSmemKeep + NQ * kKeepRing * 2 * 4 + 1024;  // + alignment slack
    static constexpr int kKeepWarp0 = NQ * 4 + 2;  // the helper warp of query tile i is kKeepWarp0 + i
    // ALiBi whose bias is linear in the key position (every visible key at or before the query) is added by
    // the tensor core: one more K = 16 step per Q K^T over two extra 64-column boxes, [1 1 0 ...] for every
    // query row and [hi lo 0 ...] of slope * column / scale for every key row of a tile (two 16-bit terms
    // carry the bias to 2^-17 relative).  Two-tile CTAs only: a single-tile CTA shares its SM.
    static constexpr bool kBiasBoxes = NQ == 2;
    static constexpr int kSmemBiasQ = (kSmemKeep + NQ * kKeepRing * 2 * 4 + 1023) / 1024 * 1024;
    static constexpr int kSmemBiasK = kSmemBiasQ + kTile * 128;
    static constexpr int kSmemBytesBias = kSmemBiasK + kTile * 128 + 1024;  // dynamic shared memory of the ALiBi kernels
};

struct TileRange {
    int lo, hi;  // KV tiles [lo, hi)
};

__device__ __forceinline__ uint32_t fast_div(const FastDiv& f, uint32_t x) {
    if (f.d == 1) return x;
    uint32_t q = __umulhi(x, f.m);
    if (q * f.d > x) --q;
    return q;
}

__device__ __forceinline__ TileRange kv_tile_range(const FwdArgs& a, int rb, int split) {
    if (rb >= a.tr) return {0, 0};
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
    if (hi < lo) hi = lo;
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

// exp2 on the FMA/ALU pipes for a pair of arguments x <= ~8: the MUFU unit (16 results per
// clock per SM) needs as long for the 128 x 128 exponentials of a tile pair as the tensor
// pipe needs for their MMAs, so part of them is computed here instead.  Round to the nearest
// integer n with the 1.5 * 2^23 trick, evaluate 2^f on f = x - n in [-0.5, 0.5] with a cubic
// (max relative error 7.5e-5, far below the 16-bit rounding of P), and add n to the exponent.
// Arguments below -126 give 2^-126 instead of 0.
__device__ __forceinline__ float2 poly_exp2_pair(float2 x) {
    x.x = fmaxf(x.x, -126.0f);
    x.y = fmaxf(x.y, -126.0f);
    const float2 magic = make_float2(12582912.0f, 12582912.0f);
    const float2 r = __fadd2_rn(x, magic);
    const float2 n = __fadd2_rn(r, make_float2(-12582912.0f, -12582912.0f));
    const float2 f = __ffma2_rn(n, make_float2(-1.0f, -1.0f), x);
    float2 p = __ffma2_rn(make_float2(0.0551716685f, 0.0551716685f), f, make_float2(0.2426111251f, 0.2426111251f));
    p = __ffma2_rn(p, f, make_float2(0.6932609677f, 0.6932609677f));
    p = __ffma2_rn(p, f, make_float2(0.9999280572f, 0.9999280572f));
    p.x = __int_as_float(__float_as_int(p.x) + (__float_as_int(r.x) << 23));
    p.y = __int_as_float(__float_as_int(p.y) + (__float_as_int(r.y) << 23));
    return p;
}

// Byte permute whose selector nibbles 8 + n give 0xff or 0x00 by the sign bit of byte n of x.
__device__ __forceinline__ uint32_t prmt_sign(uint32_t x, uint32_t selector) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %1, %2;" : "=r"(r) : "r"(x), "r"(selector));
    return r;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// Whole-warp wait: the lanes poll together (one shared-memory access per poll).  A poll is
// slow while the tensor pipe streams operands from shared memory (several hundred cycles
// were measured), so the wait is a single phase with no second look.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag) ? 1 : 0) != 0;
}

// Hardware named barriers carry the P hand-over: the 128 threads of a softmax warpgroup
// arrive (non-blocking), the MMA warp syncs.  Waking from a named barrier costs tens of
// cycles, while a poll of a shared-memory mbarrier took several hundred whenever the tensor
// pipe was streaming operands.  A named barrier cannot time out, so a softmax warp whose
// mbarrier wait gave up keeps walking its tile loop and posts every arrival it owes.
constexpr int kPBarrierThreads = 160;  // 128 softmax threads + the MMA warp (or + a keep-bit helper warp)
// Barrier ids: 0 = __syncthreads; 1 + 2i, 2 + 2i = P of query tile i (first part, complete);
// 5 + 2i + h = keep bits of half-ring h of query tile i written; 9 + 2i + h = that half-ring read.
__device__ __forceinline__ int keep_full_id(int qi, int h) { return 5 + 2 * qi + h; }
__device__ __forceinline__ int keep_empty_id(int qi, int h) { return 9 + 2 * qi + h; }
__device__ __forceinline__ void named_arrive(int id) {
    asm volatile("bar.arrive %0, %1;" ::"r"(id), "n"(kPBarrierThreads) : "memory");
}
__device__ __forceinline__ void named_sync(int id) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "n"(kPBarrierThreads) : "memory");
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "elect.sync _|P, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

// Eight (D = 128) or four (D = 64) back-to-back MMAs of one S = Q K^T tile in a single
// asm block: the descriptors differ only in the low word (start address, 16-byte units),
// which is stepped inside the block, so the issuing thread does no other work between MMAs.
// Steps for a [128 x D] tile stored as 64-column boxes: 32 bytes per k-step inside a box
// (+2 units), next box after four steps (16 KB further: +1024 - 6 units).
#define FA_QK_STEP(inc)                                                                        \
    "add.u32 qa, qa, " #inc ";\n\tadd.u32 kb, kb, " #inc ";\n\t"                                 \
    "mov.b64 da, {qa, %3};\n\tmov.b64 db, {kb, %3};\n\t"                                        \
    "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p1;\n\t"
#define FA_QK_HEAD                                                                             \
    "{\n\t.reg .pred p0, p1;\n\t.reg .b32 qa, kb;\n\t.reg .b64 da, db;\n\t"                       \
    "setp.ne.b32 p0, 0, 0;\n\tsetp.eq.b32 p1, 0, 0;\n\t"                                        \
    "mov.b32 qa, %1;\n\tmov.b32 kb, %2;\n\t"                                                    \
    "mov.b64 da, {qa, %3};\n\tmov.b64 db, {kb, %3};\n\t"                                        \
    "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p0;\n\t"
template <int D>
__device__ __forceinline__ void issue_qk_block(uint32_t d_tmem, uint32_t qa_lo, uint32_t kb_lo, uint32_t desc_hi,
                                               uint32_t idesc) {
    if constexpr (D == 128) {
        asm volatile(FA_QK_HEAD FA_QK_STEP(2) FA_QK_STEP(2) FA_QK_STEP(2) FA_QK_STEP(1018) FA_QK_STEP(2)
                         FA_QK_STEP(2) FA_QK_STEP(2) "}"
                     ::"r"(d_tmem), "r"(qa_lo), "r"(kb_lo), "r"(desc_hi), "r"(idesc)
                     : "memory");
    } else {
        asm volatile(FA_QK_HEAD FA_QK_STEP(2) FA_QK_STEP(2) FA_QK_STEP(2) "}"
                     ::"r"(d_tmem), "r"(qa_lo), "r"(kb_lo), "r"(desc_hi), "r"(idesc)
                     : "memory");
    }
}

// Eight back-to-back MMAs of O += P V over the 128 keys of a tile: P advances 8 TMEM
// columns (16 packed elements) and V 16 rows (2048 bytes = 128 descriptor units) per step.
#define FA_PV_STEP                                                                             \
    "add.u32 pa, pa, 8;\n\tadd.u32 vb, vb, 128;\n\tmov.b64 db, {vb, %3};\n\t"                    \
    "tcgen05.mma.cta_group::1.kind::f16 [%0], [pa], db, %4, p1;\n\t"
#define FA_PV_HEAD                                                                             \
    "{\n\t.reg .pred p0, p1;\n\t.reg .b32 pa, vb;\n\t.reg .b64 db;\n\t"                          \
    "setp.ne.b32 p0, %5, 0;\n\tsetp.eq.b32 p1, 0, 0;\n\t"                                        \
    "mov.b32 pa, %1;\n\tmov.b32 vb, %2;\n\tmov.b64 db, {vb, %3};\n\t"                            \
    "tcgen05.mma.cta_group::1.kind::f16 [%0], [pa], db, %4, p0;\n\t"
// k-steps [0, kSplitSteps) of a tile: issued as soon as the first kSplitSteps*16 columns of P
// are in tensor memory; the rest follow when P is complete.
constexpr int kSplitSteps = 4;
__device__ __forceinline__ void issue_pv_first(uint32_t d_tmem, uint32_t a_tmem, uint32_t vb_lo, uint32_t desc_hi,
                                               uint32_t idesc, uint32_t accumulate) {
    asm volatile(FA_PV_HEAD FA_PV_STEP FA_PV_STEP FA_PV_STEP "}"
                 ::"r"(d_tmem), "r"(a_tmem), "r"(vb_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
                 : "memory");
}
__device__ __forceinline__ void issue_pv_rest(uint32_t d_tmem, uint32_t a_tmem, uint32_t vb_lo, uint32_t desc_hi,
                                              uint32_t idesc) {
    asm volatile(FA_PV_HEAD FA_PV_STEP FA_PV_STEP FA_PV_STEP "}"
                 ::"r"(d_tmem), "r"(a_tmem + kSplitSteps * 8), "r"(vb_lo + kSplitSteps * 128), "r"(desc_hi), "r"(idesc), "r"(1u)
                 : "memory");
}

// One more k-step of S = Q K^T over the bias boxes (accumulating).
__device__ __forceinline__ void issue_qk_bias(uint32_t d_tmem, uint32_t qa_lo, uint32_t kb_lo, uint32_t desc_hi, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p1;\n\t.reg .b64 da, db;\n\t"
        "setp.eq.b32 p1, 0, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p1;\n\t}"
        ::"r"(d_tmem), "r"(qa_lo), "r"(kb_lo), "r"(desc_hi), "r"(idesc)
        : "memory");
}

template <int D, int NQ, bool kBf16, bool kAlibi, bool kDropout>
__global__ void __launch_bounds__(Cfg<D, NQ>::kThreads, NQ == 1 ? 2 : 1)
fwd_tiled_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_o,
                 const FwdArgs a) {
    using C = Cfg<D, NQ>;
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
    const uint32_t bar_s_full = bar0 + 8;                        // [NQ]
    const uint32_t bar_o_full = bar_s_full + 8 * NQ;             // [NQ]
    const uint32_t bar_k_full = bar_o_full + 8 * NQ;             // [kStages]
    const uint32_t bar_k_empty = bar_k_full + 8 * C::kStages;    // [kStages]
    const uint32_t bar_v_full = bar_k_empty + 8 * C::kStages;    // [kStages]
    const uint32_t bar_v_empty = bar_v_full + 8 * C::kStages;    // [kStages]
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + C::kSmemBar + 8 * C::kNumBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + C::kSmemBar + 8 * C::kNumBars + 4);
    volatile uint32_t* keep_tab = reinterpret_cast<volatile uint32_t*>(smem_gen + C::kSmemKeep);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
#ifdef FA_TRACE
    int tr_n = 0;
    FA_TR(90);
#endif

    // Programmatic dependent launch: let the next kernel of the stream start its own set-up as
    // soon as SMs free up, and do this kernel's set-up (index arithmetic, barriers, TMEM) before
    // waiting for the kernel in front of it; no global memory is touched before grid_dep_wait().
    grid_dep_launch_dependents();

    // The producer warp initialises every barrier (one per lane, a single instruction) and asks for
    // the tensor maps before any index arithmetic: neither depends on which tiles the CTA owns, and
    // the maps are kernel parameters, not memory of the kernel in front.
    if (warp == C::kProducerWarp) {
        if (lane < C::kNumBars) mbar_init(bar0 + 8 * lane, 1);
        if (lane == 0) {
            *abort_flag = 0;
            tma_prefetch_desc(&tmap_q);
            tma_prefetch_desc(&tmap_k);
            tma_prefetch_desc(&tmap_v);
            if (a.o_tma) tma_prefetch_desc(&tmap_o);
        }
        __syncwarp();
        if (lane == 0) mbar_fence_init();
    }

    // ---- which query tiles does this CTA own ------------------------------------
    const int trq = (a.tr + NQ - 1) / NQ;  // query blocks of NQ tiles
    // CTA order: groups of unit_group units; inside a group all units' first query block, then
    // all second ones, ...  With a causal mask the blocks are visited heaviest first, so the
    // grid is close to a longest-job-first schedule while the K/V working set of the CTAs in
    // flight (one group) stays far below the L2 size.
    // (the divisors are launch constants: multiply-high instead of the hardware's slow integer divide,
    // which sat on the path to the first TMA load)
    const uint32_t group = fast_div(a.div_group_ctas, blockIdx.x);
    const int unit0 = static_cast<int>(group) * a.unit_group;
    const bool full_group = unit0 + a.unit_group <= a.units;
    const uint32_t rem = blockIdx.x - group * a.div_group_ctas.d;
    const uint32_t bx = fast_div(full_group ? a.div_gsize : a.div_last_gsize, rem);
    const int unit = unit0 + static_cast<int>(rem - bx * (full_group ? a.div_gsize.d : a.div_last_gsize.d));
    const int kv_unit = static_cast<int>(fast_div(a.div_kv_group, static_cast<uint32_t>(unit)));  // grouped-query attention: K/V head of this unit
    const uint32_t qb_raw = fast_div(a.div_splits, bx);
    const int split = static_cast<int>(bx - qb_raw * a.div_splits.d);
    int qb = static_cast<int>(qb_raw);
    if (a.is_causal) qb = trq - 1 - qb;  // heaviest query blocks first
    FA_TR(94);
    // The producer lane puts the Q tiles in flight as soon as it knows which they are (a tile whose
    // key range then turns out empty is loaded for nothing: fully masked blocks only), the K/V tiles
    // once the ranges are known; the HBM latency of these first loads overlaps the rest of the set-up,
    // the TMEM allocation and the CTA-wide synchronisation instead of following them.
    // Every box of these first loads is issued by a lane of its own (one instruction puts them all in
    // flight: a single thread needs 100-200 cycles per TMA instruction).
    int q_tiles = 0;  // Q tiles in flight (producer warp only)
    if (warp == C::kProducerWarp) {
        grid_dep_wait();
#pragma unroll
        for (int i = 0; i < NQ; ++i) q_tiles += (qb * NQ + i < a.tr) ? 1 : 0;
        if (lane == 0 && q_tiles > 0) mbar_expect_tx(bar_q_full, q_tiles * C::kTileBytes);
        if (lane < NQ * C::kBoxes) {
            const int i = lane / C::kBoxes, b = lane % C::kBoxes;
            if (qb * NQ + i < a.tr)
                tma_load_3d(sQ + i * C::kTileBytes + b * (kTile * 128), &tmap_q, bar_q_full, b * 64,
                            (qb * NQ + i) * kTile, unit);
        }
    }
    // (the NQ ranges are worked out side by side on lanes 0..NQ-1 and handed round)
    TileRange range[NQ];
    {
        const TileRange mine = kv_tile_range(a, qb * NQ + (lane & (NQ - 1)), split);
#pragma unroll
        for (int i = 0; i < NQ; ++i) {
            range[i].lo = NQ == 1 ? mine.lo : __shfl_sync(0xffffffffu, mine.lo, i);
            range[i].hi = NQ == 1 ? mine.hi : __shfl_sync(0xffffffffu, mine.hi, i);
        }
    }
    int lo = 0x7fffffff, hi = 0;
#pragma unroll
    for (int i = 0; i < NQ; ++i) {
        if (range[i].hi > range[i].lo) {
            lo = min(lo, range[i].lo);
            hi = max(hi, range[i].hi);
        }
    }
    const int n_union = hi > lo ? hi - lo : 0;  // KV tiles streamed by this CTA: [lo, hi)
    FA_TR(95);

    // ---- set-up ----------------------------------------------------------------
    int prefilled = 0;  // K/V tiles whose loads were issued during set-up (producer warp only)
    if (warp == C::kProducerWarp) {
        if (n_union > 0) {
            prefilled = min(C::kStages, n_union);
            // lane = (tile t of the ring, K or V, box): the ring is empty, no waits
            const int t = lane / (2 * C::kBoxes), is_v = (lane / C::kBoxes) & 1, b = lane % C::kBoxes;
            if (t < prefilled && !FA_TEST_SKIPS(t)) {
                const int row = (hi - 1 - t) * kTile;  // KV tiles are walked from the last to the first
                const uint32_t bar = (is_v ? bar_v_full : bar_k_full) + 8 * t;
                if (b == 0) mbar_expect_tx(bar, C::kTileBytes);
                tma_load_3d((is_v ? sV : sK) + t * C::kTileBytes + b * (kTile * 128), is_v ? &tmap_v : &tmap_k, bar,
                            b * 64, row, kv_unit);
            }
        } else if (lane == 0 && q_tiles > 0) {
            // nothing to do for this CTA after all: its Q tiles must land before the CTA may exit
            (void)mbar_wait(bar_q_full, 0, abort_flag);
        }
    }
    if (warp == C::kMmaWarp) {
        if (n_union > 0) {
            tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), C::kTmemCols);
            tmem_relinquish();
        }
    }
    // Dropout keep bits.  One otherwise idle warp per query tile evaluates the Philox blocks of that
    // tile's stream (src/flash_forward.h:50-54,221-237) for the whole softmax warpgroup, whose four
    // warps all need the same 64 draws per KV tile: lanes 0-15 take one KV tile of a chunk, lanes
    // 16-31 the next (lane & 15 = 2*i + row-half: draws 8*i + 4*half + {0..3}), the eight blocks of a
    // row half are OR-ed into one word by three shuffles, and the words go to a ring of
    // kKeepRing tiles in shared memory, handed over a chunk at a time over named barriers.  The first
    // chunk is written here, before the CTA-wide sync, so that it is there when the first S arrives.
    const int keep_qi = warp - C::kKeepWarp0;
    int keep_tiles = 0;
    unsigned long long keep_subseq = 0, keep_first = 0;
    auto keep_chunk = [&](int chunk) {
        const int j = chunk * kKeepChunk + (lane >> 4);  // position in the walk (last KV tile first)
        uint32_t v = 0;
        if (j < keep_tiles) {
            const uint32_t k4 = philox_keep4(a.drop, keep_subseq,
                                             keep_first + 64ull * static_cast<unsigned long long>(keep_tiles - 1 - j) +
                                                 4ull * static_cast<unsigned long long>(lane & 15));
            // draw w of block i decides columns 16*i + 8*(w/2) + {0..7} of parity w%2: its keep bit goes
            // to bit 8*w + 7 - i, so that after a left shift by i the four bits of block i are the sign
            // bits of the word's four bytes (see the byte permutes of the softmax loop)
            v = ((k4 & 1u) | ((k4 & 2u) << 7) | ((k4 & 4u) << 14) | ((k4 & 8u) << 21)) << (7 - ((lane & 15) >> 1));
        }
        v |= __shfl_xor_sync(0xffffffffu, v, 2);
        v |= __shfl_xor_sync(0xffffffffu, v, 4);
        v |= __shfl_xor_sync(0xffffffffu, v, 8);
        if ((lane & 14) == 0 && j < keep_tiles)
            keep_tab[(keep_qi * 2 + (lane & 1)) * kKeepRing + (j & (kKeepRing - 1))] = v;
        __threadfence_block();
        named_arrive(keep_full_id(keep_qi, chunk & 1));
    };
    if constexpr (kDropout) {
        if (warp >= C::kKeepWarp0 && warp < C::kKeepWarp0 + NQ) {
            const TileRange kr = (keep_qi == 0) ? range[0] : range[NQ - 1];
            keep_tiles = kr.hi - kr.lo;
            keep_subseq = (a.drop.unit0 + unit) * static_cast<unsigned long long>(a.tr * a.num_splits) +
                          static_cast<unsigned long long>((qb * NQ + keep_qi) * a.num_splits + split);
            keep_first = continuation(a.drop, keep_tiles);
            FA_TR(40);
            if (keep_tiles > 0) keep_chunk(0);
            FA_TR(41);
        }
    }
    grid_dep_wait();  // every thread, before its first global access (the producer lane has passed it already)
    // every unmasked key lies at or before the query: |q - k| = q - k, the ALiBi bias is linear in the key
    const bool keys_not_after = a.is_causal || a.window_right == 0;
    constexpr bool kBias = kAlibi && C::kBiasBoxes;
    float bias_step = 0.0f;  // the bias of a column in units of the raw scores, per column
    if constexpr (kBias) bias_step = a.alibi_slopes[unit % a.heads] * kLog2e / a.scale_log2;
    // (the two 16-bit terms carry an entry to 2^-17 relative: with slopes up to 4 per column in log2 units
    // the bias is exact to 0.004, far below the 16-bit rounding of P; steeper slopes keep the softmax path.
    // fp16 operands: the largest entry, 127 columns, must also stay far inside the format's range)
    const bool bias_in_mma = kBias && keys_not_after && fabsf(bias_step * a.scale_log2) < 4.0f &&
                             (kBf16 || fabsf(bias_step) < 200.0f);
    if constexpr (kBias) {
        if (bias_in_mma && n_union > 0 && threadIdx.x < kTile) {
            const int rr = threadIdx.x;  // key row of the K box, query row of the Q box
            const float x = bias_step * static_cast<float>(rr);
            float hi_f, lo_f;
            if constexpr (kBf16) {
                const __nv_bfloat16 h = __float2bfloat16_rn(x);
                hi_f = __bfloat162float(h);
                lo_f = x - hi_f;
            } else {
                const __half h = __float2half_rn(x);
                hi_f = __half2float(h);
                lo_f = x - hi_f;
            }
            const uint32_t kw = pack2<kBf16>(hi_f, lo_f), qw = pack2<kBf16>(1.0f, 1.0f);
            const uint32_t krow = smem_base + C::kSmemBiasK + rr * 128, qrow = smem_base + C::kSmemBiasQ + rr * 128;
#pragma unroll
            for (int j = 0; j < 8; ++j) {  // 16-byte chunks of the 128-byte-swizzled row
                const uint32_t off = static_cast<uint32_t>(j ^ (rr & 7)) * 16;
                st_shared_v4(krow + off, j == 0 ? kw : 0u, 0u, 0u, 0u);
                st_shared_v4(qrow + off, j == 0 ? qw : 0u, 0u, 0u, 0u);
            }
            fence_proxy_async_smem();
        }
    }
    FA_TR(92);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    FA_TR(93);
    const uint32_t tmem_base = (n_union > 0) ? *tmem_slot : 0u;

    int fail = 0;

    // The helper warpgroup (producer, MMA issuer, two idle warps) hands most of its registers to
    // the softmax warpgroups, which hold a 128-column score row per thread.  Each register
    // regime covers one whole branch below.
    if (warp >= NQ * 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(C::kRegsHelper));
        if (n_union > 0 && warp == C::kProducerWarp) {
            // ======================= TMA producer ===================================
            if (lane == 0) {
                for (int t = prefilled; t < n_union; ++t) {
                    if (FA_TEST_SKIPS(t)) continue;
                    const int st = t % C::kStages;
                    const uint32_t ph = (t / C::kStages) & 1;
                    const int row = (hi - 1 - t) * kTile;
                    if (!mbar_wait(bar_k_empty + 8 * st, ph ^ 1, abort_flag)) { fail = 1; break; }
                    FA_TR(10);
                    mbar_expect_tx(bar_k_full + 8 * st, C::kTileBytes);
#pragma unroll
                    for (int b = 0; b < C::kBoxes; ++b)
                        tma_load_3d(sK + st * C::kTileBytes + b * (kTile * 128), &tmap_k, bar_k_full + 8 * st, b * 64, row, kv_unit);
                    if (!mbar_wait(bar_v_empty + 8 * st, ph ^ 1, abort_flag)) { fail = 2; break; }
                    FA_TR(11);
                    mbar_expect_tx(bar_v_full + 8 * st, C::kTileBytes);
#pragma unroll
                    for (int b = 0; b < C::kBoxes; ++b)
                        tma_load_3d(sV + st * C::kTileBytes + b * (kTile * 128), &tmap_v, bar_v_full + 8 * st, b * 64, row, kv_unit);
                }
            }
        } else if (n_union > 0 && warp == C::kMmaWarp) {
            // ======================= MMA issuer =====================================
            // The warp walks the loop together (it meets the softmax warpgroups at named
            // barriers); one elected lane issues the MMAs and commits.
            const bool leader = elect_one();
            constexpr uint32_t idesc_qk = make_idesc_f16(kTile, kTile, kBf16, false);
            constexpr uint32_t idesc_pv = make_idesc_f16(kTile, D, kBf16, true);
            // Descriptor words.  High word: SBO = 1024, 128-byte swizzle, version 1; low word:
            // start address (and for V the LBO of 16 KB between its two 64-column halves).
            const uint64_t dqk = make_smem_desc(0, 0, 1024);
            const uint64_t dvv = make_smem_desc(0, kTile * 128, 1024);
            const uint32_t desc_hi = static_cast<uint32_t>(dqk >> 32);
            const uint32_t q_lo = static_cast<uint32_t>(dqk) | (sQ >> 4);
            const uint32_t k_lo = static_cast<uint32_t>(dqk) | (sK >> 4);
            const uint32_t v_lo = static_cast<uint32_t>(dvv) | (sV >> 4);
            auto issue_qk = [&](int i, int st) {
                issue_qk_block<D>(tmem_base + i * kTile, q_lo + ((i * C::kTileBytes) >> 4),
                                  k_lo + ((st * C::kTileBytes) >> 4), desc_hi, idesc_qk);
                if constexpr (kBias) {
                    if (bias_in_mma)
                        issue_qk_bias(tmem_base + i * kTile, static_cast<uint32_t>(dqk) | ((smem_base + C::kSmemBiasQ) >> 4),
                                      static_cast<uint32_t>(dqk) | ((smem_base + C::kSmemBiasK) >> 4), desc_hi, idesc_qk);
                }
            };
            auto issue_pv_a = [&](int i, int st, uint32_t accumulate) {
                issue_pv_first(tmem_base + C::kTmemO + i * D, tmem_base + i * kTile,
                               v_lo + ((st * C::kTileBytes) >> 4), desc_hi, idesc_pv, accumulate);
            };
            auto issue_pv_b = [&](int i, int st) {
                issue_pv_rest(tmem_base + C::kTmemO + i * D, tmem_base + i * kTile,
                              v_lo + ((st * C::kTileBytes) >> 4), desc_hi, idesc_pv);
            };
            auto active = [&](int i, int tile) { return tile >= range[i].lo && tile < range[i].hi; };
            do {
                if (!mbar_wait_warp(bar_q_full, 0, abort_flag)) { fail = 3; break; }
                if (!mbar_wait_warp(bar_k_full, 0, abort_flag)) { fail = 4; break; }
                FA_TR(26);
                tc_fence_after_sync();
                if (leader) {
#pragma unroll
                    for (int i = 0; i < NQ; ++i) {
                        if (active(i, hi - 1)) {
                            issue_qk(i, 0);
                            umma_commit(bar_s_full + 8 * i);
                        }
                    }
                    umma_commit(bar_k_empty);
                }
                for (int t = 0; t < n_union && fail == 0; ++t) {
                    const int tile = hi - 1 - t;
                    const int st = t % C::kStages;
                    const uint32_t ph = (t / C::kStages) & 1;
                    const int st1 = (t + 1) % C::kStages;
                    const uint32_t ph1 = ((t + 1) / C::kStages) & 1;
                    const bool more = t + 1 < n_union;
                    // K/V tiles arrive long before they are needed; their barriers are looked at now,
                    // while the warp would wait for P anyway
                    if (!mbar_wait_warp(bar_v_full + 8 * st, ph, abort_flag)) { fail = 6; break; }
                    FA_TR(20);
                    if (more) {
                        if (!mbar_wait_warp(bar_k_full + 8 * st1, ph1, abort_flag)) { fail = 7; break; }
                        FA_TR(23);
                    }
#pragma unroll
                    for (int i = 0; i < NQ; ++i) {
                        if (active(i, tile)) {
                            // P V starts on the first half of P while the second half is exponentiated
                            named_sync(1 + 2 * i);
                            FA_TR(21 + 10 * i);
                            tc_fence_after_sync();
                            if (leader) issue_pv_a(i, st, tile < range[i].hi - 1 ? 1u : 0u);
                            named_sync(2 + 2 * i);
                            tc_fence_after_sync();
                            if (leader) {
                                issue_pv_b(i, st);
                                if (tile == range[i].lo) umma_commit(bar_o_full + 8 * i);
                            }
                            FA_TR(22 + 10 * i);
                        }
                        if (more && active(i, tile - 1)) {
                            if (leader) {
                                issue_qk(i, st1);
                                umma_commit(bar_s_full + 8 * i);
                            }
                            FA_TR(24 + 10 * i);
                        }
                    }
                    if (leader) {
                        umma_commit(bar_v_empty + 8 * st);
                        if (more) umma_commit(bar_k_empty + 8 * st1);
                    }
                }
            } while (false);
        } else if (kDropout && warp >= C::kKeepWarp0 && warp < C::kKeepWarp0 + NQ) {
            // ======================= dropout keep bits ==============================
            // (the first chunk was written before the CTA-wide sync)
            for (int chunk = 1; chunk * kKeepChunk < keep_tiles; ++chunk) {
                if (chunk >= 2) named_sync(keep_empty_id(keep_qi, chunk & 1));  // the softmax group has read chunk - 2
                keep_chunk(chunk);
            }
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(C::kRegsSoftmax));
        // ======================= softmax / epilogue =============================
        const int qi = warp >> 2;                        // which query tile of the CTA
        const int rb = qb * NQ + qi;                     // its 128-row block inside the unit
        const int r = threadIdx.x & 127;                 // row inside the tile
        const int row = rb * kTile + r;                  // row inside the unit
        const long long qpos = a.q_pos0 + row;
        const TileRange mine_r = (qi == 0) ? range[0] : range[NQ - 1];
        const int t_lo = mine_r.lo;
        const int n_tiles = mine_r.hi - mine_r.lo;
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t tmem_s = tmem_base + qi * kTile;          // S accumulator, 128 fp32 columns
        const uint32_t tmem_p = tmem_s;                          // P (16-bit, two per column) over S[0,64)
        const uint32_t tmem_o = tmem_base + C::kTmemO + qi * D;  // O accumulator, D fp32 columns
        const uint32_t my_s_full = bar_s_full + 8 * qi;
        const uint32_t my_o_full = bar_o_full + 8 * qi;
        float m_ref = -INFINITY;  // running max in log2 units (scaled, biased)
        float l_sum = 0.0f;
        float slope2 = 0.0f;
        if constexpr (kAlibi) slope2 = a.alibi_slopes[unit % a.heads] * kLog2e;
        const float scale2 = a.scale_log2;
        // Dropout keep bits of this row for the KV tile at hand: bit 8*(2*(g%2) + w) + 7 - g/2 <-> columns
        // 8g..8g+7 of parity w; read from the table the keep-bit helper warp of this query tile fills.
        uint32_t keep_bits = 0xffffffffu, keep_odd = 0xffffffffu;
        static_assert(kKeepChunk == 2, "the softmax loop reads a chunk's two words at once");

        for (int j = 0; j < n_tiles; ++j) {
            const int cb = t_lo + n_tiles - 1 - j;  // from the last KV tile of this query tile to the first
            const long long kbase = a.k_pos0 + static_cast<long long>(cb) * kTile;
            // columns this row may attend to inside the tile: [c_lo, c_hi] (worked out before S arrives)
            int c_lo = 0, c_hi = min(kTile - 1, a.seqlen_k - 1 - cb * kTile);
            if (a.is_causal) c_hi = static_cast<int>(min(static_cast<long long>(c_hi), qpos - kbase));
            if (a.window_right >= 0) c_hi = static_cast<int>(min(static_cast<long long>(c_hi), qpos + a.window_right - kbase));
            if (a.window_left >= 0) c_lo = static_cast<int>(max(0LL, min(qpos - a.window_left - kbase, 128LL)));
            const bool tile_masked_pre = __any_sync(0xffffffffu, c_lo > 0 || c_hi < kTile - 1);
            if constexpr (kDropout) {
                if ((j & 1) == 0) {
                    const int chunk = j / kKeepChunk;
                    // the chunk before this one has been read: its half of the ring may be refilled
                    if (chunk >= 1 && (chunk + 1) * kKeepChunk < n_tiles) named_arrive(keep_empty_id(qi, (chunk - 1) & 1));
                    named_sync(keep_full_id(qi, chunk & 1));
                    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];"
                                 : "=r"(keep_bits), "=r"(keep_odd)
                                 : "r"(smem_base + C::kSmemKeep +
                                       4u * static_cast<uint32_t>((qi * 2 + ((lane >> 3) & 1)) * kKeepRing + (chunk & 1) * kKeepChunk))
                                 : "memory");
                } else {
                    keep_bits = keep_odd;
                }
            }
            FA_TR(1);
            if (fail != 0 || !mbar_wait_warp(my_s_full, j & 1, abort_flag)) {
                // a wait gave up: keep the barrier protocol alive (the MMA warp counts on two
                // arrivals per tile from every softmax thread) and do nothing else
                fail = 8;
                named_arrive(1 + 2 * qi);
                named_arrive(2 + 2 * qi);
                continue;
            }
            FA_TR(2);
            tc_fence_after_sync();

            float s[128];
            {
                uint32_t tmp[4][32];
#pragma unroll
                for (int c = 0; c < 4; ++c) tmem_ld32(tmem_s + lane_base + c * 32, tmp[c]);
                tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < 128; ++c) s[c] = __uint_as_float(tmp[c / 32][c % 32]);
            }
            FA_TR(3);

            const bool tile_masked = tile_masked_pre;
            if (tile_masked) {
                // (two passes: a causal diagonal, the common case, needs only the upper bound)
                if (__any_sync(0xffffffffu, c_hi < kTile - 1)) {
#pragma unroll
                    for (int c = 0; c < 128; ++c)
                        if (c > c_hi) s[c] = -INFINITY;
                }
                if (__any_sync(0xffffffffu, c_lo > 0)) {
#pragma unroll
                    for (int c = 0; c < 128; ++c)
                        if (c < c_lo) s[c] = -INFINITY;
                }
            }

            // tile max in log2 units.  Without ALiBi the max is taken over the raw scores
            // (softmax_scale > 0) and the scale is folded into the exponent's FMA.
            float m_tile;
            // scores still unscaled (the scale is folded into the exponent's FMA) / the part of the ALiBi
            // bias that is constant along the row, when the tensor core has added the part linear in the column
            const bool raw_scores = !kAlibi || bias_in_mma;
            float row_bias = 0.0f;
            if constexpr (kAlibi) {
                const float dist0 = static_cast<float>(qpos - kbase);
                if (bias_in_mma) {
                    row_bias = -slope2 * dist0;
                } else if (keys_not_after) {
                    // bias of column c = slope*(c - dist0), built up pair by pair (one packed add and
                    // one packed FMA per two columns); the running sum is re-based every 16 columns
                    const float base = -slope2 * dist0;
                    const float2 step2 = make_float2(2.0f * slope2, 2.0f * slope2);
                    const float2 sc2 = make_float2(scale2, scale2);
#pragma unroll
                    for (int c0 = 0; c0 < 128; c0 += 16) {
                        float2 bias2 = make_float2(fmaf(slope2, static_cast<float>(c0), base),
                                                   fmaf(slope2, static_cast<float>(c0 + 1), base));
#pragma unroll
                        for (int c = c0; c < c0 + 16; c += 2) {
                            const float2 v2 = __ffma2_rn(make_float2(s[c], s[c + 1]), sc2, bias2);
                            s[c] = v2.x;
                            s[c + 1] = v2.y;
                            bias2 = __fadd2_rn(bias2, step2);
                        }
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < 128; ++c) s[c] = fmaf(-slope2, fabsf(dist0 - static_cast<float>(c)), s[c] * scale2);
                }
            }
            {
                float mx[4] = {s[0], s[1], s[2], s[3]};
#pragma unroll
                for (int c = 4; c < 128; c += 8) {
                    mx[0] = max3(mx[0], s[c], s[c + 1]);
                    mx[1] = max3(mx[1], s[c + 2], s[c + 3]);
                    if (c + 4 < 128) {
                        mx[2] = max3(mx[2], s[c + 4], s[c + 5]);
                        mx[3] = max3(mx[3], s[c + 6], s[c + 7]);
                    }
                }
                m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
                if constexpr (!kAlibi) m_tile *= scale2;
                else if (raw_scores) m_tile = fmaf(m_tile, scale2, row_bias);
            }
            FA_TR(4);

            // lazy rescale: keep the old reference max unless the new one is much larger
            float m_new = m_ref;
            float factor = 1.0f;
            if (m_tile > m_ref + kRescaleThreshold || m_ref == -INFINITY) {
                m_new = fmaxf(m_ref, m_tile);
                factor = (m_ref == -INFINITY) ? 0.0f : fast_exp2(m_ref - m_new);
            }
            const bool rescale = (j > 0) && (m_new != m_ref);
            if (__any_sync(0xffffffffu, rescale)) {
                // P V of the previous tile has completed (its commit precedes s_full), so O is stable.
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
            const float neg_m = (m_ref == -INFINITY) ? 0.0f : -m_ref;
            FA_TR(5);

            // P = exp2(s*scale - m), row sum over the undropped P (src/flash_forward.h:198-213, 221-237)
            float2 acc[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
            const float add_m = kAlibi ? neg_m + row_bias : neg_m;
            const float2 neg_m2 = make_float2(add_m, add_m);
            const float2 scale22 = (!kAlibi || raw_scores) ? make_float2(scale2, scale2) : make_float2(1.0f, 1.0f);
            // The pairs of kPolyMask go through poly_exp2_pair, the rest through MUFU ex2.  The
            // polynomial needs finite arguments: on tiles with masked (-inf) scores its results for those
            // elements are replaced by 0 (MUFU gives 0 by itself).
            auto exp_tile = [&](auto guard_tag) {
                constexpr uint32_t kPolyMask = kDropout ? kPolyMaskDropout : kPolyMaskPlain;
                constexpr bool kGuard = decltype(guard_tag)::value;  // the tile has masked (-inf) scores
#pragma unroll
                for (int c = 0; c < 4; ++c) {  // quarters of 32 columns
                    uint32_t pr[16];
#pragma unroll
                    for (int g = 0; g < 4; ++g) {  // 8 columns = 4 packed pairs share one dropout mask word
                        uint32_t msk = 0xffffffffu;
                        if constexpr (kDropout) {
                            // sign-replicating byte permute: bytes 0-1 of the mask from the sign of one byte of
                            // the shifted keep word (even columns), bytes 2-3 from the next (odd columns)
                            msk = prmt_sign(keep_bits << (c * 2 + (g >> 1)), (g & 1) ? 0xbbaau : 0x9988u);
                        }
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const int col = c * 32 + g * 8 + q * 2;
                            float2 x = make_float2(s[col], s[col + 1]);
                            x = __ffma2_rn(x, scale22, neg_m2);
                            float2 p;
                            if ((kPolyMask >> ((g & 1) * 4 + q)) & 1u) {
                                p = poly_exp2_pair(x);
                                if constexpr (kGuard) {
                                    // the polynomial gives 2^-126, not 0, for a masked score
                                    if (s[col] == -INFINITY) p.x = 0.0f;
                                    if (s[col + 1] == -INFINITY) p.y = 0.0f;
                                }
                            } else {
                                p.x = fast_exp2(x.x);
                                p.y = fast_exp2(x.y);
                            }
                            acc[q] = __fadd2_rn(acc[q], p);
                            pr[g * 4 + q] = pack2<kBf16>(p.x, p.y) & msk;
                        }
                    }
                    tmem_st16(tmem_p + lane_base + c * 16, pr);
                    if (c == (kSplitSteps * 16) / 32 - 1) {
                        // the first kSplitSteps*16 columns are stored: let the MMA warp start P V on them
                        tmem_wait_st();
                        tc_fence_before_sync();
                        named_arrive(1 + 2 * qi);
                        FA_TR(8);
                        FA_TR(8);
                    }
                }
            };
            if (tile_masked) exp_tile(std::true_type{});
            else exp_tile(std::false_type{});
            FA_TR(6);
            l_sum += (acc[0].x + acc[0].y) + (acc[1].x + acc[1].y) + (acc[2].x + acc[2].y) + (acc[3].x + acc[3].y);
            tmem_wait_st();
            tc_fence_before_sync();
            named_arrive(2 + 2 * qi);
            FA_TR(7);
        }

        // ---- epilogue: normalise and write O, LSE --------------------------------
        FA_TR(91);
        bool have_o = false;
        if (n_tiles > 0 && fail == 0) {
            if (mbar_wait_warp(my_o_full, 0, abort_flag)) { tc_fence_after_sync(); have_o = true; }
            else fail = 9;
        }
        FA_TR(96);
        float inv = 0.0f;
        if (l_sum > 0.0f) inv = (kDropout ? a.drop.inv_keep : 1.0f) / l_sum;
        const bool row_ok = row < a.seqlen_q;
        float lse_val = (l_sum > 0.0f) ? (m_ref * kLn2 + __logf(l_sum)) : -INFINITY;
        const long long unit_ll = unit;
        // Running result of a key sequence that arrives block by block (one launch per block: the ring
        // of a sequence sharded across GPUs): this launch's (O, LSE) is merged into the fp32 pair the
        // caller carries from launch to launch, with the algebra of the reference's combine kernel
        // (src/flash_forward_splitkv.h:359-397) in its log-sum-exp form,
        //   lse' = log(e^lse_c + e^lse),  O' = e^(lse_c - lse') O_c + e^(lse - lse') O,
        // here in the epilogue, on the row each thread already holds, instead of in a pass of its own.
        float w_old = 0.0f;  // weight of the carried row
        if (a.accum_o != nullptr) {
            const long long arow = unit_ll * a.seqlen_q + row;
            float lse_c = -INFINITY;
            if (!a.accum_first && row_ok) lse_c = a.accum_lse[arow];
            const float m = fmaxf(lse_c, lse_val);
            float lse_new = -INFINITY, w_new = 0.0f;
            if (m != -INFINITY) {
                const float e_old = __expf(lse_c - m), e_new = __expf(lse_val - m);
                const float sum = e_old + e_new;
                w_old = e_old / sum;
                w_new = e_new / sum;
                lse_new = m + __logf(sum);
            }
            inv *= w_new;
            lse_val = lse_new;
            if (row_ok) a.accum_lse[arow] = lse_new;
        }
        if (a.num_splits > 1) {
            const long long prow = (unit_ll * a.num_splits + split) * a.seqlen_q + row;
            if (row_ok) a.lse_partial[prow] = lse_val;
        } else if (a.lse != nullptr && row_ok) {
            a.lse[unit_ll * a.seqlen_q + row] = lse_val;
        }
        if (a.o_tma && have_o) {
            // 16-bit output of an unsplit launch: the rows are staged in this query tile's Q buffer
            // (free once the last Q K^T has completed, which o_full implies) in the 128-byte-swizzled
            // box layout, and each warp hands its 32 rows to the TMA unit, which writes whole lines
            // and clips rows >= seqlen_q and columns >= head_dim.
            const uint32_t stage = sQ + qi * C::kTileBytes;
            const int y0 = rb * kTile + (warp & 3) * 32;
#pragma unroll
            for (int b = 0; b < C::kBoxes; ++b) {  // a 64-column box at a time: its store runs while the next is packed
                uint32_t orow[2][32];
                tmem_ld32(tmem_o + lane_base + b * 64, orow[0]);
                tmem_ld32(tmem_o + lane_base + b * 64 + 32, orow[1]);
                tmem_wait_ld();
                const uint32_t row_addr = stage + b * (kTile * 128) + r * 128;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        const uint32_t x = pack2<kBf16>(__uint_as_float(orow[h][i]) * inv, __uint_as_float(orow[h][i + 1]) * inv);
                        const uint32_t y = pack2<kBf16>(__uint_as_float(orow[h][i + 2]) * inv, __uint_as_float(orow[h][i + 3]) * inv);
                        const uint32_t z = pack2<kBf16>(__uint_as_float(orow[h][i + 4]) * inv, __uint_as_float(orow[h][i + 5]) * inv);
                        const uint32_t w = pack2<kBf16>(__uint_as_float(orow[h][i + 6]) * inv, __uint_as_float(orow[h][i + 7]) * inv);
                        const uint32_t chunk = static_cast<uint32_t>(h * 4 + (i >> 3)) ^ static_cast<uint32_t>(r & 7);
                        st_shared_v4(row_addr + chunk * 16, x, y, z, w);
                    }
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0 && y0 < a.seqlen_q && b * 64 < a.head_dim) {
                    tma_store_3d(&tmap_o, stage + b * (kTile * 128) + (warp & 3) * (32 * 128), b * 64, y0, unit);
                    tma_store_commit();
                }
            }
            FA_TR(97);
            if (lane == 0) tma_store_wait_read();
        } else {
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
            if (a.accum_o != nullptr) {
                // merged row: read-modify-write of the carried fp32 row (each thread walks its own row;
                // the two 16-byte halves of every 32-byte sector are touched by consecutive
                // instructions), and on the sequence's last block the 16-bit output as well
                float* acc = a.accum_o + (unit_ll * a.seqlen_q + row) * a.head_dim;
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    if (col0 + i < a.head_dim) {
                        float4 v4 = make_float4(__uint_as_float(orow[i]) * inv, __uint_as_float(orow[i + 1]) * inv,
                                                __uint_as_float(orow[i + 2]) * inv, __uint_as_float(orow[i + 3]) * inv);
                        if (w_old != 0.0f) {
                            const float4 c4 = *reinterpret_cast<const float4*>(acc + col0 + i);
                            v4.x = fmaf(w_old, c4.x, v4.x);
                            v4.y = fmaf(w_old, c4.y, v4.y);
                            v4.z = fmaf(w_old, c4.z, v4.z);
                            v4.w = fmaf(w_old, c4.w, v4.w);
                        }
                        if (!a.accum_final || a.o == nullptr) *reinterpret_cast<float4*>(acc + col0 + i) = v4;
                        orow[i] = __float_as_uint(v4.x);
                        orow[i + 1] = __float_as_uint(v4.y);
                        orow[i + 2] = __float_as_uint(v4.z);
                        orow[i + 3] = __float_as_uint(v4.w);
                    }
                }
                if (a.accum_final && a.o != nullptr) {
                    if (a.o_is_fp32) {
                        float* dst = static_cast<float*>(a.o) + (unit_ll * a.seqlen_q + row) * a.head_dim;
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            if (col0 + i < a.head_dim)
                                *reinterpret_cast<uint4*>(dst + col0 + i) = make_uint4(orow[i], orow[i + 1], orow[i + 2], orow[i + 3]);
                    } else {
                        uint16_t* dst = static_cast<uint16_t*>(a.o) + (unit_ll * a.seqlen_q + row) * a.head_dim;
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            if (col0 + i < a.head_dim) {
                                uint4 v4;
                                v4.x = pack2<kBf16>(__uint_as_float(orow[i]), __uint_as_float(orow[i + 1]));
                                v4.y = pack2<kBf16>(__uint_as_float(orow[i + 2]), __uint_as_float(orow[i + 3]));
                                v4.z = pack2<kBf16>(__uint_as_float(orow[i + 4]), __uint_as_float(orow[i + 5]));
                                v4.w = pack2<kBf16>(__uint_as_float(orow[i + 6]), __uint_as_float(orow[i + 7]));
                                *reinterpret_cast<uint4*>(dst + col0 + i) = v4;
                            }
                        }
                    }
                }
                continue;
            }
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
    }

    // ---- teardown ------------------------------------------------------------------
    if (fail != 0) {
        *abort_flag = 1;
        if (a.status != nullptr) atomicExch(a.status, 100 + fail);
        // give copies that are still in flight time to land before the CTA's memory is reused
        const long long t0 = clock64();
        while (clock64() - t0 < 200000) { }
    }
    FA_TR(98);
    tc_fence_before_sync();
    __syncthreads();
    FA_TR(99);
    if (warp == C::kMmaWarp && n_union > 0) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

template <int D, int NQ, bool kBf16, bool kAlibi, bool kDropout>
cudaError_t launch_one(FwdArgs a, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                       const CUtensorMap& to, int units, cudaStream_t stream) {
    auto kern = fwd_tiled_kernel<D, NQ, kBf16, kAlibi, kDropout>;
    constexpr int smem = (kAlibi && Cfg<D, NQ>::kBiasBoxes) ? Cfg<D, NQ>::kSmemBytesBias : Cfg<D, NQ>::kSmemBytes;
    static_assert(smem <= 232448, "beyond the 227 KB a CTA may have");
    static std::atomic<bool> configured[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64 || !configured[dev].load(std::memory_order_acquire)) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev].store(true, std::memory_order_release);
    }
    const int trq = (a.tr + NQ - 1) / NQ;
    const long long per_unit = static_cast<long long>(trq) * a.num_splits;
    const long long ctas = static_cast<long long>(units) * per_unit;
    if (ctas <= 0 || ctas > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    a.div_group_ctas = make_fastdiv(static_cast<uint32_t>(std::min<long long>(a.unit_group * per_unit, 0x7fffffffLL)));
    a.div_gsize = make_fastdiv(static_cast<uint32_t>(a.unit_group));
    a.div_last_gsize = make_fastdiv(static_cast<uint32_t>(units % a.unit_group == 0 ? a.unit_group : units % a.unit_group));
    a.div_splits = make_fastdiv(static_cast<uint32_t>(a.num_splits));
    a.div_kv_group = make_fastdiv(static_cast<uint32_t>(a.kv_group));
    // launched with programmatic stream serialization: the kernel may begin its set-up while the
    // kernel before it in the stream drains
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(ctas));
    cfg.blockDim = dim3(Cfg<D, NQ>::kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, tq, tk, tv, to, a);
}

template <int D, int NQ, bool kBf16>
cudaError_t launch_flags(const FwdArgs& a, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                         const CUtensorMap& to, int units, bool alibi, bool dropout, cudaStream_t stream) {
    if (alibi) {
        return dropout ? launch_one<D, NQ, kBf16, true, true>(a, tq, tk, tv, to, units, stream)
                       : launch_one<D, NQ, kBf16, true, false>(a, tq, tk, tv, to, units, stream);
    }
    return dropout ? launch_one<D, NQ, kBf16, false, true>(a, tq, tk, tv, to, units, stream)
                   : launch_one<D, NQ, kBf16, false, false>(a, tq, tk, tv, to, units, stream);
}

template <int D, int NQ>
cudaError_t launch_dtype(const FwdArgs& a, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                         const CUtensorMap& to, int units, bool bf16, bool alibi, bool dropout, cudaStream_t stream) {
    return bf16 ? launch_flags<D, NQ, true>(a, tq, tk, tv, to, units, alibi, dropout, stream)
                : launch_flags<D, NQ, false>(a, tq, tk, tv, to, units, alibi, dropout, stream);
}

}  // namespace

cudaError_t launch_fwd_tiled(const FwdArgs& a, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                             const CUtensorMap& to, int units, bool bf16, bool dropout, cudaStream_t stream) {
    const bool alibi = a.alibi_slopes != nullptr;
    // two query tiles per CTA once a unit has more than one; a single tile (decode-like
    // shapes) keeps two independent CTAs per SM instead
    // (with two query tiles and a causal mask the pair would spend half its time on the diagonal tile that
    // only one of them can use: 277 against 308 TFLOP/s at [128,16,256,128])
    const bool pair = a.tr > 2 || (a.tr == 2 && !a.is_causal);
    if (a.head_dim <= 64) {
        return pair ? launch_dtype<64, 2>(a, tq, tk, tv, to, units, bf16, alibi, dropout, stream)
                    : launch_dtype<64, 1>(a, tq, tk, tv, to, units, bf16, alibi, dropout, stream);
    }
    return pair ? launch_dtype<128, 2>(a, tq, tk, tv, to, units, bf16, alibi, dropout, stream)
                : launch_dtype<128, 1>(a, tq, tk, tv, to, units, bf16, alibi, dropout, stream);
}

}  // namespace fa
