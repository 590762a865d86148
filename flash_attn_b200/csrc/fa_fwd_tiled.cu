// Tiled flash-attention forward for sm_100a.  Replaces the reference's
// forward_kernel (src/flash_forward.h:13-306) and forward_kernel_splitkv
// (src/flash_forward_splitkv.h:14-344).
//
// A work item is NQ (1 or 2) consecutive 128-row query tiles of one (batch, head)
// unit, optionally one KV split of them; each query tile is exactly one CTA of
// the reference's decomposition (grid (Tr*splits, H, B), src/main.cu:142-158),
// which is what the dropout streams are keyed on.  Roles by warp:
//   softmax groups (4 warps per query tile): thread r owns query row r.  S is read
//       from tensor memory (tcgen05.ld), masked / biased / exponentiated in
//       registers, the 16-bit P is written back to tensor memory over S
//       (tcgen05.st); the running (max, sum) and the lazy rescale of O live here.
//   TMA producer warp: streams the Q tiles and the K/V tiles through mbarrier
//       rings (cp.async.bulk.tensor, 128-byte swizzle).
//   MMA issuer warp: one thread issues tcgen05.mma for S_i = Q_i K^T (operands in
//       shared memory) and O_i += P_i V (P in tensor memory, V in shared memory,
//       MN-major), accumulators in tensor memory.  With NQ = 2 the two query tiles
//       alternate on the tensor pipe, so the softmax of one overlaps the MMAs of
//       the other while both share every K/V tile brought in by TMA.
// NQ = 1 (units of one or two query tiles): one CTA per item, two CTAs per SM.
// NQ = 2: a persistent kernel, one CTA per SM, which walks a list of items that the
// host scheduled for it (FwdSched).  TMEM, the barriers and the K/V ring live across
// items: the K/V tiles of consecutive items form one stream, the Q tiles of the next
// item are fetched as soon as the last Q K^T of the current one has been issued, the
// first Q K^T of the next item is issued behind the last P V of the current one, and O
// leaves through a small staging buffer per warp, so that a query tile's epilogue
// overlaps the other tile's tensor work instead of an empty SM.
// KV tiles are visited from the last to the first (the softmax is order-independent and the
// dropout draw of an element is a function of its position): with a causal mask the odd
// query tile of an item owns one KV tile more than the even one, the diagonal one, and
// walking backwards puts that solo tile at the start of the item.  The odd tile belongs to
// the softmax group that the MMA warp serves first, which is the group that finishes an
// item first: it runs the next item's solo tile while the other group is still finishing.
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
__device__ long long fa_trace_buf[16 * 4096];
__device__ unsigned int fa_claims[256 * 64];  // per CTA: the positions it claimed, in order
extern "C" int fa_claims_read(unsigned int* host_out) {
    return static_cast<int>(cudaMemcpyFromSymbol(host_out, fa_claims, sizeof(fa_claims)));
}
__device__ unsigned long long fa_cta_times[4 * 1024];  // per CTA: start, past the grid dependency wait, roles done, end (ns)
extern "C" int fa_cta_times_read(unsigned long long* host_out) {
    return static_cast<int>(cudaMemcpyFromSymbol(host_out, fa_cta_times, sizeof(fa_cta_times)));
}
__device__ __forceinline__ unsigned long long fa_globaltimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define FA_CTA_TIME(k)                                                                          \
    do {                                                                                       \
        if (threadIdx.x == 0 && blockIdx.x < 1024) fa_cta_times[4 * blockIdx.x + (k)] = fa_globaltimer(); \
    } while (0)
extern "C" int fa_trace_reset() {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, fa_trace_buf) != cudaSuccess) return -1;
    return static_cast<int>(cudaMemset(p, 0, sizeof(long long) * 16 * 4096));
}
extern "C" int fa_trace_read(long long* host_out) {
    return static_cast<int>(cudaMemcpyFromSymbol(host_out, fa_trace_buf, sizeof(long long) * 16 * 4096));
}
#define FA_TR(ev)                                                                              \
    do {                                                                                       \
        if (blockIdx.x == FA_TRACE_CTA && (threadIdx.x & 31) == 0 && tr_n < 2047) {                        \
            fa_trace_buf[(threadIdx.x >> 5) * 4096 + 2 * tr_n] = (ev);                          \
            fa_trace_buf[(threadIdx.x >> 5) * 4096 + 2 * tr_n + 1] = clock64();                 \
            ++tr_n;                                                                            \
        }                                                                                      \
    } while (0)
#else
#define FA_TR(ev) do { } while (0)
#define FA_CTA_TIME(k) do { } while (0)
#endif

namespace fa {

namespace {

constexpr float kRescaleThreshold = 8.0f;  // log2 units: rescale O only when the max grew by > 2^8
constexpr int kPolyPairsFrom = 3;  // of every 4 column pairs, pairs >= this use the polynomial exp2
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

template <int D, int NQ>
struct Cfg {
    static constexpr bool kPersist = NQ == 2;  // two query tiles per item: persistent kernel, one CTA per SM
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
    // persistent kernel: every softmax warp stages its 32 output rows, one 64-column box at a
    // time, in 4 KB of its own, so that the Q buffers are free for the next item's loads
    static constexpr int kSmemStage = kSmemV + kStages * kTileBytes;
    static constexpr int kStageBytes = kPersist ? NQ * 4 * 4096 : 0;
    static constexpr int kSmemBar = kSmemStage + kStageBytes;
    // persistent kernel: claimed items travel from the producer to the other roles through a ring
    static constexpr int kItemSlots = 4;
    static constexpr int kItemReaders = 1 + 4 * NQ;  // MMA warp + softmax warps
    static constexpr int kNumBars = 4 * NQ + 4 * kStages + (kPersist ? 2 * kItemSlots : 0);
    static constexpr int kSmemBytes = kSmemBar + 8 * kNumBars + 16 + 4 * kItemSlots + 1024;  // + alignment slack
    static_assert(kSmemBytes <= 232448, "shared memory of one CTA");
};

struct TileRange {
    int lo, hi;  // KV tiles [lo, hi)
};

__host__ __device__ __forceinline__ TileRange kv_tile_range(const FwdArgs& a, int rb, int split) {
    if (rb >= a.tr) return {0, 0};
    const long long q0 = a.q_pos0 + static_cast<long long>(rb) * kTile;
    const long long tc = a.tc;
    long long lo = 0, hi = tc;
    if (a.num_splits > 1) {  // src/flash_forward_splitkv.h:40-43
        lo = static_cast<long long>(a.tiles_per_split) * split;
        hi = lo + a.tiles_per_split < tc ? lo + a.tiles_per_split : tc;
    }
    if (a.window_left >= 0) {  // src/flash_forward.h:39
        long long w = (q0 - a.window_left - a.k_pos0) / kTile;  // truncating, like the reference
        w = w < 0 ? 0 : (w > tc ? tc : w);
        lo = lo > w ? lo : w;
    }
    if (a.window_right >= 0) {  // src/flash_forward.h:42-44
        const long long last = q0 + kTile - 1 + a.window_right - a.k_pos0;
        const long long h = last < 0 ? 0 : (last / kTile + 1 < tc ? last / kTile + 1 : tc);
        hi = hi < h ? hi : h;
    }
    if (a.is_causal) {  // src/flash_forward.h:46-48
        const long long last = q0 + kTile - 1 - a.k_pos0;
        const long long h = last < 0 ? 0 : (last / kTile + 1 < tc ? last / kTile + 1 : tc);
        hi = hi < h ? hi : h;
    }
    if (hi < lo) hi = lo;
    return {static_cast<int>(lo), static_cast<int>(hi)};
}

__device__ __forceinline__ uint32_t fast_div(const FastDiv& f, uint32_t x) {
    if (f.d == 1) return x;
    uint32_t q = __umulhi(x, f.m);
    if (q * f.d > x) --q;
    return q;
}

// Launch order of the items: groups of unit_group units; inside a group all units' first query
// block, then all second ones, ...  With a causal mask the blocks are visited heaviest first, so
// the launch is close to a longest-job-first schedule while the K/V working set of the items in
// flight (one group) stays far below the L2 size.
struct ItemPos {
    int unit, kv_unit, qb, split;
};
template <int NQ>
__host__ __device__ __forceinline__ ItemPos item_position(const FwdArgs& a, uint32_t p) {
    const int trq = (a.tr + NQ - 1) / NQ;  // query blocks of NQ tiles
#ifdef __CUDA_ARCH__
    const uint32_t g = fast_div(a.div_group_items, p);
#else
    const uint32_t g = p / a.div_group_items.d;
#endif
    const int unit0 = static_cast<int>(g) * a.unit_group;
    const uint32_t rem = p - g * a.div_group_items.d;
    const bool full = unit0 + a.unit_group <= a.units;
#ifdef __CUDA_ARCH__
    const uint32_t bx = fast_div(full ? a.div_gsize : a.div_last_gsize, rem);
#else
    const uint32_t bx = rem / (full ? a.div_gsize.d : a.div_last_gsize.d);
#endif
    ItemPos it;
    it.unit = unit0 + static_cast<int>(rem - bx * (full ? a.div_gsize.d : a.div_last_gsize.d));
    it.kv_unit = a.kv_group > 1 ? it.unit / a.kv_group : it.unit;  // grouped-query attention: K/V head of this unit
    uint32_t qb = bx;
    it.split = 0;
    if (a.num_splits > 1) {
#ifdef __CUDA_ARCH__
        qb = fast_div(a.div_splits, bx);
#else
        qb = bx / a.div_splits.d;
#endif
        it.split = static_cast<int>(bx - qb * a.div_splits.d);
    }
    it.qb = a.is_causal ? trq - 1 - static_cast<int>(qb) : static_cast<int>(qb);  // heaviest query blocks first
    return it;
}

// Query tile of softmax group i inside query block qb: the groups take the tiles in descending
// order, so that group 0, which the MMA warp serves first, owns the tile with the diagonal.
template <int NQ>
__host__ __device__ __forceinline__ int tile_of_group(int qb, int i) {
    return qb * NQ + (NQ - 1 - i);
}

template <int NQ>
struct Item {
    ItemPos pos;
    TileRange r[NQ];  // KV tiles of each softmax group's query tile
    int lo, hi;       // KV tiles streamed for the item: [lo, hi), empty when hi <= lo
};
template <int NQ>
__host__ __device__ __forceinline__ Item<NQ> make_item(const FwdArgs& a, uint32_t p) {
    Item<NQ> it;
    it.pos = item_position<NQ>(a, p);
    it.lo = 0x7fffffff;
    it.hi = 0;
#pragma unroll
    for (int i = 0; i < NQ; ++i) {
        it.r[i] = kv_tile_range(a, tile_of_group<NQ>(it.pos.qb, i), it.pos.split);
        if (it.r[i].hi > it.r[i].lo) {
            it.lo = it.r[i].lo < it.lo ? it.r[i].lo : it.lo;
            it.hi = it.r[i].hi > it.hi ? it.r[i].hi : it.hi;
        }
    }
    if (it.hi <= it.lo) it.lo = it.hi = 0;
    return it;
}

// Work distribution of the persistent kernel (NQ = 2).  The items of a launch form one list in
// launch order; the CTAs claim them one at a time from a counter in global memory, so that an SM
// that runs faster (the SMs of a B200 differ by several percent on this kernel, and a static
// split of the list left the slowest 15 % behind the mean) simply takes more of them.
//   The counter is one of kSchedSlots 64-bit words that belong to the library image; a launch is
// given the next slot in turn and a tag that is unique in the process.  High word = tag of the
// launch that owns the word, low word = claims made so far.  A claim adds one and finds either
// its own tag in what the word held, or anything else (and then restarts the word at its own
// tag): a word left behind by a launch that never finished therefore heals itself.  Every CTA makes exactly one claim
// beyond the end of the list; the CTA whose claim is the last one of the launch zeroes the
// word (tag 0 is never issued), which is what makes a captured launch replayable with the
// tag it was captured with.  Two launches that share a slot must not overlap on the device:
// with kSchedSlots in rotation that takes kSchedSlots launches in flight at once.
constexpr int kSchedSlots = 256;
__device__ unsigned long long g_sched_counter[kSchedSlots];
constexpr uint32_t kNoItem = 0xffffffffu;

__device__ __forceinline__ uint32_t claim_item(const FwdArgs& a) {
    unsigned long long* ctr = &g_sched_counter[a.sched_slot];
    const unsigned long long mine = static_cast<unsigned long long>(a.sched_tag) << 32;
    // One atomic add per claim (a compare-and-swap loop on the one word serialises the CTAs: with
    // 148 of them claiming at once only one attempt per round trip succeeds).
    unsigned long long old = atomicAdd(ctr, 1ull);
    if ((old >> 32) != a.sched_tag) {
        // The word is not this launch's yet (the add above only disturbed a count nobody needs):
        // install the tag, taking item 0, unless another CTA does so first.
        for (int tries = 0;; ++tries) {
            const unsigned long long cur = *reinterpret_cast<volatile unsigned long long*>(ctr);
            if ((cur >> 32) == a.sched_tag) {
                old = atomicAdd(ctr, 1ull);
                break;
            }
            if (atomicCAS(ctr, cur, mine + 1) == cur) {
                old = mine;
                break;
            }
            if (tries > (1 << 16)) return kNoItem;  // (never seen: every failed attempt means another CTA's succeeded)
        }
    }
    const uint32_t n = static_cast<uint32_t>(old);
    if (n + 1 == static_cast<uint32_t>(a.n_items) + gridDim.x) atomicExch(ctr, 0ull);  // the launch's last claim
    return n < static_cast<uint32_t>(a.n_items) ? n : kNoItem;
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
constexpr int kPBarrierThreads = 160;  // 128 softmax threads + the MMA warp
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
constexpr int kSplitSteps = 6;
__device__ __forceinline__ void issue_pv_first(uint32_t d_tmem, uint32_t a_tmem, uint32_t vb_lo, uint32_t desc_hi,
                                               uint32_t idesc, uint32_t accumulate) {
    asm volatile(FA_PV_HEAD FA_PV_STEP FA_PV_STEP FA_PV_STEP FA_PV_STEP FA_PV_STEP "}"
                 ::"r"(d_tmem), "r"(a_tmem), "r"(vb_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
                 : "memory");
}
__device__ __forceinline__ void issue_pv_rest(uint32_t d_tmem, uint32_t a_tmem, uint32_t vb_lo, uint32_t desc_hi,
                                              uint32_t idesc) {
    asm volatile(FA_PV_HEAD FA_PV_STEP "}"
                 ::"r"(d_tmem), "r"(a_tmem + kSplitSteps * 8), "r"(vb_lo + kSplitSteps * 128), "r"(desc_hi), "r"(idesc), "r"(1u)
                 : "memory");
}

template <int D, int NQ, bool kBf16, bool kAlibi, bool kDropout>
__global__ void __launch_bounds__(Cfg<D, NQ>::kThreads, NQ == 1 ? 2 : 1)
fwd_tiled_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_o,
                 const __grid_constant__ FwdArgs a) {
    using C = Cfg<D, NQ>;
    extern __shared__ uint8_t smem_raw[];
    // 128-byte-swizzled tiles need a 1024-byte aligned base
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t sQ = smem_base + C::kSmemQ;
    const uint32_t sK = smem_base + C::kSmemK;
    const uint32_t sV = smem_base + C::kSmemV;
    const uint32_t sStage = smem_base + C::kSmemStage;
    const uint32_t bar0 = smem_base + C::kSmemBar;
    // barrier map
    const uint32_t bar_q_full = bar0;                            // [NQ]  Q tile of group i has landed
    const uint32_t bar_q_empty = bar_q_full + 8 * NQ;            // [NQ]  last Q K^T of group i's item has completed
    const uint32_t bar_s_full = bar_q_empty + 8 * NQ;            // [NQ]
    const uint32_t bar_o_full = bar_s_full + 8 * NQ;             // [NQ]
    const uint32_t bar_k_full = bar_o_full + 8 * NQ;             // [kStages]
    const uint32_t bar_k_empty = bar_k_full + 8 * C::kStages;    // [kStages]
    const uint32_t bar_v_full = bar_k_empty + 8 * C::kStages;    // [kStages]
    const uint32_t bar_v_empty = bar_v_full + 8 * C::kStages;    // [kStages]
    const uint32_t bar_item_full = bar_v_empty + 8 * C::kStages;      // [kItemSlots] (persistent kernel)
    const uint32_t bar_item_empty = bar_item_full + 8 * C::kItemSlots;  // [kItemSlots]
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + C::kSmemBar + 8 * C::kNumBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + C::kSmemBar + 8 * C::kNumBars + 4);
    volatile uint32_t* item_ring = reinterpret_cast<volatile uint32_t*>(smem_gen + C::kSmemBar + 8 * C::kNumBars + 16);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
#ifdef FA_TRACE
    int tr_n = 0;
    FA_TR(90);
#endif
    FA_CTA_TIME(0);

    // Programmatic dependent launch: let the next kernel of the stream start its own set-up as
    // soon as SMs free up, and do this kernel's set-up (index arithmetic, barriers, TMEM) before
    // waiting for the kernel in front of it; no global memory is touched before grid_dep_wait().
    grid_dep_launch_dependents();

    // ---- set-up ----------------------------------------------------------------
    // The barriers are initialised by the lanes that use them first: the producer lane its ring
    // and Q barriers, after which it immediately puts the first item's Q tiles and the first
    // ring-full of K/V tiles in flight, so that the HBM latency of these first loads overlaps the
    // TMEM allocation and the CTA-wide synchronisation instead of following them.
    int fail = 0;
    uint32_t prod_pub = 0;   // items published so far (producer lane)
    Item<NQ> prod_item;
    bool prod_have = false;
    int prod_t = 0;          // KV tiles of prod_item already requested
    uint32_t prod_g = 0;     // KV tiles requested so far (position in the ring)
    uint32_t prod_q[NQ];     // Q tiles requested so far, per softmax group
#pragma unroll
    for (int i = 0; i < NQ; ++i) prod_q[i] = 0;

    auto load_kv_tile = [&](const Item<NQ>& it, int t, uint32_t g) __attribute__((always_inline)) {
        const int st = static_cast<int>(g % C::kStages);
        const int row = (it.hi - 1 - t) * kTile;  // KV tiles are walked from the last to the first
        mbar_expect_tx(bar_k_full + 8 * st, C::kTileBytes);
#pragma unroll
        for (int b = 0; b < C::kBoxes; ++b)
            tma_load_3d(sK + st * C::kTileBytes + b * (kTile * 128), &tmap_k, bar_k_full + 8 * st, b * 64, row, it.pos.kv_unit);
        return st;
    };
    auto load_v_tile = [&](const Item<NQ>& it, int t, int st) __attribute__((always_inline)) {
        const int row = (it.hi - 1 - t) * kTile;
        mbar_expect_tx(bar_v_full + 8 * st, C::kTileBytes);
#pragma unroll
        for (int b = 0; b < C::kBoxes; ++b)
            tma_load_3d(sV + st * C::kTileBytes + b * (kTile * 128), &tmap_v, bar_v_full + 8 * st, b * 64, row, it.pos.kv_unit);
    };
    auto load_q_tile = [&](const Item<NQ>& it, int i) __attribute__((always_inline)) {
        mbar_expect_tx(bar_q_full + 8 * i, C::kTileBytes);
#pragma unroll
        for (int b = 0; b < C::kBoxes; ++b)
            tma_load_3d(sQ + i * C::kTileBytes + b * (kTile * 128), &tmap_q, bar_q_full + 8 * i, b * 64,
                        tile_of_group<NQ>(it.pos.qb, i) * kTile, it.pos.unit);
    };

    // Producer lane: next item of this CTA that streams at least one KV tile.  Every item claimed on
    // the way (the softmax groups write zero rows for items without KV tiles) and the end of the
    // list are published to the other roles.
    auto producer_next = [&]() __attribute__((always_inline)) -> bool {
        for (;;) {
            uint32_t pos;
            if constexpr (C::kPersist) {
                pos = claim_item(a);
#ifdef FA_TRACE
                if (blockIdx.x < 256 && prod_pub < 64) fa_claims[blockIdx.x * 64 + prod_pub] = pos;
#endif
                const uint32_t slot = prod_pub % C::kItemSlots;
                if (prod_pub >= C::kItemSlots &&
                    !mbar_wait(bar_item_empty + 8 * slot, ((prod_pub / C::kItemSlots) - 1) & 1, abort_flag)) {
                    fail = 12;
                    return false;
                }
                item_ring[slot] = pos;
                mbar_arrive(bar_item_full + 8 * slot);  // (release: the store above is visible to whoever sees the phase)
                ++prod_pub;
            } else {
                pos = prod_pub++ == 0 ? blockIdx.x : kNoItem;
            }
            if (pos == kNoItem) return false;
            prod_item = make_item<NQ>(a, pos);
            if (prod_item.hi > prod_item.lo) return true;
        }
    };
    // The other roles: next published item (warp-collective).
    auto consume_item = [&](uint32_t& n_seen) __attribute__((always_inline)) -> uint32_t {
        if constexpr (C::kPersist) {
            const uint32_t slot = n_seen % C::kItemSlots;
            if (!mbar_wait_warp(bar_item_full + 8 * slot, (n_seen / C::kItemSlots) & 1, abort_flag)) {
                fail = 11;
                return kNoItem;
            }
            const uint32_t pos = item_ring[slot];
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_item_empty + 8 * slot);
            ++n_seen;
            return pos;
        } else {
            return n_seen++ == 0 ? blockIdx.x : kNoItem;
        }
    };
    auto consume_streaming_item = [&](uint32_t& n_seen, Item<NQ>* it) __attribute__((always_inline)) -> bool {
        for (;;) {
            const uint32_t pos = consume_item(n_seen);
            if (pos == kNoItem) return false;
            *it = make_item<NQ>(a, pos);
            if (it->hi > it->lo) return true;
        }
    };

    if (warp == C::kProducerWarp && lane == 0) {
        *abort_flag = 0;
        for (int i = 0; i < NQ; ++i) {
            mbar_init(bar_q_full + 8 * i, 1);
            mbar_init(bar_q_empty + 8 * i, 1);
        }
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(bar_k_full + 8 * s, 1);
            mbar_init(bar_k_empty + 8 * s, 1);
            mbar_init(bar_v_full + 8 * s, 1);
            mbar_init(bar_v_empty + 8 * s, 1);
        }
        if constexpr (C::kPersist) {
            for (int s = 0; s < C::kItemSlots; ++s) {
                mbar_init(bar_item_full + 8 * s, 1);
                mbar_init(bar_item_empty + 8 * s, C::kItemReaders);
            }
        }
        mbar_fence_init();
        prod_have = producer_next();  // (the claim counter is not data of the kernel in front: no need to wait for it)
        grid_dep_wait();
        tma_prefetch_desc(&tmap_q);
        tma_prefetch_desc(&tmap_k);
        tma_prefetch_desc(&tmap_v);
        if (a.o_tma) tma_prefetch_desc(&tmap_o);
        if (prod_have) {
#pragma unroll
            for (int i = 0; i < NQ; ++i) {
                if (prod_item.r[i].hi > prod_item.r[i].lo) {
                    load_q_tile(prod_item, i);
                    ++prod_q[i];
                }
            }
            const int pre = min(C::kStages, prod_item.hi - prod_item.lo);
            for (; prod_t < pre; ++prod_t, ++prod_g) {  // the ring is empty: no waits
                const int st = load_kv_tile(prod_item, prod_t, prod_g);
                load_v_tile(prod_item, prod_t, st);
            }
        }
    }
    if (warp == C::kMmaWarp) {
        if (lane == 0) {
            for (int i = 0; i < NQ; ++i) {
                mbar_init(bar_s_full + 8 * i, 1);
                mbar_init(bar_o_full + 8 * i, 1);
            }
            mbar_fence_init();
        }
        __syncwarp();
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), C::kTmemCols);
        tmem_relinquish();
    }
    grid_dep_wait();  // every thread, before its first global access (the producer lane has passed it already)
    FA_CTA_TIME(1);
    FA_TR(92);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    FA_TR(93);
    const uint32_t tmem_base = *tmem_slot;

    // The helper warpgroup (producer, MMA issuer, two idle warps) hands most of its registers to
    // the softmax warpgroups, which hold a 128-column score row per thread.  Each register
    // regime covers one whole branch below.
    if (warp >= NQ * 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(C::kRegsHelper));
        if (warp == C::kProducerWarp) {
            // ======================= TMA producer ===================================
            if (lane == 0) {
                bool q_owed = false;  // the Q tiles of prod_item have not been requested yet
                while (prod_have && fail == 0) {
                    const int n_union = prod_item.hi - prod_item.lo;
                    for (; prod_t < n_union; ++prod_t, ++prod_g) {
                        const int st = static_cast<int>(prod_g % C::kStages);
                        const uint32_t ph = (prod_g / C::kStages) & 1;
                        if (prod_g >= C::kStages && !mbar_wait(bar_k_empty + 8 * st, ph ^ 1, abort_flag)) { fail = 1; break; }
                        FA_TR(10);
                        load_kv_tile(prod_item, prod_t, prod_g);
                        if (q_owed) {
                            // A new item: its first K tile is in flight (its ring slot came free long ago); the
                            // Q buffer of a group is free once its last Q K^T of the previous item has completed.
                            q_owed = false;
#pragma unroll
                            for (int i = 0; i < NQ; ++i) {
                                if (prod_item.r[i].hi > prod_item.r[i].lo) {
                                    if (prod_q[i] > 0 && !mbar_wait(bar_q_empty + 8 * i, (prod_q[i] - 1) & 1, abort_flag)) { fail = 10; break; }
                                    FA_TR(12);
                                    load_q_tile(prod_item, i);
                                    ++prod_q[i];
                                }
                            }
                            if (fail != 0) break;
                        }
                        if (prod_g >= C::kStages && !mbar_wait(bar_v_empty + 8 * st, ph ^ 1, abort_flag)) { fail = 2; break; }
                        FA_TR(11);
                        load_v_tile(prod_item, prod_t, st);
                    }
                    if (fail != 0) break;
                    prod_have = producer_next();
                    prod_t = 0;
                    q_owed = true;
                }
            }
        } else if (warp == C::kMmaWarp) {
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
            auto issue_pv_a = [&](int i, int st, uint32_t accumulate) __attribute__((always_inline)) {
                issue_pv_first(tmem_base + C::kTmemO + i * D, tmem_base + i * kTile,
                               v_lo + ((st * C::kTileBytes) >> 4), desc_hi, idesc_pv, accumulate);
            };
            auto issue_pv_b = [&](int i, int st) __attribute__((always_inline)) {
                issue_pv_rest(tmem_base + C::kTmemO + i * D, tmem_base + i * kTile,
                              v_lo + ((st * C::kTileBytes) >> 4), desc_hi, idesc_pv);
            };
            auto active = [&](const TileRange& rg, int tile) __attribute__((always_inline)) { return tile >= rg.lo && tile < rg.hi; };
            // S_i = Q_i K^T for KV tile `tile` of a query tile with KV range rg, K in ring slot st; the
            // last Q K^T of an item also releases the group's Q buffer
            auto issue_qk = [&](const TileRange& rg, int i, int tile, int st) __attribute__((always_inline)) {
                if (leader) {
                    issue_qk_block<D>(tmem_base + i * kTile, q_lo + ((i * C::kTileBytes) >> 4),
                                      k_lo + ((st * C::kTileBytes) >> 4), desc_hi, idesc_qk);
                    umma_commit(bar_s_full + 8 * i);
                    if (C::kPersist && tile == rg.lo) umma_commit(bar_q_empty + 8 * i);
                }
            };
            uint32_t items_seen = 0;
            Item<NQ> cur, nxt;
            bool have = consume_streaming_item(items_seen, &cur);
            uint32_t g = 0;       // KV tiles consumed so far (position in the ring)
            uint32_t q_seen[NQ];  // Q tiles consumed so far, per softmax group
#pragma unroll
            for (int i = 0; i < NQ; ++i) q_seen[i] = 0;
            do {
                if (!have) break;
                // first Q K^T of the first item
#pragma unroll
                for (int i = 0; i < NQ; ++i) {
                    if (cur.r[i].hi > cur.r[i].lo) {
                        if (!mbar_wait_warp(bar_q_full + 8 * i, 0, abort_flag)) { fail = 3; break; }
                        ++q_seen[i];
                    }
                }
                if (fail != 0) break;
                if (!mbar_wait_warp(bar_k_full, 0, abort_flag)) { fail = 4; break; }
                FA_TR(26);
                tc_fence_after_sync();
#pragma unroll
                for (int i = 0; i < NQ; ++i)
                    if (active(cur.r[i], cur.hi - 1)) issue_qk(cur.r[i], i, cur.hi - 1, 0);
                if (leader) umma_commit(bar_k_empty);
                while (have && fail == 0) {
                    bool have_next = false;
                    const int n_union = cur.hi - cur.lo;
                    for (int t = 0; t < n_union && fail == 0; ++t, ++g) {
                        // the item after this one is asked for when its first tile comes into view; the
                        // producer has published it by then (it did so after this item's last load)
                        if (t + 1 == n_union) {
                            have_next = consume_streaming_item(items_seen, &nxt);
                            if (fail != 0) break;
                        }
                        const int tile = cur.hi - 1 - t;
                        const int st = static_cast<int>(g % C::kStages);
                        const uint32_t ph = (g / C::kStages) & 1;
                        const int st1 = static_cast<int>((g + 1) % C::kStages);
                        const uint32_t ph1 = ((g + 1) / C::kStages) & 1;
                        const bool last = t + 1 == n_union;
                        const bool more = !last || have_next;  // another KV tile follows in the stream
                        const int ntile = last ? nxt.hi - 1 : tile - 1;
                        TileRange nr[NQ];  // KV ranges of the query tiles of that tile's item
#pragma unroll
                        for (int i = 0; i < NQ; ++i) {
                            nr[i].lo = last ? nxt.r[i].lo : cur.r[i].lo;
                            nr[i].hi = last ? nxt.r[i].hi : cur.r[i].hi;
                        }
                        // Operands of the next tile's Q K^T: its K tile and, when it opens the next item, that
                        // item's Q tiles.  At an item boundary they may still be in flight, and this step's
                        // P V must not wait for them: they are then looked at when the first such Q K^T is due.
                        // Groups that sit this tile out but take the next one get their Q K^T at that moment too.
                        bool next_ready = !more;
                        auto next_operands = [&]() __attribute__((always_inline)) {
                            if (next_ready || fail != 0) return;
                            if (!mbar_wait_warp(bar_k_full + 8 * st1, ph1, abort_flag)) { fail = 7; return; }
                            if (last) {
#pragma unroll
                                for (int i = 0; i < NQ; ++i) {
                                    if (nxt.r[i].hi > nxt.r[i].lo) {
                                        if (!mbar_wait_warp(bar_q_full + 8 * i, q_seen[i] & 1, abort_flag)) { fail = 5; return; }
                                        ++q_seen[i];
                                    }
                                }
                            }
                            FA_TR(23);
                            next_ready = true;
                            tc_fence_after_sync();
#pragma unroll
                            for (int i = 0; i < NQ; ++i)
                                if (!active(cur.r[i], tile) && active(nr[i], ntile)) issue_qk(nr[i], i, ntile, st1);
                        };
                        // the P V of this step needs V
                        if (!mbar_wait_warp(bar_v_full + 8 * st, ph, abort_flag)) { fail = 6; break; }
                        FA_TR(20);
                        if (more) {
                            // Inside an item the next K tile landed long ago: its barrier is looked at now, while
                            // the warp would wait for P anyway (a poll costs hundreds of cycles while the tensor
                            // pipe streams operands, and between P V and Q K^T it would sit on the critical
                            // chain).  The same goes for a group that sits this tile out and takes the next.
                            bool idle_takes_next = false;
#pragma unroll
                            for (int i = 0; i < NQ; ++i) idle_takes_next |= !active(cur.r[i], tile) && active(nr[i], ntile);
                            if (!last || idle_takes_next) next_operands();
                            if (fail != 0) break;
                        }
#pragma unroll
                        for (int i = 0; i < NQ; ++i) {
                            if (active(cur.r[i], tile)) {
                                // P V starts on the first three quarters of P while the last is exponentiated
                                named_sync(1 + 2 * i);
                                FA_TR(21 + 10 * i);
                                tc_fence_after_sync();
                                if (leader) issue_pv_a(i, st, tile < cur.r[i].hi - 1 ? 1u : 0u);
                                named_sync(2 + 2 * i);
                                tc_fence_after_sync();
                                if (leader) {
                                    issue_pv_b(i, st);
                                    if (tile == cur.r[i].lo) umma_commit(bar_o_full + 8 * i);
                                }
                                FA_TR(22 + 10 * i);
                                if (more && active(nr[i], ntile)) {
                                    next_operands();
                                    if (fail != 0) break;
                                    issue_qk(nr[i], i, ntile, st1);
                                    FA_TR(24 + 10 * i);
                                }
                            }
                        }
                        next_operands();  // (nobody took the next tile yet: its operands are still owed a look)
                        if (fail != 0) break;
                        if (leader) {
                            umma_commit(bar_v_empty + 8 * st);
                            if (more) umma_commit(bar_k_empty + 8 * st1);
                        }
                    }
                    cur = nxt;
                    have = have_next;
                }
            } while (false);
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(C::kRegsSoftmax));
        // ======================= softmax / epilogue =============================
        const int qi = warp >> 2;                        // which softmax group of the CTA
        const int r = threadIdx.x & 127;                 // row inside the tile
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t tmem_s = tmem_base + qi * kTile;          // S accumulator, 128 fp32 columns
        const uint32_t tmem_p = tmem_s;                          // P (16-bit, two per column) over S[0,64)
        const uint32_t tmem_o = tmem_base + C::kTmemO + qi * D;  // O accumulator, D fp32 columns
        const uint32_t my_s_full = bar_s_full + 8 * qi;
        const uint32_t my_o_full = bar_o_full + 8 * qi;
        // every unmasked key lies at or before the query: |q - k| = q - k
        const bool keys_not_after = a.is_causal || a.window_right == 0;
        const float scale2 = a.scale_log2;
        uint32_t s_seen = 0;   // S tiles consumed so far by this group (phase of s_full)
        uint32_t o_seen = 0;   // items with at least one KV tile finished so far (phase of o_full)
        bool staged = false;   // a TMA store of this warp may still be reading its staging buffer

        // One item of this softmax group.  The next item is looked up (position, KV range, ALiBi slope,
        // first dropout bits) while the group waits for the last P V of the current one.
        struct GroupItem {
            int unit, split, rb, t_lo, n_tiles;
            float slope2;
            unsigned long long subseq;
            uint32_t keep_first;
        };
        // Dropout keep bits of a row for KV tile j (counted from the first KV tile of the query tile):
        // bit 2*g + w <-> columns 8g..8g+7 of parity w.  Lanes 0-15 evaluate one Philox block each
        // (lane = 2*i + row-half: draws 8*i + 4*half + {0..3}); a row gathers the eight blocks of its
        // half.  Computed one tile ahead, while the warp would otherwise wait for S.
        auto tile_keep_bits = [&](unsigned long long subseq, int j) __attribute__((always_inline)) -> uint32_t {
            if constexpr (!kDropout) return 0xffffffffu;
            uint32_t mine = 0;
            if (lane < 16) mine = philox_keep4(a.drop, subseq, 64ull * static_cast<unsigned long long>(j) + 4ull * lane);
            const int half = (lane >> 3) & 1;
            uint32_t bits = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) bits |= __shfl_sync(0xffffffffu, mine, 2 * i + half) << (4 * i);
            return bits;
        };
        uint32_t items_seen = 0;
        auto fetch_item = [&](GroupItem* it) __attribute__((always_inline)) -> bool {
            for (;;) {
                const uint32_t pos = consume_item(items_seen);
                if (pos == kNoItem) return false;
                FA_TR(100000 + static_cast<long long>(pos));
                const ItemPos ip = item_position<NQ>(a, pos);
                const int rb = tile_of_group<NQ>(ip.qb, qi);  // this group's 128-row block inside the unit
                if (rb >= a.tr) continue;                     // the unit has an odd number of query tiles
                const TileRange rg = kv_tile_range(a, rb, ip.split);
                it->unit = ip.unit;
                it->split = ip.split;
                it->rb = rb;
                it->t_lo = rg.lo;
                it->n_tiles = rg.hi - rg.lo;
                it->slope2 = 0.0f;
                if constexpr (kAlibi) it->slope2 = a.alibi_slopes[ip.unit % a.heads] * kLog2e;
                it->subseq = 0;
                if constexpr (kDropout)
                    it->subseq = (a.drop.unit0 + ip.unit) * static_cast<unsigned long long>(a.tr * a.num_splits) +
                                 static_cast<unsigned long long>(rb * a.num_splits + ip.split);
                it->keep_first = it->n_tiles > 0 ? tile_keep_bits(it->subseq, it->n_tiles - 1) : 0u;
                return true;
            }
        };
        GroupItem item;
        bool have_item = fetch_item(&item);
        while (have_item) {
        const int unit = item.unit;
        const int split = item.split;
        const int rb = item.rb;
        const int row = rb * kTile + r;                  // row inside the unit
        const long long qpos = a.q_pos0 + row;
        const int t_lo = item.t_lo;
        const int n_tiles = item.n_tiles;
        const float slope2 = item.slope2;
        const unsigned long long subseq = item.subseq;
        float m_ref = -INFINITY;  // running max in log2 units (scaled, biased)
        float l_sum = 0.0f;
        uint32_t keep_next = item.keep_first;

        for (int j = 0; j < n_tiles; ++j, ++s_seen) {
            const int cb = t_lo + n_tiles - 1 - j;  // from the last KV tile of this query tile to the first
            const long long kbase = a.k_pos0 + static_cast<long long>(cb) * kTile;
            // columns this row may attend to inside the tile: [c_lo, c_hi] (worked out before S arrives)
            int c_lo = 0, c_hi = min(kTile - 1, a.seqlen_k - 1 - cb * kTile);
            if (a.is_causal) c_hi = static_cast<int>(min(static_cast<long long>(c_hi), qpos - kbase));
            if (a.window_right >= 0) c_hi = static_cast<int>(min(static_cast<long long>(c_hi), qpos + a.window_right - kbase));
            if (a.window_left >= 0) c_lo = static_cast<int>(max(0LL, min(qpos - a.window_left - kbase, 128LL)));
            const bool tile_masked_pre = __any_sync(0xffffffffu, c_lo > 0 || c_hi < kTile - 1);
            FA_TR(1);
            if (fail != 0 || !mbar_wait_warp(my_s_full, s_seen & 1, abort_flag)) {
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
            if constexpr (kAlibi) {
                const float dist0 = static_cast<float>(qpos - kbase);
                if (keys_not_after) {
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
            const uint32_t keep_bits = keep_next;
            FA_TR(5);

            // P = exp2(s*scale - m), row sum over the undropped P (src/flash_forward.h:198-213, 221-237)
            float2 acc[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
            const float2 neg_m2 = make_float2(neg_m, neg_m);
            const float2 scale22 = make_float2(scale2, scale2);
            // On tiles without masked elements (every score finite, so no argument is -inf) pairs
            // kPolyFrom..3 of every four go through poly_exp2_pair, the rest through MUFU ex2.
            auto exp_tile = [&](auto poly_tag) {
                constexpr int kPolyFrom = decltype(poly_tag)::value;
#pragma unroll
                for (int c = 0; c < 4; ++c) {  // quarters of 32 columns
                    uint32_t pr[16];
#pragma unroll
                    for (int g = 0; g < 4; ++g) {  // 8 columns = 4 packed pairs share one dropout mask word
                        uint32_t msk = 0xffffffffu;
                        if constexpr (kDropout) {
                            const uint32_t two = (keep_bits >> (2 * (c * 4 + g))) & 3u;
                            msk = __byte_perm(0u - (two & 1u), 0u - (two >> 1), 0x7610);
                        }
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const int col = c * 32 + g * 8 + q * 2;
                            float2 x = make_float2(s[col], s[col + 1]);
                            if constexpr (kAlibi) x = __fadd2_rn(x, neg_m2);
                            else x = __ffma2_rn(x, scale22, neg_m2);
                            float2 p;
                            if (q >= kPolyFrom) {
                                p = poly_exp2_pair(x);
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
                    }
                }
            };
            if (tile_masked) exp_tile(std::integral_constant<int, 4>{});
            else exp_tile(std::integral_constant<int, kPolyPairsFrom>{});
            FA_TR(6);
            l_sum += (acc[0].x + acc[0].y) + (acc[1].x + acc[1].y) + (acc[2].x + acc[2].y) + (acc[3].x + acc[3].y);
            tmem_wait_st();
            tc_fence_before_sync();
            named_arrive(2 + 2 * qi);
            FA_TR(7);
            if (j + 1 < n_tiles) keep_next = tile_keep_bits(subseq, n_tiles - 2 - j);
        }

        // ---- epilogue: normalise and write O, LSE --------------------------------
        FA_TR(91);
        GroupItem next_item_;
        const bool have_next_item = fetch_item(&next_item_);
        bool have_o = false;
        if (n_tiles > 0) {
            if (fail == 0) {
                if (mbar_wait_warp(my_o_full, o_seen & 1, abort_flag)) { tc_fence_after_sync(); have_o = true; }
                else fail = 9;
            }
            ++o_seen;
        }
        if (fail == 0) {  // (after a failed wait the results are void; the items are still walked for the barrier protocol)
        FA_TR(96);
        float inv = 0.0f;
        if (l_sum > 0.0f) inv = (kDropout ? a.drop.inv_keep : 1.0f) / l_sum;
        const bool row_ok = row < a.seqlen_q;
        const float lse_val = (l_sum > 0.0f) ? (m_ref * kLn2 + __logf(l_sum)) : -INFINITY;
        const long long unit_ll = unit;
        if (a.num_splits > 1) {
            const long long prow = (unit_ll * a.num_splits + split) * a.seqlen_q + row;
            if (row_ok) a.lse_partial[prow] = lse_val;
        } else if (a.lse != nullptr && row_ok) {
            a.lse[unit_ll * a.seqlen_q + row] = lse_val;
        }
        if (a.o_tma) {
            // 16-bit output of an unsplit launch: each warp packs its 32 rows, one 64-column box at a
            // time, into shared memory in the 128-byte-swizzled box layout and hands them to the TMA
            // unit, which writes whole lines and clips rows >= seqlen_q and columns >= head_dim.
            // One CTA per item: the boxes are staged in the query tile's own Q buffer (free once the
            // last Q K^T has completed, which o_full implies).  Persistent kernel: in the warp's own
            // 4 KB, reused box after box, because the Q buffer is already being refilled.
            const int y0 = rb * kTile + (warp & 3) * 32;
#pragma unroll
            for (int b = 0; b < C::kBoxes; ++b) {
                uint32_t orow[2][32];
                if (have_o) {
                    tmem_ld32(tmem_o + lane_base + b * 64, orow[0]);
                    tmem_ld32(tmem_o + lane_base + b * 64 + 32, orow[1]);
                    tmem_wait_ld();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) orow[0][i] = orow[1][i] = 0u;
                }
                uint32_t packed[2][16];
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int i = 0; i < 32; i += 2)
                        packed[h][i >> 1] = pack2<kBf16>(__uint_as_float(orow[h][i]) * inv, __uint_as_float(orow[h][i + 1]) * inv);
                uint32_t box;
                if constexpr (C::kPersist) {
                    box = sStage + warp * 4096;
                    if (staged) {  // the previous box of this warp must have left the buffer
                        if (lane == 0) tma_store_wait_read();
                        __syncwarp();
                    }
                } else {
                    box = sQ + qi * C::kTileBytes + b * (kTile * 128) + (warp & 3) * (32 * 128);
                }
                const uint32_t row_addr = box + lane * 128;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t chunk = static_cast<uint32_t>(h * 4 + i) ^ static_cast<uint32_t>(lane & 7);
                        st_shared_v4(row_addr + chunk * 16, packed[h][4 * i], packed[h][4 * i + 1], packed[h][4 * i + 2],
                                     packed[h][4 * i + 3]);
                    }
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0 && y0 < a.seqlen_q && b * 64 < a.head_dim) {
                    tma_store_3d(&tmap_o, box, b * 64, y0, unit);
                    tma_store_commit();
                }
                staged = true;
            }
            FA_TR(97);
            if constexpr (!C::kPersist) {
                if (lane == 0) tma_store_wait_read();
            }
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
        item = next_item_;
        have_item = have_next_item;
        }  // items
        // the staging buffers must outlive the reads of the last TMA stores
        if (C::kPersist && staged && lane == 0) tma_store_wait_read();
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
    FA_CTA_TIME(2);
    tc_fence_before_sync();
    __syncthreads();
    FA_TR(99);
    FA_CTA_TIME(3);
    if (warp == C::kMmaWarp) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

// ------------------------------------------------------------------ host side

std::atomic<uint32_t> g_launches{0};  // persistent launches so far in this process (all kernel variants)

template <int D, int NQ, bool kBf16, bool kAlibi, bool kDropout>
cudaError_t launch_one(FwdArgs a, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                       const CUtensorMap& to, int units, int sms, cudaStream_t stream) {
    auto kern = fwd_tiled_kernel<D, NQ, kBf16, kAlibi, kDropout>;
    constexpr int smem = Cfg<D, NQ>::kSmemBytes;
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
    const int per_unit = trq * a.num_splits;
    const long long items = static_cast<long long>(units) * per_unit;
    if (items <= 0 || items > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    a.n_items = static_cast<int>(items);
    a.div_group_items = make_fastdiv(static_cast<uint32_t>(std::min<long long>(static_cast<long long>(a.unit_group) * per_unit, 0x7fffffffLL)));
    a.div_gsize = make_fastdiv(static_cast<uint32_t>(a.unit_group));
    a.div_last_gsize = make_fastdiv(static_cast<uint32_t>(units % a.unit_group == 0 ? a.unit_group : units % a.unit_group));
    a.div_splits = make_fastdiv(static_cast<uint32_t>(a.num_splits));
    // launched with programmatic stream serialization: the kernel may begin its set-up while the
    // kernel before it in the stream drains
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(Cfg<D, NQ>::kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if constexpr (NQ == 2) {
        // persistent: one CTA per SM; the claim counter of this launch (tag 0 is never issued)
        uint32_t tag = g_launches.fetch_add(1, std::memory_order_relaxed) + 1;
        if (tag == 0) tag = g_launches.fetch_add(1, std::memory_order_relaxed) + 1;
        a.sched_tag = tag;
        a.sched_slot = static_cast<int>(tag % kSchedSlots);
        cfg.gridDim = dim3(static_cast<unsigned>(std::min<long long>(items, std::max(1, sms))));
    } else {
        cfg.gridDim = dim3(static_cast<unsigned>(items));
    }
    return cudaLaunchKernelEx(&cfg, kern, tq, tk, tv, to, a);
}

template <int D, int NQ, bool kBf16>
cudaError_t launch_flags(const FwdArgs& a, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                         const CUtensorMap& to, int units, bool alibi, bool dropout, int sms, cudaStream_t stream) {
    if (alibi) {
        return dropout ? launch_one<D, NQ, kBf16, true, true>(a, tq, tk, tv, to, units, sms, stream)
                       : launch_one<D, NQ, kBf16, true, false>(a, tq, tk, tv, to, units, sms, stream);
    }
    return dropout ? launch_one<D, NQ, kBf16, false, true>(a, tq, tk, tv, to, units, sms, stream)
                   : launch_one<D, NQ, kBf16, false, false>(a, tq, tk, tv, to, units, sms, stream);
}

template <int D, int NQ>
cudaError_t launch_dtype(const FwdArgs& a, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                         const CUtensorMap& to, int units, bool bf16, bool alibi, bool dropout, int sms,
                         cudaStream_t stream) {
    return bf16 ? launch_flags<D, NQ, true>(a, tq, tk, tv, to, units, alibi, dropout, sms, stream)
                : launch_flags<D, NQ, false>(a, tq, tk, tv, to, units, alibi, dropout, sms, stream);
}

}  // namespace

cudaError_t launch_fwd_tiled(const FwdArgs& a, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                             const CUtensorMap& to, int units, bool bf16, bool dropout, int sms, cudaStream_t stream) {
    const bool alibi = a.alibi_slopes != nullptr;
    // two query tiles per item once a unit has more than two (or two without a causal mask); smaller
    // units keep two independent CTAs per SM instead
    // (with two query tiles and a causal mask the pair would spend half its time on the diagonal tile that
    // only one of them can use: 277 against 308 TFLOP/s at [128,16,256,128])
    const bool pair = a.tr > 2 || (a.tr == 2 && !a.is_causal);
    if (a.head_dim <= 64) {
        return pair ? launch_dtype<64, 2>(a, tq, tk, tv, to, units, bf16, alibi, dropout, sms, stream)
                    : launch_dtype<64, 1>(a, tq, tk, tv, to, units, bf16, alibi, dropout, sms, stream);
    }
    return pair ? launch_dtype<128, 2>(a, tq, tk, tv, to, units, bf16, alibi, dropout, sms, stream)
                : launch_dtype<128, 1>(a, tq, tk, tv, to, units, bf16, alibi, dropout, sms, stream);
}

}  // namespace fa
