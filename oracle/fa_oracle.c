/*
 * CPU oracle (test infrastructure, never part of the shipped path): plain-C
 * restatement of the reference flash-attention forward semantics.
 *
 *  - attention math: reference src/main.cu:279-388 (attention_forward_cpu),
 *    extended with seqlen_q != seqlen_k, asymmetric windows, global positions,
 *    LSE output, row subsets and the dropout keep-mask.
 *  - dropout: reference src/init_curand_states.h:7-14 (stream set-up) and
 *    src/flash_forward.h:50-54,221-237 (draw order), with the generator itself
 *    (cuRAND Philox4_32_10, CUDA Toolkit 12.9 headers; not vendored by the
 *    reference) restated from the published Philox4x32-10 algorithm.
 *  - split policy: reference src/main.cu:391-422.
 *
 * Parity: pinned by tests/golden/ (reference CPU outputs, cuRAND host KATs).
 */
#include "fa_oracle.h"
#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define TILE 128

/* ---- Philox4x32-10 ------------------------------------------------------ */

static inline void philox_round(uint32_t c[4], const uint32_t k[2]) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c[0];
    const uint64_t p1 = (uint64_t)0xCD9E8D57u * c[2];
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k[0];
    const uint32_t n1 = (uint32_t)p1;
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k[1];
    const uint32_t n3 = (uint32_t)p0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}

void fa_oracle_philox4x32_10(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4]) {
    uint32_t c[4] = {ctr[0], ctr[1], ctr[2], ctr[3]};
    uint32_t k[2] = {key[0], key[1]};
    for (int r = 0; r < 10; ++r) {
        philox_round(c, k);
        if (r < 9) { k[0] += 0x9E3779B9u; k[1] += 0xBB67AE85u; }
    }
    memcpy(out, c, sizeof c);
}

uint32_t fa_oracle_curand_draw(uint64_t seed, uint64_t subsequence, uint64_t offset, uint64_t n) {
    /* curand_init(seed, subsequence, offset): key = seed, counter high 64 bits =
     * subsequence, low 64 bits advance by one per 4 draws, offset skips draws. */
    const uint64_t idx = n + offset;
    const uint64_t blk = idx >> 2;
    uint32_t ctr[4] = {(uint32_t)blk, (uint32_t)(blk >> 32),
                       (uint32_t)subsequence, (uint32_t)(subsequence >> 32)};
    /* a carry out of the low 64 bits (offset near 2^66) is not modelled */
    uint32_t key[2] = {(uint32_t)seed, (uint32_t)(seed >> 32)};
    uint32_t out[4];
    fa_oracle_philox4x32_10(ctr, key, out);
    return out[idx & 3];
}

float fa_oracle_uniform(uint32_t x) {
    /* curand_uniform: x * 2^-32 + 2^-33, evaluated in fp32.  The product with a
     * power of two is exact, so fused and unfused evaluation agree. */
    volatile float f = (float)x;
    volatile float r = f * 2.3283064365386963e-10f;
    r = r + 1.1641532182693481e-10f;
    return r;
}

uint64_t fa_oracle_keep_threshold(float p) {
    /* uniform() is monotone in x, so the dropped set {x : uniform(x) < p} is a
     * prefix [0, T).  Binary search for T. */
    uint64_t lo = 0, hi = (uint64_t)1 << 32; /* first kept x in [lo, hi] */
    if (!(fa_oracle_uniform(0u) < p)) return 0;
    if (fa_oracle_uniform(0xFFFFFFFFu) < p) return hi;
    /* invariant: lo dropped, hi kept */
    hi = 0xFFFFFFFFull;
    while (hi - lo > 1) {
        uint64_t mid = lo + (hi - lo) / 2;
        if (fa_oracle_uniform((uint32_t)mid) < p) lo = mid; else hi = mid;
    }
    return hi;
}

/* ---- dropout draw order of the reference kernels ------------------------ */

static inline int64_t imax64(int64_t a, int64_t b) { return a > b ? a : b; }
static inline int64_t imin64(int64_t a, int64_t b) { return a < b ? a : b; }

int fa_oracle_dropout_keep(const fa_oracle_dropout_geom* g, int b, int h, int64_t row, int64_t col) {
    const int64_t Tr = (g->seqlen_q + TILE - 1) / TILE;
    const int64_t Tc = (g->seqlen_k + TILE - 1) / TILE;
    const int64_t rb = row / TILE, cb = col / TILE;
    const int splits = g->num_splits < 1 ? 1 : g->num_splits;
    /* split that owns this KV tile: flash_forward_splitkv.h:40-43 */
    const int64_t per = (Tc + splits - 1) / splits;
    const int64_t s = splits == 1 ? 0 : cb / per;
    int64_t nbmin = splits == 1 ? 0 : per * s;
    if (g->window_left >= 0) {
        /* flash_forward.h:39 / flash_forward_splitkv.h:44; C division truncates */
        int64_t w = (g->q_pos0 + rb * TILE - g->window_left - g->k_pos0) / TILE;
        nbmin = imax64(nbmin, imax64(0, w));
    }
    /* tiles left of the window are never visited by the CTA: nothing is drawn
     * for them (and every element there is masked anyway) */
    if (cb < nbmin) return 1;
    /* Later launches of a loop: the kernels store the advanced state back
     * (flash_forward.h:302-305), so launch k starts every stream 64 draws per
     * visited tile per earlier launch further on.  Visited tiles = the CTA's loop
     * range [n_block_min, n_block_max), flash_forward.h:39-48 and
     * flash_forward_splitkv.h:40-52. */
    uint64_t ahead = 0;
    if (g->launch_index > 0) {
        int64_t nbmax = splits == 1 ? Tc : imin64(per * s + per, Tc);
        const int64_t q_end = g->q_pos0 + (rb + 1) * TILE - g->k_pos0; /* (bx+1)*Br with positions */
        if (g->window_right >= 0) {
            const int64_t last = q_end - 1 + g->window_right;
            nbmax = imin64(nbmax, last < 0 ? 0 : last / TILE + 1);
        }
        if (g->causal) {
            const int64_t last = q_end - 1;
            nbmax = imin64(nbmax, last < 0 ? 0 : last / TILE + 1);
        }
        const int64_t lo = imin64(nbmin, Tc);
        if (nbmax > lo) ahead = g->launch_index * 64ull * (uint64_t)(nbmax - lo);
    }
    /* one stream per CTA: flash_forward.h:52 with grid (Tr*splits, H, B) */
    const uint64_t subseq = ((uint64_t)b * g->heads + h) * (uint64_t)(Tr * splits) + (uint64_t)(rb * splits + s);
    /* 64 draws per KV tile in c_frag[i][j] order (flash_forward.h:223-227); the
     * fragment element (i,j) of every warp/lane covers
     *   col%128 in 16*i + 8*((j%4)/2) + {lane%4*2 + j%2},  row%16 in 8*(j/4) + lane/4
     * (flash_forward.h:130-131), and every thread of the CTA draws the same
     * values, so the decision depends only on these bits of (row, col). */
    const int rr = (int)(row % TILE), cc = (int)(col % TILE);
    const int i = cc / 16;
    const int j = 4 * ((rr % 16) / 8) + 2 * ((cc % 16) / 8) + (cc % 2);
    const uint64_t n = ahead + 64ull * (uint64_t)(cb - nbmin) + 8ull * i + j;
    const uint32_t x = fa_oracle_curand_draw(g->seed, subseq, g->offset, n);
    return !(fa_oracle_uniform(x) < g->p);
}

void fa_oracle_dropout_mask(const fa_oracle_dropout_geom* g, int b, int h, uint8_t* keep) {
    for (int64_t r = 0; r < g->seqlen_q; ++r)
        for (int64_t c = 0; c < g->seqlen_k; ++c)
            keep[r * g->seqlen_k + c] = (uint8_t)fa_oracle_dropout_keep(g, b, h, r, c);
}

/* ---- attention ---------------------------------------------------------- */

static void attend_row(const fa_oracle_params* p, int b, int h, int64_t i,
                       float* scores, float* o_row, float* lse_out) {
    const int d = p->head_dim;
    const int64_t Nq = p->seqlen_q, Nk = p->seqlen_k;
    const int64_t bh = (int64_t)b * p->heads + h;
    const float* Q = p->q + (bh * Nq + i) * d;
    const float* K = p->k + bh * Nk * d;
    const float* V = p->v + bh * Nk * d;
    const int64_t qpos = p->q_pos0 + i;

    /* 1. scores = scale * q.k            main.cu:309-317 */
    for (int64_t j = 0; j < Nk; ++j) {
        float sum = 0.0f;
        const float* Kj = K + j * d;
        for (int k = 0; k < d; ++k) sum += Q[k] * Kj[k];
        scores[j] = sum * p->softmax_scale;
    }
    /* 2. ALiBi: subtract slope*|i-j|     main.cu:320-327 */
    if (p->alibi_slopes) {
        const float slope = p->alibi_slopes[h];
        for (int64_t j = 0; j < Nk; ++j) {
            int64_t dist = qpos - (p->k_pos0 + j);
            if (dist < 0) dist = -dist;
            scores[j] -= slope * (float)dist;
        }
    }
    /* 3. masks                            main.cu:330-349 (window made asymmetric) */
    for (int64_t j = 0; j < Nk; ++j) {
        const int64_t kpos = p->k_pos0 + j;
        if (p->causal && kpos > qpos) scores[j] = -INFINITY;
        if (p->window_left >= 0 && qpos - kpos > p->window_left) scores[j] = -INFINITY;
        if (p->window_right >= 0 && kpos - qpos > p->window_right) scores[j] = -INFINITY;
    }
    /* 4. softmax with max subtraction     main.cu:352-372 */
    float max_val = -INFINITY;
    for (int64_t j = 0; j < Nk; ++j) max_val = scores[j] > max_val ? scores[j] : max_val;
    if (max_val == -INFINITY) {
        /* fully masked row: the reference would produce NaN (exp(-inf+inf));
         * the replacement defines O = 0, LSE = -inf. */
        for (int k = 0; k < d; ++k) o_row[k] = 0.0f;
        if (lse_out) *lse_out = -INFINITY;
        return;
    }
    float sum = 0.0f;
    for (int64_t j = 0; j < Nk; ++j) {
        scores[j] = expf(scores[j] - max_val);
        sum += scores[j];
    }
    for (int64_t j = 0; j < Nk; ++j) scores[j] /= sum;
    if (lse_out) *lse_out = max_val + logf(sum);
    /* dropout on P, after the statistics  flash_forward.h:221-237 */
    if (p->p_dropout > 0.0f) {
        fa_oracle_dropout_geom g;
        g.seed = p->seed; g.offset = p->offset; g.p = p->p_dropout;
        g.heads = p->heads; g.seqlen_q = (int)Nq; g.seqlen_k = (int)Nk;
        g.num_splits = p->dropout_splits < 1 ? 1 : p->dropout_splits;
        g.causal = p->causal; g.window_left = p->window_left;
        g.q_pos0 = p->q_pos0; g.k_pos0 = p->k_pos0;
        g.window_right = p->window_right; g.launch_index = p->launch_index;
        const float keep_scale = 1.0f / (1.0f - p->p_dropout);
        for (int64_t j = 0; j < Nk; ++j) {
            if (scores[j] == 0.0f) continue;
            if (fa_oracle_dropout_keep(&g, b, h, i, j)) scores[j] *= keep_scale;
            else scores[j] = 0.0f;
        }
    }
    /* 5. O = P V                          main.cu:375-383 */
    for (int k = 0; k < d; ++k) {
        float acc = 0.0f;
        for (int64_t j = 0; j < Nk; ++j) acc += scores[j] * V[j * d + k];
        o_row[k] = acc;
    }
}

int fa_oracle_forward(const fa_oracle_params* p) {
    if (!p || !p->q || !p->k || !p->v || !p->o) return -1;
    if (p->batch < 1 || p->heads < 1 || p->seqlen_q < 1 || p->seqlen_k < 1 || p->head_dim < 1) return -1;
    const int64_t Nq = p->seqlen_q;
    const int64_t total = p->rows ? p->n_rows : (int64_t)p->batch * p->heads * Nq;
    int nthreads = p->num_threads;
#ifdef _OPENMP
    if (nthreads <= 0) nthreads = omp_get_max_threads();
#else
    nthreads = 1;
#endif
    int err = 0;
#ifdef _OPENMP
#pragma omp parallel num_threads(nthreads)
#endif
    {
        float* scores = (float*)malloc(sizeof(float) * (size_t)p->seqlen_k);
        if (!scores) {
            err = -2;
        } else {
#ifdef _OPENMP
#pragma omp for schedule(dynamic, 16)
#endif
            for (int64_t t = 0; t < total; ++t) {
                const int64_t flat = p->rows ? p->rows[t] : t;
                const int64_t bh = flat / Nq;
                const int64_t i = flat % Nq;
                attend_row(p, (int)(bh / p->heads), (int)(bh % p->heads), i, scores,
                           p->o + t * p->head_dim, p->lse ? p->lse + t : NULL);
            }
            free(scores);
        }
    }
    return err;
}

/* ---- split policy ------------------------------------------------------- */

static int ceil_div(int a, int b) { return (a + b - 1) / b; }

static int split_eligible(int s, int n_blocks, int seq_len) {
    /* main.cu:398-400: the split must change the per-split tile count and cut
     * the (padded) sequence into whole 128-row tiles. */
    if (seq_len % (TILE * s) != 0) return 0;
    return s == 1 || ceil_div(n_blocks, s) != ceil_div(n_blocks, s - 1);
}

int fa_oracle_num_splits_heuristic(int batch_nheads_mblocks, int num_sms, int num_n_blocks,
                                   int max_splits, int seq_len) {
    if ((float)batch_nheads_mblocks >= 4.0f * (float)num_sms) return 1;
    if (num_sms < max_splits) max_splits = num_sms;
    if (num_n_blocks < max_splits) max_splits = num_n_blocks;
    float best = 0.0f;
    for (int s = 1; s <= max_splits; ++s) {
        if (!split_eligible(s, num_n_blocks, seq_len)) continue;
        const float waves = (float)(batch_nheads_mblocks * s) / (float)num_sms;
        const float eff = waves / ceilf(waves);
        if (eff > best) best = eff;
    }
    for (int s = 1; s <= max_splits; ++s) {
        if (!split_eligible(s, num_n_blocks, seq_len)) continue;
        const float waves = (float)(batch_nheads_mblocks * s) / (float)num_sms;
        const float eff = waves / ceilf(waves);
        if (eff >= 0.85 * best) return s;
    }
    return 1;
}
