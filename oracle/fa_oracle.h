/*
 * CPU oracle for the flash-attention forward path.  TEST INFRASTRUCTURE ONLY:
 * nothing in the shipped library links, loads or calls this code; it exists so
 * that tests, the smoke check and the benchmark's cpu_baseline leg can compare
 * the CUDA kernels with a plain-C restatement of the reference algorithm.
 *
 * Parity status: PINNED.  The attention math is checked bit-for-bit against the
 * reference's own attention_forward_cpu (src/main.cu:279-388) compiled from the
 * reference sources, and the dropout generator against NVIDIA cuRAND's
 * Philox4_32_10 device API (curand_init / curand_uniform) executed on the host;
 * both sets of vectors are committed under tests/golden/.
 */
#ifndef FA_ORACLE_H
#define FA_ORACLE_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* One Philox4x32-10 block: the published Salmon et al. (SC'11) generator that
 * cuRAND's curandStatePhilox4_32_10_t implements.  ctr = 128-bit counter,
 * key = 64-bit key, out = 4 x 32-bit words. */
void fa_oracle_philox4x32_10(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4]);

/* n-th 32-bit draw of the stream curand_init(seed, subsequence, offset) followed
 * by repeated curand(): word (n+offset)%4 of the block with counter
 * ((n+offset)/4, subsequence).  Follows reference src/init_curand_states.h:12. */
uint32_t fa_oracle_curand_draw(uint64_t seed, uint64_t subsequence, uint64_t offset, uint64_t n);

/* curand_uniform's mapping of a raw draw to (0,1]: x*2^-32 + 2^-33 in fp32. */
float fa_oracle_uniform(uint32_t x);

/* Smallest raw draw that is KEPT for dropout probability p, i.e. the smallest x
 * with !(uniform(x) < p) (reference src/flash_forward.h:230).  2^32 when
 * everything is dropped. */
uint64_t fa_oracle_keep_threshold(float p);

/* Dropout geometry of one launch of the reference kernels.  num_splits == 1 is
 * forward_kernel (src/flash_forward.h:50-54,221-237), > 1 is
 * forward_kernel_splitkv (src/flash_forward_splitkv.h:40-58,236-252). */
typedef struct {
    uint64_t seed, offset;
    float p;
    int heads;            /* H: gridDim.y                                   */
    int seqlen_q;         /* rows; Tr = ceil(seqlen_q/128)                  */
    int seqlen_k;         /* columns; Tc = ceil(seqlen_k/128)               */
    int num_splits;       /* 1 = non-split launch                           */
    int causal;           /* bounds the CTA's tile range (launch_index)     */
    int window_left;      /* < 0: no local mask (n_block_min = 0)           */
    int64_t q_pos0, k_pos0; /* global positions of row 0 / column 0          */
    int window_right;     /* < 0: off; bounds the tile range (launch_index) */
    uint64_t launch_index; /* k-th launch of a loop over the same generator
                             states (flash_forward.h:302-305): every stream
                             has advanced 64 * k * (tiles its CTA visits)   */
} fa_oracle_dropout_geom;

/* 1 if P[b,h,row,col] is kept, 0 if dropped, for the reference's draw order. */
int fa_oracle_dropout_keep(const fa_oracle_dropout_geom* g, int b, int h, int64_t row, int64_t col);

/* Fills keep[seqlen_q*seqlen_k] (uint8) for one (b,h). */
void fa_oracle_dropout_mask(const fa_oracle_dropout_geom* g, int b, int h, uint8_t* keep);

typedef struct {
    const float* q;       /* [B,H,Nq,d] fp32 (16-bit-rounded values upcast)  */
    const float* k;       /* [B,H,Nk,d]                                     */
    const float* v;       /* [B,H,Nk,d]                                     */
    int batch, heads, seqlen_q, seqlen_k, head_dim;
    float softmax_scale;
    int causal;           /* masks k_pos > q_pos                            */
    int window_left;      /* masks q_pos - k_pos > window_left  (-1 = off)  */
    int window_right;     /* masks k_pos - q_pos > window_right (-1 = off)  */
    const float* alibi_slopes; /* [H] or NULL; score -= slope*|q_pos-k_pos|  */
    float p_dropout;
    uint64_t seed, offset;
    int dropout_splits;   /* launch geometry the mask follows (>= 1)        */
    int64_t q_pos0, k_pos0;
    const int64_t* rows;  /* optional subset: flat (b*H+h)*Nq + i indices   */
    int64_t n_rows;       /* number of entries in rows (ignored if NULL)    */
    float* o;             /* [B,H,Nq,d] or [n_rows,d]                       */
    float* lse;           /* [B,H,Nq]   or [n_rows]   (may be NULL)         */
    int num_threads;      /* <= 0: all available                            */
    uint64_t launch_index; /* dropout mask of the k-th launch of a loop      */
} fa_oracle_params;

/* Naive fp32 attention, restating reference src/main.cu:279-388 step by step. */
int fa_oracle_forward(const fa_oracle_params* p);

/* Reference split policy, src/main.cu:391-422. */
int fa_oracle_num_splits_heuristic(int batch_nheads_mblocks, int num_sms, int num_n_blocks,
                                   int max_splits, int seq_len);

#ifdef __cplusplus
}
#endif
#endif
