/*
 * fa_b200 -- Blackwell (sm_100a) flash-attention forward behind a plain C ABI.
 *
 * This header is the drop-in boundary for the launcher surface of
 * Yhorm26/flash_attn.  The reference has no library: its "API" is the kernel
 * argument block mykernelParamType (include/utils.h:21-44) plus the launch code
 * in main() (src/main.cu:109-205).  Each entry point below names the reference
 * item it replaces.  All pointers are plain device (or, where stated, host)
 * pointers; there are no C++ or framework types in any signature.
 *
 * Tensor layout (same as the reference, src/flash_forward.h:57-59):
 *   Q, O : [batch, heads, seqlen_q, head_dim]  contiguous
 *   K, V : [batch, heads, seqlen_k, head_dim]  contiguous
 *   LSE  : [batch, heads, seqlen_q]            fp32
 * Ownership: the caller owns every buffer including the workspace; the library
 * allocates nothing in fa_fwd and keeps no state between calls (there is no RNG
 * state array: dropout is a function of (seed, offset) only).
 * Threads: every entry point may be called from several host threads at once, on
 * the same or on different devices (the current device is the thread's, as in the
 * CUDA runtime).  fa_fwd_host and fa_launch_reference_params serialise the calls
 * of one device on its cached buffers; calls for different devices run concurrently.
 */
#ifndef FA_B200_H
#define FA_B200_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FA_B200_VERSION 100

/* element types */
#define FA_DTYPE_FP16 0
#define FA_DTYPE_BF16 1
#define FA_DTYPE_FP32 2 /* output only: the reference writes O as fp32 (include/utils.h:26) */

/* return codes: 0 on success, negative on failure; the library never exits or prints
 * (the reference's CUDA_CHECK, src/main.cu:18-25, calls exit(1)). */
#define FA_OK 0
#define FA_ERR_INVALID_ARG (-1)    /* NULL pointer, non-positive size, bad enum, misaligned pointer */
#define FA_ERR_UNSUPPORTED (-2)    /* head_dim > 128, dtype combination                            */
#define FA_ERR_WORKSPACE (-3)      /* workspace missing or smaller than fa_fwd_workspace_bytes()   */
#define FA_ERR_CUDA (-4)           /* a CUDA runtime/driver call failed                            */
#define FA_ERR_DEVICE_TIMEOUT (-5) /* a bounded device-side wait gave up (fa_fwd_host; see status)    */
#define FA_ERR_NOT_SM100 (-6)      /* the current device is not compute capability 10.x            */
#define FA_ERR_TOO_LARGE (-7)      /* size beyond a fixed limit of the entry point                 */

/*
 * Launch description.  Replaces mykernelParamType (include/utils.h:21-44) and the
 * grid dimensions the reference passes beside it (batch = gridDim.z, heads =
 * gridDim.y, src/main.cu:142).  Zero-initialise, then fill.
 */
typedef struct fa_fwd_params {
    const void* q;            /* device, dtype                                   (param.Q) */
    const void* k;            /* device, dtype                                   (param.K) */
    const void* v;            /* device, dtype                                   (param.V) */
    void* o;                  /* device, o_dtype                                 (param.O) */
    float* lse;               /* device fp32 [B,H,Nq] or NULL; natural-log sum-exp of the
                                 scaled, biased, masked scores; -inf for fully masked rows */
    int dtype;                /* FA_DTYPE_FP16 | FA_DTYPE_BF16 */
    int o_dtype;              /* same as dtype, or FA_DTYPE_FP32 */
    int batch, heads;
    int seqlen_q, seqlen_k;   /* the reference has one N for both (param.N) */
    int head_dim;             /* <= 128; multiples of 8 are read in place by TMA, other values go
                                 through a padded copy in the workspace            (param.d) */
    float softmax_scale;      /* > 0                                    (param.softmax_scale) */
    int is_causal;            /* masks k_pos > q_pos      (template flag Is_causal, main.cu:45) */
    int window_left;          /* masks q_pos - k_pos > window_left;  -1 = off (window_size_left)  */
    int window_right;         /* masks k_pos - q_pos > window_right; -1 = off (window_size_right) */
    const float* alibi_slopes;/* device fp32 [heads] or NULL; score -= slope*|q_pos-k_pos|
                                 (alibi_slopes_ptr; subtracts, as src/flash_forward.h:173) */
    float p_dropout;          /* in [0,1)                                (param.dropout_prob) */
    uint64_t seed;            /* Philox key                 (seed of init_curand_states)      */
    uint64_t offset;          /* draws skipped at the start of every stream (0 = first launch) */
    uint64_t unit0;           /* global b*H+h index of this call's first (batch, head) unit:
                                 keeps the dropout mask independent of how units are sharded  */
    int num_splits;           /* 0 = fa_num_splits_heuristic with the device's SM count,
                                 1 = no split, n = forced                  (param.split_num) */
    int64_t q_pos0, k_pos0;   /* global position of query row 0 / key column 0 (0 = reference
                                 behaviour; used to run one block of a sharded sequence)      */
    void* workspace;          /* device; split partials (param.O_tmp, param.L, param.M) */
    size_t workspace_bytes;
    int* status;              /* device int or NULL.  Every wait inside the kernels is bounded (about 2 s of SM
                                 clocks); a wait that gives up stores a code here -- 100 + n from the tiled
                                 forward kernel, 200 + n from the decode kernel, n naming the wait -- and the
                                 CTA drains and exits, leaving O and LSE undefined.  fa_fwd is asynchronous:
                                 the caller clears the word before the launch and reads it after synchronising
                                 the stream.  fa_fwd_host does both itself and returns FA_ERR_DEVICE_TIMEOUT. */
    void* stream;             /* cudaStream_t; NULL = default stream (the reference's)       */
    int heads_k;              /* K/V heads for grouped-query attention: K and V are
                                 [batch, heads_k, seqlen_k, head_dim], heads % heads_k == 0 and
                                 query head h reads K/V head h / (heads / heads_k).  0 = heads
                                 (the reference has one head count, gridDim.y, main.cu:142) */
    /* Running result over key blocks that arrive one launch at a time (a sequence sharded across
     * GPUs, whose K/V blocks travel round a ring).  When accum_o is set, the launch merges its
     * (O, LSE) into the fp32 pair in its own epilogue, with the algebra of the reference's
     * combine kernel (src/flash_forward_splitkv.h:359-397) in log-sum-exp form:
     *   lse' = log(e^lse_acc + e^lse),  O' = e^(lse_acc-lse') O_acc + e^(lse-lse') O.
     * Unsplit launches only (num_splits resolves to 1). */
    float* accum_o;           /* device fp32 [B,H,Nq,head_dim], or NULL = off                     */
    float* accum_lse;         /* device fp32 [B,H,Nq]                                             */
    int accum_flags;          /* FA_ACCUM_FIRST: nothing is carried yet (the pair is written, not
                                 read).  FA_ACCUM_FINAL: last block; o (o_dtype) and lse, where
                                 non-NULL, receive the merged result, and accum_o is left as it
                                 was (accum_lse is still updated).  Without FA_ACCUM_FINAL o may
                                 be NULL and is not written. */
    uint64_t launch_index;    /* dropout in a loop of launches: the reference's kernels write every CTA's
                                 generator state back (src/flash_forward.h:302-305), so launch k of its
                                 timing loop (src/main.cu:195-206) continues each stream 64*k*T draws
                                 further on, T = KV tiles that CTA visits (fewer under a causal or local
                                 mask, so one `offset` cannot express it).  launch_index = k reproduces
                                 the mask of that launch; 0 = the first launch. */
} fa_fwd_params;

#define FA_ACCUM_FIRST 1
#define FA_ACCUM_FINAL 2

/* Forward pass: O = dropout(softmax(scale*Q K^T - slope*|i-j| + masks)) V, LSE.
 * Replaces the launches of forward_kernel (src/flash_forward.h:13-306),
 * forward_kernel_splitkv + forward_kernel_splitkv_combine
 * (src/flash_forward_splitkv.h:14-399) and init_curand_states
 * (src/init_curand_states.h:7-14) issued by src/main.cu:128-205.
 * Asynchronous on p->stream. */
int fa_fwd(const fa_fwd_params* p);

/* Bytes of workspace fa_fwd needs for p (0 when it neither splits nor pads head_dim).
 * Replaces the cudaMalloc sizing of O_tmp/L/M at src/main.cu:160-162. */
size_t fa_fwd_workspace_bytes(const fa_fwd_params* p);

/* Split count fa_fwd will use for p (resolves num_splits == 0). */
int fa_fwd_resolve_splits(const fa_fwd_params* p);

/* The reference's split policy, same arguments and result as
 * num_splits_heuristic (src/main.cu:391-422). */
int fa_num_splits_heuristic(int batch_nheads_mblocks, int num_sms, int num_n_blocks, int max_splits,
                            int seq_len);

/* Writes the dropout keep-mask fa_fwd applies for p (1 = kept, 0 = dropped) to
 * keep[B,H,Nq,Nk] (device, uint8).  The reference cannot show its mask; this is
 * the check that the stateless generator reproduces src/flash_forward.h:221-237. */
int fa_dropout_mask(const fa_fwd_params* p, uint8_t* keep);

/* Merges a partial result into an accumulated one, row by row:
 *   lse' = log(exp(lse_acc) + exp(lse_part)),
 *   o'   = exp(lse_acc-lse') o_acc + exp(lse_part-lse') o_part.
 * o_acc fp32 [rows, head_dim], o_part of part_dtype.  The same algebra as
 * forward_kernel_splitkv_combine (src/flash_forward_splitkv.h:359-397), used to
 * chain the blocks of a sequence sharded across GPUs. */
int fa_merge_partial(float* o_acc, float* lse_acc, const void* o_part, const float* lse_part,
                     int part_dtype, int64_t rows, int head_dim, void* stream);

/* Casts the fp32 accumulator of fa_merge_partial to the 16-bit output type. */
int fa_cast_output(const float* o_acc, void* o, int o_dtype, int64_t elems, void* stream);

/* Host-buffer forward, the path the reference's main() takes around its kernel
 * (cudaMemcpy H2D src/main.cu:105-107, launch, cudaMemcpy D2H :219): q/k/v/o/lse
 * and alibi_slopes in *p are HOST pointers (pinned memory overlaps best).  Device
 * staging buffers are allocated on first use and cached per device; copies and
 * kernels are pipelined over (batch, head) slices.  Synchronous. */
int fa_fwd_host(const fa_fwd_params* p);
/* Frees the staging buffers fa_fwd_host cached. */
void fa_fwd_host_release(void);

/* Field-for-field mirror of the reference's kernel argument block mykernelParamType
 * (include/utils.h:21-44), for callers that already fill that struct. */
typedef struct fa_ref_kernel_params {
    void* Q;                  /* half*  [B,H,N,d] */
    void* K;
    void* V;
    float* O;                 /* float* [B,H,N,d]: the reference writes fp32 */
    float* O_tmp;             /* split buffers of the reference: not used (the shim keeps its own workspace) */
    float* L;
    float* M;
    int N, d, Br, Bc, Tr, Tc;
    float softmax_scale;
    float dropout_prob;
    unsigned long long seed;  /* declared but never read by the reference kernels */
    void* states;             /* curandStatePhilox4_32_10_t*: not used, dropout is stateless here */
    int window_size_left, window_size_right;
    float* alibi_slopes_ptr;
    int split_num;
} fa_ref_kernel_params;

/* Launch described the reference's way: its argument block, its grid (heads = gridDim.y, batch
 * = gridDim.z, src/main.cu:142) and the template flags of forward_kernel<Is_dropout, Is_causal,
 * Is_local, Has_alibi, ...> (src/main.cu:147-155) as run-time ints.  dropout_seed is the seed the
 * caller gave init_curand_states (src/main.cu:135).  fp16 in, fp32 out, any N, any d <= 128.
 * Runs fa_fwd underneath; the workspace it needs (split partials, padded copies for d % 8 != 0)
 * is allocated on first use and cached per device (released by fa_fwd_host_release). */
int fa_launch_reference_params(const fa_ref_kernel_params* param, int heads, int batch, int is_dropout,
                               int is_causal, int is_local, int has_alibi, unsigned long long dropout_seed,
                               void* stream);

/* Size of the built-in scratch of fa_fwd_static_scratch. */
#define FA_STATIC_SCRATCH_BYTES (32u << 20)

/* fa_fwd for callers that cannot allocate device memory -- a process whose GPU
 * memory is wholly owned by another allocator, a plugin that may not call
 * cudaMalloc, a latency-critical loop -- and therefore cannot provide
 * p->workspace for a split launch.  No counterpart in the reference, which
 * cudaMallocs its split buffers before every run (src/main.cu:160-162).
 *
 * Same arguments and results as fa_fwd, except that p->workspace and
 * p->workspace_bytes are ignored: the split partials go to a fixed
 * FA_STATIC_SCRATCH_BYTES (32 MiB) array in device global memory that belongs to
 * the library image (each GPU that loads the library holds it until exit).
 * Launches whose partials need more return FA_ERR_TOO_LARGE; the need is what
 * fa_fwd_workspace_bytes reports (batch*heads*splits*seqlen_q*(head_dim+1)*4
 * bytes, rounded up to 256).  Config 4 of the baseline (2048 units, 16 splits,
 * one query row, head_dim 128) needs 16.1 MiB.
 *
 * The call itself allocates nothing and calls no allocating routine.  The first
 * call on each device looks up the array's device address
 * (cudaGetSymbolAddress) and keeps it; make that first call outside any stream
 * capture, and make it at start-up: under the runtime's lazy module loading it is
 * this lookup that loads the module image on the device, the 32 MiB included, so
 * it can fail with FA_ERR_CUDA once another allocator holds all of the device's
 * memory.  The address kept does not survive cudaDeviceReset.  All calls on a device share the one array, which keeps whatever
 * the last call left: nothing in it needs clearing (every partial that is read
 * is written first by the same call), but two calls that overlap on the GPU --
 * different streams, or different host threads -- race on it and give wrong
 * results.  Serialise them, or use fa_fwd with separate workspaces. */
int fa_fwd_static_scratch(const fa_fwd_params* p);
size_t fa_static_scratch_bytes(void);

/*
 * Ring attention: the forward pass of ONE rank of a sequence sharded across the GPUs of an NCCL
 * communicator.  No counterpart in the reference (one GPU); the merge of the visiting key blocks is
 * the algebra of its combine kernel (src/flash_forward_splitkv.h:359-397), done in the forward
 * kernel's epilogue (accum_o above).  The sequence of 2*world*chunk_rows positions is cut into
 * 2*world chunks; rank r holds chunks r and 2*world-1-r ("zig-zag": equal causal work per rank) of Q,
 * K and V and produces the same chunks of O and LSE.  K/V travel round the ring as one message per
 * step (ncclSend to rank+1 / ncclRecv from rank-1 on comm_stream) while compute_stream runs one
 * forward launch per visible (query chunk, key chunk) pair.  Asynchronous: returns once everything is
 * enqueued; O/LSE are complete when compute_stream has drained.  The caller owns every buffer.
 * Dropout is not supported (FA_ERR_UNSUPPORTED): the reference's dropout streams are keyed on the tile
 * grid of one whole-sequence launch.  NCCL is looked up at run time (libnccl.so.2); without it only
 * world = 1 works.
 */
typedef struct fa_ring_params {
    const void* q[2];         /* device, dtype, [batch, heads,   chunk_rows, head_dim]: chunks r, 2*world-1-r */
    const void* k[2];         /* device, dtype, [batch, heads_k, chunk_rows, head_dim]                        */
    const void* v[2];
    void* o[2];               /* device, dtype, like q                                                        */
    float* lse[2];            /* device fp32 [batch, heads, chunk_rows], or NULL                               */
    int dtype;                /* FA_DTYPE_FP16 | FA_DTYPE_BF16 */
    int batch, heads, heads_k;/* heads_k = 0 means heads */
    int chunk_rows, head_dim;
    float softmax_scale;
    int is_causal, window_left, window_right;  /* on global positions, as in one unsharded launch */
    const float* alibi_slopes;/* device fp32 [heads] or NULL */
    float p_dropout;          /* must be 0 */
    int rank, world;
    void* comm;               /* ncclComm_t of the ring (may be NULL when world == 1) */
    void* message[2];         /* device, fa_ring_message_bytes() each: the K/V message at hand and the one
                                 being received ([1] may be NULL when world == 1) */
    float* accum_o[2];        /* device fp32, like q: running results (scratch; contents on return undefined) */
    float* accum_lse[2];      /* device fp32 [batch, heads, chunk_rows] */
    void* compute_stream;     /* cudaStream_t of the forward launches */
    void* comm_stream;        /* cudaStream_t of the exchange; must differ from compute_stream when world > 1.
                                 Create it with the device's greatest stream priority
                                 (cudaStreamCreateWithPriority): an attention launch keeps every SM busy with
                                 a long queue of CTAs, and the exchange's CTAs overlap it only if they are
                                 placed ahead of that queue when an SM frees up */
    int* status;              /* as in fa_fwd_params */
} fa_ring_params;
int fa_ring_fwd(const fa_ring_params* p);
/* Bytes of one K/V message buffer (K and V of the rank's two chunks). */
size_t fa_ring_message_bytes(const fa_ring_params* p);
/* Communicator helpers for callers that have no NCCL code of their own: rank 0 asks for an id
 * (128 bytes) and hands it to the other ranks by any means; every rank, with its device current,
 * then creates its communicator.  (Wrappers of ncclGetUniqueId / ncclCommInitRank / ncclCommDestroy.) */
int fa_ring_unique_id(void* id_out, size_t bytes);
int fa_ring_comm_create(void** comm_out, int world, int rank, const void* id, size_t bytes);
int fa_ring_comm_destroy(void* comm);

/* Message for a return code. */
const char* fa_strerror(int code);
int fa_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FA_B200_H */
