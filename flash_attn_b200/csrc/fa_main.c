/*
 * fa_bench -- C benchmark driver over the C ABI (include/fa_b200.h).
 *
 * The successor of the reference's main() (src/main.cu:38-251), which is launcher,
 * timing loop and self-test in one: this driver generates the inputs on the host,
 * uploads them, times fa_fwd with CUDA events (warm-up + N iterations, like
 * src/main.cu:189-213), and reports TFLOP/s or GB/s as one JSON line.  The result
 * can be dumped to a file; the tests compare that dump with the CPU oracle (the
 * reference's in-program verfiy(), src/main.cu:254-276, is replaced by that check).
 *
 *   fa_bench --config 1|2|3|4|5 [--gpus N] [--iters I] [--warmup W] [--dump FILE] [--units U] [--check]
 *
 * --check verifies sampled rows of the result against a plain fp32 attention computed here on the
 * host, and times that CPU computation (as the reference's main() does with attention_forward_cpu,
 * src/main.cu:212-225); like the reference (src/main.cu:44, 222) it runs the launch without dropout.
 *
 * With --gpus N the (batch, head) units of configs 1-4 are cut into N contiguous slices,
 * one per device, with no communication; every device gets its own stream and the job
 * time is the slowest device's.  Config 5 is ONE sequence sharded over the N devices:
 * one host thread per device runs fa_ring_fwd (K/V ring over NCCL send/recv, merge in the
 * kernel epilogue).  Plain C99: only the CUDA runtime API, pthreads and fa_b200.h.
 */
#define _POSIX_C_SOURCE 200112L /* pthread barriers under -std=c99 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>
#include <cuda_runtime_api.h>
#include "fa_b200.h"

#define CHECK_CUDA(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { \
    fprintf(stderr, "fa_bench: %s failed: %s\n", #x, cudaGetErrorString(e_)); return 1; } } while (0)
#define CHECK_FA(x) do { int rc_ = (x); if (rc_ != FA_OK) { \
    fprintf(stderr, "fa_bench: %s failed: %s\n", #x, fa_strerror(rc_)); return 1; } } while (0)

typedef struct {
    const char* name;
    int dtype, B, H, Nq, Nk, d, causal, wl, wr, alibi, splits;
    float p, sigma;
    unsigned seed;
} config_t;

static const config_t kConfigs[] = {
    {"config 1: fp16 [1,4,256,64] non-causal", FA_DTYPE_FP16, 1, 4, 256, 256, 64, 0, -1, -1, 0, 0, 0.0f, 1.0f, 0},
    {"config 2: bf16 [8,16,2048,128] causal, dropout 0.1 seed 42", FA_DTYPE_BF16, 8, 16, 2048, 2048, 128, 1, -1, -1, 0, 1, 0.1f, 1.0f, 2},
    {"config 3: bf16 [4,32,8192,128] causal + window(1024,0) + ALiBi", FA_DTYPE_BF16, 4, 32, 8192, 8192, 128, 1, 1024, 0, 1, 1, 0.0f, 1.0f, 3},
    {"config 4: decode bf16 B=64 H=32 q=1 kv=32768 d=128, 16 splits", FA_DTYPE_BF16, 64, 32, 1, 32768, 128, 0, -1, -1, 0, 16, 0.0f, 1.0f, 4},
};

/* ---- reproducible N(0, sigma^2) inputs: splitmix64 counters, sum of twelve 16-bit
 *      uniforms (integer arithmetic only, so every machine produces the same bits) ---- */
static uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    uint64_t z = x;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
static float synth_normal(uint64_t seed, uint64_t stream, uint64_t idx, float sigma) {
    const uint64_t base = idx * 3ull + (seed * 0x100000001B3ull + stream * 0x9E3779B1ull) * 0x10001ull;
    int64_t total = 0;
    for (int t = 0; t < 3; ++t) {
        const uint64_t w = splitmix64(base + (uint64_t)t);
        total += (int64_t)(w & 0xFFFF) + (int64_t)((w >> 16) & 0xFFFF) + (int64_t)((w >> 32) & 0xFFFF) + (int64_t)(w >> 48);
    }
    const double x = (double)(total * 2 - 12 * 65535) / 131072.0;
    return (float)(x * (double)sigma);
}
static uint16_t to_bf16(float f) {
    uint32_t u; memcpy(&u, &f, 4);
    if ((u & 0x7F800000u) == 0x7F800000u && (u & 0x007FFFFFu)) return (uint16_t)((u >> 16) | 0x40);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
static uint16_t to_fp16(float f) {
    uint32_t u; memcpy(&u, &f, 4);
    const uint32_t sign = (u >> 16) & 0x8000u;
    const int32_t exp = (int32_t)((u >> 23) & 0xFF) - 127 + 15;
    uint32_t man = u & 0x007FFFFFu;
    if (((u >> 23) & 0xFF) == 0xFF) return (uint16_t)(sign | 0x7C00u | (man ? 0x200u : 0u));
    if (exp >= 31) return (uint16_t)(sign | 0x7C00u);
    if (exp <= 0) {
        if (exp < -10) return (uint16_t)sign;
        man |= 0x00800000u;
        const int shift = 14 - exp;
        uint32_t h = man >> shift;
        const uint32_t rem = man & ((1u << shift) - 1u), half = 1u << (shift - 1);
        if (rem > half || (rem == half && (h & 1u))) ++h;
        return (uint16_t)(sign | h);
    }
    uint32_t h = ((uint32_t)exp << 10) | (man >> 13);
    const uint32_t rem = man & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) ++h;
    return (uint16_t)(sign | h);
}
static void fill(uint16_t* dst, size_t n, uint64_t seed, uint64_t stream, float sigma, int dtype) {
    for (size_t i = 0; i < n; ++i) {
        const float x = synth_normal(seed, stream, i, sigma);
        dst[i] = dtype == FA_DTYPE_BF16 ? to_bf16(x) : to_fp16(x);
    }
}


static float from_bf16(uint16_t h) { uint32_t u = (uint32_t)h << 16; float f; memcpy(&f, &u, 4); return f; }
static float from_fp16(uint16_t h) {
    const uint32_t sign = ((uint32_t)h & 0x8000u) << 16, exp = (h >> 10) & 0x1F, man = h & 0x3FFu;
    uint32_t u;
    if (exp == 0) {
        if (man == 0) u = sign;
        else { int e = -1; uint32_t m = man; do { ++e; m <<= 1; } while (!(m & 0x400u)); u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((m & 0x3FFu) << 13); }
    } else if (exp == 31) u = sign | 0x7F800000u | (man << 13);
    else u = sign | ((exp - 15 + 127) << 23) | (man << 13);
    float f; memcpy(&f, &u, 4); return f;
}
/* --check: the program's own verification, the successor of the reference's attention_forward_cpu + verfiy
 * (src/main.cu:212-225, 254-388) on sampled rows: plain fp32 attention of one query row over the unit's keys
 * with the launch's masks and ALiBi.  Returns the output row in out[d]. */
static void naive_row(const uint16_t* q, const uint16_t* k, const uint16_t* v, int dtype, int row, int Nk, int d,
                      float scale, int causal, int wl, int wr, float slope, long q_pos0, float* scores, float* out) {
    float mx = -INFINITY;
    const long qp = q_pos0 + row;
    for (int j = 0; j < Nk; ++j) {
        const int masked = (causal && j > qp) || (wl >= 0 && qp - j > wl) || (wr >= 0 && j - qp > wr);
        if (masked) { scores[j] = -INFINITY; continue; }
        float acc = 0.0f;
        for (int c = 0; c < d; ++c) {
            const float a = dtype == FA_DTYPE_BF16 ? from_bf16(q[(size_t)row * d + c]) : from_fp16(q[(size_t)row * d + c]);
            const float b = dtype == FA_DTYPE_BF16 ? from_bf16(k[(size_t)j * d + c]) : from_fp16(k[(size_t)j * d + c]);
            acc += a * b;
        }
        scores[j] = acc * scale - slope * (float)labs(qp - j);
        if (scores[j] > mx) mx = scores[j];
    }
    float sum = 0.0f;
    for (int j = 0; j < Nk; ++j) { scores[j] = scores[j] == -INFINITY ? 0.0f : expf(scores[j] - mx); sum += scores[j]; }
    for (int c = 0; c < d; ++c) out[c] = 0.0f;
    if (sum > 0.0f)
        for (int j = 0; j < Nk; ++j) {
            if (scores[j] == 0.0f) continue;
            const float p = scores[j] / sum;
            for (int c = 0; c < d; ++c)
                out[c] += p * (dtype == FA_DTYPE_BF16 ? from_bf16(v[(size_t)j * d + c]) : from_fp16(v[(size_t)j * d + c]));
        }
}

/* ---- config 5: bf16 [1,32,131072,128] causal, N(0, 0.5), the sequence sharded over the devices ---- */
typedef struct {
    int rank, world, iters, warmup, heads, chunk, d, rc;
    void* comm;
    const uint16_t* host_chunk[3][2];  /* one head of q, k, v for each of the rank's two chunks */
    pthread_barrier_t* barrier;
    float ms;
} ring_thread_t;

static void* ring_thread(void* arg) {
    ring_thread_t* t = (ring_thread_t*)arg;
    t->rc = 1;
    if (cudaSetDevice(t->rank) != cudaSuccess) return NULL;
    const size_t head_elems = (size_t)t->chunk * t->d, chunk_elems = head_elems * t->heads;
    cudaStream_t compute, comm;
    cudaEvent_t e0, e1;
    /* the exchange gets the highest stream priority: its few CTAs are then placed as soon as an SM
       frees up, instead of queueing behind the thousand CTAs of the attention launch it overlaps */
    int prio_least = 0, prio_greatest = 0;
    if (cudaDeviceGetStreamPriorityRange(&prio_least, &prio_greatest) != cudaSuccess) return NULL;
    if (cudaStreamCreate(&compute) != cudaSuccess ||
        cudaStreamCreateWithPriority(&comm, cudaStreamNonBlocking, prio_greatest) != cudaSuccess ||
        cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return NULL;
    fa_ring_params p;
    memset(&p, 0, sizeof(p));
    void* dev_in[3][2];
    for (int x = 0; x < 3; ++x)
        for (int i = 0; i < 2; ++i) {
            if (cudaMalloc(&dev_in[x][i], chunk_elems * 2) != cudaSuccess) return NULL;
            /* one generated head, repeated over the heads on the device */
            if (cudaMemcpy(dev_in[x][i], t->host_chunk[x][i], head_elems * 2, cudaMemcpyHostToDevice) != cudaSuccess) return NULL;
            for (int h = 1; h < t->heads; ++h)
                if (cudaMemcpy((char*)dev_in[x][i] + (size_t)h * head_elems * 2, dev_in[x][i], head_elems * 2,
                               cudaMemcpyDeviceToDevice) != cudaSuccess) return NULL;
        }
    for (int i = 0; i < 2; ++i) {
        p.q[i] = dev_in[0][i]; p.k[i] = dev_in[1][i]; p.v[i] = dev_in[2][i];
        if (cudaMalloc(&p.o[i], chunk_elems * 2) != cudaSuccess) return NULL;
        if (cudaMalloc((void**)&p.lse[i], (size_t)t->heads * t->chunk * 4) != cudaSuccess) return NULL;
        if (cudaMalloc((void**)&p.accum_o[i], chunk_elems * 4) != cudaSuccess) return NULL;
        if (cudaMalloc((void**)&p.accum_lse[i], (size_t)t->heads * t->chunk * 4) != cudaSuccess) return NULL;
    }
    p.dtype = FA_DTYPE_BF16;
    p.batch = 1; p.heads = t->heads; p.heads_k = t->heads; p.chunk_rows = t->chunk; p.head_dim = t->d;
    p.softmax_scale = 1.0f / sqrtf((float)t->d);
    p.is_causal = 1; p.window_left = p.window_right = -1;
    p.rank = t->rank; p.world = t->world; p.comm = t->comm;
    p.compute_stream = compute; p.comm_stream = comm;
    const size_t msg = fa_ring_message_bytes(&p);
    if (cudaMalloc(&p.message[0], msg) != cudaSuccess || cudaMalloc(&p.message[1], msg) != cudaSuccess) return NULL;
    for (int it = 0; it < t->warmup; ++it)
        if (fa_ring_fwd(&p) != FA_OK) return NULL;
    if (cudaDeviceSynchronize() != cudaSuccess) return NULL;
    pthread_barrier_wait(t->barrier);
    cudaEventRecord(e0, compute);
    for (int it = 0; it < t->iters; ++it)
        if (fa_ring_fwd(&p) != FA_OK) return NULL;
    cudaEventRecord(e1, compute);
    if (cudaStreamSynchronize(compute) != cudaSuccess || cudaStreamSynchronize(comm) != cudaSuccess) return NULL;
    cudaEventElapsedTime(&t->ms, e0, e1);
    pthread_barrier_wait(t->barrier);
    for (int i = 0; i < 2; ++i) {
        cudaFree((void*)p.q[i]); cudaFree((void*)p.k[i]); cudaFree((void*)p.v[i]); cudaFree(p.o[i]); cudaFree(p.lse[i]);
        cudaFree(p.accum_o[i]); cudaFree(p.accum_lse[i]); cudaFree(p.message[i]);
    }
    cudaEventDestroy(e0); cudaEventDestroy(e1); cudaStreamDestroy(compute); cudaStreamDestroy(comm);
    t->rc = 0;
    return NULL;
}

typedef struct { int g, world, rc; unsigned char* id; void** comm; } fa_bench_ci_t;
static void* fa_bench_comm_thread(void* arg) {
    fa_bench_ci_t* c = (fa_bench_ci_t*)arg;
    c->rc = 1;
    if (cudaSetDevice(c->g) != cudaSuccess) return NULL;
    if (fa_ring_comm_create(c->comm, c->world, c->g, c->id, 128) != FA_OK) return NULL;
    c->rc = 0;
    return NULL;
}

static int run_config5(int gpus, int iters, int warmup, int seq) {
    const int heads = 32, d = 128;
    if (seq % (2 * gpus * 128) != 0) { fprintf(stderr, "fa_bench: the sequence must split into 2 x gpus chunks of whole tiles\n"); return 2; }
    const int chunk = seq / (2 * gpus);
    unsigned char id[128];
    void** comms = (void**)calloc((size_t)gpus, sizeof(void*));
    ring_thread_t* th = (ring_thread_t*)calloc((size_t)gpus, sizeof(ring_thread_t));
    pthread_t* tid = (pthread_t*)calloc((size_t)gpus, sizeof(pthread_t));
    pthread_barrier_t barrier;
    pthread_barrier_init(&barrier, NULL, (unsigned)gpus);
    if (gpus > 1) CHECK_FA(fa_ring_unique_id(id, sizeof(id)));
    /* one generated head per chunk of the sequence (2 x gpus chunks), shared by q, k, v streams 0, 1, 2 */
    const size_t head_elems = (size_t)chunk * d;
    uint16_t* host = (uint16_t*)malloc(head_elems * 2 * 3 * 2 * (size_t)gpus);
    if (!host) { fprintf(stderr, "fa_bench: out of host memory\n"); return 1; }
    for (int g = 0; g < gpus; ++g) {
        const int chunks[2] = {g, 2 * gpus - 1 - g};
        for (int x = 0; x < 3; ++x)
            for (int i = 0; i < 2; ++i) {
                uint16_t* dst = host + (((size_t)g * 3 + x) * 2 + i) * head_elems;
                for (size_t e = 0; e < head_elems; ++e)
                    dst[e] = to_bf16(synth_normal(5, (uint64_t)x, (uint64_t)chunks[i] * head_elems + e, 0.5f));
                th[g].host_chunk[x][i] = dst;
            }
    }
    for (int g = 0; g < gpus; ++g) {
        th[g].rank = g; th[g].world = gpus; th[g].iters = iters; th[g].warmup = warmup;
        th[g].heads = heads; th[g].chunk = chunk; th[g].d = d; th[g].barrier = &barrier;
    }
    if (gpus > 1) {
        /* ncclCommInitRank blocks until all ranks have called it: one thread per rank */
        pthread_t* it = (pthread_t*)calloc((size_t)gpus, sizeof(pthread_t));
        fa_bench_ci_t* ci = (fa_bench_ci_t*)calloc((size_t)gpus, sizeof(fa_bench_ci_t));
        for (int g = 0; g < gpus; ++g) { ci[g].g = g; ci[g].world = gpus; ci[g].id = id; ci[g].comm = &comms[g]; pthread_create(&it[g], NULL, fa_bench_comm_thread, &ci[g]); }
        for (int g = 0; g < gpus; ++g) pthread_join(it[g], NULL);
        for (int g = 0; g < gpus; ++g) if (ci[g].rc != 0) { fprintf(stderr, "fa_bench: communicator of rank %d failed\n", g); return 1; }
        free(it); free(ci);
    }
    for (int g = 0; g < gpus; ++g) { th[g].comm = comms[g]; pthread_create(&tid[g], NULL, ring_thread, &th[g]); }
    float ms_max = 0.0f;
    int bad = 0;
    for (int g = 0; g < gpus; ++g) { pthread_join(tid[g], NULL); if (th[g].rc) bad = 1; if (th[g].ms > ms_max) ms_max = th[g].ms; }
    for (int g = 0; g < gpus; ++g) if (comms[g]) { cudaSetDevice(g); fa_ring_comm_destroy(comms[g]); }
    if (bad) { fprintf(stderr, "fa_bench: a ring rank failed\n"); return 1; }
    const double ms_iter = ms_max / iters;
    const double flops = 4.0 * heads * 0.5 * (double)seq * (double)seq * d;  /* causal convention 4*H*N^2*d/2 */
    printf("{\"driver\": \"fa_bench\", \"config\": \"config 5: bf16 [1,32,%d,128] causal, sequence ring over %d GPU(s)\", "
           "\"n_gpus\": %d, \"iters\": %d, \"ms_per_iter\": %.4f, \"tflops\": %.2f, \"chunk_rows\": %d}\n",
           seq, gpus, gpus, iters, ms_iter, flops / (ms_iter * 1e-3) / 1e12, chunk);
    free(host); free(th); free(tid); free(comms);
    pthread_barrier_destroy(&barrier);
    return 0;
}

typedef struct {
    int dev, units, unit0;
    void *q, *k, *v, *o, *ws, *slopes;
    float* lse;
    size_t ws_bytes;
    cudaStream_t stream;
    cudaEvent_t e0, e1;
    fa_fwd_params p;
} shard_t;

int main(int argc, char** argv) {
    int cfg_id = 1, gpus = 1, iters = 20, warmup = 3, units_override = 0, seq = 131072, check = 0;
    const char* dump = NULL;
    for (int i = 1; i < argc; ++i) {
        if (!strcmp(argv[i], "--config") && i + 1 < argc) cfg_id = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--gpus") && i + 1 < argc) gpus = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--iters") && i + 1 < argc) iters = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--warmup") && i + 1 < argc) warmup = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--units") && i + 1 < argc) units_override = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--dump") && i + 1 < argc) dump = argv[++i];
        else if (!strcmp(argv[i], "--seq") && i + 1 < argc) seq = atoi(argv[++i]);  /* config 5: sequence length (tests) */
        else if (!strcmp(argv[i], "--check")) check = 1;
        else { fprintf(stderr, "usage: fa_bench --config 1..5 [--gpus N] [--iters I] [--warmup W] [--units U] [--dump FILE] [--seq N] [--check]\n"); return 2; }
    }
    if (cfg_id < 1 || cfg_id > 5 || gpus < 1 || iters < 1) { fprintf(stderr, "fa_bench: bad arguments\n"); return 2; }
    if (cfg_id == 5) {
        int ndev5 = 0;
        CHECK_CUDA(cudaGetDeviceCount(&ndev5));
        if (gpus > ndev5) { fprintf(stderr, "fa_bench: %d GPUs asked, %d present\n", gpus, ndev5); return 2; }
        return run_config5(gpus, iters, warmup, seq);
    }
    config_t c = kConfigs[cfg_id - 1];
    if (check) c.p = 0.0f;  /* the verification has no dropout (src/main.cu:44, 222) */
    int units = c.B * c.H;
    if (units_override > 0 && units_override < units) units = units_override;  /* a prefix of the units (tests) */
    int ndev = 0;
    CHECK_CUDA(cudaGetDeviceCount(&ndev));
    if (gpus > ndev) { fprintf(stderr, "fa_bench: %d GPUs asked, %d present\n", gpus, ndev); return 2; }

    /* host inputs: at most `distinct` different units are generated, the rest repeat them */
    const size_t q_unit = (size_t)c.Nq * c.d, kv_unit = (size_t)c.Nk * c.d;
    const int distinct = (dump || units <= 8) ? units : 4;
    uint16_t* hq = (uint16_t*)malloc(q_unit * distinct * 2);
    uint16_t* hk = (uint16_t*)malloc(kv_unit * distinct * 2);
    uint16_t* hv = (uint16_t*)malloc(kv_unit * distinct * 2);
    float* hslopes = (float*)malloc(sizeof(float) * (size_t)units);
    if (!hq || !hk || !hv || !hslopes) { fprintf(stderr, "fa_bench: out of host memory\n"); return 1; }
    fill(hq, q_unit * distinct, c.seed, 0, c.sigma, c.dtype);
    fill(hk, kv_unit * distinct, c.seed, 1, c.sigma, c.dtype);
    fill(hv, kv_unit * distinct, c.seed, 2, c.sigma, c.dtype);
    for (int u = 0; u < units; ++u) hslopes[u] = (float)pow(2.0, -8.0 * ((u % c.H) + 1) / c.H);

    shard_t* sh = (shard_t*)calloc((size_t)gpus, sizeof(shard_t));
    for (int g = 0; g < gpus; ++g) {
        shard_t* s = &sh[g];
        const int base = units / gpus, extra = units % gpus;
        s->dev = g;
        s->unit0 = g * base + (g < extra ? g : extra);
        s->units = base + (g < extra ? 1 : 0);
        if (s->units == 0) continue;
        CHECK_CUDA(cudaSetDevice(g));
        CHECK_CUDA(cudaStreamCreate(&s->stream));
        CHECK_CUDA(cudaEventCreate(&s->e0));
        CHECK_CUDA(cudaEventCreate(&s->e1));
        CHECK_CUDA(cudaMalloc(&s->q, q_unit * s->units * 2));
        CHECK_CUDA(cudaMalloc(&s->k, kv_unit * s->units * 2));
        CHECK_CUDA(cudaMalloc(&s->v, kv_unit * s->units * 2));
        CHECK_CUDA(cudaMalloc(&s->o, q_unit * s->units * 2));
        CHECK_CUDA(cudaMalloc((void**)&s->lse, sizeof(float) * (size_t)c.Nq * s->units));
        CHECK_CUDA(cudaMalloc(&s->slopes, sizeof(float) * (size_t)s->units));
        int* first_local = (int*)malloc(sizeof(int) * (size_t)distinct);
        for (int i = 0; i < distinct; ++i) first_local[i] = -1;
        for (int u = 0; u < s->units; ++u) {  /* upload every distinct unit once, repeat it on the device */
            const int src = (s->unit0 + u) % distinct;
            char* dq = (char*)s->q + (size_t)u * q_unit * 2;
            char* dk = (char*)s->k + (size_t)u * kv_unit * 2;
            char* dv = (char*)s->v + (size_t)u * kv_unit * 2;
            if (first_local[src] < 0) {
                first_local[src] = u;
                CHECK_CUDA(cudaMemcpy(dq, hq + (size_t)src * q_unit, q_unit * 2, cudaMemcpyHostToDevice));
                CHECK_CUDA(cudaMemcpy(dk, hk + (size_t)src * kv_unit, kv_unit * 2, cudaMemcpyHostToDevice));
                CHECK_CUDA(cudaMemcpy(dv, hv + (size_t)src * kv_unit, kv_unit * 2, cudaMemcpyHostToDevice));
            } else {
                const size_t f0 = (size_t)first_local[src];
                CHECK_CUDA(cudaMemcpy(dq, (char*)s->q + f0 * q_unit * 2, q_unit * 2, cudaMemcpyDeviceToDevice));
                CHECK_CUDA(cudaMemcpy(dk, (char*)s->k + f0 * kv_unit * 2, kv_unit * 2, cudaMemcpyDeviceToDevice));
                CHECK_CUDA(cudaMemcpy(dv, (char*)s->v + f0 * kv_unit * 2, kv_unit * 2, cudaMemcpyDeviceToDevice));
            }
        }
        free(first_local);
        CHECK_CUDA(cudaMemcpy(s->slopes, hslopes + s->unit0, sizeof(float) * (size_t)s->units, cudaMemcpyHostToDevice));
        /* every slice is described as batch 1 x heads = its units, with per-unit ALiBi slopes */
        fa_fwd_params* p = &s->p;
        memset(p, 0, sizeof(*p));
        p->q = s->q; p->k = s->k; p->v = s->v; p->o = s->o; p->lse = s->lse;
        p->dtype = p->o_dtype = c.dtype;
        p->batch = 1; p->heads = s->units;
        p->seqlen_q = c.Nq; p->seqlen_k = c.Nk; p->head_dim = c.d;
        p->softmax_scale = 1.0f / sqrtf((float)c.d);
        p->is_causal = c.causal; p->window_left = c.wl; p->window_right = c.wr;
        p->alibi_slopes = c.alibi ? (const float*)s->slopes : NULL;
        p->p_dropout = c.p; p->seed = 42; p->offset = 0; p->unit0 = (uint64_t)s->unit0;
        p->num_splits = c.splits;
        p->stream = s->stream;
        s->ws_bytes = fa_fwd_workspace_bytes(p);
        if (s->ws_bytes) CHECK_CUDA(cudaMalloc(&s->ws, s->ws_bytes));
        p->workspace = s->ws; p->workspace_bytes = s->ws_bytes;
    }

    for (int it = 0; it < warmup; ++it)
        for (int g = 0; g < gpus; ++g) if (sh[g].units) { CHECK_CUDA(cudaSetDevice(g)); CHECK_FA(fa_fwd(&sh[g].p)); }
    for (int g = 0; g < gpus; ++g) if (sh[g].units) { CHECK_CUDA(cudaSetDevice(g)); CHECK_CUDA(cudaDeviceSynchronize()); }
    for (int g = 0; g < gpus; ++g) if (sh[g].units) { CHECK_CUDA(cudaSetDevice(g)); CHECK_CUDA(cudaEventRecord(sh[g].e0, sh[g].stream)); }
    for (int it = 0; it < iters; ++it)
        for (int g = 0; g < gpus; ++g) if (sh[g].units) { CHECK_CUDA(cudaSetDevice(g)); CHECK_FA(fa_fwd(&sh[g].p)); }
    float ms_max = 0.0f;
    for (int g = 0; g < gpus; ++g) if (sh[g].units) {
        CHECK_CUDA(cudaSetDevice(g));
        CHECK_CUDA(cudaEventRecord(sh[g].e1, sh[g].stream));
        CHECK_CUDA(cudaEventSynchronize(sh[g].e1));
        float ms = 0.0f;
        CHECK_CUDA(cudaEventElapsedTime(&ms, sh[g].e0, sh[g].e1));
        if (ms > ms_max) ms_max = ms;
    }
    const double ms_iter = ms_max / iters;

    /* algorithmic work: 4*d FLOP per unmasked (q,k) pair; config 2 by the 4*B*H*N^2*d/2 convention */
    double pairs = 0.0;
    if (cfg_id == 2) pairs = 0.5 * (double)c.Nq * c.Nk;
    else for (int i = 0; i < c.Nq; ++i) {
        long lo = 0, hi = c.Nk - 1;
        if (c.causal && i < hi) hi = i;
        if (c.wr >= 0 && i + c.wr < hi) hi = i + c.wr;
        if (c.wl >= 0 && i - c.wl > lo) lo = i - c.wl;
        if (hi >= lo) pairs += (double)(hi - lo + 1);
    }
    const double flops = 4.0 * c.d * pairs * units;
    const double bytes = 2.0 * units * c.d * (2.0 * c.Nk + 2.0 * c.Nq);

    /* result of the last launch: checksum, optional dump (O then LSE, device 0's slice first) */
    double checksum = 0.0;
    FILE* f = dump ? fopen(dump, "wb") : NULL;
    if (dump && !f) { fprintf(stderr, "fa_bench: cannot open %s\n", dump); return 1; }
    for (int g = 0; g < gpus; ++g) if (sh[g].units) {
        CHECK_CUDA(cudaSetDevice(g));
        const size_t n = q_unit * sh[g].units;
        uint16_t* ho = (uint16_t*)malloc(n * 2);
        CHECK_CUDA(cudaMemcpy(ho, sh[g].o, n * 2, cudaMemcpyDeviceToHost));
        for (size_t i = 0; i < n; ++i) checksum += (double)ho[i] * (double)((i % 251) + 1);
        if (f) fwrite(ho, 2, n, f);
        free(ho);
    }
    if (f) {
        for (int g = 0; g < gpus; ++g) if (sh[g].units) {
            CHECK_CUDA(cudaSetDevice(g));
            const size_t n = (size_t)c.Nq * sh[g].units;
            float* hl = (float*)malloc(n * 4);
            CHECK_CUDA(cudaMemcpy(hl, sh[g].lse, n * 4, cudaMemcpyDeviceToHost));
            fwrite(hl, 4, n, f);
            free(hl);
        }
        fclose(f);
    }

    double check_max = -1.0, check_mean = 0.0, cpu_ms_per_row = 0.0;
    int check_rows = 0;
    if (check) {
        /* sampled rows of device 0's slice: first, last, tile edges and a stride through the rest */
        shard_t* s0 = &sh[0];
        CHECK_CUDA(cudaSetDevice(0));
        float* scores = (float*)malloc(sizeof(float) * (size_t)c.Nk);
        float* want = (float*)malloc(sizeof(float) * (size_t)c.d);
        uint16_t* got = (uint16_t*)malloc(2 * (size_t)c.d);
        struct timespec t0, t1;
        clock_gettime(CLOCK_MONOTONIC, &t0);
        check_max = 0.0;
        double sum = 0.0;
        const int sample_units = s0->units < 3 ? s0->units : 3;
        for (int su = 0; su < sample_units; ++su) {
            const int u = su == 0 ? 0 : (su == 1 ? s0->units - 1 : s0->units / 2);
            const int src = (s0->unit0 + u) % distinct;
            const int rows[8] = {0, c.Nq / 2, c.Nq - 1, c.Nq > 128 ? 127 : 0, c.Nq > 128 ? 128 : 0, c.Nq > 1025 ? 1024 : 0,
                                 c.Nq > 1025 ? 1025 : 0, (int)((977u * (unsigned)(su + 1)) % (unsigned)c.Nq)};
            for (int r = 0; r < 8; ++r) {
                const int row = rows[r];
                naive_row(hq + (size_t)src * q_unit, hk + (size_t)src * kv_unit, hv + (size_t)src * kv_unit, c.dtype, row, c.Nk,
                          c.d, 1.0f / sqrtf((float)c.d), c.causal, c.wl, c.wr, c.alibi ? hslopes[s0->unit0 + u] : 0.0f,
                          0L, scores, want);
                CHECK_CUDA(cudaMemcpy(got, (char*)s0->o + ((size_t)u * q_unit + (size_t)row * c.d) * 2, 2 * (size_t)c.d,
                                      cudaMemcpyDeviceToHost));
                for (int x = 0; x < c.d; ++x) {
                    const double e = fabs((double)(c.dtype == FA_DTYPE_BF16 ? from_bf16(got[x]) : from_fp16(got[x])) - (double)want[x]);
                    if (e > check_max) check_max = e;
                    sum += e;
                }
                ++check_rows;
            }
        }
        clock_gettime(CLOCK_MONOTONIC, &t1);
        check_mean = sum / ((double)check_rows * c.d);
        cpu_ms_per_row = ((double)(t1.tv_sec - t0.tv_sec) * 1e3 + (double)(t1.tv_nsec - t0.tv_nsec) * 1e-6) / check_rows;
        free(scores); free(want); free(got);
    }

    printf("{\"driver\": \"fa_bench\", \"config\": \"%s\", \"units\": %d, \"n_gpus\": %d, \"iters\": %d, \"ms_per_iter\": %.6f, "
           "\"tflops\": %.3f, \"gbs\": %.1f, \"checksum\": %.0f",
           c.name, units, gpus, iters, ms_iter, flops / (ms_iter * 1e-3) / 1e12, bytes / (ms_iter * 1e-3) / 1e9, checksum);
    if (check) {
        /* CPU time of the whole workload, extrapolated linearly in rows from the sampled ones (1 core) */
        const double cpu_s = cpu_ms_per_row * 1e-3 * (double)c.Nq * units;
        printf(", \"check\": {\"rows\": %d, \"max_abs\": %.5f, \"mean_abs\": %.6f, \"pass\": %s, \"dropout\": \"off for the check\"}, "
               "\"cpu\": {\"cores\": 1, \"ms_per_row\": %.4f, \"seconds_whole_workload_extrapolated\": %.1f}",
               check_rows, check_max, check_mean, (check_max <= 2e-2 && check_mean <= 2e-3) ? "true" : "false", cpu_ms_per_row, cpu_s);
    }
    printf("}\n");
    if (check && !(check_max <= 2e-2 && check_mean <= 2e-3)) return 3;

    for (int g = 0; g < gpus; ++g) if (sh[g].units) {
        cudaSetDevice(g);
        cudaFree(sh[g].q); cudaFree(sh[g].k); cudaFree(sh[g].v); cudaFree(sh[g].o); cudaFree(sh[g].lse);
        cudaFree(sh[g].slopes); cudaFree(sh[g].ws);
        cudaEventDestroy(sh[g].e0); cudaEventDestroy(sh[g].e1); cudaStreamDestroy(sh[g].stream);
    }
    free(sh); free(hq); free(hk); free(hv); free(hslopes);
    return 0;
}
