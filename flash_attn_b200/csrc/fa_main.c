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
 *   fa_bench --config 1|2|3|4 [--gpus N] [--iters I] [--warmup W] [--dump FILE] [--units U]
 *
 * With --gpus N the (batch, head) units are cut into N contiguous slices, one per
 * device, with no communication; every device gets its own stream and the job time
 * is the slowest device's.  Plain C99: only the CUDA runtime API and fa_b200.h.
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
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
    int cfg_id = 1, gpus = 1, iters = 20, warmup = 3, units_override = 0;
    const char* dump = NULL;
    for (int i = 1; i < argc; ++i) {
        if (!strcmp(argv[i], "--config") && i + 1 < argc) cfg_id = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--gpus") && i + 1 < argc) gpus = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--iters") && i + 1 < argc) iters = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--warmup") && i + 1 < argc) warmup = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--units") && i + 1 < argc) units_override = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--dump") && i + 1 < argc) dump = argv[++i];
        else { fprintf(stderr, "usage: fa_bench --config 1..4 [--gpus N] [--iters I] [--warmup W] [--units U] [--dump FILE]\n"); return 2; }
    }
    if (cfg_id < 1 || cfg_id > 4 || gpus < 1 || iters < 1) { fprintf(stderr, "fa_bench: bad arguments\n"); return 2; }
    config_t c = kConfigs[cfg_id - 1];
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

    printf("{\"driver\": \"fa_bench\", \"config\": \"%s\", \"units\": %d, \"n_gpus\": %d, \"iters\": %d, \"ms_per_iter\": %.6f, "
           "\"tflops\": %.3f, \"gbs\": %.1f, \"checksum\": %.0f}\n",
           c.name, units, gpus, iters, ms_iter, flops / (ms_iter * 1e-3) / 1e12, bytes / (ms_iter * 1e-3) / 1e9, checksum);

    for (int g = 0; g < gpus; ++g) if (sh[g].units) {
        cudaSetDevice(g);
        cudaFree(sh[g].q); cudaFree(sh[g].k); cudaFree(sh[g].v); cudaFree(sh[g].o); cudaFree(sh[g].lse);
        cudaFree(sh[g].slopes); cudaFree(sh[g].ws);
        cudaEventDestroy(sh[g].e0); cudaEventDestroy(sh[g].e1); cudaStreamDestroy(sh[g].stream);
    }
    free(sh); free(hq); free(hk); free(hv); free(hslopes);
    return 0;
}
