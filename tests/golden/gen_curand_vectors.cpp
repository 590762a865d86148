// Generates tests/golden/philox_kat.json and tests/golden/dropout_mask_sim.json
// with NVIDIA cuRAND's own Philox4_32_10 device API (CUDA Toolkit headers) run on
// the host: the QUALIFIERS macro, which the headers let a includer pre-define,
// turns curand_init / curand / curand_uniform into ordinary host functions.
//
//   g++ -O2 -I/usr/local/cuda/include tests/golden/gen_curand_vectors.cpp -o /tmp/gen_curand
//   /tmp/gen_curand tests/golden
//
// Part 1 (KATs): raw draws and uniforms for several (seed, subsequence, offset).
// Part 2 (mask simulation): walks the reference kernels' loop structure literally
// -- one stream per CTA (src/flash_forward.h:50-54), 64 draws per KV tile in
// c_frag[i][j] order (:221-237), fragment (i,j) -> (row,col) of every warp/lane
// (:130-131), KV tile range (:39-48, src/flash_forward_splitkv.h:40-52) -- and
// records the keep decision of every (row, col).  The closed-form map used by
// the oracle and by the CUDA kernels is tested against these bits.
#define QUALIFIERS static inline
#include <cstdio>
#include <cstdint>
#include <cstdlib>
#include <cmath>
#include <string>
#include <vector>
#include <algorithm>
#include <cuda_runtime.h>
#include <curand_kernel.h>

static void kats(FILE* f) {
    struct C { unsigned long long seed, subseq, offset; };
    const C cases[] = {{0, 0, 0}, {42, 0, 0}, {42, 7, 0}, {48, 123456, 0}, {42, 3, 5},
                       {0x123456789abcdefULL, 0x1ffffffffULL, 1000003ULL}, {42, 2047, 64}};
    fprintf(f, "{\n \"cases\": [\n");
    const int n = sizeof(cases) / sizeof(cases[0]);
    for (int c = 0; c < n; ++c) {
        curandStatePhilox4_32_10_t st;
        curand_init(cases[c].seed, cases[c].subseq, cases[c].offset, &st);
        fprintf(f, "  {\"seed\": %llu, \"subsequence\": %llu, \"offset\": %llu, \"raw\": [",
                cases[c].seed, cases[c].subseq, cases[c].offset);
        for (int i = 0; i < 24; ++i) fprintf(f, "%s%u", i ? ", " : "", curand(&st));
        curand_init(cases[c].seed, cases[c].subseq, cases[c].offset, &st);
        fprintf(f, "], \"uniform_hex\": [");
        for (int i = 0; i < 24; ++i) {
            float u = curand_uniform(&st);
            uint32_t bits; memcpy(&bits, &u, 4);
            fprintf(f, "%s%u", i ? ", " : "", bits);
        }
        fprintf(f, "]}%s\n", c + 1 < n ? "," : "");
    }
    fprintf(f, " ],\n \"thresholds\": [\n");
    // first kept raw value for a few probabilities, by exhaustive monotone search
    const float ps[] = {0.1f, 0.5f, 0.25f, 0.01f, 0.9f, 0.0f};
    const int np = sizeof(ps) / sizeof(ps[0]);
    for (int k = 0; k < np; ++k) {
        // curand_uniform(x) = x * 2^-32 + 2^-33 (fp32); scan outward from p*2^32
        double guess = (double)ps[k] * 4294967296.0;
        long long lo = std::max(0LL, (long long)guess - 100000), hi = std::min(4294967295LL, (long long)guess + 100000);
        long long first_kept = -1;
        for (long long x = lo; x <= hi; ++x) {
            float u = _curand_uniform((unsigned int)x);
            if (!(u < ps[k])) { first_kept = x; break; }
        }
        uint32_t pb; memcpy(&pb, &ps[k], 4);
        fprintf(f, "  {\"p_bits\": %u, \"first_kept\": %lld}%s\n", pb, first_kept, k + 1 < np ? "," : "");
    }
    fprintf(f, " ]\n}\n");
}

struct SimCase { int B, H, N; float p; unsigned long long seed; int splits; int causal; int wl, wr; };

static void simulate(FILE* f, const SimCase& c, bool last) {
    const int Br = 128, Bc = 128;
    const int Tr = (c.N + Br - 1) / Br, Tc = (c.N + Bc - 1) / Bc;
    const bool local = c.wl >= 0 || c.wr >= 0;
    std::vector<uint8_t> keep((size_t)c.B * c.H * c.N * c.N, 2);  // 2 = never visited
    const int gx = Tr * c.splits, gy = c.H, gz = c.B;
    for (int bz = 0; bz < gz; ++bz) for (int by = 0; by < gy; ++by) for (int bx = 0; bx < gx; ++bx) {
        int nbmin, nbmax, rb;
        if (c.splits == 1) {
            rb = bx;
            nbmin = !local ? 0 : std::max(0, (bx * Br - c.wl) / Bc);
            nbmax = Tc;
            if (local) nbmax = std::min(nbmax, ((bx + 1) * Br + c.wr + Bc - 1) / Bc);
            if (c.causal) nbmax = std::min(nbmax, ((bx + 1) * Br + Bc - 1) / Bc);
        } else {
            rb = bx / c.splits;
            int per = (Tc + c.splits - 1) / c.splits;
            nbmin = per * (bx % c.splits);
            nbmax = std::min(nbmin + per, Tc);
            if (local) nbmin = std::max(nbmin, (rb * Br - c.wl) / Bc);
            if (local) nbmax = std::min(nbmax, ((rb + 1) * Br + c.wr + Bc - 1) / Bc);
            if (c.causal) nbmax = std::min(nbmax, ((rb + 1) * Br + Bc - 1) / Bc);
        }
        curandStatePhilox4_32_10_t st;
        const int state_idx = bz * gy * gx + by * gx + bx;
        curand_init(c.seed, state_idx, 0, &st);
        for (int iter = nbmin; iter < nbmax; ++iter) {
            bool kp[8][8];
            for (int i = 0; i < 8; ++i) for (int j = 0; j < 8; ++j) kp[i][j] = !(curand_uniform(&st) < c.p);
            for (int warp = 0; warp < 8; ++warp) for (int lane = 0; lane < 32; ++lane)
                for (int i = 0; i < 8; ++i) for (int j = 0; j < 8; ++j) {
                    int row = rb * Br + warp * 16 + lane / 4 + (j / 4) * 8;
                    int col = iter * Bc + i * 16 + (lane % 4) * 2 + (j % 4) / 2 * 8 + j % 2;
                    if (row < c.N && col < c.N)
                        keep[(((size_t)bz * c.H + by) * c.N + row) * c.N + col] = kp[i][j];
                }
        }
    }
    uint32_t pb; memcpy(&pb, &c.p, 4);
    fprintf(f, "  {\"B\": %d, \"H\": %d, \"N\": %d, \"p_bits\": %u, \"seed\": %llu, \"splits\": %d, \"causal\": %d, \"wl\": %d, \"wr\": %d,\n   \"mask\": \"",
            c.B, c.H, c.N, pb, c.seed, c.splits, c.causal, c.wl, c.wr);
    // one char per element: '0' dropped, '1' kept, '.' not visited (tile skipped); run-length free, rows concatenated
    for (size_t i = 0; i < keep.size(); ++i) fputc(keep[i] == 2 ? '.' : '0' + keep[i], f);
    fprintf(f, "\"}%s\n", last ? "" : ",");
}

int main(int argc, char** argv) {
    std::string dir = argc > 1 ? argv[1] : ".";
    FILE* f = fopen((dir + "/philox_kat.json").c_str(), "w");
    kats(f); fclose(f);
    f = fopen((dir + "/dropout_mask_sim.json").c_str(), "w");
    const SimCase cs[] = {
        {1, 2, 200, 0.1f, 42, 1, 0, -1, -1},
        {2, 1, 300, 0.1f, 42, 1, 1, -1, -1},
        {1, 1, 400, 0.25f, 48, 1, 0, 130, 5},
        {1, 2, 256, 0.1f, 7, 2, 0, -1, -1},
        {1, 1, 384, 0.5f, 9, 3, 1, -1, -1},
    };
    const int n = sizeof(cs) / sizeof(cs[0]);
    fprintf(f, "{\n \"cases\": [\n");
    for (int i = 0; i < n; ++i) simulate(f, cs[i], i + 1 == n);
    fprintf(f, " ]\n}\n");
    fclose(f);
    return 0;
}
