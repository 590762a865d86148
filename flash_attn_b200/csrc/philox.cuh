// Stateless Philox4x32-10 dropout generator.  Replaces the reference's stateful
// cuRAND set-up (src/init_curand_states.h:7-14) and its per-thread draw loop
// (src/flash_forward.h:50-54,221-237): the keep/drop decision of P[b,h,row,col]
// is a pure function of (seed, offset, launch geometry, b, h, row, col) that
// reproduces the reference's stream/draw order bit for bit.
//
// Reference order: one stream per CTA, subsequence = ((b*H+h)*Tr + rb)*splits + s;
// per 128x128 KV tile the CTA draws 64 values, draw 8*i + j deciding the
// fragment elements with  col%128 in 16*i + 8*((j%4)/2) + {0..7 of parity j%2},
// row%16 in 8*(j/4) + {0..7}.  Draw n of a stream is word n%4 of the Philox block
// with counter (n/4, subsequence) and key = seed; it is dropped iff
// x*2^-32 + 2^-33 < p in fp32, i.e. iff x < keep_threshold(p).
// Later launches of a timing loop: the kernels save the advanced state, so the CTA that
// visits T KV tiles starts launch k at draw 64*k*T of its stream (continuation()).
#pragma once
#include <cstdint>

namespace fa {

struct DropoutParams {
    uint32_t seed_lo, seed_hi;
    unsigned long long offset;      // draws skipped at the start of every stream
    unsigned long long launch_index;  // the reference writes every stream's state back (src/flash_forward.h:302-305):
                                      // launch k of a loop continues each CTA's stream 64 * k * (KV tiles that CTA
                                      // visits) draws further on; 0 = the first launch
    unsigned long long unit0;       // global (b*H+h) index of this launch's first unit
    unsigned long long threshold;   // raw draws below this are dropped (may be 2^32)
    float inv_keep;                 // 1/(1-p)
};

__host__ __device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                                       uint32_t k0, uint32_t k1, uint32_t (&out)[4]) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const unsigned long long p0 = 0xD2511F53ull * c0;
        const unsigned long long p1 = 0xCD9E8D57ull * c2;
        const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c1 ^ k0;
        const uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ c3 ^ k1;
        c1 = static_cast<uint32_t>(p1);
        c3 = static_cast<uint32_t>(p0);
        c0 = n0;
        c2 = n2;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// Draws a stream is ahead by at launch dp.launch_index when its CTA visits `tiles_visited` KV tiles per launch.
__host__ __device__ __forceinline__ unsigned long long continuation(const DropoutParams& dp, int tiles_visited) {
    return dp.launch_index * 64ull * static_cast<unsigned long long>(tiles_visited > 0 ? tiles_visited : 0);
}

// Keep bits of draws first .. first+3 of stream `subseq` (first % 4 == 0 before
// the offset is added): bit w set = draw first+w is kept.
__host__ __device__ __forceinline__ uint32_t philox_keep4(const DropoutParams& dp, unsigned long long subseq,
                                                          unsigned long long first) {
    const unsigned long long n = first + dp.offset;
    const unsigned long long blk = n >> 2;
    const uint32_t sh = static_cast<uint32_t>(n & 3);
    uint32_t w[4];
    philox4x32_10(static_cast<uint32_t>(blk), static_cast<uint32_t>(blk >> 32),
                  static_cast<uint32_t>(subseq), static_cast<uint32_t>(subseq >> 32), dp.seed_lo, dp.seed_hi, w);
    uint32_t x[4];
    if (sh == 0) {
        x[0] = w[0]; x[1] = w[1]; x[2] = w[2]; x[3] = w[3];
    } else {
        // offset not a multiple of 4: the four draws straddle two blocks
        uint32_t w2[4];
        const unsigned long long blk2 = blk + 1;
        philox4x32_10(static_cast<uint32_t>(blk2), static_cast<uint32_t>(blk2 >> 32),
                      static_cast<uint32_t>(subseq), static_cast<uint32_t>(subseq >> 32), dp.seed_lo, dp.seed_hi, w2);
        const uint32_t a[8] = {w[0], w[1], w[2], w[3], w2[0], w2[1], w2[2], w2[3]};
#pragma unroll
        for (int i = 0; i < 4; ++i) x[i] = sh == 1 ? a[i + 1] : (sh == 2 ? a[i + 2] : a[i + 3]);
    }
    uint32_t bits = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) bits |= (static_cast<unsigned long long>(x[i]) >= dp.threshold ? 1u : 0u) << i;
    return bits;
}

}  // namespace fa
