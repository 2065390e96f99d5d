/* synth.h -- seeded synthetic Maple-shaped weights and activations (shared by host C and CUDA code).
 *
 * The real checkpoint cannot be present where this library is measured, so every tensor is a pure function of
 * (seed, tensor id, element index) through a counter-based generator.  Host and device evaluate the same integer
 * arithmetic, so a slice generated on a GPU equals the same slice generated on a CPU bit for bit.
 *
 * Layout written is the reference converter's (convert.py:23-33, 79-84): a ternary matrix [rows x cols] is
 * rows*cols/4 bytes of 2-bit codes (code = t + 1 in {0,1,2}; within each 128-column group byte j holds columns
 * j, j+32, j+64, j+96 at bits 0,2,4,6) followed immediately by one fp32 scale per row.  One expert is
 * gate [512x2048], up [512x2048], down [2048x512] back to back = 798,720 bytes (layout.py:16-17 order).
 */
#ifndef MAPLE_SYNTH_H
#define MAPLE_SYNTH_H
#include <math.h>
#include <stdint.h>

#define MS_H 2048
#define MS_FF 512
#define MS_NE 256
#define MS_TOPK 8
#define MS_GU_CODES 262144u               /* 512 * 2048 / 4 */
#define MS_GU_BYTES 264192u               /* codes + 512 scales */
#define MS_DN_CODES 262144u               /* 2048 * 512 / 4 */
#define MS_DN_BYTES 270336u               /* codes + 2048 scales */
#define MS_EXPERT_BYTES 798720u           /* 2 * MS_GU_BYTES + MS_DN_BYTES */
#define MS_LAYER_BYTES 204472320ull       /* 256 experts */

#ifdef __CUDACC__
#define MS_HD __host__ __device__ static __forceinline__
#else
#define MS_HD static inline
#endif

MS_HD uint64_t ms_mix(uint64_t z) {       /* splitmix64 finaliser */
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
/* tensor ids: layer L, expert e, part 0 gate codes, 1 gate scales, 2 up codes, 3 up scales, 4 down codes, 5 down scales */
MS_HD uint64_t ms_tid(int L, int e, int part) { return ((uint64_t)L * MS_NE + (uint64_t)e) * 8 + (uint64_t)part + 1; }
MS_HD uint64_t ms_u64(uint64_t seed, uint64_t tid, uint64_t idx) { return ms_mix(ms_mix(seed ^ (tid << 36)) ^ idx); }

/* one packed byte = four codes drawn with P{0,1,2} = {0.3, 0.4, 0.3} from four 16-bit fields of one draw */
MS_HD uint8_t ms_code_byte(uint64_t seed, uint64_t tid, uint64_t idx) {
    uint64_t h = ms_u64(seed, tid, idx);
    uint32_t b = 0;
    for (int k = 0; k < 4; k++) {
        uint32_t v = (uint32_t)(h >> (16 * k)) & 0xFFFFu;
        b |= (v < 19661u ? 0u : v < 45875u ? 1u : 2u) << (2 * k);
    }
    return (uint8_t)b;
}
/* row scale ~ U(0.01, 0.05): 24 random bits, exact in fp32 on both sides */
MS_HD float ms_scale(uint64_t seed, uint64_t tid, uint64_t idx) {
    uint32_t u = (uint32_t)(ms_u64(seed, tid, idx) >> 40);
    return fmaf((float)u, 0.04f / 16777216.0f, 0.01f);   /* one explicit fused rounding: same bits on host and device */
}
#endif
