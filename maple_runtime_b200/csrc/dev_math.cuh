// dev_math.cuh -- device arithmetic that has to land on the same bits as the reference's libm calls.
#pragma once
#include <stdint.h>

// 2^(i/32) as double bits with i << 47 subtracted: the table of the double-precision expf scheme published with
// the Arm optimized routines (glibc's expf since 2.27).  The CPU test-suite checks the same scheme against libm
// expf over every float in [-104, 89].
static __device__ const unsigned long long DEV_EXP_TAB[32] = {
    0x3ff0000000000000ull, 0x3fefd9b0d3158574ull, 0x3fefb5586cf9890full, 0x3fef9301d0125b51ull,
    0x3fef72b83c7d517bull, 0x3fef54873168b9aaull, 0x3fef387a6e756238ull, 0x3fef1e9df51fdee1ull,
    0x3fef06fe0a31b715ull, 0x3feef1a7373aa9cbull, 0x3feedea64c123422ull, 0x3feece086061892dull,
    0x3feebfdad5362a27ull, 0x3feeb42b569d4f82ull, 0x3feeab07dd485429ull, 0x3feea47eb03a5585ull,
    0x3feea09e667f3bcdull, 0x3fee9f75e8ec5f74ull, 0x3feea11473eb0187ull, 0x3feea589994cce13ull,
    0x3feeace5422aa0dbull, 0x3feeb737b0cdc5e5ull, 0x3feec49182a3f090ull, 0x3feed503b23e255dull,
    0x3feee89f995ad3adull, 0x3feeff76f2fb5e47ull, 0x3fef199bdd85529cull, 0x3fef3720dcef9069ull,
    0x3fef5818dcfba487ull, 0x3fef7c97337b9b5full, 0x3fefa4afa2a490daull, 0x3fefd0765b6e4540ull};

// expf as the reference's libm computes it (maple.c:738, 829, 915 call expf): x scaled by 32/ln2, nearest integer
// split off with the 1.5*2^52 shift, cubic in the remainder, table value times 2^(k/32), one rounding to float.
template <typename TabT>
__device__ __forceinline__ float dev_expf_tab(float x, const TabT *tab) {
    if (x != x) return x;
    if (x > 89.0f) return __int_as_float(0x7f800000);
    if (x < -104.0f) return 0.0f;
    const double inv_ln2_n = 0x1.71547652b82fep+0 * 32.0, shift = 0x1.8p+52;
    const double c0 = 0x1.c6af84b912394p-5 / 32768.0, c1 = 0x1.ebfce50fac4f3p-3 / 1024.0, c2 = 0x1.62e42ff0c52d6p-1 / 32.0;
    double z = inv_ln2_n * (double)x, kd = z + shift;
    unsigned long long ki = (unsigned long long)__double_as_longlong(kd);
    kd -= shift;
    double r = z - kd;
    double s = __longlong_as_double((long long)(tab[ki & 31] + (ki << 47)));
    double p = c0 * r + c1, r2 = r * r, y = c2 * r + 1.0;
    y = p * r2 + y;
    return (float)(y * s);
}

__device__ __forceinline__ float dev_expf(float x) { return dev_expf_tab(x, DEV_EXP_TAB); }

// maple.c:827-829: g = min(g, 7), u = clamp(u, -7, 7), act = g / (1 + expf(-g)) * u
// tab: the 32-entry table above, or a copy of it in shared memory (lane-varying index: cheaper there)
template <typename TabT>
__device__ __forceinline__ float dev_silu_mul_tab(float g, float u, const TabT *tab) {
    g = g < 7.0f ? g : 7.0f;
    u = u < -7.0f ? -7.0f : (u > 7.0f ? 7.0f : u);
    return __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, dev_expf_tab(-g, tab))), u);
}
__device__ __forceinline__ float dev_silu_mul(float g, float u) { return dev_silu_mul_tab(g, u, DEV_EXP_TAB); }
