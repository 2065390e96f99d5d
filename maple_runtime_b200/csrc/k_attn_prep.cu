// k_attn_prep.cu -- the first step of the attention half of a layer (maple.c:711-717; the reference's card kernel is `qkn`,
// gpu_full.metal:32-71): per token and head, RMS norm of the query and key heads (head dimension 128; maple.c:398-402 with the layer's
// q_norm / k_norm), half-rotary embedding at the token's position on local layers (maple.c:403-411: dimensions 0..63 as pairs (i, i + 32),
// cos and sin from the host's table, maple.c:1151-1153), queries out in fp32, keys and values out in fp16 (maple.c:314-320: round to
// nearest even).  One warp per (token, head): lane l holds dimensions 4l..4l+3; the rotation partner of lanes 0-7 sits in lanes 8-15.
// The arithmetic is the compiled reference's: sum of squares in double, 1 / sqrtf(mean + 1e-6f), (x * k) * w, and for the rotation the
// fused forms its compiler emits: lo = fma(a, cos, -(b * sin)), hi = fma(b, cos, a * sin).
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include "kernels.h"
#include "launch.cuh"

extern "C" void k_count_add(long n);

#define AP_HD 128
#define AP_NH 16
#define AP_NKV 4

__global__ void __launch_bounds__(256) qk_rope_kernel(const float *__restrict__ qkv, const int *__restrict__ pos, int nb, int glob,
                                                      const float *__restrict__ qn, const float *__restrict__ kn, const float *__restrict__ cs, int cs_positions,
                                                      float *__restrict__ q, __half *__restrict__ kc, __half *__restrict__ vc, int *err) {
    const int lane = threadIdx.x & 31, item = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int heads = AP_NH + 2 * AP_NKV, b = item / heads, h = item % heads;
    if (b >= nb) return;
    float4 v = reinterpret_cast<const float4 *>(qkv + (size_t)b * (heads * AP_HD) + h * AP_HD)[lane];
    if (h >= AP_NH + AP_NKV) {      // a value head: fp16 only
        __half2 *o = reinterpret_cast<__half2 *>(vc + (size_t)b * (AP_NKV * AP_HD) + (h - AP_NH - AP_NKV) * AP_HD) + 2 * lane;
        o[0] = __halves2half2(__float2half_rn(v.x), __float2half_rn(v.y)); o[1] = __halves2half2(__float2half_rn(v.z), __float2half_rn(v.w));
        return;
    }
    double ss = (double)v.x * (double)v.x + (double)v.y * (double)v.y + ((double)v.z * (double)v.z + (double)v.w * (double)v.w);
#pragma unroll
    for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float k = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn((float)(ss / (double)AP_HD), 1e-6f)));
    const float4 w = reinterpret_cast<const float4 *>(h < AP_NH ? qn : kn)[lane];
    v.x = __fmul_rn(__fmul_rn(v.x, k), w.x); v.y = __fmul_rn(__fmul_rn(v.y, k), w.y); v.z = __fmul_rn(__fmul_rn(v.z, k), w.z); v.w = __fmul_rn(__fmul_rn(v.w, k), w.w);
    if (!glob) {
        int p = pos[b];
        if (p < 0 || p >= cs_positions) { if (lane == 0) atomicExch(err, 51); p = 0; }      // a position outside the table: flagged, not read
        // lanes 0-7: a = dimensions 0..31 (mine), b = 32..63 (lane + 8); lanes 8-15 the other way round; lanes 16-31 are not rotated
        const float4 o = make_float4(__shfl_xor_sync(0xffffffffu, v.x, 8), __shfl_xor_sync(0xffffffffu, v.y, 8), __shfl_xor_sync(0xffffffffu, v.z, 8), __shfl_xor_sync(0xffffffffu, v.w, 8));
        if (lane < 16) {
            const float4 *t = reinterpret_cast<const float4 *>(cs + ((size_t)p * 32 + 4 * (lane & 7)) * 2);      // (cos, sin) of four pairs
            const float4 t0 = t[0], t1 = t[1];
            const float c[4] = {t0.x, t0.z, t1.x, t1.z}, s[4] = {t0.y, t0.w, t1.y, t1.w};
            const float mine[4] = {v.x, v.y, v.z, v.w}, other[4] = {o.x, o.y, o.z, o.w};
            float r[4];
#pragma unroll
            for (int e = 0; e < 4; e++)
                r[e] = lane < 8 ? __fmaf_rn(mine[e], c[e], -__fmul_rn(other[e], s[e])) : __fmaf_rn(mine[e], c[e], __fmul_rn(other[e], s[e]));
            v = make_float4(r[0], r[1], r[2], r[3]);
        }
    }
    if (h < AP_NH) reinterpret_cast<float4 *>(q + (size_t)b * (AP_NH * AP_HD) + h * AP_HD)[lane] = v;
    else {
        __half2 *o = reinterpret_cast<__half2 *>(kc + (size_t)b * (AP_NKV * AP_HD) + (h - AP_NH) * AP_HD) + 2 * lane;
        o[0] = __halves2half2(__float2half_rn(v.x), __float2half_rn(v.y)); o[1] = __halves2half2(__float2half_rn(v.z), __float2half_rn(v.w));
    }
}
extern "C" void k_qk_rope(cudaStream_t st, const float *qkv, const int *pos, int nb, int glob, const float *qn, const float *kn, const float *cs, int cs_positions,
                          float *q, void *kc, void *vc, int *err) {
    if (nb <= 0) return;
    const int items = nb * (AP_NH + 2 * AP_NKV);
    launch_k(qk_rope_kernel, (items + 7) / 8, 256, 0, st, qkv, pos, nb, glob, qn, kn, cs, cs_positions, q, (__half *)kc, (__half *)vc, err);
    k_count_add(1);
}
