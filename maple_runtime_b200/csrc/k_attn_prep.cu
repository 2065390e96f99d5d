// k_attn_prep.cu -- the first step of the attention half of a layer (maple.c:711-717; the reference's card kernel is `qkn`,
// gpu_full.metal:32-71): per token and head, RMS norm of the query and key heads (head dimension 128; maple.c:398-402 with the layer's
// q_norm / k_norm), half-rotary embedding at the token's position on local layers (maple.c:403-411: dimensions 0..63 as pairs (i, i + 32),
// cos and sin from the host's table, maple.c:1151-1153), queries out in fp32, keys and values out in fp16 (maple.c:314-320: round to
// nearest even).  Lane l of a warp holds dimensions 4l..4l+3 of a head; the rotation partner of lanes 0-7 sits in lanes 8-15.
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

// One warp per (token, group of four heads): groups 0-3 the query heads, 4 the key heads, 5 the value heads; the four rows of a group are
// loaded together, so that a lane has four 16-byte loads in flight.
__global__ void __launch_bounds__(256) qk_rope_kernel(const float *__restrict__ qkv, const int *__restrict__ pos, int nb, int glob,
                                                      const float *__restrict__ qn, const float *__restrict__ kn, const float *__restrict__ cs, int cs_positions,
                                                      float *__restrict__ q, __half *__restrict__ kc, __half *__restrict__ vc, int *err) {
    const int lane = threadIdx.x & 31, item = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int b = item / 6, grp = item % 6;
    if (b >= nb) return;
    const float4 *src = reinterpret_cast<const float4 *>(qkv + (size_t)b * ((AP_NH + 2 * AP_NKV) * AP_HD) + grp * 4 * AP_HD) + lane;
    float4 v[4];
#pragma unroll
    for (int i = 0; i < 4; i++) v[i] = src[i * (AP_HD / 4)];
    if (grp == 5) {      // the value heads: fp16 only
        __half2 *o = reinterpret_cast<__half2 *>(vc + (size_t)b * (AP_NKV * AP_HD)) + 2 * lane;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            o[i * (AP_HD / 2)] = __halves2half2(__float2half_rn(v[i].x), __float2half_rn(v[i].y)); o[i * (AP_HD / 2) + 1] = __halves2half2(__float2half_rn(v[i].z), __float2half_rn(v[i].w));
        }
        return;
    }
    const float4 w = reinterpret_cast<const float4 *>(grp < 4 ? qn : kn)[lane];
    float4 c4 = make_float4(0.f, 0.f, 0.f, 0.f), s4 = c4;
    if (!glob) {
        int p = pos[b];
        if (p < 0 || p >= cs_positions) { if (lane == 0) atomicExch(err, 51); p = 0; }      // a position outside the table: flagged, not read
        if (lane < 16) {
            const float4 *t = reinterpret_cast<const float4 *>(cs + ((size_t)p * 32 + 4 * (lane & 7)) * 2);      // (cos, sin) of four pairs
            const float4 t0 = t[0], t1 = t[1];
            c4 = make_float4(t0.x, t0.z, t1.x, t1.z); s4 = make_float4(t0.y, t0.w, t1.y, t1.w);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        float4 x = v[i];
        double ss = (double)x.x * (double)x.x + (double)x.y * (double)x.y + ((double)x.z * (double)x.z + (double)x.w * (double)x.w);
#pragma unroll
        for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float k = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn((float)(ss / (double)AP_HD), 1e-6f)));
        x.x = __fmul_rn(__fmul_rn(x.x, k), w.x); x.y = __fmul_rn(__fmul_rn(x.y, k), w.y); x.z = __fmul_rn(__fmul_rn(x.z, k), w.z); x.w = __fmul_rn(__fmul_rn(x.w, k), w.w);
        if (!glob) {
            // lanes 0-7: a = dimensions 0..31 (mine), b = 32..63 (lane + 8); lanes 8-15 the other way round; lanes 16-31 are not rotated
            const float4 o = make_float4(__shfl_xor_sync(0xffffffffu, x.x, 8), __shfl_xor_sync(0xffffffffu, x.y, 8), __shfl_xor_sync(0xffffffffu, x.z, 8), __shfl_xor_sync(0xffffffffu, x.w, 8));
            if (lane < 8) x = make_float4(__fmaf_rn(x.x, c4.x, -__fmul_rn(o.x, s4.x)), __fmaf_rn(x.y, c4.y, -__fmul_rn(o.y, s4.y)), __fmaf_rn(x.z, c4.z, -__fmul_rn(o.z, s4.z)), __fmaf_rn(x.w, c4.w, -__fmul_rn(o.w, s4.w)));
            else if (lane < 16) x = make_float4(__fmaf_rn(x.x, c4.x, __fmul_rn(o.x, s4.x)), __fmaf_rn(x.y, c4.y, __fmul_rn(o.y, s4.y)), __fmaf_rn(x.z, c4.z, __fmul_rn(o.z, s4.z)), __fmaf_rn(x.w, c4.w, __fmul_rn(o.w, s4.w)));
        }
        if (grp < 4) reinterpret_cast<float4 *>(q + (size_t)b * (AP_NH * AP_HD) + (grp * 4 + i) * AP_HD)[lane] = x;
        else {
            __half2 *o2 = reinterpret_cast<__half2 *>(kc + (size_t)b * (AP_NKV * AP_HD) + i * AP_HD) + 2 * lane;
            o2[0] = __halves2half2(__float2half_rn(x.x), __float2half_rn(x.y)); o2[1] = __halves2half2(__float2half_rn(x.z), __float2half_rn(x.w));
        }
    }
}
extern "C" void k_qk_rope(cudaStream_t st, const float *qkv, const int *pos, int nb, int glob, const float *qn, const float *kn, const float *cs, int cs_positions,
                          float *q, void *kc, void *vc, int *err) {
    if (nb <= 0) return;
    const int items = nb * 6;
    launch_k(qk_rope_kernel, (items + 7) / 8, 256, 0, st, qkv, pos, nb, glob, qn, kn, cs, cs_positions, q, (__half *)kc, (__half *)vc, err);
    k_count_add(1);
}
