// k_router_umma.cu -- router logits on the tensor cores for prefill-sized batches (maple.c:870-889 computes them with AVX2
// multiply-adds), plus the selection that makes the result safe to use: sm_100a, tcgen05.mma kind::f16.
//
// logit[b][e] = sum_c W[e][c] hn[b][c], W bf16, hn fp32.  The tensor cores take fp16 operands with fp32 accumulation, so
//   * hn is split into two fp16 terms, hi = fp16(hn), lo = fp16(hn - hi) (the norm kernel writes them, k_route.cu): 22 bits of hn;
//   * W goes to fp16 once per layer: exact for every bf16 value of magnitude >= 2^-17, below that to within 2^-25;
//   * a CTA owns 128 tokens x 256 experts x one eighth of the columns (K = 2 x 256 fp16 values): 32 MMAs of 128 x 256 x 16 into one
//     accumulator of 256 tensor-memory columns.  Short accumulation chains keep the accumulator's own rounding small; the eight
//     partial sums of a token are added in a fixed order by the selection kernel.
// The logits differ from the reference's (its particular order of fp32 roundings) by a few 1e-7 of |W||hn|.  The reference's
// top-8 is reproduced all the same:
//   * router_select_kernel (one warp per token) takes the nine largest logits; if every gap between consecutive ones exceeds
//     ROUTER_GAP * |hn_b| * max_e |W_e| (a bound on both computations' error, with margin), the order of the top nine is the order the
//     reference finds, the eight indices are final and the weights are exp(l_k - l_1) / sum over the eight (equal to the reference's
//     p_k / (sum p + 1e-20) up to rounding: the softmax denominator cancels);
//   * otherwise the token is flagged: router_fix_kernel recomputes its 256 logits in the reference's exact order (eight strided
//     multiply-add chains, then the pairwise adds of maple.c:117-121) and redoes its selection with the exact softmax + top-8
//     (topk.cuh).  Ties, near-ties and all-equal rows therefore take the reference's path bit for bit.
// Indices are the reference's for every token; weights of unflagged tokens agree to ~1e-6 relative.
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include "kernels.h"
#include "launch.cuh"
#include "umma.cuh"
#include "topk.cuh"

extern "C" void k_count_add(long n);

#define HID 2048
#define NEXP 256
#define TOPK 8
#define RU_KS 8                          /* column splits */
#define RU_KCOLS (HID / RU_KS)           /* 256 columns of hn per CTA */
#define RU_KBLK (RU_KCOLS / 64)          /* 4 blocks of 64 columns (128 bytes of fp16) */
#define RU_STAGES 3
#define RU_ABYTES (128 * 128)            /* 128 tokens x 64 fp16 */
#define RU_BBYTES (256 * 128)            /* 256 experts x 64 fp16 */
#define RU_STAGE_BYTES (2 * RU_ABYTES + RU_BBYTES)
#define ROUTER_GAP 3.814697265625e-6f     /* 2^-18: the difference between the two computations stayed below 2^-23 |hn| max|W_e| over a million tokens */

// kind::f16: D fp32, A and B fp16, both K-major, M = 128, N = n
__device__ __forceinline__ uint32_t idesc_f16(uint32_t n) { return (1u << 4) | ((n >> 3) << 17) | ((128u >> 4) << 24); }
__device__ __forceinline__ void umma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// router rows bf16 [256][2048] -> fp16 [256][2048]; wnorm[0] = max over experts of the row's Euclidean norm (float bits, atomicMax)
__global__ void __launch_bounds__(256) router_w16_kernel(const uint16_t *__restrict__ W, __half *__restrict__ W16, float *__restrict__ wnorm) {
    __shared__ float sn[8];
    const int e = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const uint4 v = reinterpret_cast<const uint4 *>(W + (size_t)e * HID)[tid];
    const uint32_t ww[4] = {v.x, v.y, v.z, v.w};
    __align__(16) __half o[8]; float n2 = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float f = __uint_as_float((i & 1) ? (ww[i >> 1] & 0xFFFF0000u) : (ww[i >> 1] << 16));
        o[i] = __float2half_rn(f); n2 = fmaf(f, f, n2);
    }
    reinterpret_cast<uint4 *>(W16 + (size_t)e * HID)[tid] = *reinterpret_cast<const uint4 *>(o);
#pragma unroll
    for (int s = 16; s; s >>= 1) n2 += __shfl_xor_sync(0xffffffffu, n2, s);
    if (lane == 0) sn[wid] = n2;
    __syncthreads();
    if (tid == 0) {
        float t = 0.0f;
        for (int i = 0; i < 8; i++) t += sn[i];
        atomicMax(reinterpret_cast<int *>(wnorm), __float_as_int(sqrtf(t)));      // norms are >= 0: their bit patterns order like the values
    }
}
extern "C" void k_router_w16(cudaStream_t st, const uint16_t *router, void *w16, float *wnorm) {
    cudaMemsetAsync(wnorm, 0, 4, st);
    router_w16_kernel<<<NEXP, 256, 0, st>>>(router, (__half *)w16, wnorm);
    k_count_add(1);
}

struct RuBars { uint64_t full[RU_STAGES], empty[RU_STAGES], acc; uint32_t tmem_base; int abort_flag; };

// grid (RU_KS, token tiles of 128).  Warp 0: TMA (one lane), warp 1: tensor-memory allocation and MMA issue, warps 2-5: epilogue.
// part [RU_KS][ntok_cap][256] fp32 receives the partial sums.
__global__ void __launch_bounds__(192, 1) router_umma_kernel(const __grid_constant__ TMap amap, const __grid_constant__ TMap wmap,
                                                             float *__restrict__ part, int nb, int ntok_cap, int *err, int *__restrict__ nflagged,
                                                             unsigned *__restrict__ mask, int mask_n) {
    extern __shared__ __align__(1024) uint8_t ru_raw[];
    uint8_t *ring = (uint8_t *)(((uintptr_t)ru_raw + 1023) & ~(uintptr_t)1023);
    __shared__ RuBars sh;
    const int tid = threadIdx.x, lane = tid & 31, warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int ks = blockIdx.x, tile = blockIdx.y;
    volatile int *abortp = &sh.abort_flag;
    if (tid == 0) {
        for (int s = 0; s < RU_STAGES; s++) { mbar_init(&sh.full[s], 1); mbar_init(&sh.empty[s], 1); }
        mbar_init(&sh.acc, 1); sh.abort_flag = 0; mbar_init_fence();
    }
    if (warp == 1) tmem_alloc(&sh.tmem_base, 256);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tb = sh.tmem_base;
    if (tid == 0 && blockIdx.x == 0 && blockIdx.y == 0) *nflagged = 0;      // the selection kernel counts its flagged tokens from zero
    if (mask) {     // and sets the grouping's bits and counters: cleared here, one word per thread
        const int w = (blockIdx.y * gridDim.x + blockIdx.x) * 192 + tid;
        for (int i = w; i < mask_n; i += gridDim.x * gridDim.y * 192) mask[i] = 0u;
    }
    if (warp == 0) {
        if (lane == 0) {
            for (int kb = 0; kb < RU_KBLK; kb++) {
                const int s = kb % RU_STAGES;
                if (!mbar_wait(&sh.empty[s], ((kb / RU_STAGES) & 1) ^ 1, abortp)) break;
                const uint32_t dst = smem_u32(ring + s * RU_STAGE_BYTES);
                const int col = ks * RU_KCOLS + kb * 64;
                mbar_expect_tx(&sh.full[s], RU_STAGE_BYTES);
                tma_load_2d(dst, &amap, col, tile * 128, &sh.full[s]);                       // hi terms of 128 tokens
                tma_load_2d(dst + RU_ABYTES, &amap, HID + col, tile * 128, &sh.full[s]);      // lo terms
                tma_load_2d(dst + 2 * RU_ABYTES, &wmap, col, 0, &sh.full[s]);                 // 256 experts
            }
        }
    } else if (warp == 1) {
        const uint32_t idesc = idesc_f16(NEXP);
        const uint32_t ring0 = __shfl_sync(0xffffffffu, smem_u32(ring), 0);
        bool live = true;
#pragma unroll 1
        for (int kb = 0; kb < RU_KBLK && live; kb++) {
            const int s = kb % RU_STAGES;
            if (!mbar_wait(&sh.full[s], (kb / RU_STAGES) & 1, abortp)) { live = false; break; }
            tc_fence_after();
            const uint64_t ahi = smem_desc_k128(ring0 + s * RU_STAGE_BYTES, 0), alo = smem_desc_k128(ring0 + s * RU_STAGE_BYTES + RU_ABYTES, 0);
            const uint64_t bd = smem_desc_k128(ring0 + s * RU_STAGE_BYTES + 2 * RU_ABYTES, 0);
#pragma unroll
            for (int k = 0; k < 4; k++) {       // 16 fp16 values = 32 bytes per MMA
                if (elect_one()) umma_f16_ss(tb, ahi + 2 * k, bd + 2 * k, idesc, (kb | k) != 0);
                if (elect_one()) umma_f16_ss(tb, alo + 2 * k, bd + 2 * k, idesc, 1);
            }
            if (elect_one()) umma_commit(&sh.empty[s]);
        }
        if (live && elect_one()) umma_commit(&sh.acc);
        __syncwarp();
    } else {
        // a warp reaches the tensor-memory lanes 32 (warp % 4) ..: lane = token of the tile, columns = experts
        const int q4 = warp & 3, tok = tile * 128 + q4 * 32 + lane;
        if (mbar_wait(&sh.acc, 0, abortp)) {
            tc_fence_after();
            float *dst = part + ((size_t)ks * ntok_cap + tok) * NEXP;
#pragma unroll 1
            for (int c = 0; c < NEXP; c += 32) {
                uint32_t v[32];
                tmem_ld32(tb + ((uint32_t)(q4 * 32) << 16) + c, v);
                tmem_ld_wait();
                if (tok < nb) {
#pragma unroll
                    for (int j = 0; j < 32; j += 4) *reinterpret_cast<uint4 *>(dst + c + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tb, 256);
        if (lane == 0 && sh.abort_flag) atomicExch(err, 31);
    }
}

// one warp per token: lane l holds experts 8l..8l+7.  Adds the eight partial sums (fixed order) and the bias, stores the logits, takes the
// nine largest (lowest index first among equals), decides whether their order is safe, and writes top-8 / weights or flags the token.
__global__ void __launch_bounds__(256) router_select_kernel(const float *__restrict__ part, int ntok_cap, const float *__restrict__ bias,
                                                            const float *__restrict__ hnorm, const float *__restrict__ wnorm,
                                                            float *__restrict__ logits, int *__restrict__ top, float *__restrict__ topw,
                                                            int *__restrict__ flagged, int *__restrict__ nflagged, const uint8_t *__restrict__ router_s,
                                                            unsigned *__restrict__ mask, int mask_words, int nb) {
    {   // the flagged tokens' recomputation reads the layer's re-laid router rows (1 MB) right after this kernel: pull them into L2 now
        const unsigned line = blockIdx.x * 256u + threadIdx.x;
        if (line < NEXP * HID * 2 / 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(router_s + (size_t)line * 128));
    }
    const int lane = threadIdx.x & 31, b = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (b >= nb) return;
    float l[8];
    {
        float4 p[RU_KS][2];
#pragma unroll
        for (int s = 0; s < RU_KS; s++) {
            const float4 *r = reinterpret_cast<const float4 *>(part + ((size_t)s * ntok_cap + b) * NEXP + lane * 8);
            p[s][0] = r[0]; p[s][1] = r[1];
        }
#pragma unroll
        for (int h = 0; h < 2; h++) {
            float4 a01, a23, a45, a67;
            a01.x = p[0][h].x + p[1][h].x; a01.y = p[0][h].y + p[1][h].y; a01.z = p[0][h].z + p[1][h].z; a01.w = p[0][h].w + p[1][h].w;
            a23.x = p[2][h].x + p[3][h].x; a23.y = p[2][h].y + p[3][h].y; a23.z = p[2][h].z + p[3][h].z; a23.w = p[2][h].w + p[3][h].w;
            a45.x = p[4][h].x + p[5][h].x; a45.y = p[4][h].y + p[5][h].y; a45.z = p[4][h].z + p[5][h].z; a45.w = p[4][h].w + p[5][h].w;
            a67.x = p[6][h].x + p[7][h].x; a67.y = p[6][h].y + p[7][h].y; a67.z = p[6][h].z + p[7][h].z; a67.w = p[6][h].w + p[7][h].w;
            l[4 * h + 0] = (a01.x + a23.x) + (a45.x + a67.x); l[4 * h + 1] = (a01.y + a23.y) + (a45.y + a67.y);
            l[4 * h + 2] = (a01.z + a23.z) + (a45.z + a67.z); l[4 * h + 3] = (a01.w + a23.w) + (a45.w + a67.w);
        }
    }
    if (bias) {
        const float4 b0 = reinterpret_cast<const float4 *>(bias + lane * 8)[0], b1 = reinterpret_cast<const float4 *>(bias + lane * 8)[1];
        l[0] += b0.x; l[1] += b0.y; l[2] += b0.z; l[3] += b0.w; l[4] += b1.x; l[5] += b1.y; l[6] += b1.z; l[7] += b1.w;
    }
    {
        float4 *o = reinterpret_cast<float4 *>(logits + (size_t)b * NEXP + lane * 8);
        o[0] = make_float4(l[0], l[1], l[2], l[3]); o[1] = make_float4(l[4], l[5], l[6], l[7]);
    }
    // order-preserving keys: larger float <-> larger unsigned; 0 marks a taken entry (no finite float maps to 0)
    unsigned key[8];
#pragma unroll
    for (int i = 0; i < 8; i++) { const unsigned u = __float_as_uint(l[i]); key[i] = (u & 0x80000000u) ? ~u : (u | 0x80000000u); if (key[i] == 0u) key[i] = 1u; }
    float sel = 0.0f, gapmin = 3.0e38f, prev = 0.0f; int isel = 0;
#pragma unroll 1
    for (int k = 0; k < TOPK + 1; k++) {
        unsigned lk = key[0];
#pragma unroll
        for (int i = 1; i < 8; i++) lk = max(lk, key[i]);
        const unsigned m = __reduce_max_sync(0xffffffffu, lk);
        const int src = __ffs(__ballot_sync(0xffffffffu, lk == m)) - 1;
        int bi = 7;
#pragma unroll
        for (int i = 6; i >= 0; i--) if (key[i] == m) bi = i;
        const int be = __shfl_sync(0xffffffffu, lane * 8 + bi, src);
#pragma unroll
        for (int i = 0; i < 8; i++) if (lane == src && i == bi) key[i] = 0u;
        const float bv = __uint_as_float((m & 0x80000000u) ? (m & 0x7FFFFFFFu) : ~m);
        if (k > 0) gapmin = fminf(gapmin, prev - bv);
        prev = bv;
        if (lane == k) { sel = bv; isel = be; }
    }
    const float lmax = __shfl_sync(0xffffffffu, sel, 0);
    const float bound = ROUTER_GAP * hnorm[b] * wnorm[0];
    if (!(gapmin > bound)) {                                  // also catches NaN
        if (lane == 0) flagged[atomicAdd(nflagged, 1)] = b;
        return;
    }
    // weights in selection order: e_k / (sum_k e_k + 1e-20), e_k = exp(l_k - l_1)
    const float ek = lane < TOPK ? expf(sel - lmax) : 0.0f;
    float tsum = 0.0f;
#pragma unroll
    for (int k = 0; k < TOPK; k++) tsum += __shfl_sync(0xffffffffu, ek, k);
    if (lane < TOPK) {
        top[b * TOPK + lane] = isel; topw[b * TOPK + lane] = ek / (tsum + 1e-20f);
        if (mask) { atomicOr(&mask[(size_t)(b >> 5) * NEXP + isel], 1u << (b & 31)); atomicAdd(&mask[(size_t)NEXP * mask_words + isel], 1u); }
    }
}

// The flagged tokens over again as the reference computes them (maple.c:870-889, 117-121, 910-923).  grid (8 expert eighths, y): CTA
// (x, y) walks flagged tokens y, y + gridDim.y, ... and computes 32 experts of each: 256 threads = 8 lanes x 32 experts, the eight strided
// multiply-add chains per expert and their pairwise adds.  The last of a token's eight CTAs to finish (a counter per flagged slot, reset
// by that CTA) runs the exact softmax + top-8 on the token's finished row.
// WS: the router rows re-laid as [expert][column / 32][lane j][4 steps] bf16 (k_router_pack_small, k_router_tile.cu).
__global__ void __launch_bounds__(256) router_fix_kernel(const uint8_t *__restrict__ WS, const float *__restrict__ hn, const float *__restrict__ bias,
                                                         float *__restrict__ logits, int *__restrict__ top, float *__restrict__ topw,
                                                         const int *__restrict__ flagged, const int *__restrict__ nflagged, int *__restrict__ done,
                                                         unsigned *__restrict__ mask, int mask_words, int nb) {
    __shared__ __align__(16) float hrow[HID];
    __shared__ unsigned long long tab[32];
    __shared__ int s_last;
    const int tid = threadIdx.x, j = tid & 7, pos = tid >> 3, lane = tid & 31;
    if (tid < 32) tab[tid] = DEV_EXP_TAB[tid];
    const int total = min(*nflagged, nb);
    for (int f = blockIdx.y; f < total; f += gridDim.y) {
        const int b = flagged[f];
        __syncthreads();
        for (int i = tid; i < HID / 4; i += 256) reinterpret_cast<float4 *>(hrow)[i] = reinterpret_cast<const float4 *>(hn + (size_t)b * HID)[i];
        __syncthreads();
        const int e = blockIdx.x * 32 + pos;
        const uint8_t *wp = WS + (size_t)e * (HID * 2) + j * 8;
        float acc = 0.0f;
#pragma unroll 16
        for (int i4 = 0; i4 < 64; i4++) {
            const uint2 a = *reinterpret_cast<const uint2 *>(wp + i4 * 64);
            acc = __fmaf_rn(__uint_as_float(a.x << 16), hrow[32 * i4 + j], acc);
            acc = __fmaf_rn(__uint_as_float(a.x & 0xFFFF0000u), hrow[32 * i4 + 8 + j], acc);
            acc = __fmaf_rn(__uint_as_float(a.y << 16), hrow[32 * i4 + 16 + j], acc);
            acc = __fmaf_rn(__uint_as_float(a.y & 0xFFFF0000u), hrow[32 * i4 + 24 + j], acc);
        }
        float l = acc;      // (l0+l4)+(l1+l5) then +((l2+l6)+(l3+l7)): the same on every lane of the expert
        l = __fadd_rn(l, __shfl_xor_sync(0xffffffffu, l, 4));
        l = __fadd_rn(l, __shfl_xor_sync(0xffffffffu, l, 1));
        l = __fadd_rn(l, __shfl_xor_sync(0xffffffffu, l, 2));
        if (j == 0) logits[(size_t)b * NEXP + e] = bias ? __fadd_rn(l, bias[e]) : l;
        __threadfence();
        __syncthreads();
        if (tid == 0) s_last = atomicAdd(&done[f], 1) == (int)gridDim.x - 1;
        __syncthreads();
        if (s_last && tid < 32) {
            __threadfence();
            const float4 *lr = reinterpret_cast<const float4 *>(logits + (size_t)b * NEXP + lane * 8);
            const float4 v0 = __ldcg(lr), v1 = __ldcg(lr + 1);              // the other CTAs' values: read past L1
            float p[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
            int isel; float wsel, tsum;
            exact_topk_warp(p, lane, tab, isel, wsel, tsum);
            if (lane < TOPK) {
                top[b * TOPK + lane] = isel; topw[b * TOPK + lane] = __fdiv_rn(wsel, __fadd_rn(tsum, 1e-20f));
                if (mask) { atomicOr(&mask[(size_t)(b >> 5) * NEXP + isel], 1u << (b & 31)); atomicAdd(&mask[(size_t)NEXP * mask_words + isel], 1u); }
            }
            if (lane == 0) done[f] = 0;
        }
    }
}

extern "C" void k_router_tensor(cudaStream_t st, const RouterTensorArgs *r) {
    if (r->nb <= 0) return;
    static bool attr_done = false;
    const int smem = RU_STAGES * RU_STAGE_BYTES + 1024;
    if (!attr_done) { cudaFuncSetAttribute(router_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); attr_done = true; }
    launch_k(router_umma_kernel, dim3(RU_KS, (r->nb + 127) / 128), 192, smem, st, r->amap, r->wmap, r->part, r->nb, r->ntok_cap, r->err, r->nflagged, r->mask, NEXP * r->mask_words + NEXP);
    launch_k(router_select_kernel, (r->nb + 7) / 8, 256, 0, st, r->part, r->ntok_cap, r->bias, r->hnorm, r->wnorm, r->logits, r->top, r->topw, r->flagged, r->nflagged, (const uint8_t *)r->router_s, r->mask, r->mask_words, r->nb);
    launch_k(router_fix_kernel, dim3(8, 74), 256, 0, st, (const uint8_t *)r->router_s, r->hn, r->bias, r->logits, r->top, r->topw, r->flagged, r->nflagged, r->done, r->mask, r->mask_words, r->nb);
    k_count_add(3);
}
