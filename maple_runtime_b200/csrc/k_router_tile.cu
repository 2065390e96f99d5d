// k_router_tile.cu -- router logits for prefill-sized batches (maple.c:870-889 job_route_multi), sm_100a.
//
// logit[b][e] = hsum over eight lanes of ( sum_i W[e][8i+l] * hn[b][8i+l] ), each lane one chain of fused multiply-adds in
// increasing i, the lanes added as ((l0+l4)+(l1+l5))+((l2+l6)+(l3+l7)) (maple.c:117-121): the same bits as the CPU path.
//
// A CTA owns up to 32 tokens x 128 experts.  Eight warps hold 8 lanes x 32 positions; a position is an
// 8-token (fewer when that fills the SMs better) x 16-expert register tile, so one step of a lane costs 64 bytes of shared-memory reads (eight fp32 hidden values,
// sixteen bf16 weights) for 128 multiply-adds: half a byte per multiply-add, half of what the load path delivers at the full
// multiply-add rate.  The multiply-adds are issued two at a time (fma.rn.f32x2, each half an IEEE fused multiply-add).
// Both operands come from copies laid out for exactly this access: per 128-column chunk and 8-token (16-expert) group,
// [step i][half h][lane j][4 tokens fp32 | 8 experts bf16], so that the eight lanes of a position read 128 consecutive bytes and a
// chunk of a CTA's operands is one contiguous block.  Thread 0 streams those blocks through a four-stage ring with
// cp.async.bulk and mbarriers; every wait is bounded.
#include <cuda_runtime.h>
#include <stdint.h>
#include "kernels.h"
#include "launch.cuh"
#include "umma.cuh"

#define HID 2048
#define NEXP 256
#define RP_TOK 32
#define RP_EXP 128
#define RP_KI 16                          /* steps of 8 columns per chunk */
#define RP_NCH (HID / 8 / RP_KI)          /* 16 chunks */
#define RP_GRP (RP_KI * 256)              /* bytes of one group (8 tokens or 16 experts) in one chunk */
#define RP_HB ((RP_TOK / 8) * RP_GRP)     /* 16 KB */
#define RP_WB ((RP_EXP / 16) * RP_GRP)    /* 32 KB */
#define RP_STAGES 4
#define RP_SMEM (RP_STAGES * (RP_HB + RP_WB))

extern "C" void k_count_add(long n);

// router rows (bf16 [256][2048]) -> [expert block of 128][chunk][group of 16][i][h][j][8 experts]; once per layer
__global__ void __launch_bounds__(256) router_pack_w_kernel(const uint16_t *__restrict__ W, uint4 *__restrict__ WT) {
    const int o = blockIdx.x * 256 + threadIdx.x;
    const int j = o & 7, h = (o >> 3) & 1, i = (o >> 4) & 15, eg = (o >> 8) & 7, ch = (o >> 11) & 15, eb = o >> 15;
    const int e = eb * RP_EXP + eg * 16 + h * 8, col = (ch * RP_KI + i) * 8 + j;
    uint32_t v[4];
#pragma unroll
    for (int m = 0; m < 4; m++)
        v[m] = (uint32_t)W[(size_t)(e + 2 * m) * HID + col] | ((uint32_t)W[(size_t)(e + 2 * m + 1) * HID + col] << 16);
    WT[o] = make_uint4(v[0], v[1], v[2], v[3]);
}
// normalised hidden rows (fp32 [nb][2048]) -> [tile of 4*tt tokens][chunk][group of tt tokens in 8 slots][i][h][j][4 slots];
// slots past tt and rows past nb read as zero
__global__ void __launch_bounds__(256) router_pack_h_kernel(const float *__restrict__ hn, float4 *__restrict__ hT, int nb, int tt) {
    const int o = blockIdx.x * 256 + threadIdx.x;
    const int j = o & 7, h = (o >> 3) & 1, i = (o >> 4) & 15, tg = (o >> 8) & 3, ch = (o >> 10) & 15, tile = o >> 14;
    const int t0 = tile * 4 * tt + tg * tt, col = (ch * RP_KI + i) * 8 + j;
    float v[4];
#pragma unroll
    for (int m = 0; m < 4; m++) v[m] = (h * 4 + m < tt && t0 + h * 4 + m < nb) ? hn[(size_t)(t0 + h * 4 + m) * HID + col] : 0.0f;
    hT[o] = make_float4(v[0], v[1], v[2], v[3]);
}

__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ uint64_t pair64(uint32_t lo, uint32_t hi) {
    uint64_t r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi)); return r;
}
__device__ __forceinline__ void fma2(uint64_t &acc, uint64_t a, uint64_t b) {
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(b));
}

struct RpBars { uint64_t full[RP_STAGES], empty[RP_STAGES]; int abort; };

template <int TT>
__global__ void __maxnreg__(224) router_tile_kernel(const uint8_t *__restrict__ WT, const uint8_t *__restrict__ hT,
                                                            const float *__restrict__ bias, float *__restrict__ logits, int nb, int *err) {
    extern __shared__ __align__(128) uint8_t rp_ring[];
    __shared__ RpBars sh;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile = blockIdx.y, eb = blockIdx.x;
    if (tid == 0) {
        for (int s = 0; s < RP_STAGES; s++) { mbar_init(&sh.full[s], 1); mbar_init(&sh.empty[s], 8); }
        sh.abort = 0;
        mbar_init_fence();
    }
    __syncthreads();
    volatile int *abortp = &sh.abort;
    {
        // thread 0 is also the producer: it fills the ring before the arithmetic starts and, at the top of every chunk, refills
        // the stage that all eight warps released one chunk earlier
        const uint8_t *hsrc = hT + (size_t)tile * RP_NCH * RP_HB, *wsrc = WT + (size_t)eb * RP_NCH * RP_WB;
        auto issue = [&](int ch) {
            const int s = ch % RP_STAGES;
            const uint32_t dst = smem_u32(rp_ring) + s * (RP_HB + RP_WB);
            mbar_expect_tx(&sh.full[s], RP_HB + RP_WB);
            bulk_load(dst, hsrc + (size_t)ch * RP_HB, RP_HB, &sh.full[s]);
            bulk_load(dst + RP_HB, wsrc + (size_t)ch * RP_WB, RP_WB, &sh.full[s]);
        };
        if (tid == 0) for (int ch = 0; ch < RP_STAGES - 1; ch++) issue(ch);
        const int j = tid & 7, tg = (tid >> 3) & 3, eg = warp;      // the four positions of a warp share their sixteen experts
        uint64_t acc[TT][8];                                          // [token][expert pair], halves = experts 2m, 2m+1
#pragma unroll
        for (int a = 0; a < TT; a++)
#pragma unroll
            for (int m = 0; m < 8; m++) acc[a][m] = 0ull;
        bool live = true;
        for (int ch = 0; ch < RP_NCH && live; ch++) {
            const int s = ch % RP_STAGES, n = ch / RP_STAGES;
            if (tid == 0 && ch + RP_STAGES - 1 < RP_NCH) {
                // a wait that ran out has raised the abort flag: nothing is issued and every warp leaves at its next wait
                if (ch == 0 || mbar_wait(&sh.empty[(ch - 1) % RP_STAGES], ((ch - 1) / RP_STAGES) & 1, abortp)) issue(ch + RP_STAGES - 1);
            }
            if (!mbar_wait(&sh.full[s], n & 1, abortp)) { live = false; break; }
            const uint8_t *hp = rp_ring + s * (RP_HB + RP_WB) + tg * RP_GRP + j * 16;
            const uint8_t *wp = rp_ring + s * (RP_HB + RP_WB) + RP_HB + eg * RP_GRP + j * 16;
#pragma unroll 4
            for (int i = 0; i < RP_KI; i++) {
                const float4 h0 = *reinterpret_cast<const float4 *>(hp + i * 256), h1 = *reinterpret_cast<const float4 *>(hp + i * 256 + 128);
                const uint4 w0 = *reinterpret_cast<const uint4 *>(wp + i * 256), w1 = *reinterpret_cast<const uint4 *>(wp + i * 256 + 128);
                const uint32_t wu[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
                const float hv[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
                uint64_t wv[8], hh[8];
#pragma unroll
                for (int m = 0; m < 8; m++) wv[m] = pair64(wu[m] << 16, wu[m] & 0xFFFF0000u);
#pragma unroll
                for (int a = 0; a < TT; a++) hh[a] = pair64(__float_as_uint(hv[a]), __float_as_uint(hv[a]));
#pragma unroll
                for (int a = 0; a < TT; a++)
#pragma unroll
                    for (int m = 0; m < 8; m++) fma2(acc[a][m], wv[m], hh[a]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh.empty[s]);
        }
        if (live) {
            // every lane ends with the full sums (the additions commute pairwise); lane j stores token j's sixteen logits
            const int e0 = eb * RP_EXP + eg * 16, b0 = tile * 4 * TT + tg * TT;
            float bv[16];
#pragma unroll
            for (int c = 0; c < 16; c++) bv[c] = bias ? bias[e0 + c] : 0.0f;
#pragma unroll
            for (int a = 0; a < TT; a++) {
                float l[16];
#pragma unroll
                for (int m = 0; m < 8; m++) { l[2 * m] = __uint_as_float((uint32_t)acc[a][m]); l[2 * m + 1] = __uint_as_float((uint32_t)(acc[a][m] >> 32)); }
#pragma unroll
                for (int c = 0; c < 16; c++) {
                    float v = l[c];
                    v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 4));
                    v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 1));
                    v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 2));
                    l[c] = bias ? __fadd_rn(v, bv[c]) : v;
                }
                if (a == j && b0 + a < nb) {
                    float4 *dst = reinterpret_cast<float4 *>(logits + (size_t)(b0 + a) * NEXP + e0);
                    dst[0] = make_float4(l[0], l[1], l[2], l[3]); dst[1] = make_float4(l[4], l[5], l[6], l[7]);
                    dst[2] = make_float4(l[8], l[9], l[10], l[11]); dst[3] = make_float4(l[12], l[13], l[14], l[15]);
                }
            }
        }
    }
    __syncthreads();
    if (tid == 0 && sh.abort) atomicExch(err, 31);      // a wait ran out: the host reports it and the logits are not to be used
}

extern "C" void k_router_pack(cudaStream_t st, const uint16_t *router, void *router_t) {
    router_pack_w_kernel<<<NEXP * HID / 8 / 256, 256, 0, st>>>(router, (uint4 *)router_t);
    k_count_add(1);
}
static int g_force_tt = 0;
// pins the tokens per thread (4..8; 0 = choose by batch size); include/gmoe.h
extern "C" void gmoe_router_tile_tokens(int tt) { g_force_tt = (tt >= 4 && tt <= 8) ? tt : 0; }
template <int TT>
static void launch_tile(cudaStream_t st, const void *router_t, const float *hn, void *hT, const float *bias, float *logits, int nb, int *err) {
    static bool attr_done = false;
    if (!attr_done) { cudaFuncSetAttribute(router_tile_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, RP_SMEM); attr_done = true; }
    const int tiles = (nb + 4 * TT - 1) / (4 * TT);
    launch_k(router_pack_h_kernel, tiles * 64, 256, 0, st, hn, (float4 *)hT, nb, TT);
    launch_k(router_tile_kernel<TT>, dim3(NEXP / RP_EXP, tiles), 256, RP_SMEM, st, (const uint8_t *)router_t, (const uint8_t *)hT, bias, logits, nb, err);
}
// A thread's tile is tt tokens x 16 experts, a CTA's 4*tt tokens x 128 experts; tt in 4..8 is chosen so that the CTAs fill whole
// waves of the SMs with the least arithmetic per wave (2048 tokens: tt = 7, 148 CTAs).  hT must hold ceil(nb/16) * 256 KB.
extern "C" void k_router_logits_tile(cudaStream_t st, const void *router_t, const float *hn, void *hT, const float *bias, float *logits, int nb, int *err) {
    if (nb <= 0) return;
    static int sms = 0;
    if (!sms) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); if (sms < 1) sms = 148; }
    int best = 8; long cost = -1;
    for (int tt = 8; tt >= 4 && !g_force_tt; tt--) {
        const long ctas = 2L * ((nb + 4 * tt - 1) / (4 * tt)), c = ((ctas + sms - 1) / sms) * (tt * 8 + 5);   /* 5: the per-step cost that does not shrink with tt */
        if (cost < 0 || c < cost) { cost = c; best = tt; }
    }
    if (g_force_tt) best = g_force_tt;
    switch (best) {
    case 4: launch_tile<4>(st, router_t, hn, hT, bias, logits, nb, err); break;
    case 5: launch_tile<5>(st, router_t, hn, hT, bias, logits, nb, err); break;
    case 6: launch_tile<6>(st, router_t, hn, hT, bias, logits, nb, err); break;
    case 7: launch_tile<7>(st, router_t, hn, hT, bias, logits, nb, err); break;
    default: launch_tile<8>(st, router_t, hn, hT, bias, logits, nb, err); break;
    }
    k_count_add(2);
}

// ---------------------------------------------------------------------------------------------------------------------
// Decode batches (up to 256 tokens).  The arithmetic is a handful of microseconds of dependent multiply-adds (256 per chain), so
// the kernel is about latency: a CTA owns 8 tokens x 8 experts, fetches all 2048 columns of both in two bulk copies (64 KB of
// hidden values, 32 KB of bf16 weights, both pre-laid as [column / 32][lane j][4 steps] so that the eight lanes of a position
// read consecutive 16-byte (8-byte) pieces), waits once, and runs the 64 x 4 steps without another synchronisation.  Two CTAs
// share an SM, so the 256 CTAs of a 64-token batch are one wave.  256 threads = 8 lanes x 32 positions (8 tokens x 4 expert pairs).
// ---------------------------------------------------------------------------------------------------------------------
#define RS_TOK 8
#define RS_EXP 8
#define RS_HB (RS_TOK * HID * 4)
#define RS_WB (RS_EXP * HID * 2)
// router rows (bf16 [256][2048]) -> [expert][i4 = column / 32][lane j][4 steps]; once per layer
__global__ void __launch_bounds__(256) router_pack_w_small_kernel(const uint16_t *__restrict__ W, uint2 *__restrict__ WS) {
    const int o = blockIdx.x * 256 + threadIdx.x, j = o & 7, i4 = (o >> 3) & 63, e = o >> 9;
    uint16_t v[4];
#pragma unroll
    for (int k = 0; k < 4; k++) v[k] = W[(size_t)e * HID + (4 * i4 + k) * 8 + j];
    WS[o] = make_uint2((uint32_t)v[0] | ((uint32_t)v[1] << 16), (uint32_t)v[2] | ((uint32_t)v[3] << 16));
}
// hidden rows (fp32 [nb][2048]) -> [token][i4][lane j][4 steps]
__global__ void __launch_bounds__(256) router_pack_h_small_kernel(const float *__restrict__ hn, float4 *__restrict__ hS, int nb) {
    const int o = blockIdx.x * 256 + threadIdx.x, j = o & 7, i4 = (o >> 3) & 63, b = o >> 9;
    if (b >= nb) return;
    const float *r = hn + (size_t)b * HID + 32 * i4 + j;
    hS[o] = make_float4(r[0], r[8], r[16], r[24]);
}
// STEP: the order of the reference's single-token decode (bf_row, maple.c:146-157, called at maple.c:609): per lane two chains, one over
// columns 16m + j and one over 16m + 8 + j, added before the lanes are; otherwise one chain per lane (job_route_small/multi).
template <bool STEP>
__global__ void __launch_bounds__(256, 2) router_small_kernel(const uint8_t *__restrict__ WS, const uint8_t *__restrict__ hS, const float *__restrict__ bias,
                                                             float *__restrict__ logits, int nb, int *err) {
    extern __shared__ __align__(128) uint8_t rs_sm[];                  // hidden 64 KB, then weights 32 KB
    __shared__ uint64_t bar; __shared__ int abort_flag;
    const int tid = threadIdx.x, j = tid & 7, pos = tid >> 3, tok = pos & 7, ep = pos >> 3;
    const int b0 = blockIdx.y * RS_TOK, e0 = blockIdx.x * RS_EXP, ntok = min(RS_TOK, nb - b0);
    if (tid == 0) { mbar_init(&bar, 1); abort_flag = 0; mbar_init_fence(); }
    __syncthreads();
    if (tid == 0) {
        mbar_expect_tx(&bar, (uint32_t)(ntok * HID * 4 + RS_WB));
        bulk_load(smem_u32(rs_sm), hS + (size_t)b0 * HID * 4, (uint32_t)(ntok * HID * 4), &bar);
        bulk_load(smem_u32(rs_sm + RS_HB), WS + (size_t)e0 * HID * 2, RS_WB, &bar);
    }
    const bool ok = mbar_wait(&bar, 0, &abort_flag);
    float acc0 = 0.0f, acc1 = 0.0f, odd0 = 0.0f, odd1 = 0.0f;       // odd0/odd1: the second chain of the step order (columns 16m + 8 + j)
    if (ok && tok < ntok) {
        const uint8_t *hp = rs_sm + tok * (HID * 4) + j * 16;
        const uint8_t *w0p = rs_sm + RS_HB + (2 * ep) * (HID * 2) + j * 8, *w1p = w0p + HID * 2;
#pragma unroll 8
        for (int i4 = 0; i4 < 64; i4++) {
            const float4 h = *reinterpret_cast<const float4 *>(hp + i4 * 128);
            const uint2 a = *reinterpret_cast<const uint2 *>(w0p + i4 * 64), b = *reinterpret_cast<const uint2 *>(w1p + i4 * 64);
            acc0 = __fmaf_rn(__uint_as_float(a.x << 16), h.x, acc0); acc1 = __fmaf_rn(__uint_as_float(b.x << 16), h.x, acc1);
            if (STEP) { odd0 = __fmaf_rn(__uint_as_float(a.x & 0xFFFF0000u), h.y, odd0); odd1 = __fmaf_rn(__uint_as_float(b.x & 0xFFFF0000u), h.y, odd1); }
            else { acc0 = __fmaf_rn(__uint_as_float(a.x & 0xFFFF0000u), h.y, acc0); acc1 = __fmaf_rn(__uint_as_float(b.x & 0xFFFF0000u), h.y, acc1); }
            acc0 = __fmaf_rn(__uint_as_float(a.y << 16), h.z, acc0); acc1 = __fmaf_rn(__uint_as_float(b.y << 16), h.z, acc1);
            if (STEP) { odd0 = __fmaf_rn(__uint_as_float(a.y & 0xFFFF0000u), h.w, odd0); odd1 = __fmaf_rn(__uint_as_float(b.y & 0xFFFF0000u), h.w, odd1); }
            else { acc0 = __fmaf_rn(__uint_as_float(a.y & 0xFFFF0000u), h.w, acc0); acc1 = __fmaf_rn(__uint_as_float(b.y & 0xFFFF0000u), h.w, acc1); }
        }
        if (STEP) { acc0 = __fadd_rn(acc0, odd0); acc1 = __fadd_rn(acc1, odd1); }
    }
    // the eight lanes of a position sit in one warp: (l0+l4)+(l1+l5) then +(l2+l6)+(l3+l7), the same on every lane
    float l0 = acc0, l1 = acc1;
    l0 = __fadd_rn(l0, __shfl_xor_sync(0xffffffffu, l0, 4)); l1 = __fadd_rn(l1, __shfl_xor_sync(0xffffffffu, l1, 4));
    l0 = __fadd_rn(l0, __shfl_xor_sync(0xffffffffu, l0, 1)); l1 = __fadd_rn(l1, __shfl_xor_sync(0xffffffffu, l1, 1));
    l0 = __fadd_rn(l0, __shfl_xor_sync(0xffffffffu, l0, 2)); l1 = __fadd_rn(l1, __shfl_xor_sync(0xffffffffu, l1, 2));
    if (ok && j == 0 && tok < ntok) {
        const int e = e0 + 2 * ep;
        float *dst = logits + (size_t)(b0 + tok) * NEXP + e;
        dst[0] = bias ? __fadd_rn(l0, bias[e]) : l0; dst[1] = bias ? __fadd_rn(l1, bias[e + 1]) : l1;
    }
    if (tid == 0 && !ok) atomicExch(err, 31);
}
extern "C" void k_router_pack_small(cudaStream_t st, const uint16_t *router, void *router_s) {
    router_pack_w_small_kernel<<<NEXP * HID / 4 / 256, 256, 0, st>>>(router, (uint2 *)router_s);
    k_count_add(1);
}
static int g_step_order = 0;
// single-token calls compute their logits in the order of the reference's `step` (bf_row) instead of `step_batch` (gmoe_set_step_order)
extern "C" void k_router_step_order(int on) { g_step_order = on != 0; }
extern "C" void k_router_logits_small(cudaStream_t st, const void *router_s, const float *hn, void *hS, int relaid, const float *bias, float *logits, int nb, int *err) {
    if (nb <= 0) return;
    static bool attr_done = false;
    if (!attr_done) {
        cudaFuncSetAttribute(router_small_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, RS_HB + RS_WB);
        cudaFuncSetAttribute(router_small_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, RS_HB + RS_WB); attr_done = true;
    }
    if (!relaid) launch_k(router_pack_h_small_kernel, nb * 2, 256, 0, st, hn, (float4 *)hS, nb);
    const dim3 grid(NEXP / RS_EXP, (nb + RS_TOK - 1) / RS_TOK);
    if (g_step_order && nb == 1) launch_k(router_small_kernel<true>, grid, 256, RS_HB + RS_WB, st, (const uint8_t *)router_s, (const uint8_t *)hS, bias, logits, nb, err);
    else launch_k(router_small_kernel<false>, grid, 256, RS_HB + RS_WB, st, (const uint8_t *)router_s, (const uint8_t *)hS, bias, logits, nb, err);
    k_count_add(relaid ? 1 : 2);
}
