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
// tests: pin the tokens per thread (4..8; 0 = choose by batch size)
extern "C" void k_router_tile_force(int tt) { g_force_tt = (tt >= 4 && tt <= 8) ? tt : 0; }
template <int TT>
static void launch_tile(cudaStream_t st, const void *router_t, const float *hn, void *hT, const float *bias, float *logits, int nb, int *err) {
    static bool attr_done = false;
    if (!attr_done) { cudaFuncSetAttribute(router_tile_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, RP_SMEM); attr_done = true; }
    const int tiles = (nb + 4 * TT - 1) / (4 * TT);
    router_pack_h_kernel<<<tiles * 64, 256, 0, st>>>(hn, (float4 *)hT, nb, TT);
    router_tile_kernel<TT><<<dim3(NEXP / RP_EXP, tiles), 256, RP_SMEM, st>>>((const uint8_t *)router_t, (const uint8_t *)hT, bias, logits, nb, err);
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
