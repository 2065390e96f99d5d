// k_route.cu -- everything of the MoE half that is not a grouped GEMM or the router: RMSNorm + per-token int8,
// softmax + top-8, grouping of pairs by expert, SiLU-output int8, weighted combine.  sm_100a.
//
// Every kernel reproduces the reference's arithmetic operation by operation (order of additions, fused
// multiply-adds where the reference fuses, IEEE division and round-half-even), so its integer outputs are equal
// and its fp32 outputs are the same bits as maple.c's CPU path.  File:line citations are into maple.c.
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include "kernels.h"
#include "launch.cuh"
#include "dev_math.cuh"
#include "topk.cuh"

static long g_launches = 0;
extern "C" void k_count_reset(void) { g_launches = 0; }
extern "C" long k_count(void) { return g_launches; }
extern "C" void k_count_add(long n) { g_launches += n; }

#define HID 2048
#define NEXP 256
#define TOPK 8
#define FFN 512

// ------------------------------------------------------------------------------------------------------------
// RMSNorm (maple.c:398-402) + prep (maple.c:184-194), one warp per token: lane l holds columns 128 i + 4 l .. + 3 for i = 0..15 (every
// load and store instruction of the warp covers one contiguous run of the row, all sixteen loads are in flight together, and the three
// reductions are shuffles: no block-wide barrier).  WPC warps (tokens) per CTA: 8 for chunks, 1 for decode batches (more CTAs).
// w == NULL: x is already normalised (hn = x, not rewritten when hn == x).
// The sum of squares is accumulated in double like the reference; the tree order differs from its left-to-right
// order only below double precision, which the conversion to float absorbs.
// ------------------------------------------------------------------------------------------------------------
// hS != NULL: the normalised row is also stored as the decode router wants it, [column / 32][lane j][4 steps] (k_router_tile.cu).
// hA != NULL: the normalised row is also stored as two fp16 terms, hi = fp16(h) in columns 0..2047 and lo = fp16(h - hi) in columns
// 2048..4095 of a 4096-column row (the tensor-core router's A operand, k_router_umma.cu), and its Euclidean norm goes to hnorm.
template <int WPC>
__global__ void __launch_bounds__(WPC * 32) norm_prep_kernel(const float *__restrict__ x, const uint16_t *__restrict__ w,
                                                             float *__restrict__ hn, int8_t *__restrict__ q,
                                                             float *__restrict__ qs, int *__restrict__ qsum, float *__restrict__ hS,
                                                             __half *__restrict__ hA, float *__restrict__ hnorm, int nb) {
    const int lane = threadIdx.x & 31, b = blockIdx.x * WPC + (threadIdx.x >> 5);
    if (b >= nb) return;
    const float4 *xr = reinterpret_cast<const float4 *>(x + (size_t)b * HID) + lane;
    float4 v[16];
#pragma unroll
    for (int i = 0; i < 16; i++) v[i] = xr[32 * i];
    if (w) {
        uint2 wr[16];                                            // 4 bf16 each
#pragma unroll
        for (int i = 0; i < 16; i++) wr[i] = reinterpret_cast<const uint2 *>(w)[32 * i + lane];
        double ss = 0.0;
#pragma unroll
        for (int i = 0; i < 16; i++) ss += (double)v[i].x * (double)v[i].x + (double)v[i].y * (double)v[i].y + ((double)v[i].z * (double)v[i].z + (double)v[i].w * (double)v[i].w);
#pragma unroll
        for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float k = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn((float)(ss / (double)HID), 1e-6f)));
        float4 *hr = reinterpret_cast<float4 *>(hn + (size_t)b * HID) + lane;
#pragma unroll
        for (int i = 0; i < 16; i++) {
            v[i].x = __fmul_rn(__fmul_rn(v[i].x, k), __uint_as_float(wr[i].x << 16)); v[i].y = __fmul_rn(__fmul_rn(v[i].y, k), __uint_as_float(wr[i].x & 0xFFFF0000u));
            v[i].z = __fmul_rn(__fmul_rn(v[i].z, k), __uint_as_float(wr[i].y << 16)); v[i].w = __fmul_rn(__fmul_rn(v[i].w, k), __uint_as_float(wr[i].y & 0xFFFF0000u));
            hr[32 * i] = v[i];
        }
    } else if (hn != x) {
        float4 *hr = reinterpret_cast<float4 *>(hn + (size_t)b * HID) + lane;
#pragma unroll
        for (int i = 0; i < 16; i++) hr[32 * i] = v[i];
    }
    if (hS) {      // column c goes to (c / 32) * 32 + (c % 8) * 4 + (c / 8) % 4: granule (step / 4, lane j), slot step % 4
        float *d = hS + (size_t)b * HID;
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const int c = 128 * i + 4 * lane;                    // c % 8 is 0 or 4
            float *p = d + (c >> 5) * 32 + (c & 7) * 4 + ((c >> 3) & 3);
            p[0] = v[i].x; p[4] = v[i].y; p[8] = v[i].z; p[12] = v[i].w;
        }
    }
    float mx = 0.0f, n2 = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; i++) mx = fmaxf(fmaxf(mx, fmaxf(fabsf(v[i].x), fabsf(v[i].y))), fmaxf(fabsf(v[i].z), fabsf(v[i].w)));
    if (hA) {
        uint2 *hi_row = reinterpret_cast<uint2 *>(hA + (size_t)b * (2 * HID)) + lane, *lo_row = hi_row + HID / 4;
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const float f[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
            __align__(8) __half hi[4], lo[4];
#pragma unroll
            for (int k = 0; k < 4; k++) { hi[k] = __float2half_rn(f[k]); lo[k] = __float2half_rn(f[k] - __half2float(hi[k])); n2 = fmaf(f[k], f[k], n2); }
            hi_row[32 * i] = *reinterpret_cast<const uint2 *>(hi); lo_row[32 * i] = *reinterpret_cast<const uint2 *>(lo);
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) n2 += __shfl_xor_sync(0xffffffffu, n2, o);
        if (lane == 0) hnorm[b] = sqrtf(n2);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    const float s = mx > 0.0f ? __fdiv_rn(mx, 127.0f) : 1.0f, inv = __fdiv_rn(1.0f, s);
    int tot = 0;
    uint32_t *qr = reinterpret_cast<uint32_t *>(q + (size_t)b * HID) + lane;
#pragma unroll
    for (int i = 0; i < 16; i++) {
        const int q0 = __float2int_rn(__fmul_rn(v[i].x, inv)), q1 = __float2int_rn(__fmul_rn(v[i].y, inv)), q2 = __float2int_rn(__fmul_rn(v[i].z, inv)), q3 = __float2int_rn(__fmul_rn(v[i].w, inv));
        tot += (q0 + q1) + (q2 + q3);
        qr[32 * i] = (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) | ((uint32_t)(q2 & 0xFF) << 16) | ((uint32_t)(q3 & 0xFF) << 24);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
    if (lane == 0) { qs[b] = s; qsum[b] = tot; }
}
static void norm_launch(cudaStream_t st, const float *x, const uint16_t *w, float *hn, int8_t *q, float *qs, int *qsum, float *hS, __half *hA, float *hnorm, int nb) {
    if (nb <= 0) return;
    if (nb > 256) launch_k(norm_prep_kernel<8>, (nb + 7) / 8, 256, 0, st, x, w, hn, q, qs, qsum, hS, hA, hnorm, nb);
    else launch_k(norm_prep_kernel<1>, nb, 32, 0, st, x, w, hn, q, qs, qsum, hS, hA, hnorm, nb);
    g_launches++;
}
extern "C" void k_norm_prep(cudaStream_t st, const float *x, const uint16_t *w, float *hn, int8_t *q, float *qs, int *qsum, int nb) {
    norm_launch(st, x, w, hn, q, qs, qsum, (float *)NULL, (__half *)NULL, (float *)NULL, nb);
}
extern "C" void k_norm_prep_relaid(cudaStream_t st, const float *x, const uint16_t *w, float *hn, int8_t *q, float *qs, int *qsum, float *hS, int nb) {
    norm_launch(st, x, w, hn, q, qs, qsum, hS, (__half *)NULL, (float *)NULL, nb);
}
extern "C" void k_norm_prep_split(cudaStream_t st, const float *x, const uint16_t *w, float *hn, int8_t *q, float *qs, int *qsum, void *hA, float *hnorm, int nb) {
    norm_launch(st, x, w, hn, q, qs, qsum, (float *)NULL, (__half *)hA, hnorm, nb);
}

// (Router logits live in k_router_tile.cu.)

// ------------------------------------------------------------------------------------------------------------
// Softmax + top-8 (maple.c:910-923): one warp per token, lane l holds experts 8l..8l+7.
// p = expf(l - max); the sum runs over experts in index order (a chain through the lanes); p /= sum; eight rounds
// of "first strict maximum" (lowest index wins a tie); weights divided by (their sum in selection order + 1e-20f).
// ------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) topk_kernel(const float *__restrict__ logits, int *__restrict__ top, float *__restrict__ topw, int nb) {
    __shared__ unsigned long long tab[32];                  // the expf table beside the arithmetic (lane-varying index)
    if (threadIdx.x < 32) tab[threadIdx.x] = DEV_EXP_TAB[threadIdx.x];
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int b = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (b >= nb) return;
    const float4 *lr = reinterpret_cast<const float4 *>(logits + (size_t)b * NEXP + lane * 8);
    float4 v0 = lr[0], v1 = lr[1];
    float p[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    int isel; float wsel, tsum;
    exact_topk_warp(p, lane, tab, isel, wsel, tsum);
    if (lane < TOPK) {
        top[b * TOPK + lane] = isel;
        topw[b * TOPK + lane] = __fdiv_rn(wsel, __fadd_rn(tsum, 1e-20f));
    }
}
extern "C" void k_topk(cudaStream_t st, const float *logits, int *top, float *topw, int nb) {
    if (nb <= 0) return;
    launch_k(topk_kernel, (nb + 7) / 8, 256, 0, st, logits, top, topw, nb); g_launches++;
}

// ------------------------------------------------------------------------------------------------------------
// Grouping (maple.c:924-938) and tp (maple.c:1018-1019), deterministic without ordered atomics:
//   1. mark:  bit (b % 32) of mask[b / 32][e] is set when token b chose expert e (atomicOr: the result does not depend on order),
//             and the pairs of every expert are counted (integer adds: any order, same sum)
//   2. place: a CTA owns 128 tokens (four mask words).  Thread e scans the counts into the experts' starts (used experts numbered in
//             ascending order: NU, UE, USTART; CTA 0 writes them and the tile lists of the grouped GEMMs) and counts expert e's
//             tokens in front of the CTA's words; then one thread per token: pair slot = start + tokens in front + rank inside the
//             word; UTOK, UW, the slot of every (token, choice), and tp = the token's eight slots sorted ascending (pair index
//             order = expert order)
// ------------------------------------------------------------------------------------------------------------
__global__ void zero_words_kernel(unsigned *__restrict__ p, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = 0u;
}
__global__ void group_mark_kernel(const int *__restrict__ top, unsigned *__restrict__ mask, int mask_words, int np) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= np) return;
    int b = i >> 3, e = top[i];
    atomicOr(&mask[(size_t)(b >> 5) * NEXP + e], 1u << (b & 31));
    atomicAdd(&mask[(size_t)NEXP * mask_words + e], 1u);        // pairs per expert, kept behind the bit words
}
__global__ void __launch_bounds__(NEXP) group_place_kernel(const unsigned *__restrict__ mask, int mask_words, const int *__restrict__ top,
                                                          const float *__restrict__ topw, int *__restrict__ nu_out, int *__restrict__ ue,
                                                          int *__restrict__ estart, int *__restrict__ ustart, int *__restrict__ ecnt,
                                                          MoeTile *__restrict__ ta, int *__restrict__ nta, int tna, MoeTile *__restrict__ tb, int *__restrict__ ntb, int tnb,
                                                          int *__restrict__ utok, float *__restrict__ uw, int *__restrict__ slot, int *__restrict__ uexp,
                                                          int *__restrict__ tp, int nb) {
    __shared__ int w_cnt[8], w_used[8], w_ta[8], w_tb[8];
    __shared__ int s_pre[4][NEXP]; __shared__ unsigned s_word[4][NEXP];
    const int e = threadIdx.x, lane = e & 31, wid = e >> 5;
    const int cnt = (int)mask[(size_t)NEXP * mask_words + e];
    const int used = cnt > 0, na = (cnt + tna - 1) / tna, nb_ = (cnt + tnb - 1) / tnb;
    int c = cnt, u = used, a = na, b = nb_;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int tc = __shfl_up_sync(0xffffffffu, c, o), tu = __shfl_up_sync(0xffffffffu, u, o);
        int t1 = __shfl_up_sync(0xffffffffu, a, o), t2 = __shfl_up_sync(0xffffffffu, b, o);
        if (lane >= o) { c += tc; u += tu; a += t1; b += t2; }
    }
    if (lane == 31) { w_cnt[wid] = c; w_used[wid] = u; w_ta[wid] = a; w_tb[wid] = b; }
    __syncthreads();
    int oc = 0, ou = 0, oa = 0, ob = 0;
    for (int w = 0; w < wid; w++) { oc += w_cnt[w]; ou += w_used[w]; oa += w_ta[w]; ob += w_tb[w]; }
    const int start = oc + c - cnt, uidx = ou + u - used, ta0 = oa + a - na, tb0 = ob + b - nb_;
    if (blockIdx.x == 0) {
        if (ecnt) ecnt[e] = cnt;
        estart[e] = used ? start : -1;
        if (used) {
            ue[uidx] = e; ustart[uidx] = start;
            for (int t = 0; t < na; t++) { MoeTile m = {uidx, start + t * tna, min(tna, cnt - t * tna), e}; ta[ta0 + t] = m; }
            for (int t = 0; t < nb_; t++) { MoeTile m = {uidx, start + t * tnb, min(tnb, cnt - t * tnb), e}; tb[tb0 + t] = m; }
        }
        if (e == NEXP - 1) { const int nu = uidx + used; *nu_out = nu; ustart[nu] = start + cnt; *nta = ta0 + na; *ntb = tb0 + nb_; }
    }
    // expert e's tokens in front of this CTA's four words (coalesced: consecutive threads read consecutive experts of a word)
    const int w0 = blockIdx.x * 4;
    int pre = start;
    for (int w = 0; w < w0; w++) pre += __popc(mask[(size_t)w * NEXP + e]);
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const unsigned word = w0 + k < mask_words ? mask[(size_t)(w0 + k) * NEXP + e] : 0u;
        s_pre[k][e] = pre; s_word[k][e] = word; pre += __popc(word);
    }
    __syncthreads();
    if (e >= 128) return;
    const int tok = blockIdx.x * 128 + e;
    if (tok >= nb) return;
    const int wk = e >> 5; const unsigned below = (1u << (e & 31)) - 1u;
    int sl[TOPK];
#pragma unroll
    for (int k = 0; k < TOPK; k++) {
        const int x = top[tok * TOPK + k];
        const int r = s_pre[wk][x] + __popc(s_word[wk][x] & below);
        sl[k] = r; slot[tok * TOPK + k] = r; utok[r] = tok; uw[r] = topw[tok * TOPK + k]; if (uexp) uexp[r] = x;
    }
#pragma unroll
    for (int i = 1; i < TOPK; i++)
#pragma unroll
        for (int k = TOPK - 1; k >= 1; k--) if (k >= i && sl[k] < sl[k - 1]) { int x = sl[k]; sl[k] = sl[k - 1]; sl[k - 1] = x; }
#pragma unroll
    for (int k = 0; k < TOPK; k++) tp[tok * TOPK + k] = sl[k];
}
// Decode batches (up to 256 tokens = 2048 pairs): the whole grouping in one CTA, so that the step costs one launch instead of five, and without a
// serial walk: every pair sets its token's bit in its expert's row of a shared-memory bit table; an expert's
// count is the population of its row, a pair's place inside its expert the population below its token's bit, which is the
// reference's order (pairs of an expert in token order).  The scan over experts and the per-token sort of the eight pair slots
// follow in the same CTA.
// MAXTOK tokens at most, NT threads (the first 256 own one expert each).  Used up to 256 tokens; a 2048-token instance (160 KB of
// shared memory, 1024 threads) works but one SM takes longer over 16,384 pairs than the three kernels of the general path below.
#define GS_MAXTOK 256
template <int MAXTOK, int NT>
__global__ void __launch_bounds__(NT) group_cta_kernel(GroupArgs g) {
    constexpr int WORDS = MAXTOK / 32;
    extern __shared__ __align__(16) unsigned gs_smem[];
    unsigned (*s_mask)[WORDS] = reinterpret_cast<unsigned (*)[WORDS]>(gs_smem);                         // [NEXP][WORDS]
    int *s_slot = reinterpret_cast<int *>(gs_smem + NEXP * WORDS);                                        // [MAXTOK * TOPK]
    unsigned short (*s_wpre)[WORDS] = reinterpret_cast<unsigned short (*)[WORDS]>(s_slot + MAXTOK * TOPK); // [NEXP][WORDS] pairs before word w
    __shared__ int s_start[NEXP];
    __shared__ int w_cnt[8], w_used[8], w_ta[8], w_tb[8];
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5, nb = g.nb, np = nb * TOPK;
    for (int i = tid; i < NEXP * WORDS; i += NT) gs_smem[i] = 0u;
    __syncthreads();
    for (int i = tid; i < np; i += NT) { const int t = i >> 3; atomicOr(&s_mask[g.top[i]][t >> 5], 1u << (t & 31)); }
    __syncthreads();
    if (tid < NEXP) {
        const int e = tid;
        int cnt = 0;
#pragma unroll 8
        for (int w = 0; w < WORDS; w++) { s_wpre[e][w] = (unsigned short)cnt; cnt += __popc(s_mask[e][w]); }
        if (g.ecnt) g.ecnt[e] = cnt;
        const int used = cnt > 0, na = (cnt + g.tn_a - 1) / g.tn_a, nb_ = (cnt + g.tn_b - 1) / g.tn_b;
        int c = cnt, u = used, a = na, b = nb_;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int tc = __shfl_up_sync(0xffffffffu, c, o), tu = __shfl_up_sync(0xffffffffu, u, o);
            int t1 = __shfl_up_sync(0xffffffffu, a, o), t2 = __shfl_up_sync(0xffffffffu, b, o);
            if (lane >= o) { c += tc; u += tu; a += t1; b += t2; }
        }
        if (lane == 31) { w_cnt[wid] = c; w_used[wid] = u; w_ta[wid] = a; w_tb[wid] = b; }
        asm volatile("bar.sync 1, 256;" ::: "memory");                   // the eight warps that own experts
        int oc = 0, ou = 0, oa = 0, ob = 0;
        for (int w = 0; w < wid; w++) { oc += w_cnt[w]; ou += w_used[w]; oa += w_ta[w]; ob += w_tb[w]; }
        const int start = oc + c - cnt, uidx = ou + u - used, ta0 = oa + a - na, tb0 = ob + b - nb_;
        g.estart[e] = used ? start : -1;
        s_start[e] = start;
        if (used) {
            g.ue[uidx] = e; g.ustart[uidx] = start;
            for (int t = 0; t < na; t++) { MoeTile m = {uidx, start + t * g.tn_a, min(g.tn_a, cnt - t * g.tn_a), e}; g.tiles_a[ta0 + t] = m; }
            for (int t = 0; t < nb_; t++) { MoeTile m = {uidx, start + t * g.tn_b, min(g.tn_b, cnt - t * g.tn_b), e}; g.tiles_b[tb0 + t] = m; }
        }
        if (e == NEXP - 1) { const int nu = uidx + used; *g.nu = nu; g.ustart[nu] = start + cnt; *g.ntiles_a = ta0 + na; *g.ntiles_b = tb0 + nb_; }
    }
    __syncthreads();
    for (int i = tid; i < np; i += NT) {                             // every pair finds its place
        const int x = g.top[i], t = i >> 3, w = t >> 5;
        const int r = s_start[x] + s_wpre[x][w] + __popc(s_mask[x][w] & ((1u << (t & 31)) - 1u));
        g.utok[r] = t; g.uw[r] = g.topw[i]; if (g.uexp) g.uexp[r] = x; s_slot[i] = r;
    }
    __syncthreads();
    for (int t = tid; t < nb; t += NT) {                             // tp: the token's eight slots ascending
        int sl[TOPK];
#pragma unroll
        for (int k = 0; k < TOPK; k++) { sl[k] = s_slot[t * TOPK + k]; g.slot[t * TOPK + k] = sl[k]; }
#pragma unroll
        for (int i = 1; i < TOPK; i++)
#pragma unroll
            for (int k = TOPK - 1; k >= 1; k--) if (k >= i && sl[k] < sl[k - 1]) { int x = sl[k]; sl[k] = sl[k - 1]; sl[k - 1] = x; }
#pragma unroll
        for (int k = 0; k < TOPK; k++) g.tp[t * TOPK + k] = sl[k];
    }
}
template <int MAXTOK, int NT>
static void launch_group_cta(cudaStream_t st, const GroupArgs *g) {
    const int smem = NEXP * (MAXTOK / 32) * 4 + MAXTOK * TOPK * 4 + NEXP * (MAXTOK / 32) * 2;
    static bool attr_done = false;
    if (!attr_done) { cudaFuncSetAttribute(group_cta_kernel<MAXTOK, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); attr_done = true; }
    launch_k(group_cta_kernel<MAXTOK, NT>, 1, NT, smem, st, *g);
}
extern "C" void k_group(cudaStream_t st, const GroupArgs *g) {
    if (g->nb <= 0) return;
    if (g->nb <= 256) { launch_group_cta<256, 256>(st, g); g_launches++; return; }
    const int np = g->nb * TOPK;
    if (!g->marked) {
        const int zw = NEXP * g->mask_words + NEXP;                                           // bit words + the 256 counters behind them
        launch_k(zero_words_kernel, (zw + 1023) / 1024, 1024, 0, st, g->mask, zw);
        launch_k(group_mark_kernel, (np + 255) / 256, 256, 0, st, g->top, g->mask, g->mask_words, np);
        g_launches += 2;
    }
    launch_k(group_place_kernel, (g->nb + 127) / 128, NEXP, 0, st, g->mask, g->mask_words, g->top, g->topw, g->nu, g->ue, g->estart, g->ustart, g->ecnt,
                                                            g->tiles_a, g->ntiles_a, g->tn_a, g->tiles_b, g->ntiles_b, g->tn_b,
                                                            g->utok, g->uw, g->slot, g->uexp, g->tp, g->nb);
    g_launches += 1;
}

// ------------------------------------------------------------------------------------------------------------
// SiLU-output int8 (the prep call of maple.c:831 on 512 values): one warp per pair, 16 values per lane.
// ------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) actq_kernel(const float *__restrict__ act, int8_t *__restrict__ aq, float *__restrict__ aqs,
                                                   int *__restrict__ aqsum, int np, const int *__restrict__ np_dev) {
    if (np_dev) np = min(np, *np_dev);
    const int lane = threadIdx.x & 31, a = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (a >= np) return;
    const float4 *r = reinterpret_cast<const float4 *>(act + (size_t)a * FFN) + lane * 4;
    float v[16];
#pragma unroll
    for (int i = 0; i < 4; i++) { float4 t = r[i]; v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w; }
    float mx = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; i++) mx = fmaxf(mx, fabsf(v[i]));
#pragma unroll
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    const float s = mx > 0.0f ? __fdiv_rn(mx, 127.0f) : 1.0f, inv = __fdiv_rn(1.0f, s);
    int tot = 0; uint32_t pk[4] = {0, 0, 0, 0};
#pragma unroll
    for (int i = 0; i < 16; i++) { int qi = __float2int_rn(__fmul_rn(v[i], inv)); tot += qi; pk[i >> 2] |= (uint32_t)(qi & 0xFF) << (8 * (i & 3)); }
    reinterpret_cast<uint4 *>(aq + (size_t)a * FFN)[lane] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
#pragma unroll
    for (int o = 16; o; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
    if (lane == 0) { aqs[a] = s; aqsum[a] = tot; }
}
extern "C" void k_actq(cudaStream_t st, const float *act, int8_t *aq, float *aqs, int *aqsum, const int *np_dev, int np_max) {
    if (np_max <= 0) return;
    launch_k(actq_kernel, (np_max + 7) / 8, 256, 0, st, act, aq, aqs, aqsum, np_max, np_dev); g_launches++;
}

// ------------------------------------------------------------------------------------------------------------
// SiLU*up + int8 in one pass (maple.c:825-832) for the tensor-core path, whose GEMM stores gate and up: one warp per
// pair, 16 values per lane: columns 128 i + 4 lane .. + 3 for i = 0..3, so that every load and store instruction of the warp covers
// one contiguous run of the row.  act (optional) receives the fp32 activations for stage comparisons.
//
// The int8 row, its scale and its sum are the reference's bits in both variants.  EXACT evaluates every element with the libm-equal
// expf in double (dev_math.cuh).  The other variant evaluates act ~ g / (1 + 2^(-g log2 e)) u with the hardware's approximate
// exponential and reciprocal (relative error below SQ_EPS for every g <= 7 that does not underflow) and falls back to the exact
// evaluation only where the approximation could change a result:
//   * the row maximum: every element within 2 SQ_EPS of the approximate maximum is evaluated exactly, the exact maximum is among them;
//   * a rounded value: t = act * inv lands within |t| (2 SQ_EPS + 2^-22) of a rounding boundary (about one element in two thousand).
// ------------------------------------------------------------------------------------------------------------
#define SQ_EPS 1.2e-5f
__device__ __forceinline__ float silu_mul_approx(float g, float u) {
    g = g < 7.0f ? g : 7.0f;
    u = u < -7.0f ? -7.0f : (u > 7.0f ? 7.0f : u);
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(g * -1.4426950408889634f));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
    return g * r * u;
}
template <bool EXACT>
__global__ void __launch_bounds__(256, 4) silu_quant_kernel(const float *__restrict__ gate, const float *__restrict__ up, float *__restrict__ act,
                                                         int8_t *__restrict__ aq, float *__restrict__ aqs, int *__restrict__ aqsum, int np, const int *__restrict__ np_dev) {
    __shared__ unsigned long long tab[32];
    if (threadIdx.x < 32) tab[threadIdx.x] = DEV_EXP_TAB[threadIdx.x];
    __syncthreads();
    if (np_dev) np = min(np, *np_dev);
    const int lane = threadIdx.x & 31, a = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (a >= np) return;
    const float4 *gr = reinterpret_cast<const float4 *>(gate + (size_t)a * FFN) + lane;
    const float4 *ur = reinterpret_cast<const float4 *>(up + (size_t)a * FFN) + lane;
    float gv[16], uv[16], v[16];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float4 g = gr[32 * i], u = ur[32 * i];
        gv[4 * i] = g.x; gv[4 * i + 1] = g.y; gv[4 * i + 2] = g.z; gv[4 * i + 3] = g.w;
        uv[4 * i] = u.x; uv[4 * i + 1] = u.y; uv[4 * i + 2] = u.z; uv[4 * i + 3] = u.w;
    }
    float mx = 0.0f;
    if (EXACT) {
#pragma unroll
        for (int i = 0; i < 16; i++) { v[i] = dev_silu_mul_tab(gv[i], uv[i], tab); mx = fmaxf(mx, fabsf(v[i])); }
        if (act) {
            float4 *o = reinterpret_cast<float4 *>(act + (size_t)a * FFN) + lane;
#pragma unroll
            for (int i = 0; i < 4; i++) o[32 * i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    } else {
        float mxa = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; i++) { v[i] = silu_mul_approx(gv[i], uv[i]); mxa = fmaxf(mxa, fabsf(v[i])); }
#pragma unroll
        for (int o = 16; o; o >>= 1) mxa = fmaxf(mxa, __shfl_xor_sync(0xffffffffu, mxa, o));
        const float thr = mxa * (1.0f - 2.5f * SQ_EPS) - 1e-30f;      // every element that can be the exact maximum
#pragma unroll
        for (int i = 0; i < 16; i++) if (!(fabsf(v[i]) < thr)) mx = fmaxf(mx, fabsf(dev_silu_mul_tab(gv[i], uv[i], tab)));
#pragma unroll
        for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    const float s = mx > 0.0f ? __fdiv_rn(mx, 127.0f) : 1.0f, inv = __fdiv_rn(1.0f, s);
    int tot = 0; uint32_t pk[4] = {0, 0, 0, 0};
    if (EXACT) {
#pragma unroll
        for (int i = 0; i < 16; i++) { int qi = __float2int_rn(__fmul_rn(v[i], inv)); tot += qi; pk[i >> 2] |= (uint32_t)(qi & 0xFF) << (8 * (i & 3)); }
    } else {
        const float slack = 1e-36f * inv;                                // elements the approximation flushed to zero
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const float t = __fmul_rn(v[i], inv), big = __fadd_rn(t, 12582912.0f), r = __fsub_rn(big, 12582912.0f);      // r = t rounded to an integer, half to even
            int qi = __float_as_int(big) - 0x4B400000;
            if (!(0.5f - fabsf(__fsub_rn(t, r)) > fabsf(t) * (2.0f * SQ_EPS + 2.4e-7f) + slack))
                qi = __float2int_rn(__fmul_rn(dev_silu_mul_tab(gv[i], uv[i], tab), inv));
            tot += qi; pk[i >> 2] |= (uint32_t)(qi & 0xFF) << (8 * (i & 3));
        }
    }
#pragma unroll
    for (int i = 0; i < 4; i++) reinterpret_cast<uint32_t *>(aq + (size_t)a * FFN)[32 * i + lane] = pk[i];
#pragma unroll
    for (int o = 16; o; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
    if (lane == 0) { aqs[a] = s; aqsum[a] = tot; }
}
extern "C" void k_silu_quant(cudaStream_t st, const float *gate, const float *up, float *act, int8_t *aq, float *aqs, int *aqsum, int np, const int *np_dev) {
    if (np <= 0) return;
    if (act) launch_k(silu_quant_kernel<true>, (np + 7) / 8, 256, 0, st, gate, up, act, aq, aqs, aqsum, np, np_dev);
    else launch_k(silu_quant_kernel<false>, (np + 7) / 8, 256, 0, st, gate, up, (float *)NULL, aq, aqs, aqsum, np, np_dev);
    g_launches++;
}

// ------------------------------------------------------------------------------------------------------------
// Combine (maple.c:834): out[b] = init[b] (or 0) then, for the token's pairs in ascending pair order,
// out = fma(w, down, out) -- the order and the fused rounding of the reference's compiled loop.
// ------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) combine_kernel(const float *__restrict__ down, const float *__restrict__ uw, const int *__restrict__ tp,
                                                      const float *__restrict__ init, float *__restrict__ out, int nb) {
    const int i = blockIdx.x * 256 + threadIdx.x, b = i >> 9, c = (i & 511) * 4;
    if (b >= nb) return;
    float4 acc = init ? *reinterpret_cast<const float4 *>(init + (size_t)b * HID + c) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int k = 0; k < TOPK; k++) {
        int a = tp[b * TOPK + k]; float w = uw[a];
        float4 d = *reinterpret_cast<const float4 *>(down + (size_t)a * HID + c);
        acc.x = __fmaf_rn(w, d.x, acc.x); acc.y = __fmaf_rn(w, d.y, acc.y); acc.z = __fmaf_rn(w, d.z, acc.z); acc.w = __fmaf_rn(w, d.w, acc.w);
    }
    *reinterpret_cast<float4 *>(out + (size_t)b * HID + c) = acc;
}
extern "C" void k_combine(cudaStream_t st, const float *down, const float *uw, const int *tp, const float *init, float *out, int nb) {
    if (nb <= 0) return;
    launch_k(combine_kernel, (nb * 512 + 255) / 256, 256, 0, st, down, uw, tp, init, out, nb); g_launches++;
}
