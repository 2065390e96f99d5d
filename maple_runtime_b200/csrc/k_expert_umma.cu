// k_expert_umma.cu -- grouped ternary expert GEMMs on the 5th-generation tensor cores (tcgen05.mma kind::i8), sm_100a.
//
// One CTA = one tile (a used expert and up to 128 of its pairs) x one block of 2 x 128 weight rows:
//   gate+up: 128 gate rows and the 128 up rows of the same index (so the SiLU*up epilogue finds both in one thread);
//   down:    two consecutive blocks of 128 down rows.
// D[128 rows][N tokens] (s32, tensor memory) += A[128 rows][K] (u8 codes 0,1,2) x B[N tokens][K]^T (s8 activations).
//
// Weights never pass through shared memory: each of 256 threads owns one weight row, reads its 2-bit codes from HBM
// with 128-bit loads (128 packed bytes = 512 columns per trip, so whole 128-byte lines are consumed), expands every
// 32-bit word into four code words ((w >> 2s) & 0x03030303 is exactly the four codes of columns 32s+4j..32s+4j+3 of the
// group, in column order) and writes them with tcgen05.st into the tensor-memory A operand: lane = weight row, one
// 32-bit cell = four consecutive K values.  The activations (int8, rows gathered by token) are the B operand in shared
// memory, K-major with the 128-byte swizzle, filled by one warp with 16-byte asynchronous copies.
// Arithmetic = maple.c:425-458: out = (float)(sum(code*q) - qsum) * qs * s[r]; integer sums are exact.
//
// Roles (320 threads): warps 0-3 A rows of accumulator 0, warps 4-7 A rows of accumulator 1 (all eight do the
// epilogue), warp 8 B copies, warp 9 issues the MMAs.  Four pipeline stages; per stage a_full (8 warp arrivals),
// b_full (1), empty (tcgen05.commit).  Every wait is bounded (umma.cuh); on a timeout the CTA raises args.err, frees
// its tensor memory and returns.
//
// Tensor memory (512 columns): [0,128) accumulator 0, [128,256) accumulator 1, [256,512) four A stages of 2 x 32 columns.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include "kernels.h"
#include "dev_math.cuh"
#include "umma.cuh"

extern "C" void k_count_add(long n);

#define UM_STAGES 4
#define UM_TN 128
#define UM_BSTAGE (UM_TN * 128)

struct __align__(16) UmShared {
    uint64_t a_full[UM_STAGES], b_full[UM_STAGES], empty[UM_STAGES], acc_full;
    uint32_t tmem_base; int abort_flag;
    int tok[UM_TN]; float qs[UM_TN]; int qsum[UM_TN];
};

template <int KB, bool GATEUP>
__global__ void __launch_bounds__(320, 1) expert_umma_kernel(ExpertArgs a) {
    extern __shared__ __align__(1024) uint8_t um_smem_raw[];
    const int tile_i = blockIdx.y;
    if (tile_i >= *a.ntiles) return;
    uint8_t *bs = (uint8_t *)(((uintptr_t)um_smem_raw + 1023) & ~(uintptr_t)1023);          // UM_STAGES x 16 KB, 1024-aligned
    UmShared *sh = reinterpret_cast<UmShared *>(bs + UM_STAGES * UM_BSTAGE);
    const MoeTile tile = a.tiles[tile_i];
    const int ex = a.ue ? a.ue[tile.u] : tile.u;
    const ExpertPtrs ep = a.tab[ex];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, mb = blockIdx.x;
    const int cnt = tile.cnt, N = (cnt + 15) & ~15;
    constexpr int KBYTES = KB * 128;                                                         // bytes of one int8 activation row
    volatile int *abortp = &sh->abort_flag;

    if (tid == 0) {
        for (int s = 0; s < UM_STAGES; s++) { mbar_init(&sh->a_full[s], 8); mbar_init(&sh->b_full[s], 1); mbar_init(&sh->empty[s], 1); }
        mbar_init(&sh->acc_full, 1); sh->abort_flag = 0; mbar_init_fence();
    }
    if (warp == 9) tmem_alloc(&sh->tmem_base, 512);
    if (tid < cnt) {
        int pair = tile.p0 + tid;
        if (GATEUP) { int t = a.ptok[pair]; sh->tok[tid] = t; sh->qs[tid] = a.hqs[t]; sh->qsum[tid] = a.hqsum[t]; }
        else { sh->tok[tid] = pair; sh->qs[tid] = a.aqs[pair]; sh->qsum[tid] = a.aqsum[pair]; }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tb = sh->tmem_base;

    if (warp < 8) {
        // ---------------- A producer: one weight row per thread ----------------
        const int h = warp >> 2, row = (warp & 3) * 32 + lane;
        const uint8_t *wrow = GATEUP ? (h ? ep.uc : ep.gc) + (size_t)(mb * 128 + row) * (KBYTES / 4)
                                     : ep.dc + (size_t)((mb * 2 + h) * 128 + row) * (KBYTES / 4);
        const uint32_t a_lane = tb + ((uint32_t)((warp & 3) * 32) << 16) + 256 + h * 32;
        constexpr int NSB = KB / 4;                                                          // trips of 128 packed bytes
        uint4 cur[8], nxt[8];
#pragma unroll
        for (int i = 0; i < 8; i++) nxt[i] = __ldg(reinterpret_cast<const uint4 *>(wrow) + i);
        bool live = true;
#pragma unroll 1
        for (int sb = 0; sb < NSB && live; sb++) {
#pragma unroll
            for (int i = 0; i < 8; i++) cur[i] = nxt[i];
            if (sb + 1 < NSB) {
#pragma unroll
                for (int i = 0; i < 8; i++) nxt[i] = __ldg(reinterpret_cast<const uint4 *>(wrow + (sb + 1) * 128) + i);
            }
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const int kb = sb * 4 + q, s = kb % UM_STAGES, it = kb / UM_STAGES;
                if (!mbar_wait(&sh->empty[s], (it & 1) ^ 1, abortp)) { live = false; break; }
                tc_fence_after();
                if (a.dbg & 2) { __syncwarp(); if (lane == 0) mbar_arrive(&sh->a_full[s]); continue; }
                const uint32_t w[8] = {cur[2 * q].x, cur[2 * q].y, cur[2 * q].z, cur[2 * q].w, cur[2 * q + 1].x, cur[2 * q + 1].y, cur[2 * q + 1].z, cur[2 * q + 1].w};
                uint32_t r[32];
#pragma unroll
                for (int sft = 0; sft < 4; sft++)
#pragma unroll
                    for (int j = 0; j < 8; j++) r[sft * 8 + j] = (w[j] >> (2 * sft)) & 0x03030303u;
                tmem_st32(a_lane + s * 64, r);
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh->a_full[s]);
            }
        }
        // ---------------- epilogue: lane = weight row, columns = tokens ----------------
        if (live && mbar_wait(&sh->acc_full, 0, abortp) && !(a.dbg & 8)) {
            tc_fence_after();
            const uint32_t d_lane = tb + ((uint32_t)((warp & 3) * 32) << 16);
            const int r0 = GATEUP ? mb * 128 + row : mb * 256 + row;
            const float s0 = GATEUP ? ep.gs[r0] : ep.ds[r0], s1 = GATEUP ? ep.us[r0] : ep.ds[r0 + 128];
            for (int c0 = h * 16; c0 < N; c0 += 32) {                                        // 16-column pieces, alternating between the two warp sets
                uint32_t v0[16], v1[16];
                tmem_ld16(d_lane + c0, v0); tmem_ld16(d_lane + 128 + c0, v1);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const int n = c0 + j;
                    if (n < cnt) {
                        const int pair = tile.p0 + n, d0 = (int)v0[j] - sh->qsum[n], d1 = (int)v1[j] - sh->qsum[n];
                        const float qs = sh->qs[n];
                        const float f0 = __fmul_rn(__fmul_rn((float)d0, qs), s0), f1 = __fmul_rn(__fmul_rn((float)d1, qs), s1);
                        if (GATEUP) {
                            a.act[(size_t)pair * 512 + r0] = dev_silu_mul(f0, f1);
                            if (a.gate) { a.gate[(size_t)pair * 512 + r0] = f0; a.up[(size_t)pair * 512 + r0] = f1; }
                            if (a.gu_dots) { a.gu_dots[(size_t)pair * 1024 + r0] = d0; a.gu_dots[(size_t)pair * 1024 + 512 + r0] = d1; }
                        } else {
                            a.down[(size_t)pair * 2048 + r0] = f0; a.down[(size_t)pair * 2048 + r0 + 128] = f1;
                            if (a.dn_dots) { a.dn_dots[(size_t)pair * 2048 + r0] = d0; a.dn_dots[(size_t)pair * 2048 + r0 + 128] = d1; }
                        }
                    }
                }
            }
        }
    } else if (warp == 8) {
        // ---------------- B producer: gathered int8 rows, 16-byte asynchronous copies, two stages ahead ----------------
        const int8_t *src = GATEUP ? a.hq : a.aq;
        constexpr int AHEAD = 2;
        bool live = true;
        for (int kb = 0; kb < KB + AHEAD; kb++) {
            if (kb < KB && live) {
                const int s = kb % UM_STAGES, it = kb / UM_STAGES;
                if (!mbar_wait(&sh->empty[s], (it & 1) ^ 1, abortp)) live = false;
                else {
                    const uint32_t dst = smem_u32(bs + s * UM_BSTAGE);
                    for (int i = lane; i < cnt * 8 && !(a.dbg & 1); i += 32) {
                        const int n = i >> 3, c = i & 7;
                        cp_async16(dst + n * 128 + ((c ^ (n & 7)) << 4), src + (size_t)sh->tok[n] * KBYTES + kb * 128 + c * 16);
                    }
                }
            }
            cp_async_commit();
            if (kb >= AHEAD) {
                cp_async_wait<AHEAD>();
                proxy_fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh->b_full[(kb - AHEAD) % UM_STAGES]);
            }
        }
        cp_async_wait<0>();
    } else if (lane == 0) {
        // ---------------- MMA issuer ----------------
        const uint32_t idesc = idesc_i8_u8s8((uint32_t)N);
        bool live = true;
        for (int kb = 0; kb < KB && live; kb++) {
            const int s = kb % UM_STAGES, it = kb / UM_STAGES;
            if (!mbar_wait(&sh->a_full[s], it & 1, abortp) || !mbar_wait(&sh->b_full[s], it & 1, abortp)) { live = false; break; }
            tc_fence_after();
            const uint32_t bbase = smem_u32(bs + s * UM_BSTAGE);
#pragma unroll
            for (int k = 0; k < 4 && !(a.dbg & 4); k++) {
                const uint64_t bd = smem_desc_k128(bbase, k * 32);
                umma_i8_ts(tb, tb + 256 + s * 64 + k * 8, bd, idesc, (kb | k) != 0);
                umma_i8_ts(tb + 128, tb + 256 + s * 64 + 32 + k * 8, bd, idesc, (kb | k) != 0);
            }
            umma_commit(&sh->empty[s]);
        }
        if (live) umma_commit(&sh->acc_full);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        tmem_dealloc(tb, 512);
        if (lane == 0 && sh->abort_flag && a.err) *a.err = 1;
    }
}

template <int KB, bool GATEUP>
static void launch(cudaStream_t st, const ExpertArgs *a) {
    const size_t smem = (size_t)UM_STAGES * UM_BSTAGE + sizeof(UmShared) + 1024;
    static bool attr_done = false;
    if (!attr_done) { cudaFuncSetAttribute(expert_umma_kernel<KB, GATEUP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); attr_done = true; }
    dim3 grid(GATEUP ? 4 : 8, a->max_tiles);
    ExpertArgs b = *a;
    static int dbg = -1; if (dbg < 0) { const char *e = getenv("GMOE_UMMA_DBG"); dbg = e ? atoi(e) : 0; }
    b.dbg = dbg;
    expert_umma_kernel<KB, GATEUP><<<grid, 320, smem, st>>>(b);
    k_count_add(1);
}
extern "C" void k_gateup_umma(cudaStream_t st, const ExpertArgs *a) { if (a->max_tiles > 0) launch<16, true>(st, a); }
extern "C" void k_down_umma(cudaStream_t st, const ExpertArgs *a) { if (a->max_tiles > 0) launch<4, false>(st, a); }
