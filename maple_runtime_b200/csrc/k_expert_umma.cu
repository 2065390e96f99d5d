// k_expert_umma.cu -- grouped ternary expert GEMMs on the 5th-generation tensor cores (tcgen05.mma kind::i8), sm_100a.
//
// Work item = one tile (a used expert and up to 128 of its pairs) x one block of 2 x 128 weight rows:
//   gate+up: 128 gate rows and the 128 up rows of the same index (the SiLU*up epilogue finds both in one thread);
//   down:    256 consecutive down rows, the even ones in accumulator 0 and the odd ones in accumulator 1 (a thread of the
//            epilogue then holds two neighbouring rows and stores them as one word of the compact result row, kernels.h WIRE_*).
// D[128 rows][N tokens] (s32, tensor memory) += A[128 rows][K] (u8 codes 0,1,2) x B[N tokens][K]^T (s8 activations).
// A persistent grid (one CTA per SM) walks the items; every ring below keeps running across items, so the next item's
// weights are already on their way while the current one is multiplied.
//
// Data movement
//   weights  HBM -> shared memory, still 2-bit packed: TMA tiled copies (cp.async.bulk.tensor.2d, one tensor map per expert
//            matrix, box = 128 bytes x 128 rows, 128-byte swizzle), 32 KB stages = 256 rows x 512 columns; the swizzle makes
//            the later row-per-thread reads free of bank conflicts;
//   decode   each of 256 threads owns one weight row, reads 32 packed bytes per 128-column block, expands every 32-bit
//            word with (w >> 2s) & 0x03030303 (the four codes of columns 32s+4j..32s+4j+3 of the group, in column
//            order; convert.py:29-33) and writes the block with tcgen05.st into the tensor-memory A operand: lane = row,
//            one 32-bit cell = four consecutive K values.  Decoded weights never touch shared memory;
//   B        int8 activation rows in pair order (a gather kernel puts the tokens' rows into expert-grouped order first), TMA
//            tiled copies (box = 128 bytes x 32, 64, 96 or 128 rows, whichever covers the tile's pairs; 128-byte swizzle = the
//            K-major layout the MMA descriptor names).
// A pipeline round is two 128-column blocks: the waits and commits of the MMA warps cost about as much as four MMAs each, so
// they are paid once per eight MMAs.
// Arithmetic = maple.c:425-458: out = (float)(sum(code*q) - qsum) * qs * s[r]; integer sums are exact.  gate+up scales here;
// down stores sum(code*q) - qsum as integers and the combine applies qs and s[r] (same two roundings, same order).
//
// Warps (640 threads): 0-3 decode rows of accumulator 0, 4-7 rows of accumulator 1, 8 weight TMA, 9 B TMA, 10 and 11 MMA issue
// (one warp per accumulator: a single thread cannot issue tcgen05.mma fast enough to fill the tensor pipe at N <= 80, two can),
// 12-19 epilogue.
// Every mbarrier wait is bounded (umma.cuh): on a timeout the CTA raises args.err, frees tensor memory and returns.
//
// Tensor memory (512 columns): accumulator 0 at 0, accumulator 1 at 128 (N <= 128 columns each); A stage s at 256 + 128 s:
// rows of accumulator h, block i of the round at + 64 h + 32 i.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include "kernels.h"
#include "dev_math.cuh"
#include "umma.cuh"

extern "C" void k_count_add(long n);

#define UM_TN 128
#define UM_ASTAGES 2                 /* rounds of two 128-column blocks */
#define UM_WSTAGES 2
#define UM_BSTAGES 4                 /* rounds too: 2 x 128 rows x 128 bytes */
#define UM_WBYTES (256 * 128)
#define UM_BBYTES (2 * UM_TN * 128)
#define UM_ACOL 256

struct __align__(16) UmShared {
    uint64_t w_full[UM_WSTAGES], w_empty[UM_WSTAGES], a_full[2][UM_ASTAGES], a_empty[2][UM_ASTAGES];   // A barriers per accumulator
    uint64_t b_full[UM_BSTAGES], b_empty[UM_BSTAGES], acc_full, acc_empty;
    uint32_t tmem_base; int abort_flag;
    unsigned long long exp_tab[32];
    __align__(16) float m_qs[8][UM_TN]; __align__(16) int m_qsum[8][UM_TN];      // per epilogue warp: scale and code-sum correction of the tile's tokens
    __align__(16) unsigned long long m_dst[8][UM_TN];                             // expert parallel, down: where each token's compact row lives (a peer's memory)
};

__device__ __forceinline__ void cp_async_arrive_noinc(uint64_t *bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

template <int KB, int MODE>
__global__ void __launch_bounds__(640, 1) expert_umma_kernel(ExpertArgs a, const __grid_constant__ TMap4 bmap) {
    extern __shared__ __align__(1024) uint8_t um_smem_raw[];
    uint8_t *base = (uint8_t *)(((uintptr_t)um_smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *wsm = base;                                              // UM_WSTAGES x 32 KB packed weights
    uint8_t *bsm = base + UM_WSTAGES * UM_WBYTES;                      // UM_BSTAGES x 32 KB int8 activations (two 16 KB blocks per round)
    __shared__ UmShared sh_static;                                    // static, so that the compiler knows these accesses are shared-memory ones
    UmShared *sh = &sh_static;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr bool GATEUP = MODE == 0, DENSE = MODE == 2;
    const int MB = GATEUP ? 4 : (DENSE ? a.dense_mblocks : 8);      // 256-row blocks of the matrix (gate+up: 128 + 128)
    constexpr int NSB = KB / 4;
    const int nitems = *a.ntiles * MB;
    volatile int *abortp = &sh->abort_flag;

    if (tid == 0) {
        for (int s = 0; s < UM_WSTAGES; s++) { mbar_init(&sh->w_full[s], 1); mbar_init(&sh->w_empty[s], 8); }
        for (int s = 0; s < UM_ASTAGES; s++) for (int h = 0; h < 2; h++) { mbar_init(&sh->a_full[h][s], 4); mbar_init(&sh->a_empty[h][s], 1); }
        for (int s = 0; s < UM_BSTAGES; s++) { mbar_init(&sh->b_full[s], 1); mbar_init(&sh->b_empty[s], 2); }
        mbar_init(&sh->acc_full, 2); mbar_init(&sh->acc_empty, 8);
        sh->abort_flag = 0; mbar_init_fence();
    }
    if (tid < 32) sh->exp_tab[tid] = DEV_EXP_TAB[tid];
    if (warp == 10) tmem_alloc(&sh->tmem_base, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tb = sh->tmem_base;
    bool live = true;

    if (warp < 8) {
        // ---------------- decode: one weight row per thread, packed bytes from the shared-memory ring ----------------
        const int h = warp >> 2, R = h * 128 + (warp & 3) * 32 + lane;
        const uint32_t a_lane = tb + ((uint32_t)((warp & 3) * 32) << 16) + UM_ACOL + h * 64;
        uint32_t wcnt = 0, acnt = 0;
        for (int item = blockIdx.x; item < nitems && live; item += gridDim.x) {
#pragma unroll 1
            for (int sb = 0; sb < NSB && live; sb++, wcnt++) {
                const int ws = wcnt % UM_WSTAGES;
                if (!mbar_wait(&sh->w_full[ws], (wcnt / UM_WSTAGES) & 1, abortp)) { live = false; break; }
                const uint8_t *wr = wsm + ws * UM_WBYTES + R * 128;
#pragma unroll
                for (int rd = 0; rd < 2; rd++, acnt++) {                 // two rounds per weight stage, two 128-column blocks per round
                    const int as = acnt % UM_ASTAGES;
                    uint32_t r[32], r2[32];
                    auto decode = [&](int q, uint32_t (&o)[32]) {
                        const uint4 v0 = *reinterpret_cast<const uint4 *>(wr + (((2 * q) ^ (R & 7)) << 4));
                        const uint4 v1 = *reinterpret_cast<const uint4 *>(wr + (((2 * q + 1) ^ (R & 7)) << 4));
                        const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
                        for (int sft = 0; sft < 4; sft++)
#pragma unroll
                            for (int j = 0; j < 8; j++) o[sft * 8 + j] = (w[j] >> (2 * sft)) & 0x03030303u;
                    };
                    decode(2 * rd, r); decode(2 * rd + 1, r2);            // both blocks are ready before the stage is free
                    if (!mbar_wait(&sh->a_empty[h][as], ((acnt / UM_ASTAGES) & 1) ^ 1, abortp)) { live = false; break; }
                    tc_fence_after();
                    tmem_st32(a_lane + as * 128, r);
                    tmem_st32(a_lane + as * 128 + 32, r2);
                    tmem_st_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sh->a_full[h][as]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh->w_empty[ws]);
            }
        }
    } else if (warp == 8) {
        // ---------------- weight TMA (one lane): per stage the 128 rows of accumulator 0 and the 128 of accumulator 1 ----------------
        if (lane == 0) {
            uint32_t wcnt = 0;
            MoeTile tnext = blockIdx.x < nitems ? a.tiles[blockIdx.x / MB] : MoeTile{0, 0, 0, 0};      // one item ahead: no load latency at an item's start
            for (int item = blockIdx.x; item < nitems && live; item += gridDim.x) {
                const MoeTile tile = tnext;
                if (item + (int)gridDim.x < nitems) tnext = a.tiles[(item + gridDim.x) / MB];
                const int mb = item % MB;
                const ExpertMaps *em = a.maps + tile.ex;
                for (int sb = 0; sb < NSB && live; sb++, wcnt++) {
                    const int ws = wcnt % UM_WSTAGES;
                    if (!mbar_wait(&sh->w_empty[ws], ((wcnt / UM_WSTAGES) & 1) ^ 1, abortp)) { live = false; break; }
                    const uint32_t dst = smem_u32(wsm + ws * UM_WBYTES);
                    mbar_expect_tx(&sh->w_full[ws], UM_WBYTES);
                    if (GATEUP) {
                        tma_load_2d(dst, &em->gate, sb * 128, mb * 128, &sh->w_full[ws]);
                        tma_load_2d(dst + 128 * 128, &em->up, sb * 128, mb * 128, &sh->w_full[ws]);
                    } else {
                        tma_load_3d(dst, &em->down, sb * 128, 0, mb * 128, &sh->w_full[ws]);             // the even rows of the 256-row block
                        tma_load_3d(dst + 128 * 128, &em->down, sb * 128, 1, mb * 128, &sh->w_full[ws]);   // the odd rows
                    }
                }
            }
        }
    } else if (warp == 9) {
        // ---------------- B TMA (one lane): per round two boxes of 128 rows x 128 bytes of the pair-ordered int8 activations ----------------
        if (lane == 0) {
            uint32_t bcnt = 0;
            MoeTile tnext = blockIdx.x < nitems ? a.tiles[blockIdx.x / MB] : MoeTile{0, 0, 0, 0};
            for (int item = blockIdx.x; item < nitems && live; item += gridDim.x) {
                const MoeTile tile = tnext;
                if (item + (int)gridDim.x < nitems) tnext = a.tiles[(item + gridDim.x) / MB];
                for (int kb = 0; kb < KB && live; kb += 2, bcnt++) {
                    const int s = bcnt % UM_BSTAGES;
                    if (!mbar_wait(&sh->b_empty[s], ((bcnt / UM_BSTAGES) & 1) ^ 1, abortp)) { live = false; break; }
                    // only as many rows as the tile has pairs, in steps of 32 (the MMA reads (cnt + 15) & ~15 <= that many)
                    const int bi = tile.cnt > 0 ? (tile.cnt - 1) >> 5 : 0;
                    mbar_expect_tx(&sh->b_full[s], 2 * 128 * 32 * (bi + 1));
                    tma_load_2d(smem_u32(bsm + s * UM_BBYTES), &bmap.m[bi], kb * 128, tile.p0, &sh->b_full[s]);
                    tma_load_2d(smem_u32(bsm + s * UM_BBYTES + UM_TN * 128), &bmap.m[bi], kb * 128 + 128, tile.p0, &sh->b_full[s]);
                }
            }
        }
    } else if (warp < 12) {
        // ---------------- MMA issue: warp 10 accumulator 0, warp 11 accumulator 1 (one lane each).  Stage indices and parities are
        // carried in registers (wrap by compare), descriptors and column addresses are base + stage * constant ----------------
        if (lane == 0) {
            const int h = warp - 10;
            const uint64_t bdesc0 = smem_desc_k128(smem_u32(bsm), 0);
            const uint32_t afull0 = smem_u32(&sh->a_full[h][0]), aempty0 = smem_u32(&sh->a_empty[h][0]);
            const uint32_t bfull0 = smem_u32(&sh->b_full[0]), bempty0 = smem_u32(&sh->b_empty[0]);
            uint32_t as = 0, ap = 0, bs = 0, bp = 0, icnt = 0;
            MoeTile tnext = blockIdx.x < nitems ? a.tiles[blockIdx.x / MB] : MoeTile{0, 0, 0, 0};
            for (int item = blockIdx.x; item < nitems && live; item += gridDim.x, icnt++) {
                const MoeTile tile = tnext;
                if (item + (int)gridDim.x < nitems) tnext = a.tiles[(item + gridDim.x) / MB];
                const uint32_t idesc = idesc_i8_u8s8((uint32_t)((tile.cnt + 15) & ~15));
                if (!mbar_wait(&sh->acc_empty, (icnt & 1) ^ 1, abortp)) { live = false; break; }
                tc_fence_after();
                const uint32_t d = tb + h * 128;
#pragma unroll 1
                for (int kb = 0; kb < KB; kb += 2) {
                    if (!mbar_wait_addr(afull0 + as * 8, ap, abortp) || !mbar_wait_addr(bfull0 + bs * 8, bp, abortp)) { live = false; break; }
                    tc_fence_after();
                    const uint32_t acol = tb + UM_ACOL + as * 128 + h * 64;
                    const uint64_t bd = bdesc0 + (uint64_t)(bs * (UM_BBYTES >> 4));
                    umma_i8_ts(d, acol, bd, idesc, kb != 0);
                    umma_i8_ts(d, acol + 8, bd + 2, idesc, 1);
                    umma_i8_ts(d, acol + 16, bd + 4, idesc, 1);
                    umma_i8_ts(d, acol + 24, bd + 6, idesc, 1);
                    const uint64_t bd1 = bd + (UM_TN * 128 >> 4);
                    umma_i8_ts(d, acol + 32, bd1, idesc, 1);
                    umma_i8_ts(d, acol + 40, bd1 + 2, idesc, 1);
                    umma_i8_ts(d, acol + 48, bd1 + 4, idesc, 1);
                    umma_i8_ts(d, acol + 56, bd1 + 6, idesc, 1);
                    umma_commit_addr(aempty0 + as * 8);
                    umma_commit_addr(bempty0 + bs * 8);
                    if (++as == UM_ASTAGES) { as = 0; ap ^= 1; }
                    if (++bs == UM_BSTAGES) { bs = 0; bp ^= 1; }
                }
                if (live) umma_commit(&sh->acc_full);
            }
        }
    } else {
        // ---------------- epilogue: lane = weight row, columns = tokens; warps 12-15 take the even 16-column pieces, 16-19 the odd ----------------
        const int ew = warp - 12, q4 = warp & 3, half = ew >> 2, row = q4 * 32 + lane;   // a warp reaches the tensor-memory lanes 32 (warp % 4) ..
        uint32_t icnt = 0;
        // the item header is a chain tile -> pointer table -> scales: the tile is read two items ahead and the pointer table one item
        // ahead, so that an item starts with everything but the scale values in registers
        const int stride = gridDim.x;
        MoeTile t1 = blockIdx.x < nitems ? a.tiles[blockIdx.x / MB] : MoeTile{0, 0, 0, 0};
        MoeTile t2 = (int)blockIdx.x + stride < nitems ? a.tiles[(blockIdx.x + stride) / MB] : MoeTile{0, 0, 0, 0};
        ExpertPtrs ep1 = a.tab[t1.ex];
        for (int item = blockIdx.x; item < nitems && live; item += stride, icnt++) {
            const MoeTile tile = t1; const ExpertPtrs ep = ep1;
            t1 = t2; ep1 = a.tab[t1.ex];
            if (item + 2 * stride < nitems) t2 = a.tiles[(item + 2 * stride) / MB];
            const int mb = item % MB, cnt = tile.cnt, N = (cnt + 15) & ~15;
            const int r0 = GATEUP ? mb * 128 + row : mb * 256 + 2 * row;      // down: accumulator 0 holds row r0, accumulator 1 row r0 + 1
            const float s0 = GATEUP ? ep.gs[r0] : (DENSE ? ep.ds[r0] : 0.0f), s1 = GATEUP ? ep.us[r0] : (DENSE ? ep.ds[r0 + 1] : 0.0f);
            __syncwarp();
            for (int n = lane; n < N; n += 32) {
                const int pair = tile.p0 + (n < cnt ? n : 0), t = (GATEUP && a.ptok) ? a.ptok[pair] : pair;
                sh->m_qs[ew][n] = GATEUP ? a.hqs[t] : a.aqs[t]; sh->m_qsum[ew][n] = GATEUP ? a.hqsum[t] : (DENSE ? a.aqsum[t] : 32768 - a.aqsum[t]);
                if (MODE == 1 && a.rx_src) { const int2 sp = a.rx_src[pair]; sh->m_dst[ew][n] = (unsigned long long)(uintptr_t)(a.peer_wire[sp.x] + (size_t)sp.y * WIRE_PITCH); }
            }
            __syncwarp();
            if (!mbar_wait(&sh->acc_full, icnt & 1, abortp)) { live = false; break; }
            tc_fence_after();
            const uint32_t d_lane = tb + ((uint32_t)(q4 * 32) << 16);
            const int c_last = ((N / 16 - 1 - half) & ~1) + half;           // this warp's last piece (negative: none)
            if (half * 16 >= N) { __syncwarp(); if (lane == 0) mbar_arrive(&sh->acc_empty); }
            for (int c0 = half * 16; c0 < N; c0 += 32) {
                uint32_t v0[16], v1[16];
                tmem_ld16(d_lane + c0, v0); tmem_ld16(d_lane + 128 + c0, v1);
                tmem_ld_wait();
                if (c0 == c_last * 16) {   // the buffer is in registers: hand it back before the arithmetic
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sh->acc_empty);
                }
                const int lim = cnt - c0;                                 // tokens of this piece that exist
                if (GATEUP || DENSE) {
                    float o0[16], o1[16];
                    {   // scale and code-sum correction of the piece's 16 tokens: eight 128-bit shared-memory reads
                        const int4 *qsv = reinterpret_cast<const int4 *>(&sh->m_qsum[ew][c0]);
                        const float4 *qfv = reinterpret_cast<const float4 *>(&sh->m_qs[ew][c0]);
#pragma unroll
                        for (int g4 = 0; g4 < 4; g4++) {
                            const int4 qs4 = qsv[g4]; const float4 qf4 = qfv[g4];
                            const int qsum[4] = {qs4.x, qs4.y, qs4.z, qs4.w}; const float qs[4] = {qf4.x, qf4.y, qf4.z, qf4.w};
#pragma unroll
                            for (int k = 0; k < 4; k++) {
                                const int j = g4 * 4 + k, d0 = (int)v0[j] - qsum[k], d1 = (int)v1[j] - qsum[k];
                                o0[j] = __fmul_rn(__fmul_rn((float)d0, qs[k]), s0); o1[j] = __fmul_rn(__fmul_rn((float)d1, qs[k]), s1);
                                v0[j] = (uint32_t)d0; v1[j] = (uint32_t)d1;
                            }
                        }
                    }
                    if (DENSE) {      // fp32 rows of the projection: this thread's two neighbouring rows of every token of the piece
                        float *dp = a.down + (size_t)(tile.p0 + c0) * a.down_stride + r0;
#pragma unroll
                        for (int j = 0; j < 16; j++) if (j < lim) *reinterpret_cast<float2 *>(dp + (size_t)j * a.down_stride) = make_float2(o0[j], o1[j]);
                        continue;
                    }
                    // one base pointer per thread; the token index only adds a constant, so a store is one instruction
                    float *gp = a.gate + (size_t)(tile.p0 + c0) * 512 + r0, *up_ = a.up + (size_t)(tile.p0 + c0) * 512 + r0;
#pragma unroll
                    for (int j = 0; j < 16; j++) if (j < lim) { gp[j * 512] = o0[j]; up_[j * 512] = o1[j]; }
                    if (a.gu_dots) {
                        int *dp = a.gu_dots + (size_t)(tile.p0 + c0) * 1024 + r0;
#pragma unroll
                        for (int j = 0; j < 16; j++) if (j < lim) { dp[j * 1024] = (int)v0[j]; dp[j * 1024 + 512] = (int)v1[j]; }
                    }
                } else {
                    // compact rows: (dot + 32768) of this thread's two rows in one 32-bit word per token; the scales are applied where
                    // the rows are combined.  Values that need more than 16 bits (|dot| >= 32768) take the escape plane below.
                    uint32_t pk[16], wide = 0;
                    {
                        const int4 *qsv = reinterpret_cast<const int4 *>(&sh->m_qsum[ew][c0]);
#pragma unroll
                        for (int g4 = 0; g4 < 4; g4++) {
                            const int4 qs4 = qsv[g4]; const int bq[4] = {qs4.x, qs4.y, qs4.z, qs4.w};       // 32768 - qsum
#pragma unroll
                            for (int k = 0; k < 4; k++) {
                                const int j = g4 * 4 + k;
                                v0[j] += (uint32_t)bq[k]; v1[j] += (uint32_t)bq[k];
                                pk[j] = __byte_perm(v0[j], v1[j], 0x5410);
                                wide |= v0[j] | v1[j];
                            }
                        }
                    }
                    const bool esc = __any_sync(0xffffffffu, (wide >> 16) != 0);
                    const size_t rec0 = (size_t)a.wire_cap * WIRE_PITCH;            // the records sit behind the rows
                    const bool recw = mb == 0 && q4 == 0 && lane < 16 && lane < lim; // one warp per piece writes the tokens' records
                    if (!a.rx_src) {
                        uint8_t *rowp = a.wire + (size_t)(tile.p0 + c0) * WIRE_PITCH;
                        uint32_t *dp = reinterpret_cast<uint32_t *>(rowp) + (r0 >> 1);
#pragma unroll
                        for (int j = 0; j < 16; j++) if (j < lim) dp[j * (WIRE_PITCH / 4)] = pk[j];
                        if (recw) *reinterpret_cast<int2 *>(a.wire + rec0 + (size_t)(tile.p0 + c0 + lane) * WIRE_REC) = make_int2(__float_as_int(sh->m_qs[ew][c0 + lane]), tile.ex);
                        if (esc) {
#pragma unroll
                            for (int j = 0; j < 16; j++) if (j < lim) {
                                const uint32_t code = ((v0[j] >> 16) & 3u) | (((v1[j] >> 16) & 3u) << 2);
                                if (code) {
                                    atomicOr(reinterpret_cast<uint32_t *>(rowp + (size_t)j * WIRE_PITCH + 4096) + (r0 >> 4), code << ((r0 & 15) * 2));
                                    atomicOr(reinterpret_cast<int *>(a.wire + rec0 + (size_t)(tile.p0 + c0 + j) * WIRE_REC + 8), 1 << (r0 >> 7));
                                }
                            }
                        }
                    } else {
                        // expert parallel: each row goes to the rank that owns the token
                        const ulonglong2 *dv = reinterpret_cast<const ulonglong2 *>(&sh->m_dst[ew][c0]);
#pragma unroll
                        for (int j2 = 0; j2 < 8; j2++) {
                            const ulonglong2 d2 = dv[j2];
                            if (2 * j2 < lim) reinterpret_cast<uint32_t *>((uintptr_t)d2.x)[r0 >> 1] = pk[2 * j2];
                            if (2 * j2 + 1 < lim) reinterpret_cast<uint32_t *>((uintptr_t)d2.y)[r0 >> 1] = pk[2 * j2 + 1];
                        }
                        if (recw) {
                            const int2 sp = a.rx_src[tile.p0 + c0 + lane];
                            *reinterpret_cast<int2 *>(a.peer_wire[sp.x] + rec0 + (size_t)sp.y * WIRE_REC) = make_int2(__float_as_int(sh->m_qs[ew][c0 + lane]), tile.ex);
                        }
                        if (esc) {
#pragma unroll
                            for (int j = 0; j < 16; j++) if (j < lim) {
                                const uint32_t code = ((v0[j] >> 16) & 3u) | (((v1[j] >> 16) & 3u) << 2);
                                if (code) {
                                    const int2 sp = a.rx_src[tile.p0 + c0 + j];
                                    uint8_t *pb = a.peer_wire[sp.x];
                                    atomicOr(reinterpret_cast<uint32_t *>(pb + (size_t)sp.y * WIRE_PITCH + 4096) + (r0 >> 4), code << ((r0 & 15) * 2));
                                    atomicOr(reinterpret_cast<int *>(pb + rec0 + (size_t)sp.y * WIRE_REC + 8), 1 << (r0 >> 7));
                                }
                            }
                        }
                    }
                    if (a.dn_dots) {
                        int *ip = a.dn_dots + (size_t)(tile.p0 + c0) * 2048 + r0;
#pragma unroll
                        for (int j = 0; j < 16; j++) if (j < lim) *reinterpret_cast<int2 *>(ip + j * 2048) = make_int2((int)v0[j] - 32768, (int)v1[j] - 32768);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 10) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tb, 512);
        if (lane == 0 && sh->abort_flag && a.err) *a.err = 1;
    }
}

template <int KB, int MODE>
static void launch(cudaStream_t st, const ExpertArgs *a, const TMap4 *bmap) {
    const size_t smem = (size_t)UM_WSTAGES * UM_WBYTES + UM_BSTAGES * UM_BBYTES + 1024;
    static int sms = 0;
    if (!sms) {
        int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        cudaFuncSetAttribute(expert_umma_kernel<KB, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }
    expert_umma_kernel<KB, MODE><<<sms, 640, smem, st>>>(*a, *bmap);
    k_count_add(1);
}
extern "C" void k_gateup_umma(cudaStream_t st, const ExpertArgs *a, const TMap4 *bmap) { if (a->max_tiles > 0) launch<16, 0>(st, a, bmap); }
extern "C" void k_down_umma(cudaStream_t st, const ExpertArgs *a, const TMap4 *bmap) { if (a->max_tiles > 0) launch<4, 1>(st, a, bmap); }
/* dense projections: tab[ex].ds / maps[ex].down of a matrix of 256 * a->dense_mblocks rows x 2048 columns, B rows = the tokens' int8 rows */
extern "C" void k_dense_umma(cudaStream_t st, const ExpertArgs *a, const TMap4 *bmap) { if (a->max_tiles > 0) launch<16, 2>(st, a, bmap); }

// ---- rows of the per-token int8 matrix copied into pair (expert-grouped) order: the B operand the TMA can tile ----
__global__ void __launch_bounds__(256) gather_rows_kernel(const int8_t *__restrict__ src, const int *__restrict__ rows, int8_t *__restrict__ dst, int np) {
    // 8 pairs per CTA: each thread moves one 16-byte piece of four rows, all four loads in flight together
    const int p0 = blockIdx.x * 8 + (threadIdx.x >> 7) * 4, c = threadIdx.x & 127;
    int r[4]; uint4 v[4];
#pragma unroll
    for (int k = 0; k < 4; k++) r[k] = p0 + k < np ? rows[p0 + k] : 0;
#pragma unroll
    for (int k = 0; k < 4; k++) v[k] = reinterpret_cast<const uint4 *>(src + (size_t)r[k] * 2048)[c];
#pragma unroll
    for (int k = 0; k < 4; k++) if (p0 + k < np) reinterpret_cast<uint4 *>(dst + (size_t)(p0 + k) * 2048)[c] = v[k];
}
extern "C" void k_gather_rows(cudaStream_t st, const int8_t *src, const int *rows, int8_t *dst, int np) {
    if (np <= 0) return;
    gather_rows_kernel<<<(np + 7) / 8, 256, 0, st>>>(src, rows, dst, np);
    k_count_add(1);
}
