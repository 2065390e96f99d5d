// k_expert_umma.cu -- grouped ternary expert GEMMs on the 5th-generation tensor cores (tcgen05.mma kind::i8), sm_100a.
//
// Work item = one tile (a used expert and up to UMMA_TN = 96 of its pairs) x one block of 2 x 128 weight rows:
//   gate+up: 128 gate rows and the 128 up rows of the same index (the SiLU*up step finds both in one thread);
//   down:    256 consecutive down rows, the even ones in accumulator half 0 and the odd ones in half 1 (a thread of the
//            epilogue then holds two neighbouring rows and stores them as one word of the compact result row, kernels.h WIRE_*).
// D[128 rows][N tokens] (s32, tensor memory) += A[128 rows][K] (u8 codes 0,1,2) x B[N tokens][K]^T (s8 activations).
// A persistent grid (one CTA per SM) walks the items; every ring below keeps running across items, so the next item's
// weights are already on their way while the current one is multiplied.
//
// Data movement
//   weights  HBM -> shared memory, still 2-bit packed: TMA tiled copies (cp.async.bulk.tensor, one tensor map per expert
//            matrix, box = 128 bytes x 128 rows, 128-byte swizzle), 32 KB stages = 256 rows x 512 columns; the swizzle makes
//            the later row-per-thread reads free of bank conflicts;
//   decode   eight warps; a thread owns one row of each accumulator half and every second 128-column block: it reads 32 packed
//            bytes per row, expands every 32-bit word with (w >> 2s) & 0x03030303 (the four codes of columns 32s+4j..32s+4j+3
//            of the group, in column order; convert.py:29-33) and writes the block with tcgen05.st into the tensor-memory A
//            operand: lane = row, one 32-bit cell = four consecutive K values.  Decoded weights never touch shared memory;
//   B        int8 activation rows in pair order (a gather kernel puts the tokens' rows into expert-grouped order first), TMA
//            tiled copies (box = 128 bytes x 32, 64 or 96 rows, whichever covers the tile's pairs; 128-byte swizzle = the
//            K-major layout the MMA descriptor names), one 128-column block per stage.
// Arithmetic = maple.c:425-458: out = (float)(sum(code*q) - qsum) * qs * s[r]; integer sums are exact.  gate+up scales here;
// down stores sum(code*q) - qsum as integers and the combine applies qs and s[r] (same two roundings, same order).
//
// Warps (640 threads): 0-7 decode (warp w: tensor-memory lanes 32 (w % 4).., blocks of parity w / 4), 8 weight TMA, 9 B TMA,
// 10 and 11 MMA issue (one per accumulator half), 12-19 epilogue.
// What the tensor pipe needs from the issuing warp (measured with one-off probes): a kind::i8 MMA with A in tensor memory issues
// in ~11 cycles from an elected lane of warp-uniform code (45 from inside a `lane == 0` branch) and executes in N/2 cycles, but a
// loop iteration that waits on an mbarrier costs the issuing thread ~135 cycles more, whatever it waits for.  So the MMA warp runs
// its loop with all lanes and elects a lane per instruction; a block (8 MMAs) per wait is enough, because the MMAs themselves run at
// ~45 cycles each here: at N ~ 72 they are bound by shared-memory bandwidth (both halves read the B tile, the TMA writes it).  The producer side
// (commit -> decode warps wake -> tcgen05.st -> arrive -> MMA warp wakes) is a chain of several hundred cycles, so the A operand
// needs more than two stages to keep the pipe fed; tensor memory decides how many:
// two accumulator pairs (4 x 96 columns), so that an item's epilogue runs under the next item's MMAs, + 2 A stages of 64 columns (one
// 128-column block of both halves each); more A stages at the price of one accumulator pair measured the same.
// Every mbarrier wait is bounded (umma.cuh): on a timeout the CTA raises args.err, frees tensor memory and returns.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include "kernels.h"
#include "launch.cuh"
#include "dev_math.cuh"
#include "umma.cuh"

extern "C" void k_count_add(long n);

#define UM_TN UMMA_TN                /* 96 */
#define UM_WSTAGES 3                 /* four 128-column blocks each */
#ifndef UM_NACC
#define UM_NACC 2                    /* accumulator pairs (2 x 96 columns each): 2 = an item's epilogue runs under the next item's MMAs */
#endif
#define UM_NA ((512 - UM_NACC * 2 * UM_TN) / 64)   /* A stages in what is left of tensor memory: one 128-column block of both halves (64 columns) each */
#define UM_BSTAGES 8                 /* B stages in shared memory: one 128-column block each */
#define UM_WBYTES (256 * 128)
#define UM_BBYTES (UM_TN * 128)

struct __align__(16) UmShared {
    uint64_t w_full[UM_WSTAGES], w_empty[UM_WSTAGES], s_full[UM_NA], s_empty[UM_NA], b_full[UM_BSTAGES], b_empty[UM_BSTAGES], acc_full[UM_NACC], acc_empty[UM_NACC];
    uint32_t tmem_base; int abort_flag;
    __align__(16) float m_qs[8][UM_TN]; __align__(16) int m_qsum[8][UM_TN];      // per epilogue warp: scale and code-sum correction of the tile's tokens
    __align__(16) unsigned long long m_dst[8][UM_TN];                             // expert parallel, down: where each token's compact row lives (a peer's memory)
};

template <int KB, int MODE>
__global__ void __launch_bounds__(640, 1) expert_umma_kernel(ExpertArgs a, const __grid_constant__ TMap4 bmap) {
    extern __shared__ __align__(1024) uint8_t um_smem_raw[];
    uint8_t *base = (uint8_t *)(((uintptr_t)um_smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *wsm = base;                                              // UM_WSTAGES x 32 KB packed weights
    uint8_t *bsm = base + UM_WSTAGES * UM_WBYTES;                      // UM_BSTAGES x 12 KB int8 activations
    __shared__ UmShared sh_static;                                    // static, so that the compiler knows these accesses are shared-memory ones
    UmShared *sh = &sh_static;
    const int tid = threadIdx.x, lane = tid & 31, warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    constexpr bool GATEUP = MODE == 0, DENSE = MODE == 2, DOWN = MODE == 1;
    constexpr int NA = UM_NA;
    constexpr int NACC = UM_NACC;
    constexpr uint32_t ACOL = NACC * 2 * UM_TN;                     // first A column (behind the accumulators)
    static_assert(ACOL + NA * 64 <= 512, "tensor memory");
    static_assert(KB % 4 == 0, "blocks");
    const int MB = GATEUP ? 4 : (DENSE ? a.dense_mblocks : 8);      // 256-row blocks of the matrix (gate+up: 128 + 128)
    constexpr int NSB = KB / 4;
    volatile int *abortp = &sh->abort_flag;

    if (tid == 0) {
        for (int s = 0; s < UM_WSTAGES; s++) { mbar_init(&sh->w_full[s], 1); mbar_init(&sh->w_empty[s], 8); }
        // an A stage is full when its four decode warps have stored it, a B stage when its bytes have landed; both are empty again
        // when both issuing warps' MMAs on them have completed
        for (int s = 0; s < UM_NA; s++) { mbar_init(&sh->s_full[s], 4); mbar_init(&sh->s_empty[s], 2); }
        for (int s = 0; s < UM_BSTAGES; s++) { mbar_init(&sh->b_full[s], 1); mbar_init(&sh->b_empty[s], 2); }
        for (int b = 0; b < NACC; b++) { mbar_init(&sh->acc_full[b], 2); mbar_init(&sh->acc_empty[b], 8); }
        sh->abort_flag = 0; mbar_init_fence();
    }
    if (warp == 10) tmem_alloc(&sh->tmem_base, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tb = sh->tmem_base;
    bool live = true;
    const int nitems = *a.ntiles * MB;

    if (warp < 8) {
        // ---------------- decode: this warp's 32 rows of both halves, every second block, from the shared-memory ring ----------------
        const int q4 = warp & 3, par = warp >> 2, R = q4 * 32 + lane;       // R: row inside a half = tensor-memory lane
        const uint32_t a_lane = tb + ((uint32_t)(q4 * 32) << 16) + ACOL;
        uint32_t wcnt = 0, blk = 0;                                    // blk: blocks handed to the A ring so far (all warps count alike)
        for (int item = blockIdx.x; item < nitems && live; item += gridDim.x) {
#pragma unroll 1
            for (int sb = 0; sb < NSB && live; sb++, wcnt++, blk += 4) {
                const int ws = wcnt % UM_WSTAGES;
                if (!mbar_wait(&sh->w_full[ws], (wcnt / UM_WSTAGES) & 1, abortp)) { live = false; break; }
                const uint8_t *wr0 = wsm + ws * UM_WBYTES + R * 128, *wr1 = wr0 + 128 * 128;
#pragma unroll
                for (int qq = 0; qq < 2; qq++) {                         // this warp's two blocks of the weight stage
                    const int q = 2 * qq + par;
                    const uint32_t b = blk + q, as = b % NA, ap = ((b / NA) & 1) ^ 1;
                    uint32_t r0[32], r1[32];
                    auto decode = [&](const uint8_t *wr, uint32_t (&o)[32]) {
                        const uint4 v0 = *reinterpret_cast<const uint4 *>(wr + (((2 * q) ^ (R & 7)) << 4));
                        const uint4 v1 = *reinterpret_cast<const uint4 *>(wr + (((2 * q + 1) ^ (R & 7)) << 4));
                        const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
                        for (int sft = 0; sft < 4; sft++)
#pragma unroll
                            for (int j = 0; j < 8; j++) o[sft * 8 + j] = (w[j] >> (2 * sft)) & 0x03030303u;
                    };
                    decode(wr0, r0); decode(wr1, r1);                     // both halves are ready before the stage is asked for
                    if (!mbar_wait(&sh->s_empty[as], ap, abortp)) { live = false; break; }
                    tc_fence_after();
                    tmem_st32(a_lane + as * 64, r0);
                    tmem_st32(a_lane + as * 64 + 32, r1);
                    tmem_st_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sh->s_full[as]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh->w_empty[ws]);
            }
        }
    } else if (warp == 8) {
        // ---------------- weight TMA (one lane): per stage the 128 rows of half 0 and the 128 of half 1, 512 columns ----------------
        if (lane == 0) {
            uint32_t wcnt = 0;
            MoeTile tnext = blockIdx.x < nitems ? a.tiles[blockIdx.x / MB] : MoeTile{0, 0, 0, 0};      // one item ahead: no load latency at an item's start
            for (int item = blockIdx.x; item < nitems && live; item += gridDim.x) {
                const MoeTile tile = tnext;
                if (item + (int)gridDim.x < nitems) {
                    tnext = a.tiles[(item + gridDim.x) / MB];
                    const ExpertMaps *en = a.maps + tnext.ex;              // the next item's expert: its maps are in the descriptor cache when its copies start
                    if (GATEUP) { tma_prefetch_map(&en->gate); tma_prefetch_map(&en->up); } else tma_prefetch_map(&en->down);
                }
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
        // ---------------- B TMA (one lane): per 128-column block one box of the pair-ordered int8 activations ----------------
        if (lane == 0) {
            uint32_t bcnt = 0;
            MoeTile tnext = blockIdx.x < nitems ? a.tiles[blockIdx.x / MB] : MoeTile{0, 0, 0, 0};
            for (int item = blockIdx.x; item < nitems && live; item += gridDim.x) {
                const MoeTile tile = tnext;
                if (item + (int)gridDim.x < nitems) tnext = a.tiles[(item + gridDim.x) / MB];
                // only as many rows as the tile has pairs, in steps of 32 (the MMA reads (cnt + 15) & ~15 <= that many)
                const int bi = tile.cnt > 0 ? (tile.cnt - 1) >> 5 : 0;
                for (int kb = 0; kb < KB && live; kb++, bcnt++) {
                    const int s = bcnt % UM_BSTAGES;
                    if (!mbar_wait(&sh->b_empty[s], ((bcnt / UM_BSTAGES) & 1) ^ 1, abortp)) { live = false; break; }
                    mbar_expect_tx(&sh->b_full[s], 128 * 32 * (bi + 1));
                    tma_load_2d(smem_u32(bsm + s * UM_BBYTES), &bmap.m[bi], kb * 128, tile.p0, &sh->b_full[s]);
                }
            }
        }
    } else if (warp < 12) {
        // ---------------- MMA issue: warp 10 accumulator half 0, warp 11 half 1.  While one of them is inside a wait, the other's
        // MMAs keep the tensor pipe busy.  The whole warp walks the loop and waits; one elected lane issues and commits ----------------
        const uint32_t h = warp - 10;
        const uint64_t bdesc0 = smem_desc_k128(__shfl_sync(0xffffffffu, smem_u32(bsm), 0), 0);
        const uint32_t sfull0 = smem_u32(&sh->s_full[0]), sempty0 = smem_u32(&sh->s_empty[0]);
        const uint32_t bfull0 = smem_u32(&sh->b_full[0]), bempty0 = smem_u32(&sh->b_empty[0]);
        uint32_t as = 0, ap = 0, bs = 0, bp = 0, icnt = 0;
        int cnt_next = blockIdx.x < nitems ? a.tiles[blockIdx.x / MB].cnt : 0;
        for (int item = blockIdx.x; item < nitems && live; item += gridDim.x, icnt++) {
            const int cnt = __shfl_sync(0xffffffffu, cnt_next, 0);
            if (item + (int)gridDim.x < nitems) cnt_next = a.tiles[(item + gridDim.x) / MB].cnt;
            const uint32_t idesc = idesc_i8_u8s8((uint32_t)((cnt + 15) & ~15));
            const uint32_t buf = icnt % NACC, d = tb + buf * (2 * UM_TN) + h * UM_TN;
            if (!mbar_wait(&sh->acc_empty[buf], ((icnt / NACC) & 1) ^ 1, abortp)) { live = false; break; }
            tc_fence_after();
#pragma unroll 1
            for (int kb = 0; kb < KB; kb++) {
                if (!mbar_wait_addr(bfull0 + bs * 8, bp, abortp) || !mbar_wait_addr(sfull0 + as * 8, ap, abortp)) { live = false; break; }
                tc_fence_after();
                const uint32_t acol = tb + ACOL + as * 64 + h * 32;
                const uint64_t bd = bdesc0 + (uint64_t)(bs * (UM_BBYTES >> 4));
                // one election per instruction: a single predicated MMA stays in warp-uniform code
                if (elect_one()) umma_i8_ts(d, acol, bd, idesc, kb != 0);
                if (elect_one()) umma_i8_ts(d, acol + 8, bd + 2, idesc, 1);
                if (elect_one()) umma_i8_ts(d, acol + 16, bd + 4, idesc, 1);
                if (elect_one()) umma_i8_ts(d, acol + 24, bd + 6, idesc, 1);
                if (elect_one()) umma_commit_addr(sempty0 + as * 8);
                if (elect_one()) umma_commit_addr(bempty0 + bs * 8);
                if (++as == NA) { as = 0; ap ^= 1; }
                if (++bs == UM_BSTAGES) { bs = 0; bp ^= 1; }
            }
            if (live && elect_one()) umma_commit(&sh->acc_full[buf]);
            __syncwarp();
        }
    } else if (warp >= 12) {
        // ---------------- epilogue: lane = weight row, columns = tokens; warps 12-15 take the even 16-column pieces, 16-19 the odd ----------------
        const int ew = warp - 12, q4 = warp & 3, half = ew >> 2, row = q4 * 32 + lane;   // a warp reaches the tensor-memory lanes 32 (warp % 4) ..
        uint32_t icnt = 0;
        // An item's header is a chain tile -> (token of the pair ->) scale and code sum of its tokens, and tile -> pointer table -> row
        // scales: the tile is read two items ahead, the pointer table and the tokens' values one item ahead (into registers; they go
        // to shared memory when the item starts), so that an item starts without a dependent global read in front of it.
        const int stride = gridDim.x;
        constexpr int HN = UM_TN / 32;
        MoeTile t1 = blockIdx.x < nitems ? a.tiles[blockIdx.x / MB] : MoeTile{0, 0, 0, 0};
        MoeTile t2 = (int)blockIdx.x + stride < nitems ? a.tiles[(blockIdx.x + stride) / MB] : MoeTile{0, 0, 0, 0};
        ExpertPtrs ep1 = a.tab[t1.ex];
        float h_qs[HN]; int h_qsum[HN]; unsigned long long h_dst[HN];
        auto header_load = [&](const MoeTile &t) {      // the values of tokens lane, lane + 32, lane + 64 of tile t (clamped to its pairs)
#pragma unroll
            for (int i = 0; i < HN; i++) {
                const int n = lane + 32 * i, pair = t.p0 + (n < t.cnt ? n : 0), tk = (GATEUP && a.ptok) ? a.ptok[pair] : pair;
                h_qs[i] = GATEUP ? a.hqs[tk] : a.aqs[tk];
                h_qsum[i] = GATEUP ? a.hqsum[tk] : (DENSE ? a.aqsum[tk] : 32768 - a.aqsum[tk]);
                if (DOWN && a.rx_src) { const int2 sp = a.rx_src[pair]; h_dst[i] = (unsigned long long)(uintptr_t)(a.peer_wire[sp.x] + (size_t)sp.y * WIRE_PITCH); }
            }
        };
        if (blockIdx.x < nitems) header_load(t1);
        // the row scales of an item are read while the item before it is worked on (the pointer table they hang off has arrived by then)
        float s0n = 0.0f, s1n = 0.0f;
        auto scales_load = [&](const ExpertPtrs &e, const int it) {
            const int r = GATEUP ? (it % MB) * 128 + row : (it % MB) * 256 + 2 * row;
            s0n = GATEUP ? e.gs[r] : (DENSE ? e.ds[r] : 0.0f); s1n = GATEUP ? e.us[r] : (DENSE ? e.ds[r + 1] : 0.0f);
        };
        if (blockIdx.x < nitems) scales_load(ep1, blockIdx.x);
        for (int item = blockIdx.x; item < nitems && live; item += stride, icnt++) {
            const MoeTile tile = t1;
            const int mb = item % MB, cnt = tile.cnt, N = (cnt + 15) & ~15;
            const uint32_t buf = icnt % NACC;
            const int r0 = GATEUP ? mb * 128 + row : mb * 256 + 2 * row;      // down: half 0 holds row r0, half 1 row r0 + 1
            const float s0 = s0n, s1 = s1n;
            __syncwarp();
#pragma unroll
            for (int i = 0; i < HN; i++) {
                sh->m_qs[ew][lane + 32 * i] = h_qs[i]; sh->m_qsum[ew][lane + 32 * i] = h_qsum[i];
                if (DOWN && a.rx_src) sh->m_dst[ew][lane + 32 * i] = h_dst[i];
            }
            __syncwarp();
            t1 = t2; ep1 = a.tab[t1.ex];
            if (item + 2 * stride < nitems) t2 = a.tiles[(item + 2 * stride) / MB];
            if (item + stride < nitems) header_load(t1);                     // in flight while this item's pieces are worked on
            if (!mbar_wait(&sh->acc_full[buf], (icnt / NACC) & 1, abortp)) { live = false; break; }
            tc_fence_after();
            const uint32_t d_lane = tb + ((uint32_t)(q4 * 32) << 16) + buf * (2 * UM_TN);
            auto release = [&]() { tc_fence_before(); __syncwarp(); if (lane == 0) mbar_arrive(&sh->acc_empty[buf]); };
            auto piece = [&](const int c0, uint32_t (&v0)[16], uint32_t (&v1)[16]) {
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
                        return;
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
                }
            };
            // down: (dot + 32768) of this thread's two rows in one 32-bit word per token (the scales are applied where the rows are
            // combined); cd = two more bits per value, nonzero only when a value needs more than 16 bits (|dot| >= 32768)
            auto pack = [&](const int c0, const uint32_t (&v0)[16], const uint32_t (&v1)[16], uint32_t (&pk)[16], unsigned long long &cd) {
                const int4 *qsv = reinterpret_cast<const int4 *>(&sh->m_qsum[ew][c0]);
                cd = 0ull;
#pragma unroll
                for (int g4 = 0; g4 < 4; g4++) {
                    const int4 qs4 = qsv[g4]; const int bq[4] = {qs4.x, qs4.y, qs4.z, qs4.w};       // 32768 - qsum
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        const int j = g4 * 4 + k;
                        const uint32_t x0 = v0[j] + (uint32_t)bq[k], x1 = v1[j] + (uint32_t)bq[k];
                        pk[j] = __byte_perm(x0, x1, 0x5410);
                        cd |= (unsigned long long)(((x0 >> 16) & 3u) | (((x1 >> 16) & 3u) << 2)) << (4 * j);
                    }
                }
            };
            auto store = [&](const int c0, const uint32_t (&pk)[16], const unsigned long long cd) {
                const int lim = cnt - c0;                                 // tokens of this piece that exist
                const bool esc = __any_sync(0xffffffffu, cd != 0ull);
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
                            const uint32_t code = (uint32_t)(cd >> (4 * j)) & 15u;
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
                            const uint32_t code = (uint32_t)(cd >> (4 * j)) & 15u;
                            if (code) {
                                const int2 sp = a.rx_src[tile.p0 + c0 + j];
                                uint8_t *pb = a.peer_wire[sp.x];
                                atomicOr(reinterpret_cast<uint32_t *>(pb + (size_t)sp.y * WIRE_PITCH + 4096) + (r0 >> 4), code << ((r0 & 15) * 2));
                                atomicOr(reinterpret_cast<int *>(pb + rec0 + (size_t)sp.y * WIRE_REC + 8), 1 << (r0 >> 7));
                            }
                        }
                    }
                }
                if (a.dn_dots) {      // (dot + 32768) again from the 16 stored bits and the two escape bits: 0, +65536 or -65536 on top
                    int *ip = a.dn_dots + (size_t)(tile.p0 + c0) * 2048 + r0;
#pragma unroll
                    for (int j = 0; j < 16; j++) if (j < lim) {
                        const uint32_t code = (uint32_t)(cd >> (4 * j)) & 15u;
                        const int h0 = ((int)((code & 3u) ^ 2u) - 2) << 16, h1 = ((int)((code >> 2) ^ 2u) - 2) << 16;
                        *reinterpret_cast<int2 *>(ip + j * 2048) = make_int2((int)(pk[j] & 0xFFFFu) + h0 - 32768, (int)(pk[j] >> 16) + h1 - 32768);
                    }
                }
            };
            // this warp's pieces: c0 = 16 half, + 32, ...
            const int np = (N / 16 - half + 1) / 2;
            if (DOWN) {
                // piece by piece: 16 bits per value in registers, then the stores; the accumulators go back to the MMA warps as soon as
                // the last piece has been read
                if (np == 0) release();
#pragma unroll 1
                for (int k = 0; k < np; k++) {
                    uint32_t v0[16], v1[16], pk[16]; unsigned long long cd;
                    const int c0 = half * 16 + 32 * k;
                    tmem_ld16(d_lane + c0, v0); tmem_ld16(d_lane + UM_TN + c0, v1);
                    tmem_ld_wait();
                    if (k == np - 1) release();
                    pack(c0, v0, v1, pk, cd);
                    store(c0, pk, cd);
                }
            } else {
                // the last two pieces are copied out together and the accumulators handed back before their arithmetic (all of them
                // when there are at most two)
                if (np == 0) release();
                int c0 = half * 16;
                for (int k = 0; k < np; k++, c0 += 32) {
                    uint32_t v0[16], v1[16];
                    tmem_ld16(d_lane + c0, v0); tmem_ld16(d_lane + UM_TN + c0, v1);
                    if (np - k == 2) {
                        uint32_t w0[16], w1[16];
                        tmem_ld16(d_lane + c0 + 32, w0); tmem_ld16(d_lane + UM_TN + c0 + 32, w1);
                        tmem_ld_wait();
                        release();
                        piece(c0, v0, v1); piece(c0 + 32, w0, w1);
                        break;
                    }
                    tmem_ld_wait();
                    if (np - k == 1) release();
                    piece(c0, v0, v1);
                }
            }
            if (item + stride < nitems) scales_load(ep1, item + stride);
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
    launch_k(expert_umma_kernel<KB, MODE>, sms, 640, smem, st, *a, *bmap);
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
    launch_k(gather_rows_kernel, (np + 7) / 8, 256, 0, st, src, rows, dst, np);
    k_count_add(1);
}
