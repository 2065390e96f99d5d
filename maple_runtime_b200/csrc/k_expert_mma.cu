// k_expert_mma.cu -- grouped ternary expert GEMMs, register-decode variant for sm_100a.
//
// The 2-bit codes go from HBM straight into registers (128-bit loads), are split into four byte-wide code words per
// 32-bit word with one shift and one mask, and feed mma.sync.m16n8k32 (u8 codes x s8 activations -> s32) as the A
// operand without touching shared memory.  This is the path for decode batches (a few tokens per expert, bound by
// the weight stream) and the fallback for any token count.
//
// Arithmetic = maple.c:425-458 (tdot_multi): tot = sum(code * q) over the row, out = (float)(tot - qsum) * qs * s[r].
// Integer sums are exact, so any summation order gives the reference's int32.
//
// Column bookkeeping.  A packed row is cols/4 bytes; each 128-column group is 32 bytes and byte j holds columns
// j, j+32, j+64, j+96 at bits 0,2,4,6 (convert.py:29-33).  A K-chunk is 256 columns = 64 packed bytes.  Thread
// (g = lane/4, t = lane%4) loads bytes [16t, 16t+16) of the chunk for rows g and g+8: group G = 2*chunk + t/2, half
// h = t%2.  Word w (0..3) of that load shifted right by 2s and masked with 0x03030303 is the four codes of columns
// G*128 + 32s + 16h + 4w + (0..3).  MMA (s, p) takes words 2p and 2p+1 as its k = 4t..4t+3 and k = 16+4t..19+4t
// slices, so the B fragment of thread (g, t) is the 16 activation bytes of token g at column G*128 + 32s + 16h:
// words 2p, 2p+1 of that 16-byte piece.  Shared memory holds the tile's activations as [chunk][s][token][t][16 B],
// which makes every B-fragment fetch one conflict-free 128-bit load.
#include <cuda_runtime.h>
#include <stdint.h>
#include "kernels.h"
#include "launch.cuh"
#include "dev_math.cuh"

extern "C" void k_count_add(long n);

__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 ldg_stream(const uint8_t *p) {   // weights are read once: do not keep them in L1
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// KCH: K-chunks of 256 columns (8 for gate/up K=2048, 2 for down K=512).  NBLK: 8-token blocks per tile.
// GATEUP: rows block A = gate rows, block B = up rows of the same index, epilogue = SiLU*up;
// otherwise A and B are two consecutive 16-row blocks of the down matrix, epilogue = scale only.
template <int KCH, int NBLK, bool GATEUP>
__global__ void __launch_bounds__(128) expert_mma_kernel(ExpertArgs a) {
    constexpr int TN = NBLK * 8, KB = KCH * 256;            // tokens per tile, bytes of one int8 activation vector
    extern __shared__ __align__(16) uint8_t smem[];          // [KCH][4][TN][4][16]
    const int tile_i = blockIdx.y;
    const int ntiles = *a.ntiles;
    const MoeTile tile = a.tiles[tile_i < a.max_tiles ? tile_i : 0];      // read beside the count, not after it
    if (tile_i >= ntiles) return;
    const ExpertPtrs ep = a.tab[tile.ex];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;

    const int rows_per_cta = GATEUP ? 64 : 128;
    const int r0 = blockIdx.x * rows_per_cta + warp * (GATEUP ? 16 : 32);
    const uint8_t *wa = (GATEUP ? ep.gc : ep.dc) + (size_t)(r0 + g) * (KB / 4) + t * 16;
    const uint8_t *wb = GATEUP ? ep.uc + (size_t)(r0 + g) * (KB / 4) + t * 16 : wa + 16 * (KB / 4);
    // the weight stream starts before anything else: the first two chunks are on their way while the activations are staged
    constexpr int PF = 2;                                   // chunks in flight (more costs occupancy and loses)
    uint4 wq[PF][4];
#pragma unroll
    for (int p = 0; p < PF; p++) if (p < KCH) {
        wq[p][0] = ldg_stream(wa + p * 64); wq[p][1] = ldg_stream(wa + 8 * (KB / 4) + p * 64);
        wq[p][2] = ldg_stream(wb + p * 64); wq[p][3] = ldg_stream(wb + 8 * (KB / 4) + p * 64);
    }

    // stage the tile's activation vectors (16-byte pieces) in fragment order
    if (GATEUP || !a.act_for_down) {
        const int8_t *src = GATEUP ? a.hq : a.aq;
        for (int i = tid; i < tile.cnt * (KB / 16); i += 128) {
            int n = i / (KB / 16), q = i % (KB / 16);            // piece q covers columns 16q..16q+15
            int row = (GATEUP && a.ptok) ? a.ptok[tile.p0 + n] : tile.p0 + n;
            uint4 v = *reinterpret_cast<const uint4 *>(src + (size_t)row * KB + q * 16);
            int G = q >> 3, s = (q & 7) >> 1, h = q & 1, c = G >> 1, tt = (G & 1) * 2 + h;
            *reinterpret_cast<uint4 *>(smem + ((((c * 4 + s) * TN + n) * 4 + tt) << 4)) = v;
        }
    } else {
        // down, decode path: the SiLU outputs arrive as fp32 and are quantised here (the prep of maple.c:831), one warp per pair;
        // every row-block CTA of the tile repeats this for the tile's few pairs, the first one also stores the result
        float *s_qs = reinterpret_cast<float *>(smem + KCH * 4 * TN * 64); int *s_qsum = reinterpret_cast<int *>(s_qs + TN);
        for (int n = warp; n < tile.cnt; n += 4) {
            const int pair = tile.p0 + n;
            const float4 *r = reinterpret_cast<const float4 *>(a.act_for_down + (size_t)pair * 512) + lane * 4;
            float v[16];
#pragma unroll
            for (int i = 0; i < 4; i++) { float4 x = r[i]; v[4 * i] = x.x; v[4 * i + 1] = x.y; v[4 * i + 2] = x.z; v[4 * i + 3] = x.w; }
            float mx = 0.0f;
#pragma unroll
            for (int i = 0; i < 16; i++) mx = fmaxf(mx, fabsf(v[i]));
#pragma unroll
            for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            const float sc = mx > 0.0f ? __fdiv_rn(mx, 127.0f) : 1.0f, inv = __fdiv_rn(1.0f, sc);
            int tot = 0; uint32_t pk[4] = {0, 0, 0, 0};
#pragma unroll
            for (int i = 0; i < 16; i++) { int qi = __float2int_rn(__fmul_rn(v[i], inv)); tot += qi; pk[i >> 2] |= (uint32_t)(qi & 0xFF) << (8 * (i & 3)); }
#pragma unroll
            for (int o = 16; o; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
            // lane holds columns 16 lane .. 16 lane + 15 = piece q = lane
            const int q = lane, G = q >> 3, s = (q & 7) >> 1, h = q & 1, c = G >> 1, tt = (G & 1) * 2 + h;
            *reinterpret_cast<uint4 *>(smem + ((((c * 4 + s) * TN + n) * 4 + tt) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            if (lane == 0) { s_qs[n] = sc; s_qsum[n] = tot; }
            if (blockIdx.x == 0) {
                reinterpret_cast<uint4 *>(a.aq_out + (size_t)pair * 512)[lane] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                if (lane == 0) { a.aqs_out[pair] = sc; a.aqsum_out[pair] = tot; }
            }
        }
    }
    __syncthreads();

    int acc_a[NBLK][4], acc_b[NBLK][4];
#pragma unroll
    for (int j = 0; j < NBLK; j++)
#pragma unroll
        for (int k = 0; k < 4; k++) { acc_a[j][k] = 0; acc_b[j][k] = 0; }

#pragma unroll
    for (int c = 0; c < KCH; c++) {
        const uint4 wa0 = wq[c % PF][0], wa1 = wq[c % PF][1], wb0 = wq[c % PF][2], wb1 = wq[c % PF][3];
        if (c + PF < KCH) {   // PF chunks in flight while this one is multiplied
            wq[c % PF][0] = ldg_stream(wa + (c + PF) * 64); wq[c % PF][1] = ldg_stream(wa + 8 * (KB / 4) + (c + PF) * 64);
            wq[c % PF][2] = ldg_stream(wb + (c + PF) * 64); wq[c % PF][3] = ldg_stream(wb + 8 * (KB / 4) + (c + PF) * 64);
        }
#pragma unroll
        for (int s = 0; s < 4; s++) {
            const uint32_t m = 0x03030303u;
            uint32_t ax0 = (wa0.x >> (2 * s)) & m, ay0 = (wa0.y >> (2 * s)) & m, az0 = (wa0.z >> (2 * s)) & m, aw0 = (wa0.w >> (2 * s)) & m;
            uint32_t ax1 = (wa1.x >> (2 * s)) & m, ay1 = (wa1.y >> (2 * s)) & m, az1 = (wa1.z >> (2 * s)) & m, aw1 = (wa1.w >> (2 * s)) & m;
            uint32_t bx0 = (wb0.x >> (2 * s)) & m, by0 = (wb0.y >> (2 * s)) & m, bz0 = (wb0.z >> (2 * s)) & m, bw0 = (wb0.w >> (2 * s)) & m;
            uint32_t bx1 = (wb1.x >> (2 * s)) & m, by1 = (wb1.y >> (2 * s)) & m, bz1 = (wb1.z >> (2 * s)) & m, bw1 = (wb1.w >> (2 * s)) & m;
            const uint8_t *bs = smem + ((((c * 4 + s) * TN + g) * 4 + t) << 4);
#pragma unroll
            for (int j = 0; j < NBLK; j++) {
                uint4 q = *reinterpret_cast<const uint4 *>(bs + j * 8 * 64);
                mma_u8s8(acc_a[j], ax0, ax1, ay0, ay1, q.x, q.y);
                mma_u8s8(acc_a[j], az0, az1, aw0, aw1, q.z, q.w);
                mma_u8s8(acc_b[j], bx0, bx1, by0, by1, q.x, q.y);
                mma_u8s8(acc_b[j], bz0, bz1, bw0, bw1, q.z, q.w);
            }
        }
    }

    // epilogue: acc[j][0..3] = (row g, token 2t), (row g, token 2t+1), (row g+8, token 2t), (row g+8, token 2t+1)
    const float *sa = GATEUP ? ep.gs : ep.ds, *sb = GATEUP ? ep.us : ep.ds + 16;
    float sca[2] = {sa[r0 + g], sa[r0 + g + 8]}, scb[2] = {sb[r0 + g], sb[r0 + g + 8]};
#pragma unroll
    for (int j = 0; j < NBLK; j++)
#pragma unroll
        for (int k = 0; k < 4; k++) {
            int n = j * 8 + 2 * t + (k & 1), rr = r0 + g + (k >> 1) * 8;
            if (n >= tile.cnt) continue;
            int pair = tile.p0 + n;
            if (GATEUP) {
                int tok = a.ptok ? a.ptok[pair] : pair;
                int da = acc_a[j][k] - a.hqsum[tok], db = acc_b[j][k] - a.hqsum[tok];
                float qs = a.hqs[tok];
                float gv = __fmul_rn(__fmul_rn((float)da, qs), sca[k >> 1]), uv = __fmul_rn(__fmul_rn((float)db, qs), scb[k >> 1]);
                a.act[(size_t)pair * 512 + rr] = dev_silu_mul(gv, uv);
                if (a.gate) { a.gate[(size_t)pair * 512 + rr] = gv; a.up[(size_t)pair * 512 + rr] = uv; }
                if (a.gu_dots) { a.gu_dots[(size_t)pair * 1024 + rr] = da; a.gu_dots[(size_t)pair * 1024 + 512 + rr] = db; }
            } else {
                int qsum_p; float qs;
                if (a.act_for_down) { const float *s_qs = reinterpret_cast<const float *>(smem + KCH * 4 * TN * 64); qs = s_qs[n]; qsum_p = reinterpret_cast<const int *>(s_qs + TN)[n]; }
                else { qs = a.aqs[pair]; qsum_p = a.aqsum[pair]; }
                int da = acc_a[j][k] - qsum_p, db = acc_b[j][k] - qsum_p;
                float *drow = a.down + (size_t)pair * (a.down_stride ? a.down_stride : 2048);
                if (a.rx_src) { const int2 sp = a.rx_src[pair]; drow = a.peer_down[sp.x] + (size_t)sp.y * 2048; }   // the row goes to the token's rank
                drow[rr] = __fmul_rn(__fmul_rn((float)da, qs), sca[k >> 1]);
                drow[rr + 16] = __fmul_rn(__fmul_rn((float)db, qs), scb[k >> 1]);
                if (a.dn_dots) { a.dn_dots[(size_t)pair * 2048 + rr] = da; a.dn_dots[(size_t)pair * 2048 + rr + 16] = db; }
            }
        }
}

template <int KCH, int NBLK, bool GATEUP>
static void launch(cudaStream_t st, const ExpertArgs *a) {
    const size_t smem = (size_t)KCH * 4 * NBLK * 8 * 64 + (GATEUP ? 0 : NBLK * 8 * 8);   // + scale and code sum per pair when down quantises itself
    static bool attr_done = false;
    if (!attr_done) { cudaFuncSetAttribute(expert_mma_kernel<KCH, NBLK, GATEUP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); attr_done = true; }
    dim3 grid(GATEUP ? 8 : 16, a->max_tiles);
    launch_k(expert_mma_kernel<KCH, NBLK, GATEUP>, grid, 128, smem, st, *a);
    k_count_add(1);
}
extern "C" void k_gateup_mma(cudaStream_t st, const ExpertArgs *a, int tn) {
    if (a->max_tiles <= 0) return;
    if (tn == 8) launch<8, 1, true>(st, a); else launch<8, 4, true>(st, a);
}
extern "C" void k_down_mma(cudaStream_t st, const ExpertArgs *a, int tn) {
    if (a->max_tiles <= 0) return;
    if (tn == 8) launch<2, 1, false>(st, a); else launch<2, 4, false>(st, a);
}

// The attention projections (gpu_pre.m:200-256 gpre_dense*): the same int8 x 2-bit product with one matrix instead of 256
// experts and every token in it: K = 2048, two 16-row blocks per warp, 128 rows per CTA, tiles of 32 tokens.
extern "C" void k_dense_mma(cudaStream_t st, const ExpertArgs *a, int rows) {
    if (a->max_tiles <= 0 || rows <= 0) return;
    const size_t smem = (size_t)8 * 4 * 32 * 64 + 32 * 8;
    static bool attr_done = false;
    if (!attr_done) { cudaFuncSetAttribute(expert_mma_kernel<8, 4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); attr_done = true; }
    launch_k(expert_mma_kernel<8, 4, false>, dim3(rows / 128, a->max_tiles), 128, smem, st, *a);
    k_count_add(1);
}
