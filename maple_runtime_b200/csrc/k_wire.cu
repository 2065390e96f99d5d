// k_wire.cu -- the consumers of the compact down rows (kernels.h WIRE_*): the weighted combine of the tensor-core path and
// the conversion to fp32 rows for stage comparisons.  sm_100a.
//
// A compact row holds dot = sum(code*q) - qsum of the down projection as 16-bit (dot + 32768), plus two more bits per value in
// an escape plane that is only touched when |dot| >= 32768.  The reference's result for row r of a pair is
// (float)dot * qs * s[r] (maple.c:425-458, two roundings) and the combine adds uw * that with one fused multiply-add per pair
// in the order of tp (maple.c:834): both are done here, in that order, so the hidden state has the reference's bits.
#include <cuda_runtime.h>
#include <stdint.h>
#include "kernels.h"
#include "launch.cuh"

extern "C" void k_count_add(long n);
#define HID 2048
#define TOPK 8
#define CW_ROWS 128                 /* rows per CTA */
#define CW_WARPS 32
#define CW_EX 256                   /* entries of the down-scale pointer table */

// escape code (2 bits) -> bits 16.. of (dot + 32768): 0, +1 or -1
__device__ __forceinline__ int wire_hi(uint32_t code) { return ((int)(code ^ 2u) - 2) << 16; }
__device__ __forceinline__ float wire_scale(int dot, float qs, float s) { return __fmul_rn(__fmul_rn((float)dot, qs), s); }

// Grid (16 row blocks, token groups).  The CTA first copies into shared memory its 128-row slice of every expert's down scales
// (128 KB) and, for every pair of its tokens, {slot, weight, scale of the pair's int8 row, expert | escape bits << 8}: after that
// the walk over the tokens has no dependent global reads left.  A warp takes one token at a time: lane l owns rows 4l..4l+3 of
// the block, reads 8 bytes of each of the token's eight compact rows and chains the eight multiply-adds.
#define CW_MAXTOK 288               /* tokens per CTA the pair table is sized for */
__global__ void __launch_bounds__(CW_WARPS * 32, 1) combine_wire_kernel(uint8_t *__restrict__ wire, int np_cap, const float *const *__restrict__ dsp,
                                                                       const float *__restrict__ uw, const int *__restrict__ tp,
                                                                       const float *__restrict__ init, float *__restrict__ out, int nb, int tok_per_cta) {
    extern __shared__ __align__(16) float sds[];                       // [CW_EX][CW_ROWS] scales, then [tok_per_cta * 8] pair records
    int4 *smeta = reinterpret_cast<int4 *>(sds + CW_EX * CW_ROWS);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, rb = blockIdx.x;
    const uint8_t *recs = wire + (size_t)np_cap * WIRE_PITCH;
    const int b_begin = blockIdx.y * tok_per_cta, b_end = min(nb, b_begin + tok_per_cta);
    {   // warp w copies the scale slices of experts w, w + 32, ...: all pointer reads first, then all row reads, so that the round
        // trips overlap; the pair records' two dependent reads run beside them
        const float *p[CW_EX / CW_WARPS]; float4 v[CW_EX / CW_WARPS];
#pragma unroll
        for (int it = 0; it < CW_EX / CW_WARPS; it++) p[it] = dsp[warp + CW_WARPS * it];
        const int npair = (b_end - b_begin) * TOPK;
        int slot[(CW_MAXTOK * TOPK + CW_WARPS * 32 - 1) / (CW_WARPS * 32)];
#pragma unroll
        for (int it = 0; it < (int)(sizeof slot / sizeof slot[0]); it++) { const int i = tid + it * CW_WARPS * 32; slot[it] = i < npair ? tp[b_begin * TOPK + i] : -1; }
#pragma unroll
        for (int it = 0; it < CW_EX / CW_WARPS; it++)
            v[it] = p[it] ? reinterpret_cast<const float4 *>(p[it] + rb * CW_ROWS)[lane] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int it = 0; it < (int)(sizeof slot / sizeof slot[0]); it++) if (slot[it] >= 0) {
            const int4 rec = *reinterpret_cast<const int4 *>(recs + (size_t)slot[it] * WIRE_REC);
            smeta[tid + it * CW_WARPS * 32] = make_int4(slot[it], __float_as_int(uw[slot[it]]), rec.x, (rec.y & 0xFF) | (rec.z << 8));
        }
#pragma unroll
        for (int it = 0; it < CW_EX / CW_WARPS; it++) reinterpret_cast<float4 *>(sds)[(warp + CW_WARPS * it) * (CW_ROWS / 4) + lane] = v[it];
    }
    __syncthreads();
    for (int b = b_begin + warp; b < b_end; b += CW_WARPS) {
        const int4 *mt = smeta + (b - b_begin) * TOPK;
        uint2 raw[TOPK];
#pragma unroll
        for (int k = 0; k < TOPK; k++) raw[k] = *reinterpret_cast<const uint2 *>(wire + (size_t)mt[k].x * WIRE_PITCH + (size_t)(rb * CW_ROWS + 4 * lane) * 2);
        const size_t o = (size_t)b * HID + rb * CW_ROWS + 4 * lane;
        float4 acc = init ? *reinterpret_cast<const float4 *>(init + o) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int k = 0; k < TOPK; k++) {
            const int4 m = mt[k];
            const float w = __int_as_float(m.y), qs = __int_as_float(m.z);
            const int ex = m.w & 0xFF, escbits = m.w >> 8;
            int d[4] = {(int)(raw[k].x & 0xFFFFu) - 32768, (int)(raw[k].x >> 16) - 32768, (int)(raw[k].y & 0xFFFFu) - 32768, (int)(raw[k].y >> 16) - 32768};
            if ((escbits >> rb) & 1) {                                    // rare: some value of this row block did not fit 16 bits
                uint32_t *pw = reinterpret_cast<uint32_t *>(wire + (size_t)m.x * WIRE_PITCH + 4096) + ((rb * CW_ROWS + 4 * lane) >> 4);
                const uint32_t bits = (*pw >> ((lane & 3) * 8)) & 0xFFu;
#pragma unroll
                for (int i = 0; i < 4; i++) d[i] += wire_hi((bits >> (2 * i)) & 3u);
                __syncwarp();
                if ((lane & 3) == 0) *pw = 0u;                            // the plane is clean again for the next layer
                if (lane == 0) atomicAnd(reinterpret_cast<int *>(wire + (size_t)np_cap * WIRE_PITCH + (size_t)m.x * WIRE_REC + 8), ~(1 << rb));
            }
            const float4 s = *reinterpret_cast<const float4 *>(sds + ex * CW_ROWS + 4 * lane);
            acc.x = __fmaf_rn(w, wire_scale(d[0], qs, s.x), acc.x); acc.y = __fmaf_rn(w, wire_scale(d[1], qs, s.y), acc.y);
            acc.z = __fmaf_rn(w, wire_scale(d[2], qs, s.z), acc.z); acc.w = __fmaf_rn(w, wire_scale(d[3], qs, s.w), acc.w);
        }
        *reinterpret_cast<float4 *>(out + o) = acc;
    }
}
extern "C" void k_combine_wire(cudaStream_t st, uint8_t *wire, int np_cap, const float *const *dsp, const float *uw, const int *tp,
                               const float *init, float *out, int nb) {
    if (nb <= 0) return;
    static int sms = 0; const int smem = CW_EX * CW_ROWS * 4 + CW_MAXTOK * TOPK * 16;
    if (!sms) {
        int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        cudaFuncSetAttribute(combine_wire_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    }
    int groups = sms / (HID / CW_ROWS); if (groups < 1) groups = 1;      // one wave of CTAs: 16 row blocks x groups
    int per = (nb + groups - 1) / groups; if (per < CW_WARPS) per = CW_WARPS;
    if (per > CW_MAXTOK) per = CW_MAXTOK;                                  /* more tokens than one wave holds: more groups */
    groups = (nb + per - 1) / per;
    launch_k(combine_wire_kernel, dim3(HID / CW_ROWS, groups), CW_WARPS * 32, smem, st, wire, np_cap, dsp, uw, tp, init, out, nb, per);
    k_count_add(1);
}

// one CTA per pair, 8 rows per thread
__global__ void __launch_bounds__(256) wire_decode_kernel(const uint8_t *__restrict__ wire, int np_cap, const float *const *__restrict__ dsp,
                                                          float *__restrict__ down, int np) {
    const int a = blockIdx.x, t = threadIdx.x;
    if (a >= np) return;
    const int4 rec = *reinterpret_cast<const int4 *>(wire + (size_t)np_cap * WIRE_PITCH + (size_t)a * WIRE_REC);
    const float qs = __int_as_float(rec.x); const float *ds = dsp[rec.y];
    const uint4 raw = reinterpret_cast<const uint4 *>(wire + (size_t)a * WIRE_PITCH)[t];
    const uint32_t r4[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t bits = 0;
    if (rec.z) bits = (reinterpret_cast<const uint32_t *>(wire + (size_t)a * WIRE_PITCH + 4096)[t >> 1] >> ((t & 1) * 16)) & 0xFFFFu;
    float o[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int d = (int)((r4[i >> 1] >> ((i & 1) * 16)) & 0xFFFFu) - 32768 + wire_hi((bits >> (2 * i)) & 3u);
        o[i] = ds ? wire_scale(d, qs, ds[8 * t + i]) : 0.0f;
    }
    float4 *dst = reinterpret_cast<float4 *>(down + (size_t)a * HID + 8 * t);
    dst[0] = make_float4(o[0], o[1], o[2], o[3]); dst[1] = make_float4(o[4], o[5], o[6], o[7]);
}
extern "C" void k_wire_decode(cudaStream_t st, const uint8_t *wire, int np_cap, const float *const *dsp, float *down, int np) {
    if (np <= 0) return;
    launch_k(wire_decode_kernel, np, 256, 0, st, wire, np_cap, dsp, down, np);
    k_count_add(1);
}
