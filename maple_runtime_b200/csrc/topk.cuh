// topk.cuh -- the reference's softmax + top-8 of one token (maple.c:910-923) as a warp-level routine: lane l holds the logits of experts
// 8l..8l+7.  p = expf(l - max); the sum runs over the experts in index order (a chain through the lanes); p /= sum; eight rounds of
// "first strict maximum" (lowest index wins a tie).  Lanes 0..7 return the k-th selected expert and its probability, every lane the sum
// of the eight in selection order: weight_k = wsel / (tsum + 1e-20f).  tab: the expf table of dev_math.cuh (or a shared-memory copy).
#pragma once
#include "dev_math.cuh"

template <typename TabT>
__device__ __forceinline__ void exact_topk_warp(float (&p)[8], const int lane, const TabT *tab, int &isel, float &wsel, float &tsum) {
    float mx = -1e30f;
#pragma unroll
    for (int i = 0; i < 8; i++) mx = p[i] > mx ? p[i] : mx;
#pragma unroll
    for (int o = 16; o; o >>= 1) { float t = __shfl_xor_sync(0xffffffffu, mx, o); mx = t > mx ? t : mx; }
#pragma unroll
    for (int i = 0; i < 8; i++) p[i] = dev_expf_tab(__fsub_rn(p[i], mx), tab);
    float run = 0.0f;
    for (int l = 0; l < 32; l++) {
        if (lane == l) {
#pragma unroll
            for (int i = 0; i < 8; i++) run = __fadd_rn(run, p[i]);
        }
        run = __shfl_sync(0xffffffffu, run, l);
    }
#pragma unroll
    for (int i = 0; i < 8; i++) p[i] = __fdiv_rn(p[i], run);
    // Eight rounds of "first strict maximum" (maple.c:917-921).  Probabilities are >= +0, so their bit patterns order like the
    // values: key = bits + 1, a taken entry becomes 0.  One redux.sync gives the warp's maximum, the lowest lane holding it (and
    // the lowest of its eight entries) is the first maximum in expert order.
    unsigned key[8];
#pragma unroll
    for (int i = 0; i < 8; i++) key[i] = __float_as_uint(p[i]) + 1u;
    tsum = 0.0f; wsel = 0.0f; isel = 0;
    for (int k = 0; k < 8; k++) {
        unsigned lk = key[0];
#pragma unroll
        for (int i = 1; i < 8; i++) lk = max(lk, key[i]);
        const unsigned m = __reduce_max_sync(0xffffffffu, lk);
        const int src = __ffs(__ballot_sync(0xffffffffu, lk == m)) - 1;
        int bi = 7;
#pragma unroll
        for (int i = 6; i >= 0; i--) if (key[i] == m) bi = i;
        const int be = __shfl_sync(0xffffffffu, lane * 8 + bi, src);
        const float bv = __uint_as_float(m - 1u);
#pragma unroll
        for (int i = 0; i < 8; i++) if (lane == src && i == bi) key[i] = 0u;
        tsum = __fadd_rn(tsum, bv);
        if (lane == k) { wsel = bv; isel = be; }
    }
}
