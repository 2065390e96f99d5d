// k_ep.cu -- expert parallelism over one NVLink box: who sends which pairs where (plan), and the dispatch itself.
//
// Rank r keeps tokens r*T .. (r+1)*T-1 and the experts r*E .. (r+1)*E-1 (E = 256 / world).  Its pairs are grouped by
// global expert id (the same grouping as on one GPU), so the pairs for one destination rank are one contiguous run.
// After an exchange of the per-expert pair counts (peer stores plus arrival flags, ep_exchange_kernel) every rank can compute, without further communication, where each
// of its pairs lands in the owner's receive buffer: the owner's pairs are ordered by (expert, source rank, source
// order), i.e. global token order inside an expert.  The dispatch kernel then stores the int8 activation rows and their
// scales straight into the owners' buffers over NVLink (plain peer stores, no multicast, no TMA on peer memory), and the
// owners' down kernels store their result rows straight back into the token's rank (k_expert_*.cu).
#include <cuda_runtime.h>
#include <stdint.h>
#include "kernels.h"

extern "C" void k_count_add(long n);
#define NEXP 256

// Rendezvous of the ranks, with the count exchange folded in.  One CTA per rank (each on its own GPU): thread e stores this
// rank's count of expert e into every rank's table, after a CTA barrier threads 0..world-1 store this rank's arrival number
// into every rank's flag line (release, system scope) and wait (acquire, bounded by the clock) until every rank's arrival number
// has reached the same value in this rank's own lines.  Arrival numbers only grow, so a rank that is already one rendezvous
// ahead still satisfies the wait.
__device__ __forceinline__ unsigned long long ep_now_ns() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ void ep_rendezvous(const EpXchArgs &a) {
    __shared__ unsigned s_epoch;
    const int t = threadIdx.x;
    if (t == 0) s_epoch = *a.epoch + 1u;
    if (a.ecnt) {
        const int c = a.ecnt[t];
        for (int r = 0; r < a.world; r++) a.peer_xch[r][a.rank * NEXP + t] = c;
    }
    __syncthreads();                                     // the release stores below order the CTA's count stores before the flags
    const unsigned ep = s_epoch;
    if (t < a.world) {
        unsigned *dst = reinterpret_cast<unsigned *>(a.peer_xch[t] + EP_XCH_FLAGS) + a.rank * 16;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(dst), "r"(ep) : "memory");
        const unsigned *src = reinterpret_cast<const unsigned *>(a.xch + EP_XCH_FLAGS) + t * 16;
        const unsigned long long t0 = ep_now_ns();
        for (;;) {
            unsigned v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(src) : "memory");
            if ((int)(v - ep) >= 0) break;
            if (ep_now_ns() - t0 > a.timeout_ns) { atomicExch(a.err, 41); break; }
            __nanosleep(64);
        }
    }
    __syncthreads();
    if (t == 0) *a.epoch = ep;
}
__global__ void __launch_bounds__(NEXP) ep_exchange_kernel(EpXchArgs a) { ep_rendezvous(a); }

// one CTA, thread e = global expert
__global__ void __launch_bounds__(NEXP) ep_plan_kernel(EpPlanArgs p, EpXchArgs xc) {
    __shared__ int s_tot[NEXP], w_sum[8][4];
    if (xc.peer_xch) ep_rendezvous(xc);            // the count exchange first: every rank's counts are in all_cnt after it
    const int e = threadIdx.x, lane = e & 31, wid = e >> 5;
    const int epr = NEXP / p.world, owner = e / epr, mine = owner == p.rank;
    int tot = 0, before = 0;
    for (int s = 0; s < p.world; s++) { int c = p.all_cnt[s * NEXP + e]; if (s < p.rank) before += c; tot += c; }
    // offset of expert e inside its owner's buffer: the totals of the owner's earlier experts (a prefix sum over all experts,
    // taken relative to the owner's first expert)
    int incl = tot;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { int t = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += t; }
    if (lane == 31) w_sum[wid][0] = incl;
    __syncthreads();
    int woff = 0;
    for (int w = 0; w < wid; w++) woff += w_sum[w][0];
    s_tot[e] = woff + incl - tot;                  // exclusive prefix
    __syncthreads();
    p.dst_base[e] = s_tot[e] - s_tot[owner * epr] + before;
    __syncthreads();                               // w_sum is reused below
    // the owner's own view: only its experts count below
    const int cnt = mine ? tot : 0, used = cnt > 0;
    const int na = (cnt + p.tn_a - 1) / p.tn_a, nb = (cnt + p.tn_b - 1) / p.tn_b;
    int v[4] = {cnt, used, na, nb}, x[4] = {cnt, used, na, nb};
#pragma unroll
    for (int o = 1; o < 32; o <<= 1)
#pragma unroll
        for (int k = 0; k < 4; k++) { int t = __shfl_up_sync(0xffffffffu, x[k], o); if (lane >= o) x[k] += t; }
    if (lane == 31) for (int k = 0; k < 4; k++) w_sum[wid][k] = x[k];
    __syncthreads();
    int off[4] = {0, 0, 0, 0};
    for (int w = 0; w < wid; w++) for (int k = 0; k < 4; k++) off[k] += w_sum[w][k];
    const int start = off[0] + x[0] - v[0], uidx = off[1] + x[1] - v[1], ta0 = off[2] + x[2] - v[2], tb0 = off[3] + x[3] - v[3];
    if (used) {
        p.ue[uidx] = e; p.ustart[uidx] = start;
        for (int t = 0; t < na; t++) { MoeTile m = {uidx, start + t * p.tn_a, min(p.tn_a, cnt - t * p.tn_a), e}; p.tiles_a[ta0 + t] = m; }
        for (int t = 0; t < nb; t++) { MoeTile m = {uidx, start + t * p.tn_b, min(p.tn_b, cnt - t * p.tn_b), e}; p.tiles_b[tb0 + t] = m; }
    }
    if (e == NEXP - 1) {
        const int nu = uidx + used;
        *p.nu = nu; p.ustart[nu] = start + cnt; *p.total = start + cnt; *p.ntiles_a = ta0 + na; *p.ntiles_b = tb0 + nb;
    }
}
extern "C" void k_ep_plan(cudaStream_t st, const EpPlanArgs *p, const EpXchArgs *x) {
    EpXchArgs none = {0}; ep_plan_kernel<<<1, NEXP, 0, st>>>(*p, x ? *x : none); k_count_add(1);
}

// 128 threads per pair: the 2048-byte int8 row and its scale, code-sum correction and return address to the owner
__global__ void __launch_bounds__(256) ep_dispatch_kernel(EpDispatchArgs d) {
    const int i = blockIdx.x * 2 + (threadIdx.x >> 7), c = threadIdx.x & 127;
    if (i >= d.np) return;
    const int e = d.uexp[i], owner = e / d.experts_per_rank, tok = d.utok[i];
    const int slot = d.dst_base[e] + (i - d.ustart_of_expert[e]);
    reinterpret_cast<uint4 *>(d.peer_hq[owner] + (size_t)slot * 2048)[c] = reinterpret_cast<const uint4 *>(d.hq + (size_t)tok * 2048)[c];
    if (c == 0) { d.peer_qs[owner][slot] = d.hqs[tok]; d.peer_qsum[owner][slot] = d.hqsum[tok]; d.peer_src[owner][slot] = make_int2(d.rank, i); }
}
extern "C" void k_ep_dispatch(cudaStream_t st, const EpDispatchArgs *d) {
    if (d->np <= 0) return;
    ep_dispatch_kernel<<<(d->np + 1) / 2, 256, 0, st>>>(*d); k_count_add(1);
}

extern "C" void k_ep_exchange(cudaStream_t st, const EpXchArgs *a) { ep_exchange_kernel<<<1, NEXP, 0, st>>>(*a); k_count_add(1); }
