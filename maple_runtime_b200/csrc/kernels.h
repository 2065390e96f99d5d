/* kernels.h -- launchers of the CUDA kernels, callable from C (gpre_api.c).  Every launcher enqueues on the given
 * stream and returns; none allocates or synchronises. */
#ifndef MAPLE_KERNELS_H
#define MAPLE_KERNELS_H
#include <stdint.h>
#include <cuda_runtime_api.h>
#ifdef __cplusplus
extern "C" {
#endif

/* where one expert's six arrays live in HBM (built from the reference's GLOC/GREG tables, maple.c:1106-1131) */
typedef struct { const uint8_t *gc, *uc, *dc; const float *gs, *us, *ds; } ExpertPtrs;
/* an opaque 128-byte TMA tensor map (CUtensorMap), and the three weight matrices of one expert as 2-D byte tensors */
typedef struct __attribute__((aligned(64))) { unsigned char b[128]; } TMap;
typedef struct { TMap gate, up, down; } ExpertMaps;
/* one unit of grouped-GEMM work: used expert u, first pair p0, cnt pairs (gpu_pre.m:329-333 uses the same triple) */
typedef struct { int u, p0, cnt, ex; } MoeTile;   /* ex: index of the expert in ExpertArgs.tab / .maps */

typedef struct {
    const ExpertPtrs *tab;   /* indexed by ue[u] when ue != NULL, else by u */
    const ExpertMaps *maps;  /* same indexing; only the tcgen05 kernels read it */
    const int *ue;
    const MoeTile *tiles; const int *ntiles; int max_tiles;
    const int *ptok;         /* [np] token of each pair; NULL = the per-token arrays below are already in pair order (expert parallel) */
    /* gate+up inputs */
    const int8_t *hq; const float *hqs; const int *hqsum;          /* per token */
    float *act;              /* [np][512] */
    /* down inputs */
    const int8_t *aq; const float *aqs; const int *aqsum;          /* per pair */
    float *down;             /* [np][2048], or [np][down_stride] when down_stride != 0 (the dense projections: several matrices side by side) */
    int down_stride;
    int dense_mblocks;       /* k_dense_umma: 256-row blocks of the matrix */
    /* decode path: the down kernel quantises the fp32 SiLU outputs itself (no separate pass): act_for_down [np][512] in, and the
     * int8 rows, scales and sums it computed are also stored here for later inspection */
    const float *act_for_down; int8_t *aq_out; float *aqs_out; int *aqsum_out;
    /* optional stage outputs (NULL = off) */
    float *gate, *up; int32_t *gu_dots, *dn_dots;
    /* expert parallel: the down rows go to the rank that owns the token: rx_src[pair] = (rank, pair slot there), peer_down[rank] = its [pairs][2048] buffer */
    const int2 *rx_src; float *const *peer_down;
    /* the tcgen05 down kernel stores compact rows (see WIRE_* below) instead of fp32 ones: wire [np] rows, or in expert parallel
     * peer_wire[rank] = that rank's buffer */
    uint8_t *wire; uint8_t *const *peer_wire; int wire_cap;   /* wire_cap: pairs each such buffer is laid out for */
    int *err;                /* set to 1 by a kernel whose bounded wait ran out */
} ExpertArgs;

void k_count_reset(void); long k_count(void);

void k_norm_prep(cudaStream_t st, const float *x, const uint16_t *w, float *hn, int8_t *q, float *qs, int *qsum, int nb);
/* the same, and the normalised rows once more in the decode router's layout (hS, nb*HID*4 bytes): k_router_logits_small then takes relaid = 1 */
void k_norm_prep_relaid(cudaStream_t st, const float *x, const uint16_t *w, float *hn, int8_t *q, float *qs, int *qsum, float *hS, int nb);
/* prefill-sized batches: router_t = the layer's router rows re-laid by k_router_pack (NEXP*HID*2 bytes), hT = scratch of
 * ceil(nb/16)*16*HID*8 bytes; err receives 31 if a bounded wait inside the kernel ran out */
void k_router_pack(cudaStream_t st, const uint16_t *router, void *router_t);
/* decode batches: router_s = the rows re-laid by k_router_pack_small (NEXP*HID*2 bytes), hS = scratch of nb*HID*4 bytes */
void k_router_pack_small(cudaStream_t st, const uint16_t *router, void *router_s);
void k_router_step_order(int on);   /* nb == 1: the order of maple.c's bf_row (two chains per lane) instead of job_route_small's */
void k_router_logits_small(cudaStream_t st, const void *router_s, const float *hn, void *hS, int relaid, const float *bias, float *logits, int nb, int *err);
void k_router_logits_tile(cudaStream_t st, const void *router_t, const float *hn, void *hT, const float *bias, float *logits, int nb, int *err);
void k_topk(cudaStream_t st, const float *logits, int *top, float *topw, int nb);
/* norm + int8 as k_norm_prep, and the normalised rows once more as two fp16 terms per value (hA: [nb][4096] fp16, hi then lo) with the
 * rows' Euclidean norms (hnorm [nb]): the A operand of the tensor-core router */
void k_norm_prep_split(cudaStream_t st, const float *x, const uint16_t *w, float *hn, int8_t *q, float *qs, int *qsum, void *hA, float *hnorm, int nb);
typedef struct {
    const int *top; const float *topw; int nb;
    unsigned *mask;          /* [mask_words][256] bit words (bit b % 32 of word b / 32: token b chose the expert), then 256 counters */
    int mask_words;
    int *nu, *ue, *estart, *ustart, *utok, *slot, *tp; float *uw;
    int marked;              /* 1: the routing kernels have already set the bits and counters in mask */
    int *ecnt, *uexp;        /* optional: pairs per expert [256], expert of every pair [np] (expert parallel) */
    MoeTile *tiles_a, *tiles_b; int *ntiles_a, *ntiles_b; int tn_a, tn_b;   /* two tile lists: sizes tn_a and tn_b */
} GroupArgs;
void k_group(cudaStream_t st, const GroupArgs *g);
/* np_dev (optional, device): the pair count when only a capacity np_max is known on the host */
void k_actq(cudaStream_t st, const float *act, int8_t *aq, float *aqs, int *aqsum, const int *np_dev, int np_max);
/* SiLU*up then per-pair int8 from stored gate and up (the tensor-core path); act may be NULL */
void k_silu_quant(cudaStream_t st, const float *gate, const float *up, float *act, int8_t *aq, float *aqs, int *aqsum, int np, const int *np_dev);
void k_combine(cudaStream_t st, const float *down, const float *uw, const int *tp, const float *init, float *out, int nb);

/* register-decode + mma.sync grouped kernels (any token count; the decode-batch path); tn = 8 or 32 */
void k_gateup_mma(cudaStream_t st, const ExpertArgs *a, int tn);
/* a dense ternary matrix of `rows` rows (a multiple of 128) x 2048 columns as one "expert": tab[tile.ex].dc / .ds = its codes and
 * row scales; aq/aqs/aqsum = the int8 rows of the tokens (2048 bytes each); results go to down[token * down_stride + row] */
void k_dense_mma(cudaStream_t st, const ExpertArgs *a, int rows);
void k_down_mma(cudaStream_t st, const ExpertArgs *a, int tn);

/* tcgen05 kind::i8 grouped kernels (prefill): tiles of up to UMMA_TN tokens, codes decoded in registers into tensor memory */
#define UMMA_TN 96
/* bmap: tensor maps over the B operand rows in pair order: [pairs][2048] int8 (gate+up) or [pairs][512] int8 (down); m[i] has a box
 * of 128 bytes x 32 (i + 1) rows (the kernels use i = 0..2), so that a tile of few pairs does not pull the next experts' rows through the memory system */
typedef struct { TMap m[4]; } TMap4;
void k_gateup_umma(cudaStream_t st, const ExpertArgs *a, const TMap4 *bmap);
void k_down_umma(cudaStream_t st, const ExpertArgs *a, const TMap4 *bmap);
/* a dense matrix (rows a multiple of 256, 2048 columns) on the same kernel: maps[ex].down = its 3-D map (even / odd rows), tab[ex].ds = row
 * scales, bmap over the tokens' int8 rows, tiles of up to UMMA_TN tokens; fp32 results to down[token * down_stride + row] */
void k_dense_umma(cudaStream_t st, const ExpertArgs *a, const TMap4 *bmap);
/* dst[pair] = src[rows[pair]]: 2048-byte int8 rows put into pair (expert-grouped) order */
void k_gather_rows(cudaStream_t st, const int8_t *src, const int *rows, int8_t *dst, int np);

/* ---- the head of the attention half (k_attn_prep.cu): q/k RMS norm, half-rotary embedding, fp16 keys and values.  qkv [nb][3072]
 * = q 2048 | k 512 | v 512; pos [nb]; qn, kn [128] fp32; cs [cs_positions][32][2] (cos, sin); q [nb][2048] fp32; kc, vc [nb][512] fp16 */
void k_qk_rope(cudaStream_t st, const float *qkv, const int *pos, int nb, int glob, const float *qn, const float *kn, const float *cs, int cs_positions,
               float *q, void *kc, void *vc, int *err);

/* ---- router on the tensor cores (k_router_umma.cu): logits, top-8 and weights of nb tokens.  Tokens whose nine largest logits are
 * too close to call are recomputed in the reference's exact order of operations, so the indices are the reference's for every token;
 * weights and logits of the other tokens agree with it to ~1e-6. */
typedef struct {
    TMap amap;               /* hA [ntok_cap][4096] fp16, box 64 x 128 */
    TMap wmap;               /* the layer's router rows as fp16 [256][2048], box 64 x 256 (k_router_w16) */
    float *part;             /* [8][ntok_cap][256] partial sums */
    int nb, ntok_cap; int *err;
    const float *bias, *hnorm, *wnorm, *hn;   /* wnorm [1]: largest row norm of the layer's router (k_router_w16) */
    const void *router_s;    /* the rows re-laid by k_router_pack_small: the exact recomputation reads them */
    float *logits; int *top; float *topw;
    int *flagged, *nflagged; /* [nb], [1]: tokens that took the exact path (left for inspection) */
    unsigned *mask; int mask_words;   /* optional: the grouping's bit words and counters (GroupArgs.mask): cleared and filled here, k_group then runs with marked = 1 */
    int *done;               /* [nb] counters, zero between calls */
} RouterTensorArgs;
void k_router_w16(cudaStream_t st, const uint16_t *router, void *w16, float *wnorm);
void k_router_tensor(cudaStream_t st, const RouterTensorArgs *r);

/* ---- compact down rows (the tcgen05 path) ----
 * The down projection's results leave the expert kernel as integers and are scaled where they are combined: half the bytes of
 * fp32 rows through HBM and, in expert parallel, over NVLink.  A row of a pair is WIRE_PITCH bytes:
 *   [0, 4096)     2048 x uint16: the low 16 bits of (dot + 32768), dot = sum(code*q) - qsum in -65024..65024;
 *   [4096, 4608)  2048 x 2 bits (row r: word r/16, bits 2(r%16)..): bits 16-17 of (dot + 32768), written (OR-ed in) only when a
 *                 value does not fit 16 bits; zero otherwise and cleared again by the kernel that consumes them.
 * Behind the rows of a buffer of np_cap pairs sit np_cap records {float scale of the pair's int8 row; int index of the expert
 * in the table of down-scale pointers; int has-escapes flag; int unused}. */
#define WIRE_PITCH 4608
#define WIRE_REC 16
#define WIRE_BYTES(np_cap) ((size_t)(np_cap) * (WIRE_PITCH + WIRE_REC))
/* out[b] = init[b] (or 0) + sum over the token's pairs, in the order of tp, of uw * ((float)dot * scale * ds[expert][row]): the
 * same operations in the same order as the fp32 form (k_combine after a down kernel that scaled).  dsp[ex] = 2048 down scales. */
void k_combine_wire(cudaStream_t st, uint8_t *wire, int np_cap, const float *const *dsp, const float *uw, const int *tp,
                    const float *init, float *out, int nb);
/* fp32 rows [np][2048] from compact ones (stage comparisons); leaves the escape planes as they are */
void k_wire_decode(cudaStream_t st, const uint8_t *wire, int np_cap, const float *const *dsp, float *down, int np);

/* ---- expert parallel (k_ep.cu) ---- */
typedef struct {
    const int *all_cnt;      /* [world][256] pairs per expert of every rank */
    int rank, world;
    int *dst_base;           /* [256] where this rank's pairs of expert e start in the owner's receive buffer */
    int *nu, *ue, *ustart;   /* the owner's view of its received pairs: used local experts (global ids), starts, total at ustart[nu] */
    int *total;              /* [1] received pairs */
    MoeTile *tiles_a, *tiles_b; int *ntiles_a, *ntiles_b; int tn_a, tn_b;
} EpPlanArgs;
typedef struct {
    const int8_t *hq; const float *hqs; const int *hqsum;        /* per token, this rank */
    const int *utok, *uexp, *ustart_of_expert, *dst_base; int np, rank, experts_per_rank;
    int8_t *const *peer_hq; float *const *peer_qs; int *const *peer_qsum; int2 *const *peer_src;   /* [world] receive buffers */
} EpDispatchArgs;
void k_ep_dispatch(cudaStream_t st, const EpDispatchArgs *d);
/* Exchange buffer of a rank, written by its peers: int counts[8][256] (pairs per expert of every rank), then one 64-byte line per
 * source rank whose first word is that rank's arrival number. */
#define EP_XCH_FLAGS (8 * 256)
#define EP_XCH_INTS (EP_XCH_FLAGS + 8 * 16)
typedef struct {
    const int *ecnt;           /* this rank's [256] pairs per expert, stored into every rank's counts[rank]; NULL: rendezvous only */
    int *const *peer_xch;      /* [world] exchange buffers, this rank's own among them */
    int *xch;                  /* this rank's own */
    unsigned *epoch;           /* [1] device counter: rendezvous made so far (every rank makes the same sequence) */
    int rank, world; unsigned long long timeout_ns; int *err;
} EpXchArgs;
/* All ranks meet: everything a rank's stream did before is complete and visible before any rank's later work starts.  A wait
 * that lasts longer than timeout_ns stores 41 into *err and returns. */
void k_ep_exchange(cudaStream_t st, const EpXchArgs *a);
/* the plan; x != NULL: preceded, in the same kernel, by the rendezvous that exchanges the counts the plan reads */
void k_ep_plan(cudaStream_t st, const EpPlanArgs *p, const EpXchArgs *x);

void k_synth_experts(cudaStream_t st, uint64_t seed, int L, int e0, int ne, uint8_t *dst);

#ifdef __cplusplus
}
#endif
#endif
