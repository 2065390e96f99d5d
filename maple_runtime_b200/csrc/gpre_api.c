/* gpre_api.c -- the C host side: the reference's plug-in entry points (include/gpre.h) and this library's own
 * (include/gmoe.h) over the CUDA kernels in this directory.  Plain C; the only device code it touches is reached
 * through the launchers of kernels.h.  There is no CPU fallback: without a usable CUDA device every compute entry
 * point fails with a message. */
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>
#include <cuda.h>
#include <cuda_runtime_api.h>
#include "../../include/gpre.h"
#include "../../include/gmoe.h"
#include "kernels.h"
#include "synth.h"

void k_count_add(long n);

#define HID 2048
#define NEXP 256
#define TOPK 8
#define FFN 512
#define MAXREG 256         /* gpu_pre.m:21 has 64; synthetic layers that are generated again take new ids */
#define MAXSYNTH 64
#define MAP_CACHE 16384

static char g_err[512];
static int fail(const char *who, const char *fmt, ...) {
    va_list ap; va_start(ap, fmt);
    int n = snprintf(g_err, sizeof g_err, "%s: ", who);
    vsnprintf(g_err + n, sizeof g_err - (size_t)n, fmt, ap);
    va_end(ap);
    fprintf(stderr, "%s\n", g_err);
    return -1;
}
const char *gmoe_last_error(void) { return g_err; }
#define CU(who, call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) return fail(who, "%s: %s", #call, cudaGetErrorString(e_)); } while (0)
#define CUD(who, call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) { fail(who, "%s: %s", #call, cudaGetErrorString(e_)); return -1.0; } } while (0)

typedef struct { uint16_t *router, *post_ln; void *router_t, *router_s, *router_h; float *wnorm; TMap wmap; const float **dsp; ExpertPtrs *tab; ExpertMaps *maps; int set;
                 int e0, ne;            /* the experts this GPU holds for the layer (all 256, or one rank's shard) */
                 int synth_region;      /* region index + 1 of a synthetic layer's weights, released when the layer is replaced */ } LayerDev;

static struct {
    int ready, maxtok, maxp, mask_words, keep, path, nb_cur, ep_on;
    cudaStream_t st; cudaEvent_t e0, e1;
    void *reg[MAXREG]; size_t reg_len[MAXREG]; int nreg; double blit_s;
    LayerDev ly[GMOE_LAYERS];
    void *hT;                  /* hidden rows in the tile router's layout */
    uint8_t *wire;             /* compact down rows of the tcgen05 path + their records (kernels.h WIRE_*) */
    const float **dsp_call, *h_dsp[NEXP];   /* down-scale pointers of one gpre_moe call's experts; host staging */
    float *x, *hn, *y, *hqs, *logits, *topw, *uw, *act, *aqs, *down, *gate, *up, *bias;
    int8_t *hq, *aq;
    int *ecnt, *uexp, *hqsum, *top, *nu, *ue, *estart, *ustart, *utok, *slot, *tp, *aqsum, *ntiles_a, *ntiles_b, *gu_dots, *dn_dots;
    unsigned *mask; int *err, *h_err;
    MoeTile *tiles_a, *tiles_b;
    ExpertPtrs *tab_call;      /* the used experts of one gpre_moe call */
    ExpertMaps *maps_call, *h_maps; int8_t *hq_sorted; TMap4 bmap_hq, bmap_aq;
    struct { const void *key; ExpertMaps m; } *map_cache;   /* tensor maps of experts seen by gpre_moe, by code pointer */
    MoeTile *h_tiles; ExpertPtrs *h_tab;   /* host staging for the reference-shaped calls */
    double t_experts;          /* GPU seconds in gfull_moe, reported by gfull_report */
    float *ring; int ring_nb, ring_n;
    unsigned prof_mask; cudaEvent_t *pev; int pev_n, pev_cap; unsigned char *pev_stage; long *pev_launch;
    int fwd_timed;
    /* tensor-core router (k_router_umma.cu) */
    void *hA; float *hnorm, *rpart; int *flagged, *nflagged, *rdone; TMap amap; int router_mode;
} S;

/* ------------------------------------------------------------------------------------------------------------ */
static int dmalloc(void **p, size_t bytes) { return cudaMalloc(p, bytes ? bytes : 16) == cudaSuccess ? 0 : -1; }
#define ALLOC(field, bytes) do { if (dmalloc((void **)&S.field, (bytes))) return fail(who, "out of device memory for %d tokens (%s)", maxtok, #field); } while (0)

/* ---- TMA tensor maps (the driver's encoder, reached through the runtime so that libcuda is not a link dependency) ---- */
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode;
static int tmap_init(const char *who) {
    if (g_encode) return 0;
    void *fn = NULL; enum cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr) != cudaSuccess || !fn || qr != cudaDriverEntryPointSuccess)
        return fail(who, "the driver has no cuTensorMapEncodeTiled");
    g_encode = (EncodeTiledFn)fn; return 0;
}
/* rows x width bytes, row pitch bytes; box box_w x box_h; 128-byte swizzle; rows past the end read as zero */
static int tmap_bytes_2d(const char *who, TMap *out, const void *base, uint64_t width, uint64_t rows, uint64_t pitch, uint32_t box_w, uint32_t box_h) {
    cuuint64_t gdim[2] = {width, rows}, gstride[1] = {pitch};
    cuuint32_t box[2] = {box_w, box_h}, estr[2] = {1, 1};
    CUresult r = g_encode((CUtensorMap *)out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void *)base, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(who, "cuTensorMapEncodeTiled failed (%d) for %p, %llu x %llu", (int)r, base, (unsigned long long)rows, (unsigned long long)width);
    return 0;
}
/* fp16 matrix [rows][cols], row pitch in bytes; box box_cols x box_rows (box_cols * 2 = 128 bytes), 128-byte swizzle; rows past the end read as zero */
static int tmap_f16_2d(const char *who, TMap *out, const void *base, uint64_t cols, uint64_t rows, uint64_t pitch, uint32_t box_cols, uint32_t box_rows) {
    cuuint64_t gdim[2] = {cols, rows}, gstride[1] = {pitch};
    cuuint32_t box[2] = {box_cols, box_rows}, estr[2] = {1, 1};
    CUresult r = g_encode((CUtensorMap *)out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void *)base, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(who, "cuTensorMapEncodeTiled failed (%d) for the fp16 matrix at %p", (int)r, base);
    return 0;
}
/* the down codes [2048 rows][128 bytes] seen as [1024 row pairs][2 parities][128 bytes]: a box of 128 row pairs at parity h is the
 * even (h = 0) or odd (h = 1) rows of a 256-row block, which the tcgen05 down kernel puts into its two accumulators */
static int tmap_down_3d(const char *who, TMap *out, const void *base) {
    cuuint64_t gdim[3] = {128, 2, 1024}, gstride[2] = {128, 256};
    cuuint32_t box[3] = {128, 1, 128}, estr[3] = {1, 1, 1};
    CUresult r = g_encode((CUtensorMap *)out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, (void *)base, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(who, "cuTensorMapEncodeTiled failed (%d) for the down codes at %p", (int)r, base);
    return 0;
}
static int expert_maps(const char *who, const ExpertPtrs *e, ExpertMaps *m) {
    if (tmap_bytes_2d(who, &m->gate, e->gc, 512, 512, 512, 128, 128) || tmap_bytes_2d(who, &m->up, e->uc, 512, 512, 512, 128, 128) ||
        tmap_down_3d(who, &m->down, e->dc)) return -1;
    return 0;
}

/* the B operands of the tcgen05 kernels (int8 rows in pair order), one map per box height 32, 64, 96, 128 */
static int bmaps(const char *who, size_t pairs);
static int init_common(const char *who, int maxtok, int topk) {
    if (topk != TOPK) return fail(who, "topk %d is not supported (the kernels are built for %d)", topk, TOPK);
    if (maxtok < 1 || maxtok > GMOE_MAXTOK_LIMIT) return fail(who, "maxtok %d outside 1..%d", maxtok, GMOE_MAXTOK_LIMIT);
    if (S.ready && maxtok <= S.maxtok) return 0;
    if (S.ready) return fail(who, "already initialised for %d tokens; %d asked", S.maxtok, maxtok);
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev < 1) return fail(who, "no CUDA device (this library has no CPU path)");
    struct cudaDeviceProp pr; int dev = 0;
    CU(who, cudaGetDevice(&dev)); CU(who, cudaGetDeviceProperties(&pr, dev));
    if (pr.major != 10) return fail(who, "device %s is sm_%d%d; the kernels are built for sm_100a only", pr.name, pr.major, pr.minor);
    CU(who, cudaStreamCreateWithFlags(&S.st, cudaStreamNonBlocking));
    CU(who, cudaEventCreate(&S.e0)); CU(who, cudaEventCreate(&S.e1));
    size_t P = (size_t)maxtok * TOPK, T = (size_t)maxtok;
    S.maxtok = maxtok; S.maxp = (int)P; S.mask_words = (maxtok + 31) / 32;
    ALLOC(x, T * HID * 4); ALLOC(hn, T * HID * 4); ALLOC(y, T * HID * 4); ALLOC(hT, (T + 15) / 16 * 16 * HID * 8);
    ALLOC(hq, T * HID); ALLOC(hqs, T * 4); ALLOC(hqsum, T * 4);
    ALLOC(logits, T * NEXP * 4); ALLOC(top, P * 4); ALLOC(topw, P * 4); ALLOC(bias, NEXP * 4);
    ALLOC(ecnt, NEXP * 4); ALLOC(uexp, P * 4);
    ALLOC(mask, ((size_t)2 * NEXP * S.mask_words + NEXP) * 4); ALLOC(nu, 16); ALLOC(ue, NEXP * 4); ALLOC(estart, NEXP * 4);
    ALLOC(ustart, (NEXP + 1) * 4); ALLOC(utok, P * 4); ALLOC(uw, P * 4); ALLOC(slot, P * 4); ALLOC(tp, P * 4);
    ALLOC(tiles_a, (P / 8 + NEXP) * sizeof(MoeTile)); ALLOC(tiles_b, (P / 8 + NEXP) * sizeof(MoeTile));
    ALLOC(ntiles_a, 16); ALLOC(ntiles_b, 16);
    ALLOC(act, P * FFN * 4); ALLOC(gate, P * FFN * 4); ALLOC(up, P * FFN * 4); ALLOC(aq, P * FFN); ALLOC(aqs, P * 4); ALLOC(aqsum, P * 4); ALLOC(down, P * HID * 4);
    ALLOC(tab_call, NEXP * sizeof(ExpertPtrs)); ALLOC(err, 16); ALLOC(maps_call, NEXP * sizeof(ExpertMaps)); ALLOC(hq_sorted, P * HID);
    ALLOC(wire, WIRE_BYTES(P)); CU(who, cudaMemset(S.wire, 0, WIRE_BYTES(P))); ALLOC(dsp_call, NEXP * sizeof(void *));
    ALLOC(hA, T * HID * 4); ALLOC(hnorm, T * 4); ALLOC(rpart, (size_t)8 * T * NEXP * 4); ALLOC(flagged, T * 4); ALLOC(nflagged, 16); ALLOC(rdone, T * 4); CU(who, cudaMemset(S.rdone, 0, T * 4));
    CU(who, cudaMemset(S.hA, 0, T * HID * 4)); CU(who, cudaMemset(S.nflagged, 0, 16));
    if (tmap_init(who)) return -1;
    if (tmap_f16_2d(who, &S.amap, S.hA, 2 * HID, T, (uint64_t)2 * HID * 2, 64, 128)) return -1;
    if (bmaps(who, P)) return -1;
    CU(who, cudaMemset(S.err, 0, 16));
    CU(who, cudaHostAlloc((void **)&S.h_err, 16, cudaHostAllocDefault)); *S.h_err = 0;
    S.h_tiles = malloc(2 * (P / 8 + NEXP) * sizeof(MoeTile)); S.h_tab = malloc(NEXP * sizeof(ExpertPtrs));
    S.h_maps = aligned_alloc(64, NEXP * sizeof(ExpertMaps)); S.map_cache = aligned_alloc(64, MAP_CACHE * sizeof *S.map_cache);
    if (!S.h_tiles || !S.h_tab || !S.h_maps || !S.map_cache) return fail(who, "out of host memory");
    memset(S.map_cache, 0, MAP_CACHE * sizeof *S.map_cache);
    S.ready = 1;
    fprintf(stderr, "%s: %s, chunks up to %d tokens, %.0f MB of device workspace, weights resident in HBM\n", who, pr.name, maxtok,
            (double)(T * HID * 13 + P * (FFN * 5 + HID * 4 + 40)) / 1e6);
    return 0;
}
static int bmaps(const char *who, size_t pairs) {
    for (int i = 0; i < 4; i++)
        if (tmap_bytes_2d(who, &S.bmap_hq.m[i], S.hq_sorted, HID, pairs, HID, 128, 32 * (i + 1)) ||
            tmap_bytes_2d(who, &S.bmap_aq.m[i], S.aq, FFN, pairs, FFN, 128, 32 * (i + 1))) return -1;
    return 0;
}
int gpre_init(int maxtok, int topk) { return init_common("gpre", maxtok, topk); }
int gmoe_init(int maxtok) { return init_common("gmoe", maxtok, TOPK); }
int gmoe_set_device(int dev) { CU("gmoe", cudaSetDevice(dev)); return 0; }

static int keep_alloc(const char *who) {
    int maxtok = S.maxtok; size_t P = (size_t)S.maxp;
    if (!S.gu_dots) { ALLOC(gu_dots, P * 2 * FFN * 4); ALLOC(dn_dots, P * HID * 4); }
    return 0;
}
int gmoe_keep_stages(int keep) {
    if (!S.ready) return fail("gmoe", "not initialised");
    if (keep && keep_alloc("gmoe")) return -1;
    S.keep = keep != 0; return 0;
}
int gmoe_set_path(int path) { if (path < 0 || path > 2) return fail("gmoe", "path %d", path); S.path = path; return 0; }

/* ---- regions (gpu_pre.m:173-181) ------------------------------------------------------------------------------ */
static int region_add(const char *who, void *dev, size_t len) {
    if (S.nreg >= MAXREG) return fail(who, "more than %d regions", MAXREG);
    S.reg[S.nreg] = dev; S.reg_len[S.nreg] = len; return S.nreg++;
}
int gpre_region(const void *p, size_t len) {
    if (!S.ready) return fail("gpre", "gpre_region before gpre_init");
    size_t pg = (size_t)getpagesize();
    if (((uintptr_t)p % pg) || (len % pg) || !len) return fail("gpre", "region not page-aligned");
    if (S.nreg >= MAXREG) return fail("gpre", "more than %d regions", MAXREG);
    void *d = NULL;
    if (cudaMalloc(&d, len) != cudaSuccess) return fail("gpre", "region of %zu bytes does not fit in device memory", len);
    cudaEvent_t a, b; cudaEventCreate(&a); cudaEventCreate(&b);
    cudaEventRecord(a, S.st);
    cudaError_t e = cudaMemcpyAsync(d, p, len, cudaMemcpyHostToDevice, S.st);
    cudaEventRecord(b, S.st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(S.st);
    float ms = 0; cudaEventElapsedTime(&ms, a, b); cudaEventDestroy(a); cudaEventDestroy(b);
    if (e != cudaSuccess) { cudaFree(d); return fail("gpre", "copy of a region of %zu bytes: %s", len, cudaGetErrorString(e)); }
    S.blit_s += ms * 1e-3;
    return region_add("gpre", d, len);
}
int gpre_stage(size_t bytes) { (void)bytes; return 0; }
double gpre_blit_seconds(void) { return S.blit_s; }

/* (slot, offset) x 6 of one expert -> device pointers, with the bounds the reference leaves unchecked */
static int resolve(const char *who, const uint32_t *loc12, const int *regs, ExpertPtrs *out) {
    static const size_t need[6] = {MS_GU_CODES, MS_FF * 4, MS_GU_CODES, MS_FF * 4, MS_DN_CODES, MS_H * 4};
    const uint8_t *p[6];
    for (int m = 0; m < 6; m++) {
        uint32_t slot = loc12[m * 2], off = loc12[m * 2 + 1];
        if (slot > 3) return fail(who, "loc: region slot %u", slot);
        int id = regs[slot];
        if (id < 0 || id >= S.nreg) return fail(who, "loc: slot %u names region %d, which is not registered", slot, id);
        if ((size_t)off + need[m] > S.reg_len[id]) return fail(who, "loc: offset %u + %zu beyond region %d (%zu bytes)", off, need[m], id, S.reg_len[id]);
        if (off & ((m & 1) ? 3u : 15u)) return fail(who, "loc: offset %u is not %d-byte aligned", off, (m & 1) ? 4 : 16);
        p[m] = (const uint8_t *)S.reg[id] + off;
    }
    out->gc = p[0]; out->gs = (const float *)p[1]; out->uc = p[2]; out->us = (const float *)p[3]; out->dc = p[4]; out->ds = (const float *)p[5];
    return 0;
}

/* ---- layers ---------------------------------------------------------------------------------------------------- */
static void graphs_drop(void);
static void ep_forget_layer(int L);
static int layer_bufs(const char *who, int L) {
    if (!S.ready) return fail(who, "not initialised");
    if (L < 0 || L >= GMOE_LAYERS) return fail(who, "layer %d outside 0..%d", L, GMOE_LAYERS - 1);
    LayerDev *l = &S.ly[L];
    if (!l->router) {
        if (dmalloc((void **)&l->router, (size_t)NEXP * HID * 2) || dmalloc(&l->router_t, (size_t)NEXP * HID * 2) || dmalloc(&l->router_s, (size_t)NEXP * HID * 2) || dmalloc(&l->router_h, (size_t)NEXP * HID * 2) || dmalloc((void **)&l->wnorm, 16) || dmalloc((void **)&l->dsp, NEXP * sizeof(void *)) || dmalloc((void **)&l->post_ln, HID * 2) ||
            dmalloc((void **)&l->tab, NEXP * sizeof(ExpertPtrs)) || dmalloc((void **)&l->maps, NEXP * sizeof(ExpertMaps)))
            return fail(who, "out of device memory for layer %d", L);
        if (tmap_f16_2d(who, &l->wmap, l->router_h, HID, NEXP, (uint64_t)HID * 2, 64, 256)) return -1;
    }
    return 0;
}
int gmoe_set_layer(int L, const uint16_t *router, const uint16_t *post_ln, const uint32_t *gloc, const int *regs) {
    if (layer_bufs("gmoe", L)) return -1;
    if (!router || !gloc || !regs) return fail("gmoe", "gmoe_set_layer: null table");
    LayerDev *l = &S.ly[L];
    for (int e = 0; e < NEXP; e++) if (resolve("gmoe", gloc + e * 12, regs, &S.h_tab[e]) || expert_maps("gmoe", &S.h_tab[e], &S.h_maps[e])) return -1;
    CU("gmoe", cudaMemcpyAsync(l->maps, S.h_maps, NEXP * sizeof(ExpertMaps), cudaMemcpyHostToDevice, S.st));
    uint16_t ones[HID]; for (int i = 0; i < HID; i++) ones[i] = 0x3F80;
    CU("gmoe", cudaMemcpyAsync(l->router, router, (size_t)NEXP * HID * 2, cudaMemcpyHostToDevice, S.st));
    k_router_pack(S.st, l->router, l->router_t); k_router_pack_small(S.st, l->router, l->router_s); k_router_w16(S.st, l->router, l->router_h, l->wnorm);
    CU("gmoe", cudaMemcpyAsync(l->post_ln, post_ln ? post_ln : ones, HID * 2, cudaMemcpyHostToDevice, S.st));
    CU("gmoe", cudaMemcpyAsync(l->tab, S.h_tab, NEXP * sizeof(ExpertPtrs), cudaMemcpyHostToDevice, S.st));
    for (int e = 0; e < NEXP; e++) S.h_dsp[e] = S.h_tab[e].ds;
    CU("gmoe", cudaMemcpyAsync(l->dsp, S.h_dsp, NEXP * sizeof(void *), cudaMemcpyHostToDevice, S.st));
    CU("gmoe", cudaStreamSynchronize(S.st));
    graphs_drop(); ep_forget_layer(L);            /* replays and the gathered down scales would still name the old weights */
    l->e0 = 0; l->ne = NEXP; l->set = 1; return 0;
}
int gmoe_synth_layer(uint64_t seed, int L, int e0, int ne) {
    if (layer_bufs("gmoe", L)) return -1;
    if (e0 < 0 || ne < 1 || e0 + ne > NEXP) return fail("gmoe", "experts %d..%d outside 0..255", e0, e0 + ne - 1);
    LayerDev *l = &S.ly[L];
    uint8_t *w = NULL; size_t len = (size_t)ne * MS_EXPERT_BYTES;
    if (cudaStreamSynchronize(S.st) != cudaSuccess) return fail("gmoe", "synthetic layer %d: the stream reports an earlier error", L);
    if (l->synth_region) {                         /* the layer is generated again: its old weights go, the region id stays (empty) */
        cudaFree(S.reg[l->synth_region - 1]); S.reg[l->synth_region - 1] = NULL; S.reg_len[l->synth_region - 1] = 0; l->synth_region = 0;
    }
    l->set = 0;
    if (cudaMalloc((void **)&w, len) != cudaSuccess) return fail("gmoe", "no device memory for %d experts of layer %d", ne, L);
    const int rid = region_add("gmoe", w, len);
    if (rid < 0) { cudaFree(w); return -1; }
    l->synth_region = rid + 1;
    k_synth_experts(S.st, seed, L, e0, ne, w);
    memset(S.h_tab, 0, NEXP * sizeof(ExpertPtrs)); memset(S.h_maps, 0, NEXP * sizeof(ExpertMaps));
    for (int e = e0; e < e0 + ne; e++) {
        const uint8_t *b = w + (size_t)(e - e0) * MS_EXPERT_BYTES; ExpertPtrs *t = &S.h_tab[e];
        t->gc = b; t->gs = (const float *)(b + MS_GU_CODES); t->uc = b + MS_GU_BYTES; t->us = (const float *)(b + MS_GU_BYTES + MS_GU_CODES);
        t->dc = b + 2 * MS_GU_BYTES; t->ds = (const float *)(b + 2 * MS_GU_BYTES + MS_DN_CODES);
        if (expert_maps("gmoe", t, &S.h_maps[e])) return -1;
    }
    if (cudaMemcpyAsync(l->maps, S.h_maps, NEXP * sizeof(ExpertMaps), cudaMemcpyHostToDevice, S.st) != cudaSuccess) return fail("gmoe", "synthetic layer %d: tensor maps", L);
    uint16_t *r = malloc((size_t)NEXP * HID * 2), nw[HID];
    if (!r) return fail("gmoe", "out of host memory");
    msynth_router(seed, L, r); msynth_norm(seed, L, nw);
    cudaError_t e1 = cudaMemcpyAsync(l->router, r, (size_t)NEXP * HID * 2, cudaMemcpyHostToDevice, S.st);
    k_router_pack(S.st, l->router, l->router_t); k_router_pack_small(S.st, l->router, l->router_s); k_router_w16(S.st, l->router, l->router_h, l->wnorm);
    cudaError_t e2 = cudaMemcpyAsync(l->post_ln, nw, HID * 2, cudaMemcpyHostToDevice, S.st);
    cudaError_t e3 = cudaMemcpyAsync(l->tab, S.h_tab, NEXP * sizeof(ExpertPtrs), cudaMemcpyHostToDevice, S.st);
    for (int e = 0; e < NEXP; e++) S.h_dsp[e] = S.h_tab[e].ds;
    if (e3 == cudaSuccess) e3 = cudaMemcpyAsync(l->dsp, S.h_dsp, NEXP * sizeof(void *), cudaMemcpyHostToDevice, S.st);
    cudaError_t e4 = cudaStreamSynchronize(S.st);
    free(r);
    if (e1 || e2 || e3 || e4) return fail("gmoe", "synthetic layer %d: %s", L, cudaGetErrorString(e1 ? e1 : e2 ? e2 : e3 ? e3 : e4));
    e4 = cudaGetLastError();
    if (e4) return fail("gmoe", "synthetic layer %d: %s", L, cudaGetErrorString(e4));
    graphs_drop(); ep_forget_layer(L);
    l->e0 = e0; l->ne = ne; l->set = 1; return 0;
}

/* ---- per-stage events ------------------------------------------------------------------------------------------ */
static long g_before;
/* inside a stream capture the event becomes an event-record node of the graph, re-recorded at every replay */
static void prof_record(cudaEvent_t ev) {
    enum cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(S.st, &cs);
    if (cs == cudaStreamCaptureStatusActive) cudaEventRecordWithFlags(ev, S.st, cudaEventRecordExternal); else cudaEventRecord(ev, S.st);
}
static void prof_begin(int stage) {
    if (!(S.prof_mask >> stage & 1u)) return;
    if (S.pev_n + 2 > S.pev_cap) {
        int cap = S.pev_cap ? S.pev_cap * 2 : 1024;
        cudaEvent_t *ev = realloc(S.pev, (size_t)cap * sizeof *ev);
        unsigned char *st = realloc(S.pev_stage, (size_t)cap); long *ln = realloc(S.pev_launch, (size_t)cap * sizeof *ln);
        if (!ev || !st || !ln) return;
        for (int i = S.pev_cap; i < cap; i++) cudaEventCreate(&ev[i]);
        S.pev = ev; S.pev_stage = st; S.pev_launch = ln; S.pev_cap = cap;
    }
    g_before = k_count();
    prof_record(S.pev[S.pev_n]);
}
static void prof_end(int stage) {
    if (!(S.prof_mask >> stage & 1u) || S.pev_n + 2 > S.pev_cap) return;
    prof_record(S.pev[S.pev_n + 1]);
    S.pev_stage[S.pev_n] = (unsigned char)stage; S.pev_launch[S.pev_n] = k_count() - g_before; S.pev_n += 2;
}
int gmoe_profile(unsigned mask) { if (!S.ready) return fail("gmoe", "not initialised"); S.prof_mask = mask; return 0; }
int gmoe_profile_read(double *secs, long *launches) {
    if (!S.ready) return fail("gmoe", "not initialised");
    CU("gmoe", cudaStreamSynchronize(S.st));
    for (int s = 0; s < GMOE_STAGES; s++) { secs[s] = 0; launches[s] = 0; }
    for (int i = 0; i < S.pev_n; i += 2) {
        float ms = 0; cudaEventElapsedTime(&ms, S.pev[i], S.pev[i + 1]);
        secs[S.pev_stage[i]] += ms * 1e-3; launches[S.pev_stage[i]] += S.pev_launch[i];
    }
    S.pev_n = 0; return 0;
}

/* ---- the stages ------------------------------------------------------------------------------------------------ */
static int tile_tn(int nb) { return nb <= 256 ? 8 : 32; }

static int use_umma(int nb) { return S.path == 2 || (S.path == 0 && nb >= 512); }
static void fill_expert_args(ExpertArgs *a, const ExpertPtrs *tab, const ExpertMaps *maps, const int *ue, int nb) {
    memset(a, 0, sizeof *a);
    a->tab = tab; a->maps = maps; a->ue = ue; a->ptok = S.utok; a->err = S.err;
    if (use_umma(nb)) { a->tiles = S.tiles_b; a->ntiles = S.ntiles_b; a->max_tiles = nb * TOPK / UMMA_TN + NEXP; }
    else { a->tiles = S.tiles_a; a->ntiles = S.ntiles_a; a->max_tiles = nb * TOPK / tile_tn(nb) + NEXP; }
    a->hq = S.hq; a->hqs = S.hqs; a->hqsum = S.hqsum; a->act = S.act;
    a->aq = S.aq; a->aqs = S.aqs; a->aqsum = S.aqsum; a->down = S.down; a->wire = S.wire; a->wire_cap = S.maxp;
    if (S.keep || use_umma(nb)) { a->gate = S.gate; a->up = S.up; }          /* the tensor-core GEMM always stores gate and up */
    if (S.keep) { a->gu_dots = S.gu_dots; a->dn_dots = S.dn_dots; }
}
static void run_group_m(int nb, int marked) {
    GroupArgs g; memset(&g, 0, sizeof g); g.marked = marked && nb > 256;
    g.top = S.top; g.topw = S.topw; g.nb = nb; g.mask = S.mask; g.mask_words = S.mask_words; g.nu = S.nu; g.ue = S.ue; g.estart = S.estart;
    g.ustart = S.ustart; g.utok = S.utok; g.slot = S.slot; g.tp = S.tp; g.uw = S.uw; g.ecnt = S.ecnt; g.uexp = S.uexp;
    g.tiles_a = S.tiles_a; g.tiles_b = S.tiles_b; g.ntiles_a = S.ntiles_a; g.ntiles_b = S.ntiles_b; g.tn_a = tile_tn(nb); g.tn_b = UMMA_TN;
    k_group(S.st, &g);
    if (use_umma(nb) && !S.ep_on) k_gather_rows(S.st, S.hq, S.utok, S.hq_sorted, nb * TOPK);   /* the permute: int8 rows into pair order for the TMA */
}
static void run_group(int nb) { run_group_m(nb, 0); }
/* which: 1 gateup, 2 actq, 4 down; dsp: the down-scale pointers the tiles' expert indices name (the combine needs the same) */
static void run_experts(const ExpertPtrs *tab, const ExpertMaps *maps, const float *const *dsp, const int *ue, int nb, int which) {
    ExpertArgs a; fill_expert_args(&a, tab, maps, ue, nb);
    int tn = tile_tn(nb);
    int um = use_umma(nb);
    if (which & 1) {
        prof_begin(4);
        if (um) k_gateup_umma(S.st, &a, &S.bmap_hq); else k_gateup_mma(S.st, &a, tn);
        prof_end(4);
    }
    const int fuse_q = !um && tn == 8 && which == 7;           /* decode batches: the down kernel quantises the SiLU outputs itself */
    if (fuse_q) { a.act_for_down = S.act; a.aq_out = S.aq; a.aqs_out = S.aqs; a.aqsum_out = S.aqsum; }
    if ((which & 2) && !fuse_q) {
        prof_begin(5);
        if (um) k_silu_quant(S.st, S.gate, S.up, S.keep ? S.act : NULL, S.aq, S.aqs, S.aqsum, nb * TOPK, NULL);
        else k_actq(S.st, S.act, S.aq, S.aqs, S.aqsum, NULL, nb * TOPK);
        prof_end(5);
    }
    if (which & 4) {
        prof_begin(6);
        if (um) k_down_umma(S.st, &a, &S.bmap_aq); else k_down_mma(S.st, &a, tn);
        if (um && S.keep) k_wire_decode(S.st, S.wire, S.maxp, dsp, S.down, nb * TOPK);     /* fp32 rows for stage comparisons */
        prof_end(6);
    }
}
/* weighted combine of the pairs' down rows into out (init + sum): compact rows after the tcgen05 kernel, fp32 rows otherwise */
static void run_combine(const float *const *dsp, int nb, const float *init, float *out) {
    if (use_umma(nb)) k_combine_wire(S.st, S.wire, S.maxp, dsp, S.uw, S.tp, init, out, nb);
    else k_combine(S.st, S.down, S.uw, S.tp, init, out, nb);
}
/* router logits: batches past the decode sizes take the tiled kernel, decode batches the one-wait kernel, both on re-laid rows */
#define ROUTER_TILE_MIN 257
static void run_router_relaid(const LayerDev *l, const float *bias, int nb, int relaid) {   /* relaid: the norm kernel already wrote S.hT */
    if (nb >= ROUTER_TILE_MIN) k_router_logits_tile(S.st, l->router_t, S.hn, S.hT, bias, S.logits, nb, S.err);
    else k_router_logits_small(S.st, l->router_s, S.hn, S.hT, relaid, bias, S.logits, nb, S.err);
}
static void run_router(const LayerDev *l, const float *bias, int nb) { run_router_relaid(l, bias, nb, 0); }
/* Which router: 0 = by size (tensor cores from 512 tokens on), 1 = always the exact-order kernels, 2 = tensor cores for every size. */
int gmoe_set_step_order(int on) { graphs_drop(); k_router_step_order(on); return 0; }   /* a captured layer loop holds the kernel of the old order */
int gmoe_set_router(int mode) { if (mode < 0 || mode > 2) return fail("gmoe", "router mode %d", mode); S.router_mode = mode; return 0; }
static int tensor_router(int nb) { return S.router_mode == 2 || (S.router_mode == 0 && nb >= 512); }
int gmoe_router_flagged(void) { int n = -1; if (S.ready) { cudaMemcpyAsync(&n, S.nflagged, 4, cudaMemcpyDeviceToHost, S.st); cudaStreamSynchronize(S.st); } return n; }
/* logits, top-8 and weights on the tensor cores (needs the fp16 terms and norms that k_norm_prep_split left) */
static void run_router_tensor_m(const LayerDev *l, const float *bias, int nb, int mark) {
    RouterTensorArgs r; memset(&r, 0, sizeof r);
    r.amap = S.amap; r.wmap = l->wmap; r.part = S.rpart; r.nb = nb; r.ntok_cap = S.maxtok; r.err = S.err;
    r.bias = bias; r.hnorm = S.hnorm; r.wnorm = l->wnorm; r.hn = S.hn; r.router_s = l->router_s;
    r.logits = S.logits; r.top = S.top; r.topw = S.topw; r.flagged = S.flagged; r.nflagged = S.nflagged; r.done = S.rdone;
    if (mark && nb > 256) { r.mask = S.mask; r.mask_words = S.mask_words; }      /* the grouping's bits and counters come out of the routing kernels */
    k_router_tensor(S.st, &r);
}
static void run_router_tensor(const LayerDev *l, const float *bias, int nb) { run_router_tensor_m(l, bias, nb, 0); }
/* norm + int8 of the layer's input; decode batches also get the router's layout in the same pass */
static int run_norm(const float *x, const uint16_t *w, int nb) {
    if (tensor_router(nb)) { k_norm_prep_split(S.st, x, w, S.hn, S.hq, S.hqs, S.hqsum, S.hA, S.hnorm, nb); return 0; }
    if (nb < ROUTER_TILE_MIN) { k_norm_prep_relaid(S.st, x, w, S.hn, S.hq, S.hqs, S.hqsum, (float *)S.hT, nb); return 1; }
    k_norm_prep(S.st, x, w, S.hn, S.hq, S.hqs, S.hqsum, nb); return 0;
}
/* the MoE half of layer L on the device buffers: norm != 0: x -> hn -> ... -> x += ; else hn -> ... -> y */
static void run_layer(int L, int nb, int norm, const float *bias) {
    LayerDev *l = &S.ly[L];
    prof_begin(0); const int relaid = run_norm(norm ? S.x : S.hn, norm ? l->post_ln : NULL, nb); prof_end(0);
    const int tr = tensor_router(nb);
    if (tr) { prof_begin(1); run_router_tensor_m(l, bias, nb, 1); prof_end(1); }
    else {
        prof_begin(1); run_router_relaid(l, bias, nb, relaid); prof_end(1);
        prof_begin(2); k_topk(S.st, S.logits, S.top, S.topw, nb); prof_end(2);
    }
    prof_begin(3); run_group_m(nb, tr); prof_end(3);
    run_experts(l->tab, l->maps, (const float *const *)l->dsp, S.ue, nb, 7);
    prof_begin(7);
    if (norm) run_combine((const float *const *)l->dsp, nb, S.x, S.x); else run_combine((const float *const *)l->dsp, nb, NULL, S.y);
    prof_end(7);
}
static int g_ep_call;      /* set while an expert-parallel entry point runs its checks */
static int ep_rank_shard(int *e0, int *ne);
static int check_call(const char *who, int L, int nb) {
    if (!S.ready) return fail(who, "not initialised");
    if (L < 0 || L >= GMOE_LAYERS || !S.ly[L].set) return fail(who, "layer %d has no weights", L);
    if (nb < 1 || nb > S.maxtok) return fail(who, "%d tokens outside 1..%d", nb, S.maxtok);
    const LayerDev *l = &S.ly[L];
    if (g_ep_call) {
        int e0 = 0, ne = 0; ep_rank_shard(&e0, &ne);
        if (l->e0 > e0 || l->e0 + l->ne < e0 + ne) return fail(who, "layer %d holds experts %d..%d, this rank needs %d..%d", L, l->e0, l->e0 + l->ne - 1, e0, e0 + ne - 1);
    } else {
        /* after gmoe_ep_init the work buffers are sized and filled for the expert-parallel path only */
        if (S.ep_on) return fail(who, "expert parallelism is set up: use the gmoe_ep_* entry points");
        if (l->e0 != 0 || l->ne != NEXP) return fail(who, "layer %d holds only experts %d..%d (an expert-parallel shard); a single-GPU call needs all %d", L, l->e0, l->e0 + l->ne - 1, NEXP);
    }
    return 0;
}
static const float *bias_dev(const float *bias) {
    if (!bias) return NULL;
    cudaMemcpyAsync(S.bias, bias, NEXP * 4, cudaMemcpyHostToDevice, S.st);
    return S.bias;
}
static double finish(const char *who) {
    cudaMemcpyAsync(S.h_err, S.err, 4, cudaMemcpyDeviceToHost, S.st);
    cudaError_t e = cudaStreamSynchronize(S.st);
    if (e == cudaSuccess && *S.h_err) {
        const int code = *S.h_err;
        *S.h_err = 0; cudaMemsetAsync(S.err, 0, 4, S.st);
        /* a down pass that no combine followed leaves escape bits behind; they are only ever OR-ed into */
        cudaMemsetAsync(S.wire, 0, WIRE_BYTES((size_t)S.maxp), S.st);
        fail(who, "a kernel gave up waiting (code %d: %s); results are invalid", code,
             code == 41 ? "a rank did not arrive at the expert-parallel rendezvous" : code == 31 ? "router operand ring" : "barrier inside an expert kernel");
        return -1.0;
    }
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) { fail(who, "%s", cudaGetErrorString(e)); return -1.0; }
    float ms = 0; cudaEventElapsedTime(&ms, S.e0, S.e1);
    return ms * 1e-3;
}

/* ---- the layer loop as a CUDA graph: one launch per call instead of a dozen per layer -------------------------------------
 * Every kernel takes its sizes from device memory, so the sequence for (nb, l0, nl, bias?, path) is the same every time and can
 * be replayed.  The second call with a key captures it (the first runs plainly, so that one-time set-up calls made by the
 * launchers happen outside a capture).  Per-stage events are captured as event-record nodes, so gmoe_profile_read then reports the
 * last replay.  Not used while stages are kept or when GMOE_GRAPH=0 is set.  Under expert parallelism the ranks make the same calls
 * in the same order, so they capture and replay together; nothing on that path calls NCCL. */
#define NGRAPH 64
static struct { int nb, l0, nl, bias, path, prof, ep, seen; long launches; cudaGraphExec_t exec; } GR[NGRAPH];
static int g_graph_on = -1;
static long g_graph_launches;
long gmoe_graph_launches(void) { return g_graph_launches; }
/* forget every captured layer loop: the weights or the work buffers a replay names have changed */
static void graphs_drop(void) {
    if (S.st) cudaStreamSynchronize(S.st);
    for (int i = 0; i < NGRAPH; i++) { if (GR[i].exec) cudaGraphExecDestroy(GR[i].exec); memset(&GR[i], 0, sizeof GR[i]); }
}
static int graphs_on(void) {
    if (g_graph_on < 0) { const char *e = getenv("GMOE_GRAPH"); g_graph_on = !(e && e[0] == '0'); }
    return g_graph_on && !S.keep;
}
int gmoe_set_graph(int on) { g_graph_on = on != 0; return 0; }
static int run_layer_ep(int L, int nb, const float *bias);
static int layers_run(int nb, int l0, int nl, const float *bd, int ep) {
    for (int L = l0; L < l0 + nl; L++) { if (ep) { if (run_layer_ep(L, nb, bd)) return -1; } else run_layer(L, nb, 1, bd); }
    return 0;
}
static int layers_enqueue_ep(int nb, int l0, int nl, const float *bd, int ep) {
    if (!graphs_on()) return layers_run(nb, l0, nl, bd, ep);
    int k = -1, free_k = -1;
    for (int i = 0; i < NGRAPH; i++) {
        if (GR[i].seen && GR[i].nb == nb && GR[i].l0 == l0 && GR[i].nl == nl && GR[i].bias == (bd != NULL) && GR[i].path == S.path + 8 * S.router_mode && GR[i].prof == (int)S.prof_mask && GR[i].ep == ep) { k = i; break; }
        if (!GR[i].seen && free_k < 0) free_k = i;
    }
    if (k < 0) {   /* first sight: run plainly and remember the key */
        if (layers_run(nb, l0, nl, bd, ep)) return -1;
        if (free_k < 0) {   /* table full: the slots are reused in turn */
            static int victim;
            free_k = victim; victim = (victim + 1) % NGRAPH;
            cudaStreamSynchronize(S.st);
            if (GR[free_k].exec) cudaGraphExecDestroy(GR[free_k].exec);
            memset(&GR[free_k], 0, sizeof GR[free_k]);
        }
        if (free_k >= 0) { GR[free_k].nb = nb; GR[free_k].l0 = l0; GR[free_k].nl = nl; GR[free_k].bias = bd != NULL; GR[free_k].path = S.path + 8 * S.router_mode; GR[free_k].prof = (int)S.prof_mask; GR[free_k].ep = ep; GR[free_k].seen = 1; GR[free_k].exec = NULL; }
        return 0;
    }
    if (!GR[k].exec) {
        cudaGraph_t g = NULL; long before = k_count();
        if (cudaStreamBeginCapture(S.st, cudaStreamCaptureModeThreadLocal) != cudaSuccess) return layers_run(nb, l0, nl, bd, ep);
        int bad = layers_run(nb, l0, nl, bd, ep);
        cudaError_t e = cudaStreamEndCapture(S.st, &g);
        GR[k].launches = k_count() - before;
        if (e == cudaSuccess && !bad) e = cudaGraphInstantiate(&GR[k].exec, g, 0);
        if (g) cudaGraphDestroy(g);
        if (bad) { GR[k].exec = NULL; GR[k].seen = 2; return -1; }
        if (e != cudaSuccess) { GR[k].exec = NULL; GR[k].seen = 2; cudaGetLastError(); return fail("gmoe", "graph capture of the layer loop: %s", cudaGetErrorString(e)); }
    } else k_count_add(GR[k].launches);
    CU("gmoe", cudaGraphLaunch(GR[k].exec, S.st));
    g_graph_launches++;
    return 0;
}
static int layers_enqueue(int nb, int l0, int nl, const float *bd) { return layers_enqueue_ep(nb, l0, nl, bd, 0); }

double gmoe_moe(int L, const float *x, int nb, float *y, const float *bias) {
    if (check_call("gmoe", L, nb)) return -1.0;
    CUD("gmoe", cudaMemcpyAsync(S.hn, x, (size_t)nb * HID * 4, cudaMemcpyHostToDevice, S.st));
    const float *bd = bias_dev(bias);
    cudaEventRecord(S.e0, S.st);
    run_layer(L, nb, 0, bd);
    cudaEventRecord(S.e1, S.st);
    CUD("gmoe", cudaMemcpyAsync(y, S.y, (size_t)nb * HID * 4, cudaMemcpyDeviceToHost, S.st));
    S.nb_cur = nb;
    return finish("gmoe");
}
int gmoe_forward_dev(int nb, int l0, int nl, const float *bias) {
    for (int L = l0; L < l0 + nl; L++) if (check_call("gmoe", L, nb)) return -1;
    const float *bd = bias_dev(bias);
    cudaEventRecord(S.e0, S.st);
    if (layers_enqueue(nb, l0, nl, bd)) return -1;
    cudaEventRecord(S.e1, S.st);
    S.nb_cur = nb;
    return 0;
}
int gmoe_chunks_upload(const float *x, int nb, int nchunks) {
    if (!S.ready || nb < 1 || nb > S.maxtok || nchunks < 1) return fail("gmoe", "ring of %d chunks of %d tokens", nchunks, nb);
    if (S.ring) { cudaFree(S.ring); S.ring = NULL; }
    size_t bytes = (size_t)nchunks * nb * HID * 4;
    if (cudaMalloc((void **)&S.ring, bytes) != cudaSuccess) return fail("gmoe", "no device memory for %d chunks", nchunks);
    CU("gmoe", cudaMemcpyAsync(S.ring, x, bytes, cudaMemcpyHostToDevice, S.st)); CU("gmoe", cudaStreamSynchronize(S.st));
    S.ring_nb = nb; S.ring_n = nchunks; return 0;
}
int gmoe_forward_chunk(int chunk, int nb, int l0, int nl, const float *bias) {
    if (!S.ring || nb != S.ring_nb || chunk < 0 || chunk >= S.ring_n) return fail("gmoe", "chunk %d of %d tokens is not in the ring", chunk, nb);
    for (int L = l0; L < l0 + nl; L++) if (check_call("gmoe", L, nb)) return -1;
    const float *bd = bias_dev(bias);
    cudaEventRecord(S.e0, S.st);
    cudaMemcpyAsync(S.x, S.ring + (size_t)chunk * nb * HID, (size_t)nb * HID * 4, cudaMemcpyDeviceToDevice, S.st);
    if (layers_enqueue(nb, l0, nl, bd)) return -1;
    cudaEventRecord(S.e1, S.st);
    S.nb_cur = nb; return 0;
}
double gmoe_sync(void) { if (!S.ready) { fail("gmoe", "not initialised"); return -1.0; } return finish("gmoe"); }
int gmoe_x_upload(const float *x, int nb) {
    if (!S.ready || nb < 1 || nb > S.maxtok) return fail("gmoe", "upload of %d tokens", nb);
    CU("gmoe", cudaMemcpyAsync(S.x, x, (size_t)nb * HID * 4, cudaMemcpyHostToDevice, S.st)); S.nb_cur = nb; return 0;
}
int gmoe_x_download(float *x, int nb) {
    if (!S.ready || nb < 1 || nb > S.maxtok) return fail("gmoe", "download of %d tokens", nb);
    CU("gmoe", cudaMemcpyAsync(x, S.x, (size_t)nb * HID * 4, cudaMemcpyDeviceToHost, S.st));
    CU("gmoe", cudaStreamSynchronize(S.st)); return 0;
}
double gmoe_forward(float *x, int nb, int l0, int nl, const float *bias) {   /* the seconds include both copies */
    for (int L = l0; L < l0 + nl; L++) if (check_call("gmoe", L, nb)) return -1.0;
    const float *bd = bias_dev(bias);
    cudaEventRecord(S.e0, S.st);
    CUD("gmoe", cudaMemcpyAsync(S.x, x, (size_t)nb * HID * 4, cudaMemcpyHostToDevice, S.st));
    if (layers_enqueue(nb, l0, nl, bd)) return -1.0;
    CUD("gmoe", cudaMemcpyAsync(x, S.x, (size_t)nb * HID * 4, cudaMemcpyDeviceToHost, S.st));
    cudaEventRecord(S.e1, S.st);
    S.nb_cur = nb;
    return finish("gmoe");
}
/* ---- host in / host out without waiting: up to two chunks outstanding (see gmoe.h) ------------------------------------
 * A chunk goes host -> xin[k] on one copy stream, xin[k] -> x, the layer loop, x -> xout[k] on the library's stream, xout[k] -> host on
 * a second copy stream; k alternates.  Events order the three streams and guard the two staging slots against their reuse. */
static struct {
    cudaStream_t in, out; int ready, seq, done;          /* seq: chunks submitted, done: chunks waited for */
    float *xin[2], *xout[2]; size_t cap;                /* staging slots on the card, cap floats each */
    cudaEvent_t mark, start[2], loaded[2], taken[2], ran[2], stored[2];
    int *h_err;                                          /* pinned: the kernels' error word as each chunk left it */
} PIPE;
static int pipe_setup(int nb) {
    if (!PIPE.ready) {
        CU("gmoe", cudaStreamCreateWithFlags(&PIPE.in, cudaStreamNonBlocking)); CU("gmoe", cudaStreamCreateWithFlags(&PIPE.out, cudaStreamNonBlocking));
        CU("gmoe", cudaEventCreate(&PIPE.mark));
        for (int k = 0; k < 2; k++) {
            CU("gmoe", cudaEventCreate(&PIPE.start[k])); CU("gmoe", cudaEventCreate(&PIPE.stored[k]));
            CU("gmoe", cudaEventCreateWithFlags(&PIPE.loaded[k], cudaEventDisableTiming)); CU("gmoe", cudaEventCreateWithFlags(&PIPE.taken[k], cudaEventDisableTiming));
            CU("gmoe", cudaEventCreateWithFlags(&PIPE.ran[k], cudaEventDisableTiming));
        }
        if (cudaHostAlloc((void **)&PIPE.h_err, 2 * sizeof(int), cudaHostAllocDefault) != cudaSuccess) return fail("gmoe", "no pinned memory");
        PIPE.h_err[0] = PIPE.h_err[1] = 0;
        CU("gmoe", cudaEventRecord(PIPE.mark, PIPE.in));
        PIPE.ready = 1;
    }
    const size_t need = (size_t)nb * HID;
    if (need > PIPE.cap) {
        if (PIPE.seq != PIPE.done) return fail("gmoe", "a larger chunk while chunks are outstanding");
        for (int k = 0; k < 2; k++) { cudaFree(PIPE.xin[k]); cudaFree(PIPE.xout[k]); PIPE.xin[k] = PIPE.xout[k] = NULL; }
        PIPE.cap = 0;
        for (int k = 0; k < 2; k++)
            if (dmalloc((void **)&PIPE.xin[k], need * 4) || dmalloc((void **)&PIPE.xout[k], need * 4)) return fail("gmoe", "no device memory for the staging slots of %d tokens", nb);
        PIPE.cap = need;
    }
    return 0;
}
static int ep_layer_scales(int L);
int gmoe_forward_submit(const float *x_in, float *x_out, int nb, int l0, int nl, const float *bias) {
    if (!S.ready) return fail("gmoe", "not initialised");
    if (PIPE.seq - PIPE.done >= 2) return fail("gmoe", "two chunks are outstanding: gmoe_forward_wait first");
    g_ep_call = S.ep_on;
    for (int L = l0; L < l0 + nl; L++) if (check_call("gmoe", L, nb) || (S.ep_on && ep_layer_scales(L))) { g_ep_call = 0; return -1; }
    g_ep_call = 0;
    if (pipe_setup(nb)) return -1;
    const float *bd = bias_dev(bias);
    const int k = PIPE.seq & 1; const size_t bytes = (size_t)nb * HID * 4;
    if (PIPE.seq >= 2) CU("gmoe", cudaStreamWaitEvent(PIPE.in, PIPE.taken[k], 0));           /* the slot's previous chunk has been moved into x */
    CU("gmoe", cudaEventRecord(PIPE.start[k], PIPE.in));
    CU("gmoe", cudaMemcpyAsync(PIPE.xin[k], x_in, bytes, cudaMemcpyHostToDevice, PIPE.in));
    CU("gmoe", cudaEventRecord(PIPE.loaded[k], PIPE.in));
    CU("gmoe", cudaStreamWaitEvent(S.st, PIPE.loaded[k], 0));
    CU("gmoe", cudaMemcpyAsync(S.x, PIPE.xin[k], bytes, cudaMemcpyDeviceToDevice, S.st));
    CU("gmoe", cudaEventRecord(PIPE.taken[k], S.st));
    if (layers_enqueue_ep(nb, l0, nl, bd, S.ep_on)) return -1;
    if (PIPE.seq >= 2) CU("gmoe", cudaStreamWaitEvent(S.st, PIPE.stored[k], 0));             /* the slot's previous result has left the card */
    CU("gmoe", cudaMemcpyAsync(PIPE.xout[k], S.x, bytes, cudaMemcpyDeviceToDevice, S.st));
    CU("gmoe", cudaEventRecord(PIPE.ran[k], S.st));
    CU("gmoe", cudaStreamWaitEvent(PIPE.out, PIPE.ran[k], 0));
    CU("gmoe", cudaMemcpyAsync(x_out, PIPE.xout[k], bytes, cudaMemcpyDeviceToHost, PIPE.out));
    CU("gmoe", cudaMemcpyAsync(&PIPE.h_err[k], S.err, 4, cudaMemcpyDeviceToHost, PIPE.out));
    CU("gmoe", cudaEventRecord(PIPE.stored[k], PIPE.out));
    S.nb_cur = nb; PIPE.seq++;
    return 0;
}
double gmoe_forward_wait(void) {
    if (!PIPE.ready || PIPE.seq == PIPE.done) { fail("gmoe", "gmoe_forward_wait: nothing outstanding"); return -1.0; }
    const int k = PIPE.done & 1;
    PIPE.done++;
    cudaError_t e = cudaEventSynchronize(PIPE.stored[k]);
    if (e != cudaSuccess) { fail("gmoe", "%s", cudaGetErrorString(e)); return -1.0; }
    if (PIPE.h_err[k]) {
        const int code = PIPE.h_err[k];
        PIPE.h_err[k] = 0; cudaStreamSynchronize(S.st); cudaMemsetAsync(S.err, 0, 4, S.st); cudaMemsetAsync(S.wire, 0, WIRE_BYTES((size_t)S.maxp), S.st);
        fail("gmoe", "a kernel gave up waiting (code %d); results are invalid", code);
        return -1.0;
    }
    float ms = 0.0f;
    if (cudaEventElapsedTime(&ms, PIPE.mark, PIPE.stored[k]) != cudaSuccess) { fail("gmoe", "event timing"); return -1.0; }
    return (double)ms * 1e-3;
}
int gmoe_forward_mark(void) {
    if (!S.ready) return fail("gmoe", "not initialised");
    if (pipe_setup(1)) return -1;
    if (PIPE.seq != PIPE.done) return fail("gmoe", "gmoe_forward_mark with chunks outstanding");
    CU("gmoe", cudaStreamSynchronize(S.st)); CU("gmoe", cudaStreamSynchronize(PIPE.out));
    CU("gmoe", cudaEventRecord(PIPE.mark, PIPE.in));
    return 0;
}
int gmoe_post_norm(int L, int nb, float *logits) {
    if (check_call("gmoe", L, nb)) return -1;
    LayerDev *l = &S.ly[L];
    k_norm_prep(S.st, S.x, l->post_ln, S.hn, S.hq, S.hqs, S.hqsum, nb);
    run_router(l, NULL, nb);
    if (logits) CU("gmoe", cudaMemcpyAsync(logits, S.logits, (size_t)nb * NEXP * 4, cudaMemcpyDeviceToHost, S.st));
    CU("gmoe", cudaStreamSynchronize(S.st));
    return 0;
}

/* ---- page-locking the host's own buffers ---------------------------------------------------------------------------
 * The reference's card path reads and writes the host's hidden-state arrays in place (unified memory, gpu_pre.m:318-385); here they cross
 * PCIe, and from pageable memory that runs at a quarter of the link's rate.  maple.c holds those arrays for the life of the process
 * (HNB, YB: static).  With the policy on (gpre_pin_policy(1), or GPRE_PIN_HOST=1 in the environment when the library initialises: no
 * change to the host's source), a buffer of 1 MB or more that a reference-shaped call sees a second time at the same address and length
 * is page-locked where it lies (cudaHostRegister) and stays so; the copies then run at the rate of pinned memory.  A registration that
 * fails is forgotten and the buffer stays pageable.  Off by default: a host that frees a registered buffer and maps new memory at the
 * same address would have the card read the old pages.  Turning the policy off releases every registration. */
#define PIN_SLOTS 64
static struct { const void *p; size_t len; int seen, pinned; } PIN[PIN_SLOTS];
static int pin_on = -1;      /* -1: not decided yet (the environment is read at the first call) */
int gpre_pin_policy(int on) {
    pin_on = on != 0;
    if (!pin_on) {
        if (S.ready) cudaStreamSynchronize(S.st);
        for (int i = 0; i < PIN_SLOTS; i++) { if (PIN[i].pinned && cudaHostUnregister((void *)PIN[i].p) != cudaSuccess) cudaGetLastError(); }
        memset(PIN, 0, sizeof PIN);
    }
    return 0;
}
static void host_buffer_seen(const void *p, size_t len) {
    if (pin_on < 0) { const char *e = getenv("GPRE_PIN_HOST"); pin_on = e && e[0] == '1'; }
    if (!pin_on || !p || len < (1u << 20)) return;
    int free_i = -1;
    for (int i = 0; i < PIN_SLOTS; i++) {
        if (PIN[i].p == p && PIN[i].len == len) {
            if (!PIN[i].pinned && PIN[i].seen == 1) {
                PIN[i].seen = 2;
                if (cudaHostRegister((void *)p, len, cudaHostRegisterDefault) == cudaSuccess) PIN[i].pinned = 1; else cudaGetLastError();
            }
            return;
        }
        if (!PIN[i].p && free_i < 0) free_i = i;
    }
    if (free_i >= 0) { PIN[free_i].p = p; PIN[free_i].len = len; PIN[free_i].seen = 1; PIN[free_i].pinned = 0; }
}

/* ---- the reference-shaped calls: grouping supplied by the host ---------------------------------------------------- */
static int upload_grouping(const char *who, int nb, int nu, const uint32_t *loc, const int *regs, const int *ustart,
                           const int *ptok, const float *pw, const int *tp) {
    if (!S.ready) return fail(who, "not initialised");
    if (S.ep_on) return fail(who, "expert parallelism is set up: use the gmoe_ep_* entry points");
    if (nb < 1 || nb > S.maxtok) return fail(who, "%d tokens outside 1..%d", nb, S.maxtok);
    if (nu < 1 || nu > NEXP) return fail(who, "%d used experts outside 1..%d", nu, NEXP);
    int np = ustart[nu];
    if (np != nb * TOPK) return fail(who, "%d pairs for %d tokens (need %d per token)", np, nb, TOPK);
    if (ustart[0] != 0) return fail(who, "ustart[0] = %d", ustart[0]);
    int tn = tile_tn(nb), nt = 0, ntb = 0;
    MoeTile *h_tb = S.h_tiles + ((size_t)S.maxp / 8 + NEXP);
    for (int u = 0; u < nu; u++) {
        if (ustart[u + 1] <= ustart[u]) return fail(who, "used expert %d has no pairs", u);
        if (resolve(who, loc + u * 12, regs, &S.h_tab[u])) return -1;
        {   /* tensor maps of this expert: encoded the first time its codes are seen */
            size_t hsh = ((uintptr_t)S.h_tab[u].gc >> 8) % MAP_CACHE;
            if (S.map_cache[hsh].key != (const void *)S.h_tab[u].gc) {
                if (expert_maps(who, &S.h_tab[u], &S.map_cache[hsh].m)) return -1;
                S.map_cache[hsh].key = S.h_tab[u].gc;
            }
            S.h_maps[u] = S.map_cache[hsh].m;
        }
        for (int p = ustart[u]; p < ustart[u + 1]; p += tn) {   /* gpu_pre.m:329-333 */
            MoeTile m = {u, p, ustart[u + 1] - p < tn ? ustart[u + 1] - p : tn, u}; S.h_tiles[nt++] = m;
        }
        for (int p = ustart[u]; p < ustart[u + 1]; p += UMMA_TN) {
            MoeTile m = {u, p, ustart[u + 1] - p < UMMA_TN ? ustart[u + 1] - p : UMMA_TN, u}; h_tb[ntb++] = m;
        }
    }
    for (int a = 0; a < np; a++) if (ptok[a] < 0 || ptok[a] >= nb) return fail(who, "ptok[%d] = %d", a, ptok[a]);
    for (int i = 0; i < np; i++) if (tp[i] < 0 || tp[i] >= np) return fail(who, "tp[%d] = %d", i, tp[i]);
    for (int u = 0; u < NEXP; u++) S.h_dsp[u] = u < nu ? S.h_tab[u].ds : NULL;
    CU(who, cudaMemcpyAsync(S.dsp_call, S.h_dsp, NEXP * sizeof(void *), cudaMemcpyHostToDevice, S.st));
    CU(who, cudaMemcpyAsync(S.tab_call, S.h_tab, (size_t)nu * sizeof(ExpertPtrs), cudaMemcpyHostToDevice, S.st));
    CU(who, cudaMemcpyAsync(S.maps_call, S.h_maps, (size_t)nu * sizeof(ExpertMaps), cudaMemcpyHostToDevice, S.st));
    CU(who, cudaMemcpyAsync(S.tiles_a, S.h_tiles, (size_t)nt * sizeof(MoeTile), cudaMemcpyHostToDevice, S.st));
    CU(who, cudaMemcpyAsync(S.ntiles_a, &nt, 4, cudaMemcpyHostToDevice, S.st));
    CU(who, cudaMemcpyAsync(S.tiles_b, h_tb, (size_t)ntb * sizeof(MoeTile), cudaMemcpyHostToDevice, S.st));
    CU(who, cudaMemcpyAsync(S.ntiles_b, &ntb, 4, cudaMemcpyHostToDevice, S.st));
    CU(who, cudaMemcpyAsync(S.ustart, ustart, (size_t)(nu + 1) * 4, cudaMemcpyHostToDevice, S.st));
    CU(who, cudaMemcpyAsync(S.nu, &nu, 4, cudaMemcpyHostToDevice, S.st));
    CU(who, cudaMemcpyAsync(S.utok, ptok, (size_t)np * 4, cudaMemcpyHostToDevice, S.st));
    CU(who, cudaMemcpyAsync(S.uw, pw, (size_t)np * 4, cudaMemcpyHostToDevice, S.st));
    CU(who, cudaMemcpyAsync(S.tp, tp, (size_t)np * 4, cudaMemcpyHostToDevice, S.st));
    CU(who, cudaStreamSynchronize(S.st));   /* the host staging arrays are reused by the next call */
    return 0;
}
double gpre_moe(const float *x, int nb, int nu, const uint32_t *loc, const int *regs, const int *next,
                const int *ustart, const int *ptok, const float *pw, const int *tp, float *y) {
    (void)next;
    if (upload_grouping("gpre", nb, nu, loc, regs, ustart, ptok, pw, tp)) return -1.0;
    host_buffer_seen(x, (size_t)nb * HID * 4); host_buffer_seen(y, (size_t)nb * HID * 4);
    CUD("gpre", cudaMemcpyAsync(S.hn, x, (size_t)nb * HID * 4, cudaMemcpyHostToDevice, S.st));
    cudaEventRecord(S.e0, S.st);
    k_norm_prep(S.st, S.hn, NULL, S.hn, S.hq, S.hqs, S.hqsum, nb);
    if (use_umma(nb)) k_gather_rows(S.st, S.hq, S.utok, S.hq_sorted, nb * TOPK);
    run_experts(S.tab_call, S.maps_call, (const float *const *)S.dsp_call, NULL, nb, 7);
    run_combine((const float *const *)S.dsp_call, nb, NULL, S.y);
    cudaEventRecord(S.e1, S.st);
    CUD("gpre", cudaMemcpyAsync(y, S.y, (size_t)nb * HID * 4, cudaMemcpyDeviceToHost, S.st));
    S.nb_cur = nb;
    return finish("gpre");
}
void gfull_begin(const float *x, int nb, int pos0) {
    (void)pos0;
    if (!S.ready || nb < 1 || nb > S.maxtok) { fail("gfull", "gfull_begin with %d tokens", nb); return; }
    host_buffer_seen(x, (size_t)nb * HID * 4);
    cudaMemcpyAsync(S.x, x, (size_t)nb * HID * 4, cudaMemcpyHostToDevice, S.st); S.nb_cur = nb;
}
void gfull_moe(int nu, const uint32_t *loc, const int *regs, const int *ustart, const int *ptok, const float *pw, const int *tp) {
    int nb = S.nb_cur;
    if (upload_grouping("gfull", nb, nu, loc, regs, ustart, ptok, pw, tp)) return;
    cudaEventRecord(S.e0, S.st);
    if (use_umma(nb)) k_gather_rows(S.st, S.hq, S.utok, S.hq_sorted, nb * TOPK);
    run_experts(S.tab_call, S.maps_call, (const float *const *)S.dsp_call, NULL, nb, 7);            /* hq/hqs/hqsum were left by gmoe_post_norm */
    run_combine((const float *const *)S.dsp_call, nb, S.x, S.x);
    cudaEventRecord(S.e1, S.st);
    S.fwd_timed = 1;
}
void gfull_read(float *x, const uint16_t **ko) {
    if (ko) *ko = NULL;
    if (!S.ready) { fail("gfull", "not initialised"); return; }
    if (x) { host_buffer_seen(x, (size_t)S.nb_cur * HID * 4); cudaMemcpyAsync(x, S.x, (size_t)S.nb_cur * HID * 4, cudaMemcpyDeviceToHost, S.st); }
    cudaError_t e = cudaStreamSynchronize(S.st);
    if (e != cudaSuccess) fail("gfull", "%s", cudaGetErrorString(e));
    else if (S.fwd_timed) { float ms = 0; cudaEventElapsedTime(&ms, S.e0, S.e1); S.t_experts += ms * 1e-3; S.fwd_timed = 0; }
}
void gfull_write_x(const float *x) {
    if (!S.ready) return;
    cudaMemcpyAsync(S.x, x, (size_t)S.nb_cur * HID * 4, cudaMemcpyHostToDevice, S.st); cudaStreamSynchronize(S.st);
}
int gfull_maxtok(void) { return S.maxtok; }
void gfull_report(void) { fprintf(stderr, "gfull: card %.2f s experts\n", S.t_experts); }

/* ---- parity hooks ----------------------------------------------------------------------------------------------- */
static int named(const char *name, void **p, size_t *cap) {
    size_t T = (size_t)S.maxtok, P = (size_t)S.maxp;
    struct { const char *n; void *p; size_t cap; } tab[] = {
        {"x", S.x, T * HID * 4}, {"hn", S.hn, T * HID * 4}, {"y", S.y, T * HID * 4}, {"hq", S.hq, T * HID}, {"hqs", S.hqs, T * 4},
        {"hqsum", S.hqsum, T * 4}, {"logits", S.logits, T * NEXP * 4}, {"top", S.top, P * 4}, {"topw", S.topw, P * 4},
        {"nu", S.nu, 4}, {"ue", S.ue, NEXP * 4}, {"ustart", S.ustart, (NEXP + 1) * 4}, {"utok", S.utok, P * 4}, {"uw", S.uw, P * 4},
        {"tp", S.tp, P * 4}, {"gate", S.gate, P * FFN * 4}, {"up", S.up, P * FFN * 4}, {"act", S.act, P * FFN * 4}, {"aq", S.aq, P * FFN},
        {"aqs", S.aqs, P * 4}, {"aqsum", S.aqsum, P * 4}, {"down", S.down, P * HID * 4}, {"gu_dots", S.gu_dots, P * 2 * FFN * 4},
        {"dn_dots", S.dn_dots, P * HID * 4}, {"bias", S.bias, NEXP * 4}};
    for (size_t i = 0; i < sizeof tab / sizeof tab[0]; i++) if (!strcmp(tab[i].n, name)) { *p = tab[i].p; *cap = tab[i].cap; return 0; }
    return -1;
}
int gmoe_peek(const char *name, void *dst, size_t bytes) {
    void *p; size_t cap;
    if (!S.ready) return fail("gmoe", "not initialised");
    if (named(name, &p, &cap)) return fail("gmoe", "no buffer named %s", name);
    if (!p) return fail("gmoe", "buffer %s is only kept after gmoe_keep_stages(1)", name);
    if (bytes > cap) return fail("gmoe", "%zu bytes asked of %s, which holds %zu", bytes, name, cap);
    CU("gmoe", cudaMemcpyAsync(dst, p, bytes, cudaMemcpyDeviceToHost, S.st)); CU("gmoe", cudaStreamSynchronize(S.st)); return 0;
}
int gmoe_poke(const char *name, const void *src, size_t bytes) {
    void *p; size_t cap;
    if (!S.ready) return fail("gmoe", "not initialised");
    if (named(name, &p, &cap)) return fail("gmoe", "no buffer named %s", name);
    if (!p) return fail("gmoe", "buffer %s is only kept after gmoe_keep_stages(1)", name);
    if (bytes > cap) return fail("gmoe", "%zu bytes given for %s, which holds %zu", bytes, name, cap);
    CU("gmoe", cudaMemcpyAsync(p, src, bytes, cudaMemcpyHostToDevice, S.st)); CU("gmoe", cudaStreamSynchronize(S.st)); return 0;
}
int gmoe_stage(const char *name, int L, int nb) {
    if (check_call("gmoe", L, nb)) return -1;
    LayerDev *l = &S.ly[L];
    cudaEventRecord(S.e0, S.st);
    if (!strcmp(name, "norm")) k_norm_prep(S.st, S.x, l->post_ln, S.hn, S.hq, S.hqs, S.hqsum, nb);
    else if (!strcmp(name, "prep")) k_norm_prep(S.st, S.hn, NULL, S.hn, S.hq, S.hqs, S.hqsum, nb);
    else if (!strcmp(name, "router")) run_router(l, NULL, nb);
    else if (!strcmp(name, "router_bias")) run_router(l, S.bias, nb);
    else if (!strcmp(name, "router_tensor") || !strcmp(name, "router_tensor_bias")) {      /* from hn: fp16 terms, logits, top-8, weights */
        k_norm_prep_split(S.st, S.hn, NULL, S.hn, S.hq, S.hqs, S.hqsum, S.hA, S.hnorm, nb);
        run_router_tensor(l, name[13] ? S.bias : NULL, nb);
    }
    else if (!strcmp(name, "topk")) k_topk(S.st, S.logits, S.top, S.topw, nb);
    else if (!strcmp(name, "group")) run_group(nb);
    else if (!strcmp(name, "gateup")) { if (use_umma(nb)) k_gather_rows(S.st, S.hq, S.utok, S.hq_sorted, nb * TOPK); run_experts(l->tab, l->maps, (const float *const *)l->dsp, S.ue, nb, 1); }
    else if (!strcmp(name, "actq")) run_experts(l->tab, l->maps, (const float *const *)l->dsp, S.ue, nb, 2);
    else if (!strcmp(name, "down")) { if (use_umma(nb)) cudaMemsetAsync(S.wire, 0, WIRE_BYTES((size_t)S.maxp), S.st);   /* a repeated stage must not find the previous run's escape bits */
        run_experts(l->tab, l->maps, (const float *const *)l->dsp, S.ue, nb, 4); }
    else if (!strcmp(name, "combine_y")) run_combine((const float *const *)l->dsp, nb, NULL, S.y);
    else if (!strcmp(name, "combine_x")) run_combine((const float *const *)l->dsp, nb, S.x, S.x);
    else return fail("gmoe", "no stage named %s", name);
    cudaEventRecord(S.e1, S.st);
    return finish("gmoe") < 0 ? -1 : 0;
}

int gmoe_region_count(void) { return S.nreg; }
int gmoe_region_read(int region, size_t off, void *dst, size_t bytes) {
    if (!S.ready || region < 0 || region >= S.nreg) return fail("gmoe", "no region %d", region);
    if (off + bytes > S.reg_len[region]) return fail("gmoe", "bytes %zu..%zu beyond region %d (%zu bytes)", off, off + bytes, region, S.reg_len[region]);
    CU("gmoe", cudaMemcpyAsync(dst, (const uint8_t *)S.reg[region] + off, bytes, cudaMemcpyDeviceToHost, S.st));
    CU("gmoe", cudaStreamSynchronize(S.st)); return 0;
}

/* ---- utilities ---------------------------------------------------------------------------------------------------- */
long gmoe_launch_count(void) { return k_count(); }
void *gmoe_pinned_alloc(size_t bytes) { void *p = NULL; if (cudaHostAlloc(&p, bytes, cudaHostAllocDefault) != cudaSuccess) { fail("gmoe", "no pinned memory (%zu bytes)", bytes); return NULL; } return p; }
void gmoe_pinned_free(void *p) { if (p) cudaFreeHost(p); }
int gmoe_device_info(char *name, int namelen, int *sms, size_t *hbm_bytes) {
    int dev = 0; struct cudaDeviceProp pr;
    CU("gmoe", cudaGetDevice(&dev)); CU("gmoe", cudaGetDeviceProperties(&pr, dev));
    if (name && namelen > 0) { strncpy(name, pr.name, (size_t)namelen - 1); name[namelen - 1] = 0; }
    if (sms) *sms = pr.multiProcessorCount;
    if (hbm_bytes) *hbm_bytes = pr.totalGlobalMem;
    return 0;
}

/* ---- entry points of the reference ABI that are outside the MoE path (see gpre.h) ---------------------------------- */
int gfull_init(int ctx, int maxtok, int win, const float *norms, const uint16_t *router, const float *cs) {
    (void)ctx; (void)maxtok; (void)win; (void)norms; (void)router; (void)cs;
    fprintf(stderr, "gfull: attention on the card is not part of this library\n"); return -1;
}
double gfull_attn(int L, int glob, float *rl) { (void)L; (void)glob; (void)rl; return 0.0; }
/* ---- the head of the attention half on the card: q/k norm, rotary embedding, fp16 cache rows (see gmoe.h) -------------------- */
static struct { float *cs; int positions; float *qkv, *q, *norms; void *kc, *vc; int *pos; int cap; } AT;
int gmoe_rope_table(const float *cs, int positions) {
    if (!S.ready) return fail("gmoe", "not initialised");
    if (!cs || positions < 1 || positions > (1 << 20)) return fail("gmoe", "rope table of %d positions", positions);
    CU("gmoe", cudaStreamSynchronize(S.st));
    if (AT.cs) { cudaFree(AT.cs); AT.cs = NULL; AT.positions = 0; }
    if (dmalloc((void **)&AT.cs, (size_t)positions * 64 * 4)) return fail("gmoe", "no device memory for the rope table");
    CU("gmoe", cudaMemcpyAsync(AT.cs, cs, (size_t)positions * 64 * 4, cudaMemcpyHostToDevice, S.st)); CU("gmoe", cudaStreamSynchronize(S.st));
    AT.positions = positions; return 0;
}
double gmoe_qk_rope(const float *qkv, const int *pos, int nb, int glob, const float *qn, const float *kn, float *q, uint16_t *kc, uint16_t *vc) {
    if (!S.ready) { fail("gmoe", "not initialised"); return -1.0; }
    if (nb < 1 || nb > S.maxtok) { fail("gmoe", "gmoe_qk_rope: %d tokens outside 1..%d", nb, S.maxtok); return -1.0; }
    if (!qkv || !pos || !qn || !kn || !q || !kc || !vc) { fail("gmoe", "gmoe_qk_rope: null argument"); return -1.0; }
    if (!glob && !AT.cs) { fail("gmoe", "gmoe_qk_rope on a local layer before gmoe_rope_table"); return -1.0; }
    if (!glob) for (int b = 0; b < nb; b++) if (pos[b] < 0 || pos[b] >= AT.positions) { fail("gmoe", "gmoe_qk_rope: position %d of token %d outside the table (%d positions)", pos[b], b, AT.positions); return -1.0; }
    if (nb > AT.cap) {
        cudaStreamSynchronize(S.st);
        cudaFree(AT.qkv); cudaFree(AT.q); cudaFree(AT.kc); cudaFree(AT.vc); cudaFree(AT.pos); cudaFree(AT.norms); AT.cap = 0;
        AT.qkv = AT.q = AT.norms = NULL; AT.kc = AT.vc = NULL; AT.pos = NULL;
        const size_t T = (size_t)S.maxtok;
        if (dmalloc((void **)&AT.qkv, T * 3072 * 4) || dmalloc((void **)&AT.q, T * 2048 * 4) || dmalloc(&AT.kc, T * 512 * 2) || dmalloc(&AT.vc, T * 512 * 2) ||
            dmalloc((void **)&AT.pos, T * 4) || dmalloc((void **)&AT.norms, 256 * 4)) { fail("gmoe", "no device memory for the attention head of %d tokens", S.maxtok); return -1.0; }
        AT.cap = S.maxtok;
    }
    CUD("gmoe", cudaMemcpyAsync(AT.qkv, qkv, (size_t)nb * 3072 * 4, cudaMemcpyHostToDevice, S.st));
    CUD("gmoe", cudaMemcpyAsync(AT.pos, pos, (size_t)nb * 4, cudaMemcpyHostToDevice, S.st));
    CUD("gmoe", cudaMemcpyAsync(AT.norms, qn, 128 * 4, cudaMemcpyHostToDevice, S.st));
    CUD("gmoe", cudaMemcpyAsync(AT.norms + 128, kn, 128 * 4, cudaMemcpyHostToDevice, S.st));
    cudaEventRecord(S.e0, S.st);
    k_qk_rope(S.st, AT.qkv, AT.pos, nb, glob, AT.norms, AT.norms + 128, AT.cs, AT.positions, AT.q, AT.kc, AT.vc, S.err);
    cudaEventRecord(S.e1, S.st);
    CUD("gmoe", cudaMemcpyAsync(q, AT.q, (size_t)nb * 2048 * 4, cudaMemcpyDeviceToHost, S.st));
    CUD("gmoe", cudaMemcpyAsync(kc, AT.kc, (size_t)nb * 512 * 2, cudaMemcpyDeviceToHost, S.st));
    CUD("gmoe", cudaMemcpyAsync(vc, AT.vc, (size_t)nb * 512 * 2, cudaMemcpyDeviceToHost, S.st));
    return finish("gmoe");
}

/* ---- the attention projections (gpu_pre.m:200-256): every layer's q,k,v (group 2L) and o (group 2L+1) resident on the card.
 * y[nb][rows of the group] = the group's matrices times prep(x[nb][2048]): the expert product with one matrix and all tokens.
 * gpre_dense_add copies into a host staging area (the caller's memory need not outlive the call, as with the reference);
 * gpre_dense_done puts every group's matrices side by side on the card, so that a group is one matrix of all its rows. */
#define DGRP 48
static struct {
    uint8_t *hcodes; float *hscales;            /* staged on the host until gpre_dense_done */
    uint8_t *codes; float *scales;              /* on the card: [rows][512] codes, [rows] scales */
    int rows, staged; ExpertMaps maps;          /* maps.down: the 3-D map of the tcgen05 kernel (rows a multiple of 256) */
} DG[DGRP];
static float *DY; static int DY_tok, DY_rows, dense_bad;
static TMap4 bmap_tok;                          /* the tokens' int8 rows [maxtok][2048] as the B operand */
void gpre_dense_add(int g, const uint8_t *codes, const float *scales, int rows, int cols) {
    if (!S.ready) { fail("gpre", "gpre_dense_add before gpre_init"); dense_bad = 1; return; }
    if (g < 0 || g >= DGRP || DG[g].codes) { fail("gpre", "gpre_dense_add: group %d (outside 0..%d or already on the card)", g, DGRP - 1); dense_bad = 1; return; }
    if (cols != HID || rows < 128 || (rows % 128)) { fail("gpre", "gpre_dense_add: %d x %d (needs 2048 columns and a multiple of 128 rows)", rows, cols); dense_bad = 1; return; }
    const size_t old = (size_t)DG[g].rows, add = (size_t)rows;
    uint8_t *hc = realloc(DG[g].hcodes, (old + add) * (HID / 4)); float *hs = realloc(DG[g].hscales, (old + add) * 4);
    if (hc) DG[g].hcodes = hc;
    if (hs) DG[g].hscales = hs;
    if (!hc || !hs) { fail("gpre", "gpre_dense_add: out of host memory"); dense_bad = 1; return; }
    memcpy(hc + old * (HID / 4), codes, add * (HID / 4)); memcpy(hs + old, scales, add * 4);
    DG[g].rows += rows; DG[g].staged = 1;
}
int gpre_dense_done(int maxtok) {
    if (!S.ready) return fail("gpre", "gpre_dense_done before gpre_init");
    if (dense_bad) return -1;                       /* the message of the failed add stands; the caller keeps the projections on the CPU */
    if (maxtok < 1 || maxtok > S.maxtok) return fail("gpre", "gpre_dense_done: %d tokens, initialised for %d", maxtok, S.maxtok);
    int ymax = 0;
    for (int g = 0; g < DGRP; g++) {
        if (DG[g].rows > ymax) ymax = DG[g].rows;
        if (!DG[g].staged) continue;
        const size_t cb = (size_t)DG[g].rows * (HID / 4), sb = (size_t)DG[g].rows * 4;
        if (dmalloc((void **)&DG[g].codes, cb) || dmalloc((void **)&DG[g].scales, sb)) return fail("gpre", "no room for the attention projections of group %d", g);
        CU("gpre", cudaMemcpy(DG[g].codes, DG[g].hcodes, cb, cudaMemcpyHostToDevice));
        CU("gpre", cudaMemcpy(DG[g].scales, DG[g].hscales, sb, cudaMemcpyHostToDevice));
        free(DG[g].hcodes); free(DG[g].hscales); DG[g].hcodes = NULL; DG[g].hscales = NULL; DG[g].staged = 0;
        if (DG[g].rows % 256 == 0) {   /* [rows/2 row pairs][2 parities][512 bytes], box = 128 row pairs x 1 parity x 128 bytes */
            cuuint64_t gdim[3] = {HID / 4, 2, (cuuint64_t)DG[g].rows / 2}, gstride[2] = {HID / 4, HID / 2};
            cuuint32_t box[3] = {128, 1, 128}, estr[3] = {1, 1, 1};
            CUresult r = g_encode((CUtensorMap *)&DG[g].maps.down, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, DG[g].codes, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return fail("gpre", "cuTensorMapEncodeTiled failed (%d) for the projections of group %d", (int)r, g);
        }
    }
    if (!ymax) return fail("gpre", "gpre_dense_done: no matrices were added");
    if (!DY || maxtok > DY_tok || ymax > DY_rows) {
        cudaFree(DY); DY = NULL;
        if (dmalloc((void **)&DY, (size_t)maxtok * ymax * 4)) return fail("gpre", "no room for the attention projections' results");
        DY_tok = maxtok; DY_rows = ymax;
    }
    for (int i = 0; i < 4; i++) if (tmap_bytes_2d("gpre", &bmap_tok.m[i], S.hq, HID, (uint64_t)S.maxtok, HID, 128, 32 * (i + 1))) return -1;
    return 0;
}
double gpre_dense(int g, const float *x, int nb, float *y) {
    if (!S.ready || !DY) { fail("gpre", "gpre_dense before gpre_dense_done"); return -1.0; }
    if (g < 0 || g >= DGRP || !DG[g].codes) { fail("gpre", "gpre_dense: group %d has no matrices on the card", g); return -1.0; }
    if (nb < 1 || nb > DY_tok) { fail("gpre", "gpre_dense: %d tokens outside 1..%d", nb, DY_tok); return -1.0; }
    const int ys = DG[g].rows, um = nb >= 512 && ys % 256 == 0, tn = um ? UMMA_TN : 32, nt = (nb + tn - 1) / tn;
    memset(S.h_tab, 0, sizeof(ExpertPtrs));
    S.h_tab[0].dc = DG[g].codes; S.h_tab[0].ds = DG[g].scales;
    for (int i = 0; i < nt; i++) { MoeTile t = {0, i * tn, nb - i * tn < tn ? nb - i * tn : tn, 0}; S.h_tiles[i] = t; }
    CUD("gpre", cudaMemcpyAsync(S.hn, x, (size_t)nb * HID * 4, cudaMemcpyHostToDevice, S.st));
    CUD("gpre", cudaMemcpyAsync(S.tab_call, S.h_tab, sizeof(ExpertPtrs), cudaMemcpyHostToDevice, S.st));
    CUD("gpre", cudaMemcpyAsync(S.maps_call, &DG[g].maps, sizeof(ExpertMaps), cudaMemcpyHostToDevice, S.st));
    CUD("gpre", cudaMemcpyAsync(S.tiles_a, S.h_tiles, (size_t)nt * sizeof(MoeTile), cudaMemcpyHostToDevice, S.st));
    CUD("gpre", cudaMemcpyAsync(S.ntiles_a, &nt, 4, cudaMemcpyHostToDevice, S.st));
    cudaEventRecord(S.e0, S.st);
    k_norm_prep(S.st, S.hn, NULL, S.hn, S.hq, S.hqs, S.hqsum, nb);          /* prep of maple.c:184-194 per token */
    ExpertArgs a; memset(&a, 0, sizeof a);
    a.tab = S.tab_call; a.maps = S.maps_call; a.tiles = S.tiles_a; a.ntiles = S.ntiles_a; a.max_tiles = nt; a.err = S.err;
    a.aq = S.hq; a.aqs = S.hqs; a.aqsum = S.hqsum; a.down = DY; a.down_stride = ys; a.dense_mblocks = ys / 256;
    if (um) k_dense_umma(S.st, &a, &bmap_tok); else k_dense_mma(S.st, &a, ys);
    cudaEventRecord(S.e1, S.st);
    CUD("gpre", cudaMemcpyAsync(y, DY, (size_t)nb * ys * 4, cudaMemcpyDeviceToHost, S.st));
    S.nb_cur = nb;
    return finish("gpre");
}
int gpu_head_init(const uint16_t *w, int rows, int cols) { (void)w; (void)rows; (void)cols; return -1; }
int gpu_head_init_i8(const int8_t *w, const float *scale, int rows, int cols) { (void)w; (void)scale; (void)rows; (void)cols; return -1; }
void gpu_head_run(const float *x, float *y) { (void)x; (void)y; }
void gpu_head_run_multi(const float *x, int n, float *y) { (void)x; (void)n; (void)y; }
int gpux_init(int layers, int slots) { (void)layers; (void)slots; return -1; }
void gpux_upload(int L, int slot, const uint8_t *gc, const float *gs, const uint8_t *uc, const float *us, const uint8_t *dc, const float *ds) {
    (void)L; (void)slot; (void)gc; (void)gs; (void)uc; (void)us; (void)dc; (void)ds;
}
void *gpux_begin(int L, const float *x, int n, const int *slots) { (void)L; (void)x; (void)n; (void)slots; return NULL; }
void gpux_end(void *h, float *out, int n) { (void)h; (void)out; (void)n; }
void *gpux_begin_multi(int L, const float *x, int nb, int nu, const int *slots, const int *pstart, const int *ptok) {
    (void)L; (void)x; (void)nb; (void)nu; (void)slots; (void)pstart; (void)ptok; return NULL;
}
void gpux_end_multi(void *h, float *out, int np) { (void)h; (void)out; (void)np; }

/* ================================================================================================================
 * Expert parallelism across the GPUs of one NVLink box (one process per GPU).  The reference has no counterpart
 * (single process, single device).  Rank r keeps its own tokens and the experts r*E .. (r+1)*E-1, E = 256 / world.
 * Per layer: local norm / router / top-8 / grouping -> exchange of the per-expert pair counts (peer stores and arrival
 * flags, k_ep.cu) -> every rank stores its int8 rows straight into the owners' receive buffers (peer stores over NVLink)
 * -> rendezvous -> the owners run gate+up, SiLU+int8 and down on what they received, the down epilogue stores each
 * result row straight into the token's rank -> rendezvous -> local combine, in the same order as on one GPU, so the
 * hidden state is the same bits as without expert parallelism.  NCCL is used to form the group and for the benchmark's
 * max-over-ranks; nothing on the data path calls it.
 * ================================================================================================================ */
#include <dlfcn.h>
#include <nccl.h>

static struct {
    int rank, world, epr; size_t rcap;
    void *lib; ncclComm_t comm;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *);
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int);
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t);
    const char *(*GetErrorString)(ncclResult_t);
    int *xch; unsigned *epoch; unsigned long long timeout_ns;   /* exchange buffer (counts + arrival flags), rendezvous counter */
    int *all_cnt, *dst_base, *total, *nu_r, *ue_r, *ustart_r, *rx_qsum; float *rx_qs; int2 *rx_src; double *red;
    void *peer[7][8];                       /* opened buffers of every rank: rx rows, rx scales, rx sums, rx return addresses, down rows, exchange, compact down rows */
    void **peer_dev[7];
    float *ds_all[GMOE_LAYERS]; const float **dsp[GMOE_LAYERS];   /* every expert's down scales gathered per layer, and the pointer table over them */                     /* the same tables in device memory */
} EP;

static int ep_rank_shard(int *e0, int *ne) { *e0 = EP.rank * EP.epr; *ne = EP.epr; return 0; }
/* layer L got new weights: the down scales gathered from all ranks are stale */
static void ep_forget_layer(int L) {
    if (EP.ds_all[L]) { cudaFree(EP.ds_all[L]); EP.ds_all[L] = NULL; }
    if (EP.dsp[L]) { cudaFree((void *)EP.dsp[L]); EP.dsp[L] = NULL; }
}
static int ep_nccl(const char *who) {
    if (EP.lib) return 0;
    EP.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!EP.lib) return fail(who, "libnccl.so.2 cannot be loaded: %s", dlerror());
#define SYM(field, name) do { *(void **)&EP.field = dlsym(EP.lib, name); if (!EP.field) return fail(who, "libnccl has no %s", name); } while (0)
    SYM(GetUniqueId, "ncclGetUniqueId"); SYM(CommInitRank, "ncclCommInitRank"); SYM(AllGather, "ncclAllGather");
    SYM(AllReduce, "ncclAllReduce"); SYM(GetErrorString, "ncclGetErrorString");
#undef SYM
    return 0;
}
#define NC(who, call) do { ncclResult_t r_ = (call); if (r_ != ncclSuccess) return fail(who, "%s: %s", #call, EP.GetErrorString(r_)); } while (0)

int gmoe_ep_unique_id(void *out128) {
    if (ep_nccl("gmoe")) return -1;
    ncclUniqueId id; NC("gmoe", EP.GetUniqueId(&id)); memcpy(out128, &id, sizeof id); return 0;
}
#define EP_REALLOC(field, bytes) do { cudaFree(S.field); S.field = NULL; if (dmalloc((void **)&S.field, (bytes))) return fail("gmoe", "expert parallel: no device memory for %s", #field); } while (0)
#define EP_ALLOC(field, bytes) do { if (dmalloc((void **)&EP.field, (bytes))) return fail("gmoe", "expert parallel: no device memory for %s", #field); } while (0)
int gmoe_ep_init(int rank, int world, const void *id128) {
    if (!S.ready) return fail("gmoe", "gmoe_ep_init before gmoe_init");
    if (S.ep_on) return fail("gmoe", "expert parallelism is already set up");
    graphs_drop();                              /* the buffers reallocated below are named by every captured layer loop */
    if (world < 1 || world > 8 || (NEXP % world) || rank < 0 || rank >= world) return fail("gmoe", "rank %d of %d", rank, world);
    if (ep_nccl("gmoe")) return -1;
    ncclUniqueId id; memcpy(&id, id128, sizeof id);
    NC("gmoe", EP.CommInitRank(&EP.comm, world, id, rank));
    EP.rank = rank; EP.world = world; EP.epr = NEXP / world; EP.rcap = (size_t)world * S.maxp;
    const size_t R = EP.rcap;
    /* everything indexed by received pairs grows to the worst case: every pair of every rank lands here */
    EP_REALLOC(hq_sorted, R * HID); EP_REALLOC(gate, R * FFN * 4); EP_REALLOC(up, R * FFN * 4); EP_REALLOC(act, R * FFN * 4);
    EP_REALLOC(aq, R * FFN); EP_REALLOC(aqs, R * 4); EP_REALLOC(aqsum, R * 4);
    EP_REALLOC(tiles_a, (R / 8 + NEXP) * sizeof(MoeTile)); EP_REALLOC(tiles_b, (R / 8 + NEXP) * sizeof(MoeTile));
    if (S.gu_dots) { EP_REALLOC(gu_dots, R * 2 * FFN * 4); EP_REALLOC(dn_dots, R * HID * 4); }
    if (bmaps("gmoe", R)) return -1;
    EP_ALLOC(xch, EP_XCH_INTS * 4); EP_ALLOC(epoch, 16); EP.all_cnt = EP.xch; EP.timeout_ns = 10000000000ull;
    CU("gmoe", cudaMemset(EP.xch, 0, EP_XCH_INTS * 4)); CU("gmoe", cudaMemset(EP.epoch, 0, 16));
    EP_ALLOC(dst_base, NEXP * 4); EP_ALLOC(total, 16); EP_ALLOC(nu_r, 16); EP_ALLOC(ue_r, NEXP * 4);
    EP_ALLOC(ustart_r, (NEXP + 1) * 4); EP_ALLOC(rx_qs, R * 4); EP_ALLOC(rx_qsum, R * 4); EP_ALLOC(rx_src, R * sizeof(int2)); EP_ALLOC(red, 64);
    for (int k = 0; k < 7; k++) if (dmalloc((void **)&EP.peer_dev[k], 8 * sizeof(void *))) return fail("gmoe", "expert parallel: no device memory");
    S.ep_on = 1;
    return 0;
}
/* 7 x 64 bytes: the handles other ranks need to store into this rank's buffers */
int gmoe_ep_handles(void *out448) {
    if (!S.ep_on) return fail("gmoe", "gmoe_ep_handles before gmoe_ep_init");
    void *p[7] = {S.hq_sorted, EP.rx_qs, EP.rx_qsum, EP.rx_src, S.down, EP.xch, S.wire};
    for (int k = 0; k < 7; k++) CU("gmoe", cudaIpcGetMemHandle((cudaIpcMemHandle_t *)((char *)out448 + 64 * k), p[k]));
    return 0;
}
/* all: world x 7 x 64 bytes, rank-major, as gathered from gmoe_ep_handles */
int gmoe_ep_connect(const void *all) {
    if (!S.ep_on) return fail("gmoe", "gmoe_ep_connect before gmoe_ep_init");
    void *mine[7] = {S.hq_sorted, EP.rx_qs, EP.rx_qsum, EP.rx_src, S.down, EP.xch, S.wire};
    for (int r = 0; r < EP.world; r++) for (int k = 0; k < 7; k++) {
        if (r == EP.rank) { EP.peer[k][r] = mine[k]; continue; }
        cudaIpcMemHandle_t h; memcpy(&h, (const char *)all + ((size_t)r * 7 + k) * 64, 64);
        CU("gmoe", cudaIpcOpenMemHandle(&EP.peer[k][r], h, cudaIpcMemLazyEnablePeerAccess));
    }
    for (int k = 0; k < 7; k++) CU("gmoe", cudaMemcpy(EP.peer_dev[k], EP.peer[k], 8 * sizeof(void *), cudaMemcpyHostToDevice));
    return 0;
}
/* every rank's earlier work on its stream is complete before any rank's later work starts; with cnt, every rank also receives
 * every rank's pairs per expert */
static int ep_barrier(const int *cnt) {
    EpXchArgs a = {cnt, (int *const *)EP.peer_dev[5], EP.xch, EP.epoch, EP.rank, EP.world, EP.timeout_ns, S.err};
    k_ep_exchange(S.st, &a); return 0;
}
/* The combine scales the compact down rows where the token lives, so every rank needs every expert's 2048 down scales: gathered
 * once per layer (NCCL all-gather of 256/world x 8 KB per rank), the first time the layer runs in expert parallel.  Every rank
 * runs the same layers, so the ranks make these calls together. */
static int ep_layer_scales(int L) {
    if (EP.dsp[L]) return 0;
    LayerDev *l = &S.ly[L];
    float *send = NULL;
    if (dmalloc((void **)&EP.ds_all[L], (size_t)NEXP * HID * 4) || dmalloc((void **)&EP.dsp[L], NEXP * sizeof(void *)) || dmalloc((void **)&send, (size_t)EP.epr * HID * 4))
        return fail("gmoe", "expert parallel: no device memory for the down scales of layer %d", L);
    CU("gmoe", cudaMemcpyAsync(S.h_tab, l->tab, NEXP * sizeof(ExpertPtrs), cudaMemcpyDeviceToHost, S.st));
    CU("gmoe", cudaStreamSynchronize(S.st));
    for (int k = 0; k < EP.epr; k++) {
        const float *src = S.h_tab[EP.rank * EP.epr + k].ds;
        if (!src) return fail("gmoe", "expert parallel: rank %d has no weights for its expert %d of layer %d", EP.rank, EP.rank * EP.epr + k, L);
        CU("gmoe", cudaMemcpyAsync(send + (size_t)k * HID, src, HID * 4, cudaMemcpyDeviceToDevice, S.st));
    }
    NC("gmoe", EP.AllGather(send, EP.ds_all[L], (size_t)EP.epr * HID, ncclFloat, EP.comm, S.st));
    for (int e = 0; e < NEXP; e++) S.h_dsp[e] = EP.ds_all[L] + (size_t)e * HID;
    CU("gmoe", cudaMemcpyAsync(EP.dsp[L], S.h_dsp, NEXP * sizeof(void *), cudaMemcpyHostToDevice, S.st));
    CU("gmoe", cudaStreamSynchronize(S.st));
    cudaFree(send);
    return 0;
}
static int run_layer_ep(int L, int nb, const float *bias) {
    LayerDev *l = &S.ly[L];
    const int tn = tile_tn(nb), um = use_umma(nb);
    prof_begin(0); const int relaid = run_norm(S.x, l->post_ln, nb); prof_end(0);
    const int tr = tensor_router(nb);
    if (tr) { prof_begin(1); run_router_tensor_m(l, bias, nb, 1); prof_end(1); }
    else {
        prof_begin(1); run_router_relaid(l, bias, nb, relaid); prof_end(1);
        prof_begin(2); k_topk(S.st, S.logits, S.top, S.topw, nb); prof_end(2);
    }
    prof_begin(3);
    run_group_m(nb, tr);
    EpPlanArgs p = {EP.all_cnt, EP.rank, EP.world, EP.dst_base, EP.nu_r, EP.ue_r, EP.ustart_r, EP.total, S.tiles_a, S.tiles_b, S.ntiles_a, S.ntiles_b, tn, UMMA_TN};
    EpXchArgs xc = {S.ecnt, (int *const *)EP.peer_dev[5], EP.xch, EP.epoch, EP.rank, EP.world, EP.timeout_ns, S.err};
    k_ep_plan(S.st, &p, &xc);
    EpDispatchArgs d = {S.hq, S.hqs, S.hqsum, S.utok, S.uexp, S.estart, EP.dst_base, nb * TOPK, EP.rank, EP.epr,
                        (int8_t *const *)EP.peer_dev[0], (float *const *)EP.peer_dev[1], (int *const *)EP.peer_dev[2], (int2 *const *)EP.peer_dev[3]};
    k_ep_dispatch(S.st, &d);
    if (ep_barrier(NULL)) return -1;
    prof_end(3);
    ExpertArgs a; memset(&a, 0, sizeof a);
    a.tab = l->tab; a.maps = l->maps; a.ue = EP.ue_r; a.err = S.err; a.ptok = NULL;
    a.tiles = um ? S.tiles_b : S.tiles_a; a.ntiles = um ? S.ntiles_b : S.ntiles_a; a.max_tiles = (int)(EP.rcap / (um ? UMMA_TN : tn)) + NEXP;
    a.hq = S.hq_sorted; a.hqs = EP.rx_qs; a.hqsum = EP.rx_qsum; a.act = S.act; a.aq = S.aq; a.aqs = S.aqs; a.aqsum = S.aqsum; a.down = S.down;
    a.rx_src = EP.rx_src; a.peer_down = (float *const *)EP.peer_dev[4]; a.peer_wire = (uint8_t *const *)EP.peer_dev[6]; a.wire = S.wire; a.wire_cap = S.maxp;
    if (S.keep || um) { a.gate = S.gate; a.up = S.up; }
    if (S.keep) { a.gu_dots = S.gu_dots; a.dn_dots = S.dn_dots; }
    prof_begin(4); if (um) k_gateup_umma(S.st, &a, &S.bmap_hq); else k_gateup_mma(S.st, &a, tn); prof_end(4);
    prof_begin(5);
    if (um) k_silu_quant(S.st, S.gate, S.up, S.keep ? S.act : NULL, S.aq, S.aqs, S.aqsum, (int)EP.rcap, EP.total);
    else k_actq(S.st, S.act, S.aq, S.aqs, S.aqsum, EP.total, (int)EP.rcap);
    prof_end(5);
    prof_begin(6); if (um) k_down_umma(S.st, &a, &S.bmap_aq); else k_down_mma(S.st, &a, tn); prof_end(6);
    prof_begin(7);
    if (ep_barrier(NULL)) return -1;
    if (um && S.keep) k_wire_decode(S.st, S.wire, S.maxp, (const float *const *)EP.dsp[L], S.down, nb * TOPK);
    run_combine((const float *const *)EP.dsp[L], nb, S.x, S.x);
    prof_end(7);
    return 0;
}
/* The residual stream of this rank's nb tokens through layers l0 .. l0+nl-1, experts sharded over the ranks.
 * Device-resident form (gmoe_x_upload / gmoe_x_download, gmoe_chunks_upload); asynchronous; every rank calls it with the same nb. */
int gmoe_ep_forward_dev(int chunk, int nb, int l0, int nl, const float *bias) {
    if (!S.ep_on) return fail("gmoe", "expert parallelism is not set up");
    g_ep_call = 1;
    for (int L = l0; L < l0 + nl; L++) if (check_call("gmoe", L, nb) || ep_layer_scales(L)) { g_ep_call = 0; return -1; }
    g_ep_call = 0;
    const float *bd = bias_dev(bias);
    cudaEventRecord(S.e0, S.st);
    if (chunk >= 0) {
        if (!S.ring || nb != S.ring_nb || chunk >= S.ring_n) return fail("gmoe", "chunk %d of %d tokens is not in the ring", chunk, nb);
        cudaMemcpyAsync(S.x, S.ring + (size_t)chunk * nb * HID, (size_t)nb * HID * 4, cudaMemcpyDeviceToDevice, S.st);
    }
    if (layers_enqueue_ep(nb, l0, nl, bd, 1)) return -1;
    cudaEventRecord(S.e1, S.st);
    S.nb_cur = nb; return 0;
}
/* Host in/out, like gmoe_forward. */
double gmoe_ep_forward(float *x, int nb, int l0, int nl, const float *bias) {
    if (!S.ep_on) { fail("gmoe", "expert parallelism is not set up"); return -1.0; }
    g_ep_call = 1;
    for (int L = l0; L < l0 + nl; L++) if (check_call("gmoe", L, nb) || ep_layer_scales(L)) { g_ep_call = 0; return -1.0; }
    g_ep_call = 0;
    const float *bd = bias_dev(bias);
    cudaEventRecord(S.e0, S.st);
    CUD("gmoe", cudaMemcpyAsync(S.x, x, (size_t)nb * HID * 4, cudaMemcpyHostToDevice, S.st));
    if (layers_enqueue_ep(nb, l0, nl, bd, 1)) return -1.0;
    CUD("gmoe", cudaMemcpyAsync(x, S.x, (size_t)nb * HID * 4, cudaMemcpyDeviceToHost, S.st));
    cudaEventRecord(S.e1, S.st);
    S.nb_cur = nb;
    return finish("gmoe");
}
/* max over ranks of a host value (the benchmark's device-measured seconds), and with it a barrier: NCCL on the library's stream */
int gmoe_ep_allmax(double *v) {
    if (!S.ep_on) return fail("gmoe", "expert parallelism is not set up");
    CU("gmoe", cudaMemcpyAsync(EP.red + 2, v, 8, cudaMemcpyHostToDevice, S.st));
    NC("gmoe", EP.AllReduce(EP.red + 2, EP.red + 3, 1, ncclDouble, ncclMax, EP.comm, S.st));
    CU("gmoe", cudaMemcpyAsync(v, EP.red + 3, 8, cudaMemcpyDeviceToHost, S.st));
    CU("gmoe", cudaStreamSynchronize(S.st)); return 0;
}
/* A rendezvous in which one of two arrivals never comes (no second rank exists): the wait must give up after `ms` milliseconds
 * with the error code that the data path reports.  Returns that code (41), 0 if the wait returned without it, -1 on a CUDA error.
 * Needs gmoe_init only. */
int gmoe_ep_timeout_selftest(int ms) {
    if (!S.ready) return fail("gmoe", "not initialised");
    int *xch = NULL, **tab = NULL; unsigned *epoch = NULL; int code = -1;
    if (dmalloc((void **)&xch, EP_XCH_INTS * 4) || dmalloc((void **)&tab, 8 * sizeof(void *)) || dmalloc((void **)&epoch, 16)) return fail("gmoe", "no device memory");
    int *h_tab[8] = {xch, xch, 0, 0, 0, 0, 0, 0};
    if (cudaMemset(xch, 0, EP_XCH_INTS * 4) == cudaSuccess && cudaMemset(epoch, 0, 16) == cudaSuccess &&
        cudaMemcpy(tab, h_tab, sizeof h_tab, cudaMemcpyHostToDevice) == cudaSuccess) {
        EpXchArgs a = {NULL, (int *const *)tab, xch, epoch, 0, 2, (unsigned long long)(ms > 0 ? ms : 1) * 1000000ull, S.err};
        k_ep_exchange(S.st, &a);
        if (cudaMemcpyAsync(S.h_err, S.err, 4, cudaMemcpyDeviceToHost, S.st) == cudaSuccess && cudaStreamSynchronize(S.st) == cudaSuccess) {
            code = *S.h_err; *S.h_err = 0; cudaMemsetAsync(S.err, 0, 4, S.st); cudaStreamSynchronize(S.st);
        }
    }
    cudaFree(xch); cudaFree(tab); cudaFree(epoch);
    return code < 0 ? fail("gmoe", "rendezvous self-test: %s", cudaGetErrorString(cudaGetLastError())) : code;
}
/* received pairs of the last layer on this rank (load balance report) */
int gmoe_ep_received(void) { int t = -1; if (S.ep_on) { cudaMemcpyAsync(&t, EP.total, 4, cudaMemcpyDeviceToHost, S.st); cudaStreamSynchronize(S.st); } return t; }
