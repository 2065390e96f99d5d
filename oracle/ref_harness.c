/* ref_harness.c -- TEST INFRASTRUCTURE ONLY (never linked into the product library).
 *
 * Drives the UNMODIFIED reference runtime (maple.c) on synthetic inputs without copying it:
 * the reference's single translation unit is textually included from where it lies on this
 * machine (-DMAPLE_C="path"), its main() is renamed, and the functions below call the
 * reference's own static functions for the mixture-of-experts half of a layer:
 *   rmsnorm (maple.c:398), prep (184), job_route_small/multi (853/870), job_topk (910),
 *   group_pairs (924), jobB_gateup (471) -> tdot_multi (425), the SiLU*up + prep loop (825-832),
 *   jobB_down (498), the combine loop (834) and the worker pool run()/worker (89-108);
 * and for the first step of the attention half: rmsnorm + rope (403-411) + to_f16 (314-320) as step_batch calls them (711-717).
 * Outputs land in oracle/_ref/ only (libmaple_ref.so: IEEE build, the parity pin;
 * libmaple_ref_fast.so: the reference's documented -ffast-math build, the timed CPU baseline).
 */
#ifndef MAPLE_C
#error "build with -DMAPLE_C=\"/path/to/maple.c\""
#endif
#define main maple_reference_main
#include MAPLE_C
#undef main

#define RH_EXPERT_BYTES 798720  /* gate codes 262144 | gate scales 2048 | up codes | up scales | down codes 262144 | down scales 8192 */

static int RH_WORKERS = 1;  /* threads already running, counting the caller */

/* NT threads in total, workers spinning as maple.c:1091 starts them. Threads can only be added. */
int rh_threads(int nt) {
    if (nt < 1) nt = 1;
    if (nt < RH_WORKERS) nt = RH_WORKERS;  /* the reference has no way to stop a worker */
    NT = nt;
    for (int i = RH_WORKERS; i < nt; i++) { pthread_t th; pthread_create(&th, NULL, worker, (void *)(intptr_t)i); }
    RH_WORKERS = nt;
    return NT;
}

/* Point layer L at caller-owned arrays: router bf16 [256x2048], post_ln bf16 [2048], and the 256
 * experts stored back to back in the converter's order (convert.py:79-84: codes then row scales). */
void rh_set_layer(int L, const uint16_t *router, const uint16_t *post_ln, const uint8_t *experts) {
    Layer *l = &LY[L];
    l->router.p = router; l->router.rows = NE; l->router.cols = H;
    l->post_ln.p = post_ln; l->post_ln.rows = H; l->post_ln.cols = 1;
    for (int e = 0; e < NE; e++) {
        const uint8_t *b = experts + (size_t)e * RH_EXPERT_BYTES;
        l->eg[e].p = b;                 l->eg[e].s = (const float *)(b + 262144);          l->eg[e].rows = FF; l->eg[e].cols = H;
        l->eu[e].p = b + 264192;        l->eu[e].s = (const float *)(b + 264192 + 262144); l->eu[e].rows = FF; l->eu[e].cols = H;
        l->ed[e].p = b + 528384;        l->ed[e].s = (const float *)(b + 528384 + 262144); l->ed[e].rows = H;  l->ed[e].cols = FF;
    }
}

void rh_prep(const float *x, int n, int8_t *q, float *qs, int32_t *qsum) {
    static Vin v; prep(&v, x, n); memcpy(q, v.q, (size_t)n); *qs = v.qs; *qsum = v.qsum;
}
void rh_rmsnorm(float *out, const float *x, const uint16_t *w, int n) { BF b = {w, n, 1}; rmsnorm(out, x, &b, n); }
float rh_expf(float x) { return expf(x); }
float rh_tdot(const uint8_t *codes, const float *scales, int rows, int cols, int r, const float *x) {
    static Vin v; T2 w = {codes, scales, rows, cols}; prep(&v, x, cols); return tdot(&w, r, &v);
}

typedef struct {            /* every pointer may be NULL = not wanted */
    float *logits;          /* [nb][256]  RLG before job_topk overwrites it */
    int *top; float *topw;  /* [nb][8]    TOPB, TWB */
    int *nu, *ue, *ustart;  /* [1], [256], [257] */
    int *utok; float *uw;   /* [nb*8] */
    int *tp;                /* [nb*8]    maple.c:1018-1019 */
    int8_t *hq; float *hqs; int32_t *hqsum;   /* [nb][2048], [nb], [nb]   VHB */
    float *gate, *up, *act; /* [nb*8][512] */
    int8_t *aq; float *aqs; int32_t *aqsum;   /* [nb*8][512], [nb*8], [nb*8]   VAB */
    float *down;            /* [nb*8][2048] */
} rh_dump;

/* The MoE half of step_batch (maple.c:732-835) for nb tokens of layer L.
 * norm != 0: x is the residual stream, hn = rmsnorm(x, post_ln) first and the result is added into x
 * (x is updated in place, the CPU path of maple.c:733-834).
 * norm == 0: x already holds the normalised hidden state, and y receives sum_k w_k * expert_k(x) only
 * (what gpre_moe returns, maple.c:763-784 with GPRE_CHECK).  Returns pairs, or -1. */
int rh_moe(int L, float *x, int nb, int norm, float *y, const float *bias, rh_dump *d) {
    if (nb < 1 || nb > BMAX || L < 0 || L >= NL) return -1;
    BN = nb; BL = &LY[L];
    static int poss[BMAX];
    for (int b = 0; b < nb; b++) {
        if (norm) { memcpy(XB[b], x + (size_t)b * H, sizeof XB[b]); rmsnorm(HNB[b], XB[b], &BL->post_ln, H); }
        else { memset(XB[b], 0, sizeof XB[b]); memcpy(HNB[b], x + (size_t)b * H, sizeof HNB[b]); }
        prep(&VHB[b], HNB[b], H);
    }
    if (nb <= 32) run(job_route_small, NULL, NE); else run(job_route_multi, NULL, (nb + 7) / 8);
    if (bias) for (int b = 0; b < nb; b++) for (int e = 0; e < NE; e++) RLG[b][e] += bias[e];
    if (d && d->logits) memcpy(d->logits, RLG, sizeof(float) * NE * nb);
    run(job_topk, NULL, nb);
    int na = group_pairs(nb, poss, L);
    static int tp[BMAX * TOPK], fl[BMAX];
    memset(fl, 0, sizeof(int) * nb);
    for (int a = 0; a < na; a++) { int b = UTOK[a]; tp[b * TOPK + fl[b]++] = a; }
    run(jobB_gateup, NULL, NU * 2 * FF);
    for (int a = 0; a < na; a++) {
        for (int k = 0; k < FF; k++) {
            float g = GATEB[a][k] < 7.0f ? GATEB[a][k] : 7.0f, u = UPB[a][k];
            u = u < -7.0f ? -7.0f : (u > 7.0f ? 7.0f : u);
            ACTB[a][k] = g / (1.0f + expf(-g)) * u;
        }
        prep(&VAB[a], ACTB[a], FF);
    }
    run(jobB_down, NULL, NU * H);
    for (int a = 0; a < na; a++) { float *xo = XB[UTOK[a]]; for (int i = 0; i < H; i++) xo[i] += UW[a] * DOWNB[a][i]; }
    if (norm) memcpy(x, XB, sizeof(float) * H * nb); else if (y) memcpy(y, XB, sizeof(float) * H * nb);
    if (d) {
        if (d->top) memcpy(d->top, TOPB, sizeof(int) * TOPK * nb);
        if (d->topw) memcpy(d->topw, TWB, sizeof(float) * TOPK * nb);
        if (d->nu) *d->nu = NU;
        if (d->ue) memcpy(d->ue, UE, sizeof(int) * NU);
        if (d->ustart) memcpy(d->ustart, USTART, sizeof(int) * (NU + 1));
        if (d->utok) memcpy(d->utok, UTOK, sizeof(int) * na);
        if (d->uw) memcpy(d->uw, UW, sizeof(float) * na);
        if (d->tp) memcpy(d->tp, tp, sizeof(int) * TOPK * nb);
        for (int b = 0; b < nb; b++) {
            if (d->hq) memcpy(d->hq + (size_t)b * H, VHB[b].q, H);
            if (d->hqs) d->hqs[b] = VHB[b].qs;
            if (d->hqsum) d->hqsum[b] = VHB[b].qsum;
        }
        if (d->gate) memcpy(d->gate, GATEB, sizeof(float) * FF * na);
        if (d->up) memcpy(d->up, UPB, sizeof(float) * FF * na);
        if (d->act) memcpy(d->act, ACTB, sizeof(float) * FF * na);
        for (int a = 0; a < na; a++) {
            if (d->aq) memcpy(d->aq + (size_t)a * FF, VAB[a].q, FF);
            if (d->aqs) d->aqs[a] = VAB[a].qs;
            if (d->aqsum) d->aqsum[a] = VAB[a].qsum;
        }
        if (d->down) memcpy(d->down, DOWNB, sizeof(float) * H * na);
    }
    return na;
}

/* nlayers MoE blocks over one chunk, x updated in place layer after layer; returns seconds (maple.c:47 clock). */
double rh_stack(float *x, int nb, int l0, int nlayers, const float *bias) {
    double t0 = now();
    for (int L = l0; L < l0 + nlayers; L++) if (rh_moe(L, x, nb, 1, NULL, bias, NULL) < 0) return -1.0;
    return now() - t0;
}
/* The head of the attention half as step_batch runs it (maple.c:711-717): per token, RMS norm of every query and key head with the
 * layer's q_norm / k_norm, half-rotary embedding at the token's position on local layers (maple.c:403-411), keys and values to fp16
 * (maple.c:314-320).  q [nb][NH*HD] and k [nb][NKV*HD] are updated in place; kc, vc [nb][NKV*HD] receive the cache rows. */
void rh_qk_rope(float *q, float *k, const float *v, const uint16_t *qn, const uint16_t *kn, const int *pos, int nb, int glob, uint16_t *kc, uint16_t *vc) {
    for (int i = 0; i < ROT / 2; i++) INV_FREQ[i] = 1.0 / pow(10000.0, (2.0 * i) / ROT);      /* maple.c:1085 */
    BF bq = {qn, HD, 1}, bk = {kn, HD, 1};
    for (int b = 0; b < nb; b++) {
        for (int h = 0; h < NH; h++) { float *p = q + ((size_t)b * NH + h) * HD; rmsnorm(p, p, &bq, HD); if (!glob) rope(p, pos[b]); }
        for (int h = 0; h < NKV; h++) { float *p = k + ((size_t)b * NKV + h) * HD; rmsnorm(p, p, &bk, HD); if (!glob) rope(p, pos[b]); }
        to_f16(kc + (size_t)b * NKV * HD, k + (size_t)b * NKV * HD, NKV * HD);
        to_f16(vc + (size_t)b * NKV * HD, v + (size_t)b * NKV * HD, NKV * HD);
    }
}
/* the (cos, sin) table maple.c hands to gfull_init (maple.c:1151-1153): cs[pos][32][2] */
void rh_rope_table(float *cs, int positions) {
    for (int i = 0; i < ROT / 2; i++) INV_FREQ[i] = 1.0 / pow(10000.0, (2.0 * i) / ROT);
    for (int pos = 0; pos < positions; pos++) for (int i = 0; i < ROT / 2; i++) {
        double f = pos * INV_FREQ[i]; cs[(pos * 32 + i) * 2] = (float)cos(f); cs[(pos * 32 + i) * 2 + 1] = (float)sin(f);
    }
}
int rh_bmax(void) { return BMAX; }
