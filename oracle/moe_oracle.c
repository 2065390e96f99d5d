/* moe_oracle.c -- TEST INFRASTRUCTURE ONLY: a scalar CPU restatement of the reference's int8 x ternary
 * mixture-of-experts path.  Nothing in the product library includes, links or calls this file; tests, the smoke
 * check and the CPU-baseline leg of the benchmark use it as the checker.
 *
 * Parity is PINNED: tests compare every stage of this file bit for bit with the reference's own maple.c compiled
 * from its sources (oracle/_ref, built by oracle/Makefile from ref_harness.c), and with fixtures that build wrote
 * under tests/golden/.  Each function cites the reference lines it restates.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define H 2048
#define FF 512
#define NE 256
#define TOPK 8
#define GU_BYTES 264192
#define EXPERT_BYTES 798720


/* a small static-split parallel for (no OpenMP on the build machines) */
#include <pthread.h>
#include <unistd.h>
typedef void (*orc_job)(void *arg, int i0, int i1);
typedef struct { orc_job fn; void *arg; int i0, i1; } orc_span;
static void *orc_tramp(void *p) { orc_span *s = p; s->fn(s->arg, s->i0, s->i1); return NULL; }
static int ORC_NT;
int orc_threads(int nt) { if (nt > 0) ORC_NT = nt > 64 ? 64 : nt; if (!ORC_NT) { long c = sysconf(_SC_NPROCESSORS_ONLN); ORC_NT = c < 1 ? 1 : c > 64 ? 64 : (int)c; } return ORC_NT; }
static void par_for(int n, int grain, orc_job fn, void *arg) {
    int nt = orc_threads(0); if (nt > (n + grain - 1) / grain) nt = (n + grain - 1) / grain;
    if (nt <= 1) { fn(arg, 0, n); return; }
    pthread_t th[64]; orc_span sp[64];
    for (int t = 0; t < nt; t++) { sp[t] = (orc_span){fn, arg, (int)((long)n * t / nt), (int)((long)n * (t + 1) / nt)}; pthread_create(&th[t], NULL, orc_tramp, &sp[t]); }
    for (int t = 0; t < nt; t++) pthread_join(th[t], NULL);
}

static inline float bf16_f32(uint16_t v) { union { uint32_t u; float f; } c = {(uint32_t)v << 16}; return c.f; }  /* maple.c:48 */

/* maple.c:184-194 prep: absmax int8 of one vector; qs = mx/127 (1 when all zero), round-half-even, total of q */
void orc_prep(const float *x, int n, int8_t *q, float *qs, int32_t *qsum) {
    float mx = 0.0f;
    for (int i = 0; i < n; i++) { float a = fabsf(x[i]); if (a > mx) mx = a; }
    float s = mx > 0.0f ? mx / 127.0f : 1.0f, inv = 1.0f / s;
    int32_t tot = 0;
    for (int i = 0; i < n; i++) { int v = (int)lrintf(x[i] * inv); q[i] = (int8_t)v; tot += v; }
    *qs = s; *qsum = tot;
}

/* maple.c:398-402 rmsnorm: sum of squares in double, k = 1/sqrtf((float)(ss/n) + 1e-6f), out = x*k*w */
void orc_rmsnorm(float *out, const float *x, const uint16_t *w, int n) {
    double ss = 0.0;
    for (int i = 0; i < n; i++) ss += (double)x[i] * (double)x[i];
    float k = 1.0f / sqrtf((float)(ss / n) + 1e-6f);
    for (int i = 0; i < n; i++) { float t = x[i] * k; out[i] = t * bf16_f32(w[i]); }
}

/* The single-precision exponential the CUDA kernels evaluate: the table-driven double-precision scheme published
 * with the Arm optimized routines and used by glibc >= 2.27 (N = 32 table of 2^(i/32), cubic in r, result rounded
 * once to float).  The reference calls libm expf (maple.c:738, 829, 915); tests check this model against libm on
 * every float the path can produce, so the GPU can be bit-identical without calling libm. */
static uint64_t EXP_TAB[32]; static int EXP_READY;
static void exp_init(void) {
    for (int i = 0; i < 32; i++) {
        double d = (double)exp2l((long double)i / 32.0L); uint64_t u; memcpy(&u, &d, 8);
        EXP_TAB[i] = u - ((uint64_t)i << 47);
    }
    EXP_READY = 1;
}
/* The head of the attention half (maple.c:711-717): RMS norm of the query and key heads (398-402), half-rotary embedding on local layers
 * (403-411; cos and sin from the table maple.c:1151-1153 builds: cs[pos][32][2]) in the fused forms the reference's compiler emits
 * (lo = fma(a, cos, -(b sin)), hi = fma(b, cos, a sin): pinned against the compiled reference by tests/test_oracle.py), keys and values
 * to fp16 with round to nearest even (314-320).  q [nb][16*128], k [nb][4*128] in place; kc, vc [nb][512]. */
static uint16_t orc_f16(float f) {      /* IEEE binary16, round to nearest even, as vcvtps2ph with rounding mode 0 */
    uint32_t x; memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u; x &= 0x7FFFFFFFu;
    if (x >= 0x7F800000u) return (uint16_t)(sign | 0x7C00u | (x > 0x7F800000u ? 0x200u | ((x >> 13) & 0x3FFu) : 0u));
    if (x >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);                       /* rounds to infinity */
    if (x < 0x33000001u) return (uint16_t)sign;                                     /* below half of the smallest subnormal */
    int e = (int)(x >> 23) - 127; uint32_t m = (x & 0x7FFFFFu) | 0x800000u;
    int shift = e < -14 ? 13 + (-14 - e) : 13;                                      /* subnormal results lose more bits */
    uint32_t h = m >> shift, rem = m & ((1u << shift) - 1u), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (h & 1u))) h++;
    if (e < -14) return (uint16_t)(sign | h);                                       /* h may carry into the smallest normal: same bit pattern */
    return (uint16_t)(sign | (((uint32_t)(e + 15) << 10) + (h - 0x400u)));          /* a mantissa carry bumps the exponent */
}
void orc_qk_rope(float *q, float *k, const float *v, const uint16_t *qn, const uint16_t *kn, const int *pos, const float *cs, int nb, int glob,
                 uint16_t *kc, uint16_t *vc) {
    for (int b = 0; b < nb; b++) {
        for (int h = 0; h < 20; h++) {
            float *p = h < 16 ? q + ((size_t)b * 16 + h) * 128 : k + ((size_t)b * 4 + (h - 16)) * 128;
            orc_rmsnorm(p, p, h < 16 ? qn : kn, 128);
            if (!glob) {
                const float *t = cs + (size_t)pos[b] * 64;
                for (int i = 0; i < 32; i++) {
                    const float a = p[i], bb = p[i + 32], c = t[2 * i], s = t[2 * i + 1];
                    p[i] = fmaf(a, c, -(bb * s)); p[i + 32] = fmaf(bb, c, a * s);
                }
            }
        }
        for (int i = 0; i < 512; i++) { kc[(size_t)b * 512 + i] = orc_f16(k[(size_t)b * 512 + i]); vc[(size_t)b * 512 + i] = orc_f16(v[(size_t)b * 512 + i]); }
    }
}
void orc_exp_table(uint64_t *out) { if (!EXP_READY) exp_init(); memcpy(out, EXP_TAB, sizeof EXP_TAB); }
float orc_expf_model(float x) {
    if (!EXP_READY) exp_init();
    if (x != x) return x;
    if (x > 89.0f) return INFINITY;
    if (x < -104.0f) return 0.0f;
    const double inv_ln2_n = 0x1.71547652b82fep+0 * 32.0, shift = 0x1.8p+52;
    const double c0 = 0x1.c6af84b912394p-5 / 32768.0, c1 = 0x1.ebfce50fac4f3p-3 / 1024.0, c2 = 0x1.62e42ff0c52d6p-1 / 32.0;
    double z = inv_ln2_n * (double)x, kd = z + shift;
    uint64_t ki; memcpy(&ki, &kd, 8);
    kd -= shift;
    double r = z - kd;
    uint64_t t = EXP_TAB[ki & 31] + (ki << 47);
    double s; memcpy(&s, &t, 8);
    double p = c0 * r + c1, r2 = r * r, y = c2 * r + 1.0;
    y = p * r2 + y;
    return (float)(y * s);
}

/* counts floats in [lo_bits, hi_bits] (stepping by stride through the bit patterns, both signs) where the model
 * and libm expf differ */
long orc_expf_check(uint32_t lo_bits, uint32_t hi_bits, uint32_t stride) {
    long bad = 0;
    for (uint64_t u = lo_bits; u <= hi_bits; u += stride) {
        uint32_t b = (uint32_t)u; float x, a, m;
        for (int sg = 0; sg < 2; sg++) {
            uint32_t bb = b | (sg ? 0x80000000u : 0u); memcpy(&x, &bb, 4);
            a = expf(x); m = orc_expf_model(x);
            if (memcmp(&a, &m, 4)) bad++;
        }
    }
    return bad;
}

/* maple.c:870-889 job_route_multi (== 853-869 job_route_small per (token, expert)): eight partial sums, lane j
 * takes columns j, j+8, ... in order with one fused multiply-add each; maple.c:117-121 hsum adds lanes as
 * ((l0+l4)+(l1+l5)) + ((l2+l6)+(l3+l7)). */
void orc_router_logits(const uint16_t *router, const float *hn, int nb, float *logits) {
    for (int b = 0; b < nb; b++) for (int e = 0; e < NE; e++) {
        const uint16_t *w = router + (size_t)e * H; const float *x = hn + (size_t)b * H;
        float l[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int c = 0; c < H; c += 8) for (int j = 0; j < 8; j++) l[j] = fmaf(bf16_f32(w[c + j]), x[c + j], l[j]);
        float a0 = l[0] + l[4], a1 = l[1] + l[5], a2 = l[2] + l[6], a3 = l[3] + l[7];
        logits[(size_t)b * NE + e] = (a0 + a1) + (a2 + a3);
    }
}
/* maple.c:146-157 bf_row, the order single-token decode uses (maple.c:609): two 8-lane accumulators over
 * 16-column steps, added lane-wise, then the same hsum. */
void orc_router_logits_step(const uint16_t *router, const float *hn, float *logits) {
    for (int e = 0; e < NE; e++) {
        const uint16_t *w = router + (size_t)e * H;
        float a[8] = {0}, c8[8] = {0};
        for (int c = 0; c < H; c += 16) for (int j = 0; j < 8; j++) {
            a[j] = fmaf(bf16_f32(w[c + j]), hn[c + j], a[j]);
            c8[j] = fmaf(bf16_f32(w[c + 8 + j]), hn[c + 8 + j], c8[j]);
        }
        float l[8]; for (int j = 0; j < 8; j++) l[j] = a[j] + c8[j];
        float a0 = l[0] + l[4], a1 = l[1] + l[5], a2 = l[2] + l[6], a3 = l[3] + l[7];
        logits[e] = (a0 + a1) + (a2 + a3);
    }
}

/* maple.c:910-923 job_topk (twins 735-744, 608-617): softmax in place, then 8 times the first strict maximum;
 * weights renormalised over the 8 by (sum + 1e-20f). */
void orc_topk(float *lg, int *top, float *w) {
    float mx = -1e30f, sum = 0.0f, tsum = 0.0f;
    for (int e = 0; e < NE; e++) if (lg[e] > mx) mx = lg[e];
    for (int e = 0; e < NE; e++) { lg[e] = expf(lg[e] - mx); sum += lg[e]; }
    for (int e = 0; e < NE; e++) lg[e] /= sum;
    for (int k = 0; k < TOPK; k++) {
        int best = 0; for (int e = 1; e < NE; e++) if (lg[e] > lg[best]) best = e;
        top[k] = best; w[k] = lg[best]; tsum += lg[best]; lg[best] = -1.0f;
    }
    for (int k = 0; k < TOPK; k++) w[k] /= (tsum + 1e-20f);
}

/* maple.c:924-938 group_pairs + 1018-1019 tp: used experts ascending, pairs of one expert in token order;
 * tp[b*8+j] = the j-th smallest pair index of token b.  Returns the number of pairs. */
int orc_group(const int *top, const float *tw, int nb, int *nu_out, int *ue, int *ustart, int *utok, float *uw, int *tp) {
    int cnt[NE] = {0}, uidx[NE], fill[NE] = {0}, nu = 0, na = 0;
    for (int i = 0; i < nb * TOPK; i++) cnt[top[i]]++;
    for (int e = 0; e < NE; e++) if (cnt[e]) { uidx[e] = nu; ue[nu] = e; ustart[nu++] = na; na += cnt[e]; }
    ustart[nu] = na;
    for (int b = 0; b < nb; b++) for (int s = 0; s < TOPK; s++) {
        int u = uidx[top[b * TOPK + s]], slot = ustart[u] + fill[u]++;
        utok[slot] = b; uw[slot] = tw[b * TOPK + s];
    }
    int *fl = calloc((size_t)nb, sizeof(int));
    for (int a = 0; a < na; a++) { int b = utok[a]; tp[b * TOPK + fl[b]++] = a; }
    free(fl);
    *nu_out = nu;
    return na;
}

/* maple.c:216-224 the scalar form of tdot: sum of code * q over one packed row (the caller subtracts qsum) */
int32_t orc_dot(const uint8_t *row, int cols, const int8_t *q) {
    int32_t tot = 0;
    for (int g = 0; g < cols / 128; g++) {
        const uint8_t *p = row + g * 32; const int8_t *qg = q + g * 128;
        for (int j = 0; j < 32; j++) {
            uint8_t b = p[j];
            tot += (b & 3) * qg[j] + ((b >> 2) & 3) * qg[32 + j] + ((b >> 4) & 3) * qg[64 + j] + (b >> 6) * qg[96 + j];
        }
    }
    return tot;
}
/* a faster equal: unpack the row once to (code - 1), then plain dot products (int32, exact) */
static void unpack_row(const uint8_t *row, int cols, int8_t *t) {
    for (int g = 0; g < cols / 128; g++) for (int j = 0; j < 32; j++) {
        uint8_t b = row[g * 32 + j]; int8_t *o = t + g * 128 + j;
        o[0] = (int8_t)((b & 3) - 1); o[32] = (int8_t)(((b >> 2) & 3) - 1); o[64] = (int8_t)(((b >> 4) & 3) - 1); o[96] = (int8_t)((b >> 6) - 1);
    }
}
static inline int32_t dot_i8(const int8_t *a, const int8_t *b, int n) { int32_t s = 0; for (int i = 0; i < n; i++) s += (int32_t)a[i] * b[i]; return s; }

/* maple.c:471-479 jobB_gateup -> 425-458 tdot_multi: out = (float)(tot - qsum) * qs * s[r] for every pair of
 * every used expert. experts[u] points at that expert's 798,720 bytes. dots (optional) receives tot - qsum. */
typedef struct { const uint8_t *const *experts; int nu; const int *ustart, *utok; const int8_t *hq; const float *hqs; float *gate, *up; int32_t *dots; } gu_arg;
static void gu_job(void *p, int j0, int j1) {
    gu_arg *g = p;
    for (int job = j0; job < j1; job++) {
        int u = job / (2 * FF), k = job % (2 * FF);
        const uint8_t *ex = g->experts[u] + (k < FF ? 0 : GU_BYTES);
        int r = k < FF ? k : k - FF;
        const float *sc = (const float *)(ex + 262144);
        int8_t t[H]; unpack_row(ex + (size_t)r * (H / 4), H, t);
        for (int a = g->ustart[u]; a < g->ustart[u + 1]; a++) {
            int b = g->utok[a];
            int32_t d = dot_i8(t, g->hq + (size_t)b * H, H);   /* == orc_dot(row, q) - qsum[b] */
            float v = (float)d * g->hqs[b] * sc[r];
            if (k < FF) g->gate[(size_t)a * FF + r] = v; else g->up[(size_t)a * FF + r] = v;
            if (g->dots) g->dots[(size_t)a * 2 * FF + k] = d;
        }
    }
}
void orc_gateup(const uint8_t *const *experts, int nu, const int *ustart, const int *utok,
                const int8_t *hq, const float *hqs, const int32_t *hqsum, float *gate, float *up, int32_t *dots) {
    (void)hqsum;
    gu_arg g = {experts, nu, ustart, utok, hq, hqs, gate, up, dots};
    par_for(nu * 2 * FF, 64, gu_job, &g);
}

/* maple.c:825-832: g = min(g,7), u = clamp(u,-7,7), act = g/(1+expf(-g))*u, then prep over the 512 values */
typedef struct { const float *gate, *up; float *act; int8_t *aq; float *aqs; int32_t *aqsum; } act_arg;
static void act_job(void *p, int a0, int a1) {
    act_arg *g = p;
    for (int a = a0; a < a1; a++) {
        float *o = g->act + (size_t)a * FF;
        for (int k = 0; k < FF; k++) {
            float gt = g->gate[(size_t)a * FF + k], u = g->up[(size_t)a * FF + k];
            gt = gt < 7.0f ? gt : 7.0f; u = u < -7.0f ? -7.0f : (u > 7.0f ? 7.0f : u);
            float q = gt / (1.0f + expf(-gt));
            o[k] = q * u;
        }
        orc_prep(o, FF, g->aq + (size_t)a * FF, &g->aqs[a], &g->aqsum[a]);
    }
}
void orc_act(const float *gate, const float *up, int np, float *act, int8_t *aq, float *aqs, int32_t *aqsum) {
    act_arg g = {gate, up, act, aq, aqs, aqsum};
    par_for(np, 16, act_job, &g);
}

/* maple.c:498-505 jobB_down: down[a][k] = (float)(tot - qsum_a) * qs_a * s[k], K = 512 */
typedef struct { const uint8_t *const *experts; const int *ustart; const int8_t *aq; const float *aqs; float *down; int32_t *dots; } dn_arg;
static void dn_job(void *p, int j0, int j1) {
    dn_arg *g = p;
    for (int job = j0; job < j1; job++) {
        int u = job / H, k = job % H;
        const uint8_t *ex = g->experts[u] + 2 * GU_BYTES;
        const float *sc = (const float *)(ex + 262144);
        int8_t t[FF]; unpack_row(ex + (size_t)k * (FF / 4), FF, t);
        for (int a = g->ustart[u]; a < g->ustart[u + 1]; a++) {
            int32_t d = dot_i8(t, g->aq + (size_t)a * FF, FF);
            g->down[(size_t)a * H + k] = (float)d * g->aqs[a] * sc[k];
            if (g->dots) g->dots[(size_t)a * H + k] = d;
        }
    }
}
void orc_down(const uint8_t *const *experts, int nu, const int *ustart, const int8_t *aq, const float *aqs,
              const int32_t *aqsum, float *down, int32_t *dots) {
    (void)aqsum;
    dn_arg g = {experts, ustart, aq, aqs, down, dots};
    par_for(nu * H, 256, dn_job, &g);
}

/* maple.c:834: x[utok[a]] += uw[a] * down[a] in pair order.  The reference's compiler fuses each multiply-add
 * (GCC contracts by default when the target has FMA), so the restatement uses fmaf; pinned against oracle/_ref. */
void orc_combine(float *x, const int *utok, const float *uw, const float *down, int np) {
    for (int a = 0; a < np; a++) {
        float *xo = x + (size_t)utok[a] * H; const float *d = down + (size_t)a * H; float w = uw[a];
        for (int i = 0; i < H; i++) xo[i] = fmaf(w, d[i], xo[i]);
    }
}

typedef struct {            /* same fields as the reference harness dump; NULL = not wanted */
    float *logits; int *top; float *topw; int *nu, *ue, *ustart; int *utok; float *uw; int *tp;
    int8_t *hq; float *hqs; int32_t *hqsum; float *gate, *up, *act; int8_t *aq; float *aqs; int32_t *aqsum; float *down;
    int32_t *gu_dots, *dn_dots;   /* [np][1024], [np][2048]: tot - qsum (not in the reference harness) */
} orc_dump;

#define KEEP(ptr, type, n) type *ptr##_ = d && d->ptr ? d->ptr : (type *)malloc(sizeof(type) * (size_t)(n))
#define DROP(ptr) do { if (!(d && d->ptr)) free(ptr##_); } while (0)

/* The MoE half of one layer (maple.c:732-835). experts_base: the layer's 256 experts back to back.
 * norm/x/y/bias as in the reference harness: norm != 0 updates the residual stream x in place,
 * norm == 0 takes x as the normalised hidden state and writes the weighted expert sum to y. */
int orc_moe(const uint16_t *router, const uint16_t *post_ln, const uint8_t *experts_base, float *x, int nb, int norm,
            float *y, const float *bias, orc_dump *d) {
    int np = nb * TOPK;
    float *hn = malloc(sizeof(float) * (size_t)nb * H);
    if (norm) for (int b = 0; b < nb; b++) orc_rmsnorm(hn + (size_t)b * H, x + (size_t)b * H, post_ln, H);
    else memcpy(hn, x, sizeof(float) * (size_t)nb * H);
    KEEP(hq, int8_t, (size_t)nb * H); KEEP(hqs, float, nb); KEEP(hqsum, int32_t, nb);
    for (int b = 0; b < nb; b++) orc_prep(hn + (size_t)b * H, H, hq_ + (size_t)b * H, &hqs_[b], &hqsum_[b]);
    KEEP(logits, float, (size_t)nb * NE);
    orc_router_logits(router, hn, nb, logits_);
    if (bias) for (int b = 0; b < nb; b++) for (int e = 0; e < NE; e++) logits_[(size_t)b * NE + e] += bias[e];
    KEEP(top, int, np); KEEP(topw, float, np);
    float *pr = malloc(sizeof(float) * NE);
    for (int b = 0; b < nb; b++) { memcpy(pr, logits_ + (size_t)b * NE, sizeof(float) * NE); orc_topk(pr, top_ + b * TOPK, topw_ + b * TOPK); }
    free(pr);
    int nu; KEEP(ue, int, NE); KEEP(ustart, int, NE + 1); KEEP(utok, int, np); KEEP(uw, float, np); KEEP(tp, int, np);
    orc_group(top_, topw_, nb, &nu, ue_, ustart_, utok_, uw_, tp_);
    if (d && d->nu) *d->nu = nu;
    const uint8_t *ex[NE]; for (int u = 0; u < nu; u++) ex[u] = experts_base + (size_t)ue_[u] * EXPERT_BYTES;
    KEEP(gate, float, (size_t)np * FF); KEEP(up, float, (size_t)np * FF); KEEP(act, float, (size_t)np * FF);
    KEEP(aq, int8_t, (size_t)np * FF); KEEP(aqs, float, np); KEEP(aqsum, int32_t, np); KEEP(down, float, (size_t)np * H);
    orc_gateup(ex, nu, ustart_, utok_, hq_, hqs_, hqsum_, gate_, up_, d ? d->gu_dots : NULL);
    orc_act(gate_, up_, np, act_, aq_, aqs_, aqsum_);
    orc_down(ex, nu, ustart_, aq_, aqs_, aqsum_, down_, d ? d->dn_dots : NULL);
    if (norm) orc_combine(x, utok_, uw_, down_, np);
    else { memset(y, 0, sizeof(float) * (size_t)nb * H); orc_combine(y, utok_, uw_, down_, np); }
    DROP(hq); DROP(hqs); DROP(hqsum); DROP(logits); DROP(top); DROP(topw); DROP(ue); DROP(ustart); DROP(utok); DROP(uw);
    DROP(tp); DROP(gate); DROP(up); DROP(act); DROP(aq); DROP(aqs); DROP(aqsum); DROP(down);
    free(hn);
    return np;
}
