/* synth_host.c -- host side of the synthetic-workload generator (see synth.h).  Plain C, no CUDA. */
#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <unistd.h>
#include <string.h>
#include "synth.h"
#include "../../include/gmoe.h"

/* One expert (798,720 bytes, converter layout) of layer L into dst. */
void msynth_expert(uint64_t seed, int L, int e, uint8_t *dst) {
    static const uint32_t off[3] = {0, MS_GU_BYTES, 2 * MS_GU_BYTES};
    static const uint32_t ncode[3] = {MS_GU_CODES, MS_GU_CODES, MS_DN_CODES};
    static const uint32_t nrow[3] = {MS_FF, MS_FF, MS_H};
    for (int m = 0; m < 3; m++) {
        uint8_t *c = dst + off[m];
        uint64_t tc = ms_tid(L, e, 2 * m), ts = ms_tid(L, e, 2 * m + 1);
        for (uint32_t i = 0; i < ncode[m]; i++) c[i] = ms_code_byte(seed, tc, i);
        float *s = (float *)(c + ncode[m]);
        for (uint32_t r = 0; r < nrow[m]; r++) s[r] = ms_scale(seed, ts, r);
    }
}

/* Experts e0 .. e0+ne-1 of layer L, back to back; split over the host's cores. */
typedef struct { uint64_t seed; int L, e0, e1; uint8_t *dst; int base; } ms_span;
static void *ms_span_run(void *p) {
    ms_span *s = p;
    for (int e = s->e0; e < s->e1; e++) msynth_expert(s->seed, s->L, e, s->dst + (size_t)(e - s->base) * MS_EXPERT_BYTES);
    return NULL;
}
void msynth_experts(uint64_t seed, int L, int e0, int ne, uint8_t *dst) {
    long nc = sysconf(_SC_NPROCESSORS_ONLN);
    int nt = nc < 1 ? 1 : nc > 32 ? 32 : (int)nc;
    if (nt > ne) nt = ne;
    pthread_t th[32]; ms_span sp[32];
    for (int t = 0; t < nt; t++) {
        sp[t] = (ms_span){seed, L, e0 + (int)((long)ne * t / nt), e0 + (int)((long)ne * (t + 1) / nt), dst, e0};
        if (pthread_create(&th[t], NULL, ms_span_run, &sp[t])) { ms_span_run(&sp[t]); th[t] = 0; }
    }
    for (int t = 0; t < nt; t++) if (th[t]) pthread_join(th[t], NULL);
}

static float ms_bf16_round(float f, uint16_t *out) {   /* round to nearest even, as a bf16 store does */
    uint32_t u; memcpy(&u, &f, 4);
    u += 0x7FFFu + ((u >> 16) & 1u);
    u &= 0xFFFF0000u;
    *out = (uint16_t)(u >> 16);
    memcpy(&f, &u, 4); return f;
}
static float ms_normal(uint64_t seed, uint64_t tid, uint64_t idx) {   /* Box-Muller on two 24-bit uniforms */
    uint64_t h = ms_u64(seed, tid, idx);
    float u1 = ((float)(uint32_t)(h >> 40) + 1.0f) * (1.0f / 16777216.0f);   /* (0, 1] */
    float u2 = (float)(uint32_t)((h >> 16) & 0xFFFFFFu) * (1.0f / 16777216.0f);
    return sqrtf(-2.0f * logf(u1)) * cosf(6.28318530717958647692f * u2);
}

/* Router of layer L: N(0, 1/sqrt(2048)) drawn in fp32, then rounded to bf16 (the reference stores bf16, maple.c:39). */
void msynth_router(uint64_t seed, int L, uint16_t *dst) {
    const float sd = 1.0f / sqrtf((float)MS_H);
    uint64_t tid = ms_tid(L, 0, 6);
    for (uint32_t i = 0; i < (uint32_t)MS_NE * MS_H; i++) ms_bf16_round(ms_normal(seed, tid, i) * sd, &dst[i]);
}
/* RMSNorm weight of layer L: ones (bf16 0x3F80). */
void msynth_norm(uint64_t seed, int L, uint16_t *dst) { (void)seed; (void)L; for (int i = 0; i < MS_H; i++) dst[i] = 0x3F80; }

/* nb hidden vectors ~ N(0,1), fp32. stream distinguishes independent batches. */
void msynth_hidden(uint64_t seed, uint64_t stream, int nb, float *dst) {
    uint64_t tid = (1ull << 26) + stream;
    for (size_t i = 0; i < (size_t)nb * MS_H; i++) dst[i] = ms_normal(seed, tid, i);
}
/* Router bias b_e = ln(256 p_e), p_e proportional to rank(e)^-s, rank a seeded permutation of 1..256. */
void msynth_zipf_bias(uint64_t seed, double s, float *bias) {
    int perm[MS_NE]; double p[MS_NE], z = 0;
    for (int i = 0; i < MS_NE; i++) perm[i] = i;
    for (int i = MS_NE - 1; i > 0; i--) {   /* Fisher-Yates on the counter generator */
        int j = (int)(ms_u64(seed, (1ull << 27), (uint64_t)i) % (uint64_t)(i + 1));
        int t = perm[i]; perm[i] = perm[j]; perm[j] = t;
    }
    for (int r = 0; r < MS_NE; r++) { p[r] = pow((double)(r + 1), -s); z += p[r]; }
    for (int r = 0; r < MS_NE; r++) bias[perm[r]] = (float)log(256.0 * p[r] / z);
}
