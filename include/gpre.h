/* gpre.h -- the reference runtime's GPU plug-in ABI for its "--gpupre" expert path, served by CUDA kernels for
 * sm_100a.  Every prototype below is the one maple.c declares under -DGPU_HEAD (maple.c:247-272); a maple.c built
 * with -DGPU_HEAD links against libgpre_cuda.so in place of gpu_head.m / gpu_exp.m / gpu_pre.m.
 *
 * Only the mixture-of-experts functions do work.  The output head, the expert cache, the dense attention
 * projections and the whole-layer attention driver are outside this library: their entry points exist so the
 * reference links, and they answer "unavailable" exactly the way the reference expects (non-zero from *_init),
 * which makes maple.c keep those parts on its own CPU path (maple.c:1096-1105, 1141, 1154-1158).
 *
 * All pointers are host pointers owned by the caller and are only read (or written) during the call.
 * The library keeps one CUDA context, one stream and its device buffers in file-scope state, as the reference's
 * plug-in does (gpu_pre.m:22-36); calls come from one thread; there is no teardown call in this ABI.
 */
#ifndef GPRE_H
#define GPRE_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* gpu_pre.m:266-316 / maple.c:257, called at maple.c:1105.  Allocates device buffers for chunks of up to maxtok
 * tokens with topk experts each (topk must be 8).  Returns 0, or -1 after a "gpre: ..." line on stderr. */
int gpre_init(int maxtok, int topk);

/* gpu_pre.m:173-181 / maple.c:258, called at maple.c:1125.  Registers a page-aligned span of an mmapped shard.
 * The reference wraps the span without copying; here the span is copied into HBM once (a B200 holds every
 * expert of the model).  Returns a region id 0..63, or -1 (not page aligned, too many regions, out of memory). */
int gpre_region(const void *p, size_t len);

/* gpu_pre.m:318-385 / maple.c:259, called at maple.c:763.  The experts of one layer for a chunk:
 *   x      [nb][2048] fp32, the normalised hidden state (after the post-attention RMSNorm)
 *   nu     used experts; loc [nu][12] = six (region slot 0..3, byte offset) pairs per used expert:
 *          gate codes, gate scales, up codes, up scales, down codes, down scales (maple.c:276, 1120)
 *   regs   [4] region ids behind slots 0..3, -1 = unused; next [4]: the next layer's regions (a prefetch hint,
 *          ignored: the weights are already resident)
 *   ustart [nu+1], ptok [np], pw [np] with np = ustart[nu]: pairs grouped by used expert (maple.c:749-755)
 *   tp     [nb][topk]: each token's pair indices, ascending (maple.c:761-762)
 *   y      [nb][2048] fp32 out = sum_k w_k * expert_k(x), WITHOUT the residual (the caller adds, maple.c:784)
 * Arithmetic is the reference's int8 x ternary CPU path (maple.c:425-458, 825-834), not the Metal kernels' fp32
 * activations.  Synchronous.  Returns the seconds the GPU spent (CUDA events), or a negative value after a
 * "gpre: ..." line when an argument is rejected (bad region, offset beyond the region, np > maxtok*topk). */
double gpre_moe(const float *x, int nb, int nu, const uint32_t *loc, const int *regs, const int *next,
                const int *ustart, const int *ptok, const float *pw, const int *tp, float *y);

/* gpu_pre.m:183-187 / maple.c:260.  Staging buffer for weights in VRAM: nothing to do here (regions already
 * live in HBM), returns 0. */
int gpre_stage(size_t bytes);
/* gpu_pre.m:258-264 / maple.c:264: seconds spent copying regions into HBM. */
double gpre_blit_seconds(void);

/* gpu_pre.m:508-566 / maple.c:268, called at maple.c:1021: the asynchronous form.  Same tables as gpre_moe, but
 * the normalised hidden state is the device-resident one (left by gmoe_post_norm, which stands in for the tail of
 * gfull_attn, gpu_pre.m:486-493) and the result is ADDED into the device-resident hidden state set by
 * gfull_begin.  Queued on the library's stream, not waited for (gpu_pre.m:562-564). */
void gfull_moe(int nu, const uint32_t *loc, const int *regs, const int *ustart, const int *ptok, const float *pw,
               const int *tp);
/* gpu_pre.m:433-436 / maple.c:266: a new chunk, nb hidden vectors copied to the device. pos0 is unused here. */
void gfull_begin(const float *x, int nb, int pos0);
/* gpu_pre.m:569-584 / maple.c:269: waits, copies the hidden state back. ko (the card's K/V rows) is set to NULL:
 * attention is not part of this library. */
void gfull_read(float *x, const uint16_t **ko);
/* gpu_pre.m:586 / maple.c:270 */
void gfull_write_x(const float *x);
/* gpu_pre.m:587 / maple.c:271 */
int gfull_maxtok(void);
/* gpu_pre.m:589-594 / maple.c:272: prints the GPU seconds spent in the experts. */
void gfull_report(void);

/* ---- the attention projections q,k,v,o: the same int8 x ternary product with one matrix and every token in it ----
 * gpu_pre.m:211-216 / maple.c:264, called at maple.c:1137-1139: adds one matrix (2048 columns, a multiple of 128 rows) to group g
 * (layer * 2 for q,k,v; layer * 2 + 1 for o); its outputs follow the group's earlier ones.  Copies codes and scales to the card. */
void gpre_dense_add(int g, const uint8_t *codes, const float *scales, int rows, int cols);
/* gpu_pre.m:217-233 / maple.c:265, called at maple.c:1141: 0 when every added matrix is on the card, else -1 (the caller then keeps
 * the projections on the CPU, as the reference does when its buffers do not fit). */
int gpre_dense_done(int maxtok);
/* gpu_pre.m:235-256 / maple.c:266: y[nb][rows of the group] = the group's matrices times prep(x[nb][2048]) (tdot_multi of
 * maple.c:459-470: per-token absmax int8, int32 dot, (float)(tot - qsum) * qs * s[r]).  Returns GPU seconds, -1.0 on error. */
double gpre_dense(int g, const float *x, int nb, float *y);

/* ---- present so the reference links; not part of the MoE path; each reports "unavailable" ---- */
int gfull_init(int ctx, int maxtok, int win, const float *norms, const uint16_t *router, const float *cs); /* -1: maple.c:1154-1156 falls back to experts-only */
double gfull_attn(int L, int glob, float *rl);                                   /* never reached after gfull_init fails; returns 0 */
int gpu_head_init(const uint16_t *w, int rows, int cols);                        /* -1: maple.c:1096 */
int gpu_head_init_i8(const int8_t *w, const float *scale, int rows, int cols);   /* -1: maple.c:1100 */
void gpu_head_run(const float *x, float *y);
void gpu_head_run_multi(const float *x, int n, float *y);
int gpux_init(int layers, int slots);                                            /* -1: maple.c:1103 */
void gpux_upload(int L, int slot, const uint8_t *gc, const float *gs, const uint8_t *uc, const float *us, const uint8_t *dc, const float *ds);
void *gpux_begin(int L, const float *x, int n, const int *slots);
void gpux_end(void *h, float *out, int n);
void *gpux_begin_multi(int L, const float *x, int nb, int nu, const int *slots, const int *pstart, const int *ptok);
void gpux_end_multi(void *h, float *out, int np);

#ifdef __cplusplus
}
#endif
#endif
