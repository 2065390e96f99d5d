/* gmoe.h -- entry points this library ADDS next to the reference's plug-in ABI (gpre.h).
 *
 * The reference keeps softmax/top-8 and the grouping of pairs on the host between two GPU calls
 * (maple.c:1015-1021).  Here the whole mixture-of-experts half of a layer runs on the device:
 *   RMSNorm (maple.c:398-402) -> per-token absmax int8 (184-194) -> router logits (870-889) -> softmax + top-8
 *   (910-923) -> grouping by expert (924-938, 1018-1019) -> gate+up (471-479, 425-458) -> SiLU*up + per-pair int8
 *   (825-832) -> down (498-505) -> weighted combine into the hidden state (834).
 * Plain C ABI: pointers and sizes only.  Host pointers unless a name says _dev.
 * Every int-returning function returns 0 on success and -1 after a "gmoe: ..." line on stderr;
 * gmoe_last_error() returns that line.
 */
#ifndef GMOE_H
#define GMOE_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

#define GMOE_LAYERS 24
#define GMOE_MAXTOK_LIMIT 16384

/* ---- set-up ------------------------------------------------------------------------------------------------ */
/* Same as gpre_init(maxtok, 8) (maple.c:1105) plus the routing workspace; maxtok <= GMOE_MAXTOK_LIMIT. */
int gmoe_init(int maxtok);
/* A converted checkpoint directory (shard-0000N.bin + layout.bin, maple.c:61-81, layout.py) straight into HBM: layers
 * file_layer0 .. file_layer0+nl-1 of the directory become layers dst_layer0 .. of this library, through gpre_region and
 * gmoe_set_layer exactly as maple.c:1106-1131 builds its regions and GLOC; with_dense != 0 also adds every layer's q,k,v (group
 * 2L) and o (group 2L+1) with gpre_dense_add (call gpre_dense_done afterwards).  0, or -1 with gmoe_load_error(). */
int gmoe_load_layers(const char *dir, int file_layer0, int nl, int dst_layer0, int with_dense);
const char *gmoe_load_error(void);
/* Selects the CUDA device of this process (call before gmoe_init / gpre_init; one process per GPU). */
int gmoe_set_device(int dev);
/* Layer L's tables in the reference's own form: router bf16 [256][2048] (Layer.router, maple.c:39), post-attention
 * RMSNorm weight bf16 [2048] (Layer.post_ln), gloc = GLOC[L] [256][12] and regs = GREG[L] [4] as maple.c:1106-1131
 * builds them for regions registered with gpre_region.  post_ln may be NULL when only normalised input is used. */
int gmoe_set_layer(int L, const uint16_t *router, const uint16_t *post_ln, const uint32_t *gloc, const int *regs);
/* Synthetic layer L generated in HBM by the device generator (synth.h), registered like gmoe_set_layer.
 * e0/ne: only experts e0..e0+ne-1 are materialised (expert-parallel shards); e0 = 0, ne = 256 for all. */
int gmoe_synth_layer(uint64_t seed, int L, int e0, int ne);

/* ---- one layer, host buffers (the drop-in shape of gpre_moe with routing on the device) ---------------------- */
/* x [nb][2048] normalised hidden state; y [nb][2048] = sum_k w_k expert_k(x), no residual; bias [256] added to
 * the router logits before the softmax (NULL = none; the reference has no bias, benchmarks use it for skew).
 * Synchronous; returns GPU seconds or a negative value. */
double gmoe_moe(int L, const float *x, int nb, float *y, const float *bias);

/* ---- the residual stream through nl layers starting at l0 ----------------------------------------------------- */
/* Host in/out: per layer hn = rmsnorm(x, post_ln), x += moe(hn) (maple.c:733-834).  Returns the seconds on the
 * device timeline from the start of the host-to-device copy of x to the end of the copy back. */
double gmoe_forward(float *x, int nb, int l0, int nl, const float *bias);
/* The same without waiting, for hosts that stream chunks: gmoe_forward_submit queues the copy of x_in (pinned host memory) to the
 * card, the layers and the copy of the result to x_out (pinned; may be x_in) and returns; at most two chunks may be outstanding, so that
 * one chunk's copies run beside the other's kernels (three streams, two staging slots on the card).  gmoe_forward_wait waits for the
 * oldest outstanding chunk; its x_out is then complete.  It returns the seconds on the device timeline from the last gmoe_forward_mark
 * (or the first submit) to the end of that chunk's copy back, or a negative value.  After gmoe_ep_init the expert-parallel layer loop
 * runs (every rank submits and waits alike).  Other entry points must not be called while chunks are outstanding.  No counterpart in
 * the reference (maple.c:1015-1023 waits for every call). */
int gmoe_forward_submit(const float *x_in, float *x_out, int nb, int l0, int nl, const float *bias);
double gmoe_forward_wait(void);
int gmoe_forward_mark(void);

/* on = 1: the reference-shaped calls (gpre_moe, gfull_begin, gfull_read) page-lock a host buffer of 1 MB or more where it lies when
 * they see it a second time at the same address and length, and leave it so: maple.c keeps its hidden-state arrays for the life of the
 * process (HNB, YB, maple.c:763), and copies from and to page-locked memory run at several times the rate of pageable memory.
 * on = 0 (default) releases every such registration and stops making new ones.  GPRE_PIN_HOST=1 in the environment turns the policy on
 * for a host whose source is not touched.  Only for hosts that do not free those buffers while the library may still see them: memory
 * mapped later at a freed, still registered address would be read through the old pages.  No counterpart in the reference (its card
 * path shares memory with the host). */
int gpre_pin_policy(int on);

/* ---- the head of the attention half of a layer, on the card (the reference's kernel `qkn`, gpu_full.metal:32-71; its CPU form
 * maple.c:711-717).  Per token and head: RMS norm of the 16 query and 4 key heads (head dimension 128; qn, kn [128] fp32 as gfull_init
 * receives them, maple.c:1148), on local layers (glob == 0) the half-rotary embedding at the token's position (dimensions 0..63 as pairs
 * (i, i + 32), maple.c:403-411) with cos and sin from the table the host builds for gfull_init (maple.c:1151-1153:
 * cs[position][32][2] = (cos, sin), handed over once with gmoe_rope_table), queries out in fp32, keys and values out in fp16 (the rows
 * the KV cache receives, maple.c:716-717).  qkv [nb][3072] = q 2048 | k 512 | v 512 (the q,k,v projections' output, gpre_dense group 2L);
 * pos [nb]; q [nb][2048]; kc, vc [nb][512] fp16.  Host pointers, synchronous; returns the kernel's seconds or a negative value.  Results
 * are the compiled reference's bits.  This is the first piece of the attention half; attention itself, the cache and the output head
 * are not on the card (gfull_init answers "unavailable"). */
int gmoe_rope_table(const float *cs, int positions);
double gmoe_qk_rope(const float *qkv, const int *pos, int nb, int glob, const float *qn, const float *kn, float *q, uint16_t *kc, uint16_t *vc);
/* Device-resident form: upload once, run (asynchronous, on the library's stream), download. */
int gmoe_x_upload(const float *x, int nb);
int gmoe_x_download(float *x, int nb);
int gmoe_forward_dev(int nb, int l0, int nl, const float *bias);
/* A ring of input chunks kept in HBM so a benchmark step starts with its input resident: chunk c of nchunks, each
 * nb tokens.  gmoe_forward_chunk copies chunk c into the hidden state (device to device) and runs the layers,
 * asynchronously like gmoe_forward_dev. */
int gmoe_chunks_upload(const float *x, int nb, int nchunks);
int gmoe_forward_chunk(int chunk, int nb, int l0, int nl, const float *bias);
/* The layer loop of gmoe_forward* is replayed as a CUDA graph from the second call with the same (nb, l0, nl) on (one launch per
 * call).  on = 0 switches that off (also: environment GMOE_GRAPH=0), e.g. to time every stage with gmoe_profile. */
int gmoe_set_graph(int on);
/* How many times a captured layer loop has been replayed since load (tests use it to know that a call was a replay). */
long gmoe_graph_launches(void);
/* Waits for the stream; returns the GPU seconds between the last gmoe_forward_dev's first and last kernel. */
double gmoe_sync(void);
/* rmsnorm(post_ln[L]) of the device-resident hidden state + int8 + router logits: the part of gfull_attn
 * (gpu_pre.m:486-501) that feeds the experts.  logits [nb][256] may be NULL. Synchronous. */
int gmoe_post_norm(int L, int nb, float *logits);

/* ---- expert parallelism across the GPUs of one NVLink box (no counterpart in the reference, which is single-device) ---- */
/* One process per GPU.  Rank r keeps its own tokens and experts r*E .. (r+1)*E-1 (E = 256/world; gmoe_synth_layer or
 * gmoe_set_layer give each rank at least its own experts).  Set-up: rank 0 calls gmoe_ep_unique_id and hands the 128 bytes
 * to every rank; every rank calls gmoe_ep_init (after gmoe_init), then gmoe_ep_handles; the 448-byte results of all ranks,
 * concatenated in rank order, go to gmoe_ep_connect on every rank.  Then gmoe_ep_forward* replace gmoe_forward*: same
 * arguments, same result bits, every rank calls them together with the same nb. */
int gmoe_ep_unique_id(void *out128);
int gmoe_ep_init(int rank, int world, const void *id128);
int gmoe_ep_handles(void *out448);
int gmoe_ep_connect(const void *all_handles);
/* chunk >= 0: start from chunk `chunk` of the ring (gmoe_chunks_upload); -1: from the device-resident hidden state */
int gmoe_ep_forward_dev(int chunk, int nb, int l0, int nl, const float *bias);
double gmoe_ep_forward(float *x, int nb, int l0, int nl, const float *bias);
int gmoe_ep_allmax(double *v);            /* max over ranks (also a barrier) */
int gmoe_ep_received(void);               /* pairs this rank's experts received in the last layer */
/* The ranks meet through arrival flags in each other's memory; a wait longer than 10 s makes the call fail (code 41 in the
 * message).  This runs such a wait with a missing peer and a limit of `ms` milliseconds on this GPU alone and returns the code. */
int gmoe_ep_timeout_selftest(int ms);

/* ---- parity hooks: named device buffers of the last call, and single stages ---------------------------------- */
/* Names: x hn y hq hqs hqsum logits top topw nu ue ustart utok uw tp gate up act aq aqs aqsum down gu_dots dn_dots */
int gmoe_peek(const char *name, void *dst, size_t bytes);
int gmoe_poke(const char *name, const void *src, size_t bytes);
/* keep = 1: the expert kernels also store gate, up and the int32 dot products (tot - qsum). */
int gmoe_keep_stages(int keep);
/* Runs one stage on the device buffers for nb tokens of layer L: "norm" (x->hn,hq..), "prep" (hn->hq..),
 * "router", "router_tensor" (hn -> logits, top-8, weights on the tensor-core path), "topk", "group", "gateup", "actq", "down", "combine_y" (y = sum), "combine_x" (x += sum). */
int gmoe_stage(const char *name, int L, int nb);
/* Router: 0 = by size (default): batches of 512 tokens and more compute the logits on the tensor cores (fp16 x 2 terms, fp32
 * accumulation) and recompute, in the reference's exact order of operations, every token whose nine largest logits are closer than an
 * error bound; 1 = always the exact-order kernels (logits, weights and everything downstream have the reference's bits);
 * 2 = tensor cores for every batch size.  In all modes the top-8 indices are the reference's (maple.c:910-923). */
int gmoe_set_router(int mode);
/* The reference computes a lone token's router logits in two different orders: `step` (token-by-token decode, maple.c:609) calls
 * bf_row (maple.c:146-157: two multiply-add chains per lane), `step_batch` (prefill chunks and --multi, maple.c:734) calls
 * job_route_small (853-869: one chain per lane).  The bits differ, so a near-tie can choose differently.  on = 1: calls with one
 * token use the `step` order; on = 0 (default): the `step_batch` order for every size. */
int gmoe_set_step_order(int on);
/* tokens of the last tensor-core router call that took the exact path */
int gmoe_router_flagged(void);
/* 0 = grouped kernels chosen by size (default), 1 = force the mma.sync register-decode kernels,
 * 2 = force the tcgen05 kernels. */
int gmoe_set_path(int path);
/* The exact-order router kernel for batches above 256 tokens gives each thread tt tokens x 16 experts; tt = 4..8 pins that
 * (every value gives the same bits), 0 = choose by batch size (default). */
void gmoe_router_tile_tokens(int tt);
/* Copies bytes [off, off+bytes) of a registered region (gpre_region id, or the id a synthetic layer got: regions are
 * numbered in registration order) back to the host, to check what lives in HBM. */
int gmoe_region_read(int region, size_t off, void *dst, size_t bytes);
int gmoe_region_count(void);

/* ---- grouping without any allocation ------------------------------------------------------------------------------ */
/* No counterpart in the reference (its grouping is host code, maple.c:924-938); added for callers that cannot
 * allocate device memory when they need the grouping: a server working inside a memory budget fixed at start-up, a
 * plug-in inside another runtime's pool, a latency path where cudaMalloc's device-wide synchronisation is not
 * acceptable.  Same result as the grouping stage of gmoe_moe (NU, UE, USTART, UTOK, UW, tp of maple.c:924-938,
 * 1018-1019), computed with scratch that is a fixed array inside the loaded library (about 270 KB per GPU, held until
 * the process exits) instead of buffers from cudaMalloc.  All pointers are DEVICE pointers owned by the caller:
 *   top [nb][8] expert ids, topw [nb][8] routing weights  ->  nu [1], ue [256], ustart [257], utok [nb*8], uw [nb*8],
 *   tp [nb*8].  stream: a cudaStream_t (NULL = the default stream); the work is queued there, not waited for.
 * Limit: 1 <= nb <= GMOE_NOALLOC_MAXTOK; more is rejected with -2 and a message.  Returns 0, -1 (null pointer),
 * -2 (too many tokens), -3 (CUDA error), each with a "gmoe: ..." line on stderr.
 * The first call on a GPU looks up the array's device address (cudaGetSymbolAddress); make that first call before
 * any stream capture starts.  The array is shared by every call and keeps the previous call's contents; the masks
 * are cleared at the start of each call.  Calls that overlap on the GPU race on it: order them. */
#define GMOE_NOALLOC_MAXTOK 2048
int gmoe_group_noalloc(const int *top, const float *topw, int nb, int *nu, int *ue, int *ustart, int *utok, float *uw,
                       int *tp, void *stream);

/* ---- per-stage timing (the reference's GPRE_PROF=1 split, gpu_pre.m:349-365) ------------------------------------ */
/* mask: bit s set = CUDA events are recorded around stage s of every layer (0 norm+int8, 1 router, 2 top-8, 3 grouping,
 * 4 gate+up, 5 SiLU int8, 6 down, 7 combine).  gmoe_profile_read waits for the stream, adds up the recorded intervals
 * into secs[8] / launches[8] (kernel launches timed) and clears them. */
#define GMOE_STAGES 8
int gmoe_profile(unsigned mask);
int gmoe_profile_read(double *secs, long *launches);

/* ---- check of the tensor-core building blocks ------------------------------------------------------------------------ */
/* d[128][n] = a[128][k] (unsigned bytes) x b[n][k]^T (signed bytes), k = 128*kblocks, on one CTA with tcgen05.mma
 * kind::i8; mode 0 stages A in shared memory, mode 1 writes A to tensor memory.  Host pointers.  0 = ran,
 * -1 = bad arguments or CUDA error, -2 = the MMA never signalled completion. */
int gmoe_umma_selftest(const uint8_t *a, const int8_t *b, int n, int kblocks, int mode, int32_t *d);

/* The rate at which this GPU executes tcgen05.mma kind::i8 (M = 128, N = n, K = 32, operands resident in shared memory, one CTA per
 * SM, iters x 4 MMAs each), timed with CUDA events: 1e12 integer operations per second, or a negative value.  The roofline
 * denominator of the grouped expert GEMMs; n = 256 and iters >= 20000 give a run of some tens of milliseconds. */
double gmoe_i8_peak(int n, int iters);

/* ---- utilities -------------------------------------------------------------------------------------------------- */
const char *gmoe_last_error(void);
long gmoe_launch_count(void);             /* kernels launched by this library since load */
void *gmoe_pinned_alloc(size_t bytes);    /* page-locked host memory for x/y so copies overlap */
void gmoe_pinned_free(void *p);
int gmoe_device_info(char *name, int namelen, int *sms, size_t *hbm_bytes);

/* ---- synthetic workload (host side; synth.h gives the generator) ------------------------------------------------ */
void msynth_expert(uint64_t seed, int L, int e, uint8_t *dst);                 /* 798,720 bytes */
void msynth_experts(uint64_t seed, int L, int e0, int ne, uint8_t *dst);
void msynth_router(uint64_t seed, int L, uint16_t *dst);                       /* bf16 [256][2048] */
void msynth_norm(uint64_t seed, int L, uint16_t *dst);                         /* bf16 [2048] */
void msynth_hidden(uint64_t seed, uint64_t stream, int nb, float *dst);        /* fp32 [nb][2048] ~ N(0,1) */
void msynth_zipf_bias(uint64_t seed, double s, float *bias);                   /* fp32 [256] */

#ifdef __cplusplus
}
#endif
#endif
