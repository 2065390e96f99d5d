// noalloc_group.cu -- grouping of (token, expert) pairs for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need the grouping: a serving loop that
// runs under a fixed memory budget handed out at start-up, a plug-in living inside another runtime's memory pool, or
// code on a latency path where an allocation (a device-wide synchronising call) is not acceptable.  For them this
// file offers one entry point, gmoe_group_noalloc, that does the same work as the library's grouping stage but keeps
// its scratch in a fixed array that is part of the loaded module instead of in buffers obtained from cudaMalloc.
//
// The scratch (NA_SCRATCH_BYTES, about 270 KB) exists once per GPU that loads the library and stays until the
// process exits.  It bounds the call: at most NA_MAXTOK = 2048 tokens.  Every call uses the same array and finds
// the previous call's contents in it; the part that has to start at zero (the token bit masks) is cleared on the
// caller's stream at the start of each call.  Two calls that overlap on the GPU (different streams, or different
// host threads) would both write the array: callers must order them.
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdint.h>
#include "kernels.h"
#include "../../include/gmoe.h"

#define NA_MAXTOK GMOE_NOALLOC_MAXTOK
#define NA_WORDS (NA_MAXTOK / 32)
#define NA_TILES (NA_MAXTOK * 8 / 8 + 256)

struct NaScratch {
    unsigned mask[256 * NA_WORDS + 256]; // bit b % 32 of word [b / 32][e]: token b chose expert e; then one counter per expert (all zero at the start of a call)
    int estart[256];
    int slot[NA_MAXTOK * 8];
    MoeTile tiles_a[NA_TILES], tiles_b[NA_TILES];
    int ntiles_a[4], ntiles_b[4];
};
#define NA_SCRATCH_BYTES sizeof(NaScratch)

// Lives in the module's device image.  In host code this name is only a handle for the runtime: the device address
// comes from cudaGetSymbolAddress, once per device, below.
static __device__ __align__(256) unsigned char g_na_scratch[NA_SCRATCH_BYTES];

#define NA_MAXDEV 64
static NaScratch *g_na_dev[NA_MAXDEV];   // device address of the array on each GPU, filled on the first call there

extern "C" int gmoe_group_noalloc(const int *top, const float *topw, int nb, int *nu, int *ue, int *ustart, int *utok,
                                  float *uw, int *tp, void *stream) {
    if (!top || !topw || !nu || !ue || !ustart || !utok || !uw || !tp) {
        fprintf(stderr, "gmoe: gmoe_group_noalloc: null pointer argument\n"); return -1;
    }
    if (nb < 1 || nb > NA_MAXTOK) {
        fprintf(stderr, "gmoe: gmoe_group_noalloc: %d tokens, but the built-in scratch holds 1..%d (use the allocating path for more)\n", nb, NA_MAXTOK);
        return -2;
    }
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= NA_MAXDEV) {
        fprintf(stderr, "gmoe: gmoe_group_noalloc: no current CUDA device (%s)\n", cudaGetErrorString(e)); return -3;
    }
    if (!g_na_dev[dev]) {   // set-up, first call on this device: ask the runtime where the array lives on it
        void *p = NULL;
        e = cudaGetSymbolAddress(&p, g_na_scratch);
        if (e != cudaSuccess || !p) {
            fprintf(stderr, "gmoe: gmoe_group_noalloc: cudaGetSymbolAddress: %s\n", cudaGetErrorString(e)); return -3;
        }
        g_na_dev[dev] = static_cast<NaScratch *>(p);
    }
    NaScratch *s = g_na_dev[dev];
    GroupArgs g;
    g.top = top; g.topw = topw; g.nb = nb; g.marked = 0;
    g.mask = s->mask; g.mask_words = (nb + 31) / 32;
    g.nu = nu; g.ue = ue; g.estart = s->estart; g.ustart = ustart; g.utok = utok; g.slot = s->slot; g.tp = tp; g.uw = uw;
    g.ecnt = NULL; g.uexp = NULL;
    g.tiles_a = s->tiles_a; g.tiles_b = s->tiles_b; g.ntiles_a = s->ntiles_a; g.ntiles_b = s->ntiles_b; g.tn_a = 8; g.tn_b = UMMA_TN;
    k_group(static_cast<cudaStream_t>(stream), &g);   // above 256 tokens: clears the masks and counters (cudaMemsetAsync), then two kernels; up to 256: one kernel with its masks in shared memory; no allocation either way
    e = cudaGetLastError();
    if (e != cudaSuccess) { fprintf(stderr, "gmoe: gmoe_group_noalloc: launch failed: %s\n", cudaGetErrorString(e)); return -3; }
    return 0;
}
