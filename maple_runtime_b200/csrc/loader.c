/* loader.c -- a converted checkpoint directory straight into HBM: the walk over layout.bin that maple.c does at start-up
 * (maple.c:61-81 load, 1106-1131 regions and GLOC), for hosts that use the gmoe_* entry points and have no table of their own.
 *
 * Directory (convert.py, layout.py:1-22): shard-00001.bin .. shard-00009.bin and layout.bin, a sequence of packed 26-byte records
 * {u8 kind ('b' bf16 | 't' ternary), u8 shard 0..8, u64 data offset, u64 scale offset, u32 rows, u32 cols} in the fixed order
 * embeddings, head, final norm, then per layer: input norm, post-attention norm, q norm, k norm, router, q, k, v, o and, for each
 * of the 256 experts, gate, up, down.  A directory may hold fewer than 24 layers (synthetic ones do).
 *
 * Per layer and shard the page-aligned span of the layer's expert tensors becomes one region (gpre_region copies it to the card
 * once), the twelve (slot, offset) words per expert are what maple.c calls GLOC, and gmoe_set_layer takes both together with the
 * router and post-attention norm rows.  Optionally the q,k,v and o matrices go to the card as the dense groups 2L and 2L+1. */
#include <errno.h>
#include <stdarg.h>
#include <fcntl.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include "../../include/gpre.h"
#include "../../include/gmoe.h"

#define NSHARD 9
#define NEXP 256
#define RECS_HEAD 3
#define RECS_LAYER (5 + 4 + 3 * NEXP)

typedef struct __attribute__((packed)) { uint8_t kind, file; uint64_t off, soff; uint32_t rows, cols; } LayoutRec;

static char g_load_err[512];
const char *gmoe_load_error(void) { return g_load_err; }
static int lfail(const char *fmt, ...) {
    va_list ap; va_start(ap, fmt); vsnprintf(g_load_err, sizeof g_load_err, fmt, ap); va_end(ap);
    fprintf(stderr, "gmoe_load: %s\n", g_load_err); return -1;
}

typedef struct { const uint8_t *p; size_t len; } Shard;
static void unmap_all(Shard *sh) { for (int k = 0; k < NSHARD; k++) if (sh[k].p) munmap((void *)sh[k].p, sh[k].len); }

/* tensor bytes inside a shard, with the bounds and alignment the kernels rely on */
static const uint8_t *span(const Shard *sh, int file, uint64_t off, size_t len, unsigned align) {
    if (file < 0 || file >= NSHARD || !sh[file].p || off > sh[file].len || len > sh[file].len - off || (off & (align - 1))) return NULL;
    return sh[file].p + off;
}

int gmoe_load_layers(const char *dir, int file_layer0, int nl, int dst_layer0, int with_dense) {
    g_load_err[0] = 0;
    if (!dir || nl < 1 || file_layer0 < 0 || dst_layer0 < 0 || dst_layer0 + nl > GMOE_LAYERS) return lfail("bad arguments (%s, %d layers to %d)", dir ? dir : "(null)", nl, dst_layer0);
    char path[1200];
    Shard sh[NSHARD]; memset(sh, 0, sizeof sh);
    for (int k = 0; k < NSHARD; k++) {              /* a directory need not have all nine; a record that names a missing one fails below */
        snprintf(path, sizeof path, "%s/shard-%05d.bin", dir, k + 1);
        int fd = open(path, O_RDONLY);
        if (fd < 0) continue;
        struct stat st;
        if (fstat(fd, &st) == 0 && st.st_size > 0) {
            void *p = mmap(NULL, (size_t)st.st_size, PROT_READ, MAP_SHARED, fd, 0);
            if (p != MAP_FAILED) { sh[k].p = p; sh[k].len = (size_t)st.st_size; }
        }
        close(fd);
    }
    snprintf(path, sizeof path, "%s/layout.bin", dir);
    FILE *f = fopen(path, "rb");
    if (!f) { unmap_all(sh); return lfail("%s: %s", path, strerror(errno)); }
    LayoutRec *rec = malloc(sizeof(LayoutRec) * RECS_LAYER);
    uint32_t *gloc = malloc(sizeof(uint32_t) * NEXP * 12);
    int rc = -1;
    if (!rec || !gloc) { lfail("out of host memory"); goto out; }
    const size_t pg = (size_t)getpagesize();
    for (int i = 0; i < nl; i++) {
        const int FL = file_layer0 + i, L = dst_layer0 + i;
        if (fseek(f, (long)sizeof(LayoutRec) * (RECS_HEAD + (long)FL * RECS_LAYER), SEEK_SET) != 0 ||
            fread(rec, sizeof(LayoutRec), RECS_LAYER, f) != RECS_LAYER) { lfail("%s has no layer %d", path, FL); goto out; }
        /* 0 in_ln, 1 post_ln, 2 q_norm, 3 k_norm, 4 router, 5..8 q k v o, 9.. experts (gate, up, down) */
        for (int k = 0; k < 5; k++) if (rec[k].kind != 'b') { lfail("%s: layer %d record %d is not bf16", path, FL, k); goto out; }
        for (int k = 5; k < RECS_LAYER; k++) if (rec[k].kind != 't') { lfail("%s: layer %d record %d is not ternary", path, FL, k); goto out; }
        if (rec[1].rows * (rec[1].cols ? rec[1].cols : 1) != 2048 || rec[4].rows != NEXP || rec[4].cols != 2048) { lfail("%s: layer %d: post-attention norm or router of another shape", path, FL); goto out; }
        const uint8_t *post_ln = span(sh, rec[1].file, rec[1].off, 2048 * 2, 2), *router = span(sh, rec[4].file, rec[4].off, (size_t)NEXP * 2048 * 2, 2);
        if (!post_ln || !router) { lfail("%s: layer %d: norm or router outside its shard", path, FL); goto out; }
        /* pass 1: the span of this layer's expert bytes in every shard */
        size_t lo[NSHARD], hi[NSHARD]; int slot[NSHARD], regs[4] = {-1, -1, -1, -1}, ns = 0;
        for (int k = 0; k < NSHARD; k++) { lo[k] = SIZE_MAX; hi[k] = 0; slot[k] = -1; }
        for (int e = 0; e < NEXP; e++) for (int m = 0; m < 3; m++) {
            const LayoutRec *r = &rec[9 + e * 3 + m];
            const uint32_t rows = m < 2 ? 512 : 2048, cols = m < 2 ? 2048 : 512;
            if (r->rows != rows || r->cols != cols) { lfail("%s: layer %d expert %d: matrix of another shape", path, FL, e); goto out; }
            const size_t clen = (size_t)rows * cols / 4, slen = (size_t)rows * 4;
            if (!span(sh, r->file, r->off, clen, 16) || !span(sh, r->file, r->soff, slen, 4)) { lfail("%s: layer %d expert %d: tensor outside its shard or misaligned", path, FL, e); goto out; }
            if (r->off < lo[r->file]) lo[r->file] = r->off;
            if (r->soff < lo[r->file]) lo[r->file] = r->soff;
            if (r->off + clen > hi[r->file]) hi[r->file] = r->off + clen;
            if (r->soff + slen > hi[r->file]) hi[r->file] = r->soff + slen;
        }
        for (int k = 0; k < NSHARD; k++) if (hi[k]) {
            lo[k] = lo[k] / pg * pg; hi[k] = (hi[k] + pg - 1) / pg * pg;
            if (hi[k] > sh[k].len) hi[k] = sh[k].len;                          /* the last page of a file may be short: copy what exists */
            if (ns == 4) { lfail("%s: layer %d spans more than 4 shards", path, FL); goto out; }
            size_t len = hi[k] - lo[k];
            int id;
            if (len % pg) {                                                    /* gpre_region wants whole pages: pad a private copy */
                size_t padded = (len + pg - 1) / pg * pg; void *tmp = NULL;
                if (posix_memalign(&tmp, pg, padded)) { lfail("out of host memory"); goto out; }
                memcpy(tmp, sh[k].p + lo[k], len); memset((char *)tmp + len, 0, padded - len);
                id = gpre_region(tmp, padded); free(tmp);
            } else id = gpre_region(sh[k].p + lo[k], len);
            if (id < 0) { lfail("%s: layer %d: the card refused a region (%s)", path, FL, gmoe_last_error()); goto out; }
            slot[k] = ns; regs[ns++] = id;
        }
        /* pass 2: (slot, offset inside the region) for codes and scales of gate, up, down */
        for (int e = 0; e < NEXP; e++) for (int m = 0; m < 3; m++) {
            const LayoutRec *r = &rec[9 + e * 3 + m];
            gloc[e * 12 + m * 4 + 0] = (uint32_t)slot[r->file]; gloc[e * 12 + m * 4 + 1] = (uint32_t)(r->off - lo[r->file]);
            gloc[e * 12 + m * 4 + 2] = (uint32_t)slot[r->file]; gloc[e * 12 + m * 4 + 3] = (uint32_t)(r->soff - lo[r->file]);
        }
        if (gmoe_set_layer(L, (const uint16_t *)router, (const uint16_t *)post_ln, gloc, regs) != 0) { lfail("layer %d: %s", L, gmoe_last_error()); goto out; }
        if (with_dense) for (int m = 0; m < 4; m++) {
            const LayoutRec *r = &rec[5 + m];
            const uint8_t *c = span(sh, r->file, r->off, (size_t)r->rows * r->cols / 4, 16), *s = span(sh, r->file, r->soff, (size_t)r->rows * 4, 4);
            if (!c || !s) { lfail("%s: layer %d: projection %d outside its shard", path, FL, m); goto out; }
            gpre_dense_add(L * 2 + (m == 3), c, (const float *)s, (int)r->rows, (int)r->cols);
        }
    }
    rc = 0;
out:
    free(rec); free(gloc); fclose(f); unmap_all(sh);
    return rc;
}
