// umma.cuh -- the sm_100a primitives the grouped expert GEMMs are built from, as inline PTX: mbarriers with bounded
// waits, tensor-memory allocation, tcgen05.mma kind::i8 (A from shared memory or from tensor memory), tcgen05.commit,
// tcgen05.ld / tcgen05.st, and the shared-memory / instruction descriptors.
#pragma once
#include <stdint.h>

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- mbarrier ----------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One poll.  The suspend-time hint lets the hardware park the thread until the phase completes (or the hint runs out) instead of
// returning at once: a waiting warp then does not take issue slots from the warps that are working.
#define MBAR_HINT_NS 20000u
__device__ __forceinline__ bool mbar_try_addr(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity), "r"(MBAR_HINT_NS) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_try(uint64_t *bar, uint32_t parity) { return mbar_try_addr(smem_u32(bar), parity); }
// Every wait is bounded: after MBAR_SPINS failed polls (each parks for up to MBAR_HINT_NS) the waiter gives up, raises *abort
// (shared memory, seen by all roles of the CTA) and returns false; callers then leave their loops, free tensor memory and return.
#define MBAR_SPINS (1u << 16)
__device__ __forceinline__ bool mbar_wait_addr(uint32_t bar, uint32_t parity, volatile int *abort) {
    if (mbar_try_addr(bar, parity)) return true;
    for (uint32_t i = 0; i < MBAR_SPINS; i++) {
        if (mbar_try_addr(bar, parity)) return true;
        if (*abort) return false;
    }
    *abort = 1;
    return false;
}
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort) { return mbar_wait_addr(smem_u32(bar), parity, abort); }

// One lane of a fully active warp (the same one every time).  tcgen05.mma is issued by a single thread; issuing it from the elected
// lane inside warp-uniform control flow keeps its operands in uniform registers.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred P1;\n\telect.sync _|P1, 0xffffffff;\n\tselp.u32 %0, 1, 0, P1;\n\t}" : "=r"(pred));
    return pred != 0;
}

// ---- tensor memory ---------------------------------------------------------------------------------------------
// one warp, all lanes: allocates ncols (power of two >= 32) columns, the address lands in *dst (shared memory)
__device__ __forceinline__ void tmem_alloc(uint32_t *dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void proxy_fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- descriptors -------------------------------------------------------------------------------------------------
// K-major operand in shared memory, 128-byte swizzle: row r of the tile is the 128 bytes at base + 128 r (8-row
// groups 1024 bytes apart), and inside a row the 16-byte piece c sits at position c ^ (r & 7).  base is 1024-aligned;
// byte_off (a multiple of 32) selects the 32-byte K-slice of one MMA.
__device__ __forceinline__ uint64_t smem_desc_k128(uint32_t base, uint32_t byte_off) {
    uint64_t d = 0;
    d |= (uint64_t)(((base + byte_off) >> 4) & 0x3FFF);        // start address
    d |= (uint64_t)1 << 16;                                      // leading byte offset (unused with a swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;                            // stride between 8-row groups
    d |= (uint64_t)1 << 46;                                      // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                                      // 128-byte swizzle
    return d;
}
// kind::i8: D s32, A unsigned 8-bit (ternary codes 0,1,2), B signed 8-bit, both K-major, M = 128, N = n (multiple of 16)
__device__ __forceinline__ uint32_t idesc_i8_u8s8(uint32_t n) {
    return (2u << 4) | (0u << 7) | (1u << 10) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

// ---- MMA ---------------------------------------------------------------------------------------------------------
// D[tmem] (+)= A[smem] * B[smem]^T ; one thread issues
__device__ __forceinline__ void umma_i8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]^T : A is 128 lanes x 8 columns, each 32-bit cell four consecutive K values
__device__ __forceinline__ void umma_i8_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// the mbarrier gets one arrival when every MMA issued so far by this thread has finished
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void umma_commit_addr(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ---- tensor memory <-> registers: thread t of warp w touches lane 32 (w % 4) + t, 32 consecutive columns ------------
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                   "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
                   "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
                   "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                   "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
                   "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
                   "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
                   "r"(r[30]), "r"(r[31]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---- TMA: 2-D tiled bulk tensor copy global -> shared, completion counted in bytes on an mbarrier -------------------
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// x = innermost coordinate (elements; times the element size a multiple of 16 bytes), y = row
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const void *tmap, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst_smem), "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}

// the 3-D form: x = innermost coordinate (same alignment rule), y, z = the outer two
__device__ __forceinline__ void tma_load_3d(uint32_t dst_smem, const void *tmap, int x, int y, int z, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst_smem), "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar)) : "memory");
}

// pulls a tensor map into the descriptor cache ahead of its first use: a copy through a map that is not there waits for it, and the copies
// queued behind it wait too
__device__ __forceinline__ void tma_prefetch_map(const void *tmap) { asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory"); }

// ---- asynchronous 16-byte copies global -> shared (gathered activation rows) -------------------------------------
__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
