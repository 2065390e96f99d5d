// k_umma_selftest.cu -- a one-CTA check of the tcgen05 building blocks (umma.cuh) against integer arithmetic a host
// can redo: D[128][n] = A[128][k] (u8) x B[n][k]^T (s8), A either staged in shared memory or written to tensor memory.
// Used by the test-suite before the grouped kernels are trusted.
#include <cuda_runtime.h>
#include <stdint.h>
#include "umma.cuh"

extern "C" void k_count_add(long n);

// k = 128 * kblocks.  A and B row-major [rows][k] in global memory.  mode 0: A from shared memory, 1: A from tensor memory.
__global__ void __launch_bounds__(128) umma_selftest_kernel(const uint8_t *__restrict__ A, const int8_t *__restrict__ B, int n, int kblocks,
                                                            int mode, int32_t *__restrict__ D, int *__restrict__ status) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_base;
    __shared__ int abort_flag;
    const int tid = threadIdx.x, warp = tid >> 5;
    const int K = kblocks * 128;
    uint8_t *As = smem, *Bs = smem + (size_t)kblocks * 128 * 128;   // [kb][row][128], swizzled
    if (tid == 0) { mbar_init(&bar, 1); abort_flag = 0; mbar_init_fence(); }
    if (warp == 0) tmem_alloc(&tmem_base, 512);
    // operands -> shared memory, 16 bytes per access, piece c of row r at c ^ (r & 7)
    for (int i = tid; i < 128 * K / 16; i += 128) {
        int r = i / (K / 16), c = i % (K / 16), kb = c >> 3, cc = c & 7;
        uint4 v = *reinterpret_cast<const uint4 *>(A + (size_t)r * K + c * 16);
        *reinterpret_cast<uint4 *>(As + ((size_t)kb * 128 + r) * 128 + ((cc ^ (r & 7)) << 4)) = v;
    }
    for (int i = tid; i < n * K / 16; i += 128) {
        int r = i / (K / 16), c = i % (K / 16), kb = c >> 3, cc = c & 7;
        uint4 v = *reinterpret_cast<const uint4 *>(B + (size_t)r * K + c * 16);
        *reinterpret_cast<uint4 *>(Bs + ((size_t)kb * n + r) * 128 + ((cc ^ (r & 7)) << 4)) = v;
    }
    proxy_fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tb = tmem_base, d_col = 0, a_col = 256;
    if (mode == 1) {   // A into tensor memory: lane = row, 32 columns per 128-column block
        for (int kb = 0; kb < kblocks && kb < 8; kb++) {
            uint32_t r[32];
            const uint32_t *src = reinterpret_cast<const uint32_t *>(A + (size_t)tid * K + kb * 128);
#pragma unroll
            for (int j = 0; j < 32; j++) r[j] = src[j];
            tmem_st32(tb + ((uint32_t)(warp * 32) << 16) + a_col + kb * 32, r);
        }
        tmem_st_wait();
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
    }
    if (tid == 0) {
        const uint32_t idesc = idesc_i8_u8s8((uint32_t)n);
        for (int kb = 0; kb < kblocks; kb++)
            for (int k = 0; k < 4; k++) {
                uint64_t bd = smem_desc_k128(smem_u32(Bs + (size_t)kb * n * 128), k * 32);
                if (mode == 0) umma_i8_ss(tb + d_col, smem_desc_k128(smem_u32(As + (size_t)kb * 128 * 128), k * 32), bd, idesc, (kb | k) != 0);
                else umma_i8_ts(tb + d_col, tb + a_col + kb * 32 + k * 8, bd, idesc, (kb | k) != 0);
            }
        umma_commit(&bar);
    }
    __syncwarp();
    bool ok = mbar_wait(&bar, 0, &abort_flag);
    tc_fence_after();
    if (ok) {
        for (int c0 = 0; c0 < n; c0 += 16) {
            uint32_t r[16];
            tmem_ld16(tb + ((uint32_t)(warp * 32) << 16) + d_col + c0, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; j++) D[(size_t)tid * n + c0 + j] = (int32_t)r[j];
        }
    } else if (tid == 0) *status = 1;
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tb, 512);
}

// Device pointers.  Returns 0 after queueing; *status (device int) becomes 1 if the MMA never signalled completion.
extern "C" int k_umma_selftest(cudaStream_t st, const uint8_t *A, const int8_t *B, int n, int kblocks, int mode, int32_t *D, int *status) {
    if (n < 16 || n > 256 || (n & 15) || kblocks < 1 || kblocks > 4) return -1;
    size_t smem = (size_t)kblocks * 128 * (128 + n) + 1024;
    cudaFuncSetAttribute(umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    umma_selftest_kernel<<<1, 128, smem, st>>>(A, B, n, kblocks, mode, D, status);
    k_count_add(1);
    return 0;
}
