// k_i8_peak.cu -- what the tensor cores of this GPU deliver in tcgen05.mma kind::i8: the denominator of the grouped GEMMs' roofline.
// One CTA per SM; an elected lane of a warp-uniform loop issues M = 128, K = 32 MMAs with both operands resident in shared memory
// (constant bytes: no memory traffic), N = n columns of one tensor-memory accumulator; the loop is timed with CUDA events by the
// caller.  2 * 128 * n * 32 integer operations per MMA.
#include <cuda_runtime.h>
#include <stdint.h>
#include "umma.cuh"

extern "C" void k_count_add(long n);

__global__ void __launch_bounds__(128, 1) i8_peak_kernel(int n, int iters, int *status) {
    extern __shared__ __align__(1024) uint8_t pk_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)pk_raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t bar; __shared__ uint32_t tmem; __shared__ int ab;
    const int tid = threadIdx.x;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    if (tid == 0) { mbar_init(&bar, 1); ab = 0; mbar_init_fence(); }
    if (warp == 0) tmem_alloc(&tmem, 256);
    for (int i = tid; i < (128 * 128 + 256 * 128) / 4; i += 128) ((uint32_t *)smem)[i] = 0x01020102u ^ (uint32_t)(i * 2654435761u & 0x03030303u);
    proxy_fence_async_smem(); tc_fence_before(); __syncthreads(); tc_fence_after();
    const uint32_t tb = tmem;
    if (warp == 0) {
        const uint32_t idesc = idesc_i8_u8s8((uint32_t)n);
        const uint32_t sbase = __shfl_sync(0xffffffffu, smem_u32(smem), 0);
        const uint64_t ad = smem_desc_k128(sbase, 0), bd = smem_desc_k128(sbase + 128 * 128, 0);
        for (int it = 0; it < iters; it++) {
#pragma unroll
            for (int k = 0; k < 4; k++) { if (elect_one()) umma_i8_ss(tb, ad + 2 * k, bd + 2 * k, idesc, 1); }
        }
        if (elect_one()) umma_commit(&bar);
        __syncwarp();
        if (!mbar_wait(&bar, 0, &ab) && (tid & 31) == 0) *status = 1;
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tb, 256);
}

// Queues `launches` launches of iters x 4 MMAs on every SM; *status (device) becomes 1 if a completion never arrived.
extern "C" int k_i8_peak(cudaStream_t st, int n, int iters, int sms, int *status) {
    if (n < 16 || n > 256 || (n & 15) || iters < 1) return -1;
    static bool attr_done = false;
    if (!attr_done) { cudaFuncSetAttribute(i8_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024); attr_done = true; }
    i8_peak_kernel<<<sms, 128, 60 * 1024, st>>>(n, iters, status);
    k_count_add(1);
    return 0;
}
