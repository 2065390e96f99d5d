// k_synth.cu -- device side of the synthetic-weight generator (synth.h): fills experts in HBM with the same bytes
// the host generator (synth_host.c) produces, so a 4.9 GB model never crosses PCIe.
#include <cuda_runtime.h>
#include "kernels.h"
#include "synth.h"

extern "C" void k_count_add(long n);

__global__ void __launch_bounds__(256) synth_experts_kernel(uint64_t seed, int L, int e0, uint32_t *__restrict__ dst, size_t nwords) {
    const size_t wpe = MS_EXPERT_BYTES / 4;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nwords; i += (size_t)gridDim.x * blockDim.x) {
        const int e = e0 + (int)(i / wpe);
        uint32_t o = (uint32_t)(i % wpe) * 4u, m = 0;             // byte offset inside the expert; matrix 0 gate, 1 up, 2 down
        if (o >= 2 * MS_GU_BYTES) { m = 2; o -= 2 * MS_GU_BYTES; } else if (o >= MS_GU_BYTES) { m = 1; o -= MS_GU_BYTES; }
        uint32_t v;
        if (o < MS_GU_CODES) {
            const uint64_t tc = ms_tid(L, e, 2 * m);
            v = (uint32_t)ms_code_byte(seed, tc, o) | ((uint32_t)ms_code_byte(seed, tc, o + 1) << 8) |
                ((uint32_t)ms_code_byte(seed, tc, o + 2) << 16) | ((uint32_t)ms_code_byte(seed, tc, o + 3) << 24);
        } else {
            v = __float_as_uint(ms_scale(seed, ms_tid(L, e, 2 * m + 1), (o - MS_GU_CODES) / 4));
        }
        dst[i] = v;
    }
}
extern "C" void k_synth_experts(cudaStream_t st, uint64_t seed, int L, int e0, int ne, uint8_t *dst) {
    if (ne <= 0) return;
    const size_t nwords = (size_t)ne * (MS_EXPERT_BYTES / 4);
    synth_experts_kernel<<<148 * 8, 256, 0, st>>>(seed, L, e0, reinterpret_cast<uint32_t *>(dst), nwords);
    k_count_add(1);
}
