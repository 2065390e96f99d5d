/* selftest_api.c -- host entry of the tcgen05 building-block check (k_umma_selftest.cu). */
#include <stdio.h>
#include <stdint.h>
#include <cuda_runtime_api.h>
#include "../../include/gmoe.h"

int k_umma_selftest(cudaStream_t st, const uint8_t *A, const int8_t *B, int n, int kblocks, int mode, int32_t *D, int *status);

int gmoe_umma_selftest(const uint8_t *a, const int8_t *b, int n, int kblocks, int mode, int32_t *d) {
    size_t K = (size_t)kblocks * 128;
    uint8_t *da = NULL; int8_t *db = NULL; int32_t *dd = NULL; int *ds = NULL; int hs = 0, rc = -1;
    if (n < 16 || n > 256 || (n & 15) || kblocks < 1 || kblocks > 4) { fprintf(stderr, "gmoe: selftest: n %d, kblocks %d\n", n, kblocks); return -1; }
    if (cudaMalloc((void **)&da, 128 * K) || cudaMalloc((void **)&db, (size_t)n * K) || cudaMalloc((void **)&dd, (size_t)128 * n * 4) ||
        cudaMalloc((void **)&ds, 4)) { fprintf(stderr, "gmoe: selftest: no device memory\n"); goto out; }
    cudaMemcpy(da, a, 128 * K, cudaMemcpyHostToDevice); cudaMemcpy(db, b, (size_t)n * K, cudaMemcpyHostToDevice);
    cudaMemset(dd, 0xFF, (size_t)128 * n * 4); cudaMemset(ds, 0, 4);
    if (k_umma_selftest(0, da, db, n, kblocks, mode, dd, ds)) goto out;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { fprintf(stderr, "gmoe: selftest: %s\n", cudaGetErrorString(e)); goto out; }
    cudaMemcpy(d, dd, (size_t)128 * n * 4, cudaMemcpyDeviceToHost); cudaMemcpy(&hs, ds, 4, cudaMemcpyDeviceToHost);
    if (hs) { fprintf(stderr, "gmoe: selftest: the MMA did not signal completion within the wait limit\n"); rc = -2; goto out; }
    rc = 0;
out:
    cudaFree(da); cudaFree(db); cudaFree(dd); cudaFree(ds);
    return rc;
}

int k_i8_peak(cudaStream_t st, int n, int iters, int sms, int *status);
/* include/gmoe.h: measured tcgen05.mma kind::i8 rate of this GPU, in units of 1e12 integer operations per second */
double gmoe_i8_peak(int n, int iters) {
    int dev = 0, sms = 0, hs = 0, *ds = NULL; float ms = 0; double tops = -1.0;
    cudaEvent_t a = NULL, b = NULL;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) { fprintf(stderr, "gmoe: i8 peak: no CUDA device\n"); return -1.0; }
    if (cudaMalloc((void **)&ds, 4) != cudaSuccess) { fprintf(stderr, "gmoe: i8 peak: no device memory\n"); return -1.0; }
    cudaMemset(ds, 0, 4); cudaEventCreate(&a); cudaEventCreate(&b);
    if (k_i8_peak(0, n, iters, sms, ds)) { fprintf(stderr, "gmoe: i8 peak: n %d, iters %d\n", n, iters); goto out; }   /* warm-up */
    cudaEventRecord(a, 0);
    k_i8_peak(0, n, iters, sms, ds);
    cudaEventRecord(b, 0);
    if (cudaDeviceSynchronize() != cudaSuccess) { fprintf(stderr, "gmoe: i8 peak: %s\n", cudaGetErrorString(cudaGetLastError())); goto out; }
    cudaMemcpy(&hs, ds, 4, cudaMemcpyDeviceToHost);
    if (hs) { fprintf(stderr, "gmoe: i8 peak: an MMA completion never arrived\n"); goto out; }
    cudaEventElapsedTime(&ms, a, b);
    tops = 2.0 * 128.0 * n * 32.0 * 4.0 * iters * sms / (ms * 1e-3) / 1e12;
out:
    cudaFree(ds); if (a) cudaEventDestroy(a); if (b) cudaEventDestroy(b);
    return tops;
}
