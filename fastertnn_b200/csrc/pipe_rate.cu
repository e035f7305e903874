// Issue-rate microbenchmarks: the denominators for "fraction of the integer pipe" figures.
// Each kernel runs eight independent dependency chains of one instruction kind per thread at
// full occupancy; the result is thread-instructions per second over the whole GPU.
#include "internal.h"

namespace {

template <int OP>
__global__ void __launch_bounds__(1024) pipe_rate_kernel(uint32_t* out, int iters, uint32_t k) {
    uint32_t a[8];
#pragma unroll
    for (int i = 0; i < 8; i++) a[i] = threadIdx.x * 2654435761u + i * 40503u + k;
    for (int it = 0; it < iters; it++) {
#pragma unroll
        for (int u = 0; u < 8; u++) {
#pragma unroll
            for (int i = 0; i < 8; i++) {
                if (OP == 0) asm volatile("lop3.b32 %0, %0, %1, %2, 0x96;" : "+r"(a[i]) : "r"(a[(i + 1) & 7]), "r"(k));
                else if (OP == 1) asm volatile("popc.b32 %0, %0;" : "+r"(a[i]));
                else asm volatile("add.u32 %0, %0, %1;" : "+r"(a[i]) : "r"(k));
            }
        }
    }
    uint32_t s = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) s ^= a[i];
    out[blockIdx.x * blockDim.x + threadIdx.x] = s;
}

}  // namespace

// Tensor pipe: an issue-bound loop of tcgen05.mma on operands resident in shared memory.
static int tensor_rate(tnns_cuda_ctx* ctx, bool f4, double* giga_per_s) {
    const int iters = 2000;  // x 4 MMAs per block: under a millisecond
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    float best = 1e30f;
    double ops = 0;
    int rc = TNNS_OK;
    for (int rep = 0; rep < 5 && rc == TNNS_OK; rep++) {
        cudaEventRecord(e0, (cudaStream_t)0);
        rc = tnns_launch_mma_rate(ctx, f4, iters, &ops, (cudaStream_t)0);
        cudaEventRecord(e1, (cudaStream_t)0);
        cudaEventSynchronize(e1);
        float ms = 0;
        cudaEventElapsedTime(&ms, e0, e1);
        if (rep > 0 && ms < best) best = ms;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (rc != TNNS_OK) return rc;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return tnns_fail(TNNS_ERR_CUDA, "tensor-rate kernel failed: %s", cudaGetErrorString(e));
    *giga_per_s = ops / (best * 1e-3) / 1e9;
    return TNNS_OK;
}

// op: 0 = LOP3, 1 = POPC, 2 = IADD: result in 1e9 thread-instructions per second.
// op: 3 = tcgen05.mma kind::i8, 4 = kind::mxf4 (block scales): result in 1e9 operations
// (2*M*N*K) per second.
extern "C" int tnns_cuda_pipe_rate(tnns_cuda_ctx* ctx, int op, double* giga_per_s) {
    if (!ctx || !giga_per_s) return tnns_fail(TNNS_ERR_INVALID, "NULL argument");
    if (op < 0 || op > 4) return tnns_fail(TNNS_ERR_INVALID, "unknown instruction kind %d", op);
    TNNS_CUDA_TRY(cudaSetDevice(ctx->device));
    if (op >= 3) return tensor_rate(ctx, op == 4, giga_per_s);
    const int blocks = ctx->sm_count * 2, threads = 1024, iters = 2000;
    uint32_t* d = nullptr;
    TNNS_CUDA_TRY(cudaMalloc(&d, (size_t)blocks * threads * 4));
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    float best = 1e30f;
    for (int rep = 0; rep < 4; rep++) {
        cudaEventRecord(e0, 0);
        if (op == 0) pipe_rate_kernel<0><<<blocks, threads>>>(d, iters, 0x9E3779B9u);
        else if (op == 1) pipe_rate_kernel<1><<<blocks, threads>>>(d, iters, 0x9E3779B9u);
        else pipe_rate_kernel<2><<<blocks, threads>>>(d, iters, 0x9E3779B9u);
        tnns_count_launch();
        cudaEventRecord(e1, 0);
        cudaEventSynchronize(e1);
        float ms = 0;
        cudaEventElapsedTime(&ms, e0, e1);
        if (rep > 0 && ms < best) best = ms;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaError_t e = cudaGetLastError();
    cudaFree(d);
    if (e != cudaSuccess) return tnns_fail(TNNS_ERR_CUDA, "pipe-rate kernel failed: %s", cudaGetErrorString(e));
    *giga_per_s = (double)blocks * threads * iters * 64.0 / (best * 1e-3) / 1e9;
    return TNNS_OK;
}
