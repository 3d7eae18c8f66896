// A check of the bounded waits themselves: a kernel waits on a barrier that nothing ever arrives on, with a short
// limit, and must come back with the status of a wait that ran out, leaving the context usable.  Every spin of the
// product kernels (TMA rings, tensor-memory accumulators) goes through the same mbar_wait with a limit of about two
// seconds; a run-out there records a code in the kernel's status word (ops.tc_status()) instead of hanging the GPU.
#include "common.cuh"
#include "tma.cuh"

namespace {

__global__ void wait_runs_out_kernel(long long limit, int* status, long long* waited) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const long long t0 = clock64();
    const bool ok = mbar_wait(smem_u32(&bar), 0, limit);      // phase 0 never completes: nobody arrives
    if (threadIdx.x == 0) {
        *status = ok ? 0 : 1;
        *waited = clock64() - t0;
    }
}

}  // namespace

// Runs the kernel with the given limit (cycles; at most 2e8, a tenth of a second).  *status: what the kernel recorded
// (1: the wait ran out, as it must; 0: it did not); *waited_cycles: how long its thread waited.
Q6K_API int q6k_selftest_wait_runs_out(long long limit_cycles, int* status, long long* waited_cycles, cudaStream_t st) {
    Q6K_REQUIRE(limit_cycles > 0 && limit_cycles <= 200000000LL && status && waited_cycles, "selftest: a limit of %lld cycles (1 to 2e8)", limit_cycles);
    int* d_status = nullptr;
    long long* d_waited = nullptr;
    if (cudaMalloc(&d_status, sizeof(int)) != cudaSuccess || cudaMalloc(&d_waited, sizeof(long long)) != cudaSuccess) {
        cudaFree(d_status);
        return q6k_check_launch("selftest: allocation");
    }
    q6k_launch(wait_runs_out_kernel, 1, 32, 0, st, limit_cycles, d_status, d_waited);
    const bool ok = cudaStreamSynchronize(st) == cudaSuccess && cudaMemcpy(status, d_status, sizeof(int), cudaMemcpyDeviceToHost) == cudaSuccess &&
                    cudaMemcpy(waited_cycles, d_waited, sizeof(long long), cudaMemcpyDeviceToHost) == cudaSuccess;
    cudaFree(d_status);
    cudaFree(d_waited);
    return ok ? 0 : q6k_fail("selftest: the kernel could not be run or read back: %s", cudaGetErrorString(cudaGetLastError()));
}
