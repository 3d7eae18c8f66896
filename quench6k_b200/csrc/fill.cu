// Random weights made on the device: the kernel twin of the host's generator (fill_normal.h says
// how the two produce the same bits).  One pass over the tensor, nothing read.
#include "common.cuh"
#include "fill_normal.h"

namespace {

template <typename T>
__global__ void fill_normal_kernel(T* out, long long n, unsigned long long start, unsigned long long key, float std, float mean) {
    pdl_enter();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = from_f32<T>(q6k_fill::element(key, start + (unsigned long long)i, std, mean));
}

}  // namespace

// out[i] = dtype(normal(key, start + i) * std + mean) for i < n; dtype: float32 or bfloat16.
Q6K_API int q6k_fill_normal(void* out, int dtype, long long n, long long start, unsigned long long key, float std, float mean, cudaStream_t st) {
    if (n == 0) return 0;
    Q6K_REQUIRE(n > 0 && start >= 0, "fill_normal: bad range start=%lld n=%lld", start, n);
    const int threads = 256;
    const long long blocks = (n + threads - 1) / threads;
    const int grid = (int)(blocks < 148LL * 32 ? blocks : 148LL * 32);
    Q6K_DISPATCH(dtype, q6k_launch(fill_normal_kernel<T>, grid, threads, 0, st, (T*)out, n, (unsigned long long)start, key, std, mean););
    return q6k_check_launch("fill_normal");
}
