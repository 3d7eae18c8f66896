// Shared device helpers and the error convention of the exported launchers.
//
// Every exported function returns 0 on success or a non-zero code after storing a message that
// q6k_last_error() returns.  Nothing here allocates device memory: callers pass every buffer.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#define Q6K_API extern "C" __attribute__((visibility("default")))

enum { Q6K_F32 = 0, Q6K_BF16 = 1 };

int q6k_fail(const char* fmt, ...);           // stores the message, returns 1
int q6k_check_launch(const char* what);       // cudaGetLastError -> message

#define Q6K_REQUIRE(cond, ...)                   \
    do {                                         \
        if (!(cond)) return q6k_fail(__VA_ARGS__); \
    } while (0)

template <typename T> struct q6k_type;
template <> struct q6k_type<float> { static constexpr int code = Q6K_F32; };
template <> struct q6k_type<__nv_bfloat16> { static constexpr int code = Q6K_BF16; };

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
// The value as it will be stored in T, as a float (rounding through T).
template <typename T> __device__ __forceinline__ float round_to(float v) { return to_f32(from_f32<T>(v)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Sum over the block in a fixed order (warp results added in warp order); every thread gets it.
// `red` holds at least 32 floats.  Safe to call repeatedly.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = 0.0f;
    for (int i = 0; i < nw; ++i) t += red[i];
    return t;
}

// Programmatic dependent launch (the reference launches every Flint kernel this way,
// crates/cuda/kernels/common.cuh:82-99): a kernel lets the next one in the stream be scheduled as
// soon as all of its own blocks are resident, and itself touches no global memory before every
// earlier kernel has completed.  Every kernel calls pdl_enter() first, so stream order holds for
// memory while launch latency and block scheduling overlap the predecessor's tail.  Measured on
// B200 under CUDA-graph replay the attribute made a decode step 3 % slower (5.00 vs 4.85 ms), so it
// is off unless Q6K_PDL=1 is set; without the attribute both instructions are no-ops.
__device__ __forceinline__ void pdl_enter() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

bool q6k_pdl_enabled();       // Q6K_PDL=1 in the environment switches the launch attribute on

template <typename... KArgs, typename... Args>
cudaError_t q6k_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = q6k_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Dispatch on a dtype code: body sees `T`.
#define Q6K_DISPATCH(code, ...)                                              \
    do {                                                                     \
        if ((code) == Q6K_F32) { using T = float; __VA_ARGS__ }              \
        else if ((code) == Q6K_BF16) { using T = __nv_bfloat16; __VA_ARGS__ } \
        else return q6k_fail("unknown dtype code %d", (int)(code));          \
    } while (0)
