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
// crates/cuda/kernels/common.cuh:82-99).  A launch that carries the attribute may begin as soon as
// every block of the kernel before it has executed pdl_launch() (or ended); it must execute
// pdl_wait() before it touches anything an earlier kernel writes or reads, since pdl_wait() returns
// only when the kernel before it has completed and its memory is visible.  Every kernel calls
// pdl_enter() first (the wait, then the signal) unless it has work that needs no earlier result: the
// products set themselves up and fetch weights before they wait, and signal first.  Waiting before
// signalling is what lets such a kernel also read, before its wait, what the kernel before its
// predecessor wrote (a pair list two kernels old): its predecessor, if it is an ordinary kernel,
// lets nobody start before it has itself seen everything older complete, whatever the launch mode.  A kernel that
// allocates tensor memory calls pdl_launch() only after the allocation, so that a successor cannot
// take the columns one of its own blocks still needs.  Without the attribute both are no-ops.
// Pointers to anything an earlier kernel of the step writes carry no __restrict__: a load through a `const __restrict__`
// pointer counts as read-only for the kernel's lifetime, and the compiler may move it ahead of pdl_wait() (it did, in
// the matrix-vector kernel: a step replayed from a CUDA graph then read activations that were not written yet).
// Only weights keep the qualifier.
//
// Measured on B200 under CUDA-graph replay, the attribute costs about 0.3 us per launch when the
// kernel has nothing to overlap (a decode step with it on every launch: 4.93 vs 4.86 ms), so only
// launches that have such work carry it.  The environment variable Q6K_PDL overrides:
// "0" no launch, "1" every launch, unset or "gemm" only those marked.
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_enter() {
    pdl_wait();
    pdl_launch();
}
// 16 bytes that the kernel before this one may have written, read after pdl_wait(): a volatile asm load, which the compiler
// keeps behind the (volatile asm) wait.  A plain load through a `const __restrict__` pointer counts as read-only for the
// kernel's lifetime and may be moved ahead of the wait, where the data is not there yet.
__device__ __forceinline__ uint4 ld_after_wait(const void* p) {
    uint4 v;
    asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// Data that a step reads once (weights, a request's keys and values) is fetched with this policy: its lines are the
// first to leave the L2 cache again, so that what is read again soon (activations, partial sums, the kernels'
// own code) stays there.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
// 16 bytes of such data (read-only for the kernel's lifetime), past L1.
__device__ __forceinline__ uint4 ld_once(const void* p, uint64_t policy) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0, %1, %2, %3}, [%4], %5;" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p), "l"(policy));
    return v;
}

int q6k_pdl_mode();           // 0: never, 1: every launch, 2: launches marked as overlapping

template <typename... KArgs, typename... Args>
cudaError_t q6k_launch_as(bool overlaps, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    const int mode = q6k_pdl_mode();
    cfg.numAttrs = (mode == 1 || (mode == 2 && overlaps)) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
cudaError_t q6k_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    return q6k_launch_as(false, kernel, grid, block, smem, st, static_cast<Args&&>(args)...);
}

// Dispatch on a dtype code: body sees `T`.
#define Q6K_DISPATCH(code, ...)                                              \
    do {                                                                     \
        if ((code) == Q6K_F32) { using T = float; __VA_ARGS__ }              \
        else if ((code) == Q6K_BF16) { using T = __nv_bfloat16; __VA_ARGS__ } \
        else return q6k_fail("unknown dtype code %d", (int)(code));          \
    } while (0)
