// Dense products of a step of 3 to 16 tokens: out[t, n] = sum_k x[t, k] w[n, k], bfloat16 operands,
// FP32 sums, on mma.sync with the weights as the M side (16 output rows per instruction) and the
// tokens as the N side (8 per instruction).
//
// Like the matrix-vector kernel (gemv.cu) this is a stream of weights with as little around it as
// possible: no tensor memory, no barriers, no split of K over blocks whose partial sums would have
// to meet in another kernel.  Nothing goes through shared memory on the way in either.  The sum
// over k may be taken in any order as long as both operands agree on it, so a lane does not fetch
// the scattered element pairs of the instruction's operand layout: it fetches 16 contiguous
// bytes of a weight row (and of a token's activations), eight consecutive k, and hands them to two
// instructions as if they were the layout's pairs; the four lanes that share a row cover 64
// contiguous bytes per load.  A block of eight warps owns 16 output rows (or 32), its warps split
// K, every lane has all its loads of a stretch of 128 k in flight before the first instruction,
// and the warps' sums meet in shared memory, added in warp order.
#include "common.cuh"

namespace {

constexpr int SK_WARPS = 8;

__device__ __forceinline__ void sk_mma(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

enum { SK_STORE = 0, SK_ADD = 1, SK_SWIGLU = 2 };

// grid: ceil(N / (16 RB)).  NB: blocks of 8 tokens (1 or 2); RB: blocks of 16 output rows per warp; every warp of the
// block works on the same rows and takes every eighth stretch of K; LOADS: 16-byte loads per lane and row in flight at
// once (a stretch is 32 LOADS elements of k: 4 for the usual widths, 8 for long rows, which then take fewer turns).
template <int NB, int RB, int EPI, int LOADS>
__global__ void __launch_bounds__(SK_WARPS * 32) gemm_skinny_kernel(const __nv_bfloat16* x, long long ldx, int T_,
                                                                    const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ w2,
                                                                    void* out, long long ldo, int N, int K, int k_slice, long long slice_stride) {
    // The weights are a model's and older than any kernel of the step: their first stretch is asked for while the kernel
    // launched before this one still runs (programmatic dependent launch); the activations and the output wait for it.
    pdl_launch();
    bool waited = false;
    const uint64_t once = l2_evict_first_policy();
    constexpr bool DUAL = EPI == SK_SWIGLU;
    constexpr int MATS = DUAL ? 2 : 1;
    __shared__ float meet[SK_WARPS][MATS * RB * NB * 4 * 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, quad = lane >> 2, pair = lane & 3;
    const int n0 = blockIdx.x * RB * 16;
    float acc[MATS][RB][NB][4];
#pragma unroll
    for (int m = 0; m < MATS; ++m)
#pragma unroll
        for (int rb = 0; rb < RB; ++rb)
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) acc[m][rb][nb][0] = acc[m][rb][nb][1] = acc[m][rb][nb][2] = acc[m][rb][nb][3] = 0.0f;
    // this lane's two weight rows of every row block (clamped: a ragged last block reads a valid row and drops the sums)
    const __nv_bfloat16* wrow[MATS][RB][2];
#pragma unroll
    for (int rb = 0; rb < RB; ++rb)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const long long r = min(n0 + rb * 16 + quad + 8 * h, N - 1);
            wrow[0][rb][h] = w + r * K + pair * 8;
            if (DUAL) wrow[1][rb][h] = w2 + r * K + pair * 8;
        }
    const __nv_bfloat16* xrow[NB];
    bool live[NB];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
        live[nb] = nb * 8 + quad < T_;
        xrow[nb] = x + (long long)(live[nb] ? nb * 8 + quad : 0) * ldx + pair * 8;
    }
    constexpr int STRETCH = 32 * LOADS;
    // blockIdx.y: a slice of K of its own (k_slice elements), whose sums go to a slice of the output (plain stores only)
    const int k_begin = blockIdx.y * k_slice, k_end = min(K, k_begin + k_slice);
    for (int k0 = k_begin + warp * STRETCH; k0 < k_end; k0 += SK_WARPS * STRETCH) {
        uint4 a[MATS][RB][2][LOADS], b[NB][LOADS];
#pragma unroll
        for (int j = 0; j < LOADS; ++j) {
            const int k = k0 + j * 32;                       // the lane's eight elements start at k + 8 pair
            const bool in = k + pair * 8 < k_end;            // K and the slices are multiples of 8: a lane's 16 bytes are inside or outside as a whole
#pragma unroll
            for (int m = 0; m < MATS; ++m)
#pragma unroll
                for (int rb = 0; rb < RB; ++rb)
#pragma unroll
                    for (int h = 0; h < 2; ++h) a[m][rb][h][j] = in ? ld_once(wrow[m][rb][h] + k, once) : make_uint4(0, 0, 0, 0);
        }
        if (!waited) {
            pdl_wait();
            waited = true;
        }
#pragma unroll
        for (int j = 0; j < LOADS; ++j) {
            const int k = k0 + j * 32;
            const bool in = k + pair * 8 < k_end;
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
                b[nb][j] = in && live[nb] ? ld_after_wait(xrow[nb] + k) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int j = 0; j < LOADS; ++j)
#pragma unroll
            for (int m = 0; m < MATS; ++m)
#pragma unroll
                for (int rb = 0; rb < RB; ++rb)
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb) {
                        const uint4 lo = a[m][rb][0][j], hi = a[m][rb][1][j], t = b[nb][j];
                        sk_mma(acc[m][rb][nb], lo.x, hi.x, lo.y, hi.y, t.x, t.y);
                        sk_mma(acc[m][rb][nb], lo.z, hi.z, lo.w, hi.w, t.z, t.w);
                    }
    }
    if (!waited) pdl_wait();                  // a warp without a stretch of its own
    // the warps' sums, fragment by fragment: [matrix][row block][token block][4] per lane
    constexpr int PER_LANE = MATS * RB * NB * 4;
#pragma unroll
    for (int m = 0; m < MATS; ++m)
#pragma unroll
        for (int rb = 0; rb < RB; ++rb)
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                for (int i = 0; i < 4; ++i) meet[warp][(((m * RB + rb) * NB + nb) * 4 + i) * 32 + lane] = acc[m][rb][nb][i];
    __syncthreads();
    // thread -> (row block, token block, element of the fragment, lane of the fragment): rows quad (+8), tokens 2 pair (+1)
    for (int idx = threadIdx.x; idx < RB * NB * 4 * 32; idx += SK_WARPS * 32) {
        const int ln = idx & 31, i = (idx >> 5) & 3, nb = (idx >> 7) % NB, rb = (idx >> 7) / NB;
        const int n = n0 + rb * 16 + (ln >> 2) + 8 * (i >> 1), t = nb * 8 + 2 * (ln & 3) + (i & 1);
        float s = 0.0f, s2 = 0.0f;
#pragma unroll
        for (int q = 0; q < SK_WARPS; ++q) {
            s += meet[q][idx];
            if (DUAL) s2 += meet[q][RB * NB * 4 * 32 + idx];
        }
        if (n >= N || t >= T_) continue;
        const long long at = (long long)blockIdx.y * slice_stride + (long long)t * ldo + n;
        if (EPI == SK_SWIGLU) reinterpret_cast<__nv_bfloat16*>(out)[at] = __float2bfloat16_rn(s / (1.0f + __expf(-s)) * s2);
        else if (EPI == SK_ADD) reinterpret_cast<float*>(out)[at] += s;
        else reinterpret_cast<float*>(out)[at] = s;
    }
    (void)PER_LANE;
}

template <int NB, int RB, int LOADS>
int skinny_launch(int epi, cudaStream_t st, const __nv_bfloat16* x, long long ldx, int T_, const __nv_bfloat16* w, const __nv_bfloat16* w2, void* out,
                  long long ldo, int N, int K, int slices, int k_slice, long long slice_stride) {
    const dim3 grid((N + RB * 16 - 1) / (RB * 16), slices);
    if (epi == SK_SWIGLU) q6k_launch_as(true, gemm_skinny_kernel<NB, 1, SK_SWIGLU, 4>, (N + 15) / 16, SK_WARPS * 32, 0, st, x, ldx, T_, w, w2, out, ldo, N, K, K, 0LL);
    else if (epi == SK_ADD) q6k_launch_as(true, gemm_skinny_kernel<NB, RB, SK_ADD, LOADS>, grid, SK_WARPS * 32, 0, st, x, ldx, T_, w, w2, out, ldo, N, K, K, 0LL);
    else q6k_launch_as(true, gemm_skinny_kernel<NB, RB, SK_STORE, LOADS>, grid, SK_WARPS * 32, 0, st, x, ldx, T_, w, w2, out, ldo, N, K, k_slice, slice_stride);
    return q6k_check_launch("gemm_skinny");
}

}  // namespace

// Whether a bfloat16 product of `tokens` rows with an [N, K] matrix should come here rather than to the tcgen05 kernel
// (which splits K over blocks and leaves partial sums at these sizes).  Measured on B200 inside a CUDA graph, weights
// from HBM: [5120, 2048] 6.7 against 8.3 us at 8 tokens, the [151936, 2048] LM head 92 against 102 us (91 against 100 at
// one token); with few rows ([2048, 4096]: 128 blocks of 16 rows) it is the slower one (10 against 7 us).  One or two
// tokens against a matrix that is no LM head go to the matrix-vector kernel.
Q6K_API int q6k_gemm_skinny_preferred(int tokens, int N, int K) {
    if (tokens < 1 || tokens > 16 || K % 8 || K < 512 || N < 4096) return 0;
    return tokens >= 3 || (long long)N * K > (64LL << 20);
}

// Slices of K for a plain product whose caller can add partial sums itself, when the matrix has too few rows to give
// every SM two blocks of 16 (the o projection of a decode step): as many as bring the blocks to two per SM, each slice a
// multiple of 1,024 elements (eight warps' stretches) and at least that long.  0: not for this kernel.
Q6K_API int q6k_gemm_skinny_slices(int tokens, int N, int K) {
    if (tokens < 3 || tokens > 16 || K % 8 || N < 512 || N >= 4096 || K < 2048) return 0;
    const int blocks = (N + 15) / 16;
    int slices = (2 * 148 + blocks - 1) / blocks;
    if (slices > K / 1024) slices = K / 1024;
    if (slices < 2) return 0;
    const int k_slice = ((K + slices - 1) / slices + 1023) / 1024 * 1024;    // as q6k_gemm_skinny cuts it
    return (K + k_slice - 1) / k_slice;
}

// x: bfloat16 [tokens <= 16, K] (row pitch ldx elements); w (and w2 for the SwiGLU epilogue): bfloat16 [N, K]; out: FP32
// [tokens, N] (epi 0 store, 1 add) or bfloat16 [tokens, N] (epi 2: silu(x w^T) * (x w2^T)), row pitch ldo.
// slices > 1 (epi 0 only): K is cut into that many slices, slice z's sums go to out + z * slice_stride floats.
Q6K_API int q6k_gemm_skinny(const void* x, long long ldx, int tokens, const void* w, const void* w2, int N, int K, void* out, long long ldo, int epi,
                            int slices, long long slice_stride, cudaStream_t st) {
    if (tokens == 0) return 0;
    Q6K_REQUIRE(tokens >= 1 && tokens <= 16, "gemm_skinny: %d tokens (1 to 16)", tokens);
    Q6K_REQUIRE(N > 0 && K > 0 && K % 8 == 0 && ldx % 8 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0 && ((uintptr_t)w2 & 15) == 0,
                "gemm_skinny: K=%d and the row pitch %lld must be multiples of 8 and the operands 16-byte aligned", K, ldx);
    Q6K_REQUIRE(epi >= 0 && epi <= 2 && (epi == SK_SWIGLU) == (w2 != nullptr), "gemm_skinny: epilogue %d with%s a second matrix", epi, w2 ? "" : "out");
    Q6K_REQUIRE(slices >= 1 && (slices == 1 || epi == SK_STORE), "gemm_skinny: %d slices of K with epilogue %d", slices, epi);
    const int k_slice = slices == 1 ? K : ((K + slices - 1) / slices + 1023) / 1024 * 1024;
    const __nv_bfloat16 *xp = (const __nv_bfloat16*)x, *wp = (const __nv_bfloat16*)w, *w2p = (const __nv_bfloat16*)w2;
    // 32 rows per block where that still gives every SM two blocks; 16 otherwise
    const bool wide = N >= 148 * 2 * 32, deep = k_slice >= 4096 && !wide;          // long rows and few of them: eight loads per row at once
#define SK_GO(NB_, RB_, LOADS_) skinny_launch<NB_, RB_, LOADS_>(epi, st, xp, ldx, tokens, wp, w2p, out, ldo, N, K, slices, k_slice, slice_stride)
    if (tokens <= 8) {
        if (wide) return SK_GO(1, 2, 4);
        if (deep) return SK_GO(1, 1, 8);
        return SK_GO(1, 1, 4);
    }
    if (deep) return SK_GO(2, 1, 8);
    return SK_GO(2, 1, 4);
#undef SK_GO
}
