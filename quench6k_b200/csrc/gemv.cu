// Matrix-vector products for steps of one to four tokens: out[t, n] = sum_k x[t, k] w[n, k], bfloat16
// operands, FP32 sums.  (The reference runs its small-T products on dedicated GEMV kernels too:
// crates/cuda/kernels/flint.cu:589-824, there on 4-bit weights.)
//
// With so few tokens a product is a stream of weights and nothing else, and what decides its time
// is how soon the whole stream is in flight and how little surrounds it: no tensor memory to
// allocate, no barriers to initialise, no partial sums to meet in another kernel.  A block of
// eight warps owns a few output rows; KW of its warps split K between them in strides of 256
// elements (16 bytes per lane: one coalesced 512-byte line per row and stride, read past L1 since
// nothing is read twice), the other 8 / KW-fold of the block takes further rows, so that for the
// usual widths a lane issues all its loads at once and the whole matrix is asked for within the
// first microsecond.  The tokens' activations come through L1; every lane multiplies its eight
// weights with its eight activations of every token in FP32; the lanes' sums meet in five
// shuffles and the KW warps' sums in shared memory, added in warp order.
//
// Three shapes of call: a dense product (all tokens against one matrix), a product per (token,
// expert) pair (row pair / pair_div of x against the matrix of pair_expert[pair]; one token per
// block row), and either of them with a second matrix and the SwiGLU epilogue
// act = silu(x w^T) * (x w2^T) in bfloat16.
#include "common.cuh"

namespace {

constexpr int GEMV_WARPS = 8;

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __bfloat1622float2(p[i]);
        f[2 * i] = t.x, f[2 * i + 1] = t.y;
    }
}

enum { GEMV_STORE = 0, GEMV_ADD = 1, GEMV_SWIGLU = 2 };

// grid (ceil(N / ((GEMV_WARPS / KW) * ROWS)), pairs or 1).  TT: tokens handled together (dense calls; 1 for pair calls);
// ROWS: output rows of a warp; KW: warps that share a row's K.
template <int TT, int ROWS, int KW, int EPI>
__global__ void __launch_bounds__(GEMV_WARPS * 32, 4) gemv_kernel(const __nv_bfloat16* x, long long ldx, const __nv_bfloat16* __restrict__ w,
                                                               const __nv_bfloat16* __restrict__ w2, long long expert_stride,
                                                               const int* pair_expert, int pair_div, void* out,
                                                               long long ldo, int N, int K, int early) {
    // early: the weights (and the pair list) are older than the kernel before this one, so they may be asked for
    // before that kernel has ended (programmatic dependent launch); the activations and the output wait for it
    if (!early) pdl_wait();                   // an ordinary kernel: the wait first, then the signal (see common.cuh)
    pdl_launch();
    const uint64_t once = l2_evict_first_policy();
    constexpr bool DUAL = EPI == GEMV_SWIGLU;
    constexpr int RG = GEMV_WARPS / KW;                                   // groups of warps along the rows
    constexpr int SUMS = ROWS * TT * (DUAL ? 2 : 1);
    __shared__ float meet[GEMV_WARPS][SUMS];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, kw = warp % KW, rg = warp / KW;
    const int n0 = (blockIdx.x * RG + rg) * ROWS;
    long long xrow = 0, orow = 0;
    if (pair_expert) {
        const int pair = blockIdx.y, e = pair_expert[pair];
        w += (long long)e * expert_stride;
        if (DUAL) w2 += (long long)e * expert_stride;
        xrow = pair / pair_div, orow = pair;
    }
    float acc[ROWS][TT], acc2[DUAL ? ROWS : 1][TT];
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
#pragma unroll
        for (int t = 0; t < TT; ++t) {
            acc[r][t] = 0.0f;
            if (DUAL) acc2[r][t] = 0.0f;
        }
    if (n0 < N)
        for (int k0 = (kw * 32 + lane) * 8; k0 < K; k0 += KW * 256) {
            uint4 wv[ROWS], w2v[DUAL ? ROWS : 1], xv[TT];
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                const long long row = n0 + r < N ? n0 + r : N - 1;      // a ragged last group reads a valid row and drops the sum
                wv[r] = ld_once(w + row * K + k0, once);
                if (DUAL) w2v[r] = ld_once(w2 + row * K + k0, once);
            }
            if (early) {
                pdl_wait();                                              // the weights are on their way; now the kernel before must be done
                early = 0;
            }
#pragma unroll
            for (int t = 0; t < TT; ++t) xv[t] = ld_after_wait(x + (xrow + t) * ldx + k0);
            float xf[TT][8];
#pragma unroll
            for (int t = 0; t < TT; ++t) unpack8(xv[t], xf[t]);
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                float wf[8];
                unpack8(wv[r], wf);
#pragma unroll
                for (int t = 0; t < TT; ++t)
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[r][t] = fmaf(wf[i], xf[t][i], acc[r][t]);
                if (DUAL) {
                    unpack8(w2v[r], wf);
#pragma unroll
                    for (int t = 0; t < TT; ++t)
#pragma unroll
                        for (int i = 0; i < 8; ++i) acc2[r][t] = fmaf(wf[i], xf[t][i], acc2[r][t]);
                }
            }
        }
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
#pragma unroll
        for (int t = 0; t < TT; ++t) {
            const float s = warp_sum(acc[r][t]);
            if (lane == 0) meet[warp][r * TT + t] = s;
            if (DUAL) {
                const float s2 = warp_sum(acc2[r][t]);
                if (lane == 0) meet[warp][ROWS * TT + r * TT + t] = s2;
            }
        }
    if (early) pdl_wait();                                                // a warp without a stride of its own
    __syncthreads();
    // one thread per (row group, row, token): the KW warps' sums in warp order
    const int idx = threadIdx.x;
    if (idx >= RG * ROWS * TT) return;
    const int g = idx / (ROWS * TT), rt = idx % (ROWS * TT), r = rt / TT, t = rt % TT;
    const int n = (blockIdx.x * RG + g) * ROWS + r;
    if (n >= N) return;
    float s = 0.0f, s2 = 0.0f;
#pragma unroll
    for (int q = 0; q < KW; ++q) {
        s += meet[g * KW + q][rt];
        if (DUAL) s2 += meet[g * KW + q][ROWS * TT + rt];
    }
    const long long at = (orow + t) * ldo + n;
    if (EPI == GEMV_SWIGLU) reinterpret_cast<__nv_bfloat16*>(out)[at] = __float2bfloat16_rn(s / (1.0f + __expf(-s)) * s2);
    else if (EPI == GEMV_ADD) reinterpret_cast<float*>(out)[at] += s;
    else reinterpret_cast<float*>(out)[at] = s;
}

template <int TT, int ROWS, int KW>
int gemv_launch(int early, int epi, int blocks_y, cudaStream_t st, const __nv_bfloat16* x, long long ldx, const __nv_bfloat16* w, const __nv_bfloat16* w2,
                long long expert_stride, const int* pair_expert, int pair_div, void* out, long long ldo, int N, int K) {
    const int per_block = (GEMV_WARPS / KW) * ROWS;
    const dim3 grid((N + per_block - 1) / per_block, blocks_y);
    const bool over = early != 0;
    if (epi == GEMV_SWIGLU) q6k_launch_as(over, gemv_kernel<TT, ROWS, KW, GEMV_SWIGLU>, grid, GEMV_WARPS * 32, 0, st, x, ldx, w, w2, expert_stride, pair_expert, pair_div, out, ldo, N, K, early);
    else if (epi == GEMV_ADD) q6k_launch_as(over, gemv_kernel<TT, ROWS, KW, GEMV_ADD>, grid, GEMV_WARPS * 32, 0, st, x, ldx, w, w2, expert_stride, pair_expert, pair_div, out, ldo, N, K, early);
    else q6k_launch_as(over, gemv_kernel<TT, ROWS, KW, GEMV_STORE>, grid, GEMV_WARPS * 32, 0, st, x, ldx, w, w2, expert_stride, pair_expert, pair_div, out, ldo, N, K, early);
    return q6k_check_launch("gemv");
}

template <int TT, int ROWS>
int gemv_launch_k(int early, int kw, int epi, int blocks_y, cudaStream_t st, const __nv_bfloat16* x, long long ldx, const __nv_bfloat16* w, const __nv_bfloat16* w2,
                  long long es, const int* pe, int pd, void* out, long long ldo, int N, int K) {
    if (kw == 8) return gemv_launch<TT, ROWS, 8>(early, epi, blocks_y, st, x, ldx, w, w2, es, pe, pd, out, ldo, N, K);
    if (kw == 4) return gemv_launch<TT, ROWS, 4>(early, epi, blocks_y, st, x, ldx, w, w2, es, pe, pd, out, ldo, N, K);
    if (kw == 2) return gemv_launch<TT, ROWS, 2>(early, epi, blocks_y, st, x, ldx, w, w2, es, pe, pd, out, ldo, N, K);
    return gemv_launch<TT, ROWS, 1>(early, epi, blocks_y, st, x, ldx, w, w2, es, pe, pd, out, ldo, N, K);
}

}  // namespace

// The most tokens a dense call takes, and whether a product of this shape should come here rather than to the
// tensor-core kernel: with one or two tokens and a matrix that is no LM head, this kernel starts sooner and streams as fast.
Q6K_API int q6k_gemv_max_tokens() { return 4; }
Q6K_API int q6k_gemv_preferred(int tokens, int N, int K) {
    return tokens >= 1 && tokens <= 2 && K % 8 == 0 && K >= 256 && N >= 1 && (long long)N * K <= (64LL << 20);
}

// x: bfloat16 [tokens, K] (row pitch ldx elements, rows on 16 bytes); w (and w2 for the SwiGLU epilogue): bfloat16 [N, K], or
// [experts, N, K] with pair_expert (int32 [pairs]) naming each pair's expert, pair y using row y / pair_div of x and
// writing row y of out.  out: FP32 [rows, N] (epi 0 store, 1 add) or bfloat16 [rows, N] (epi 2), row pitch ldo.
// early != 0: the weights and the pair list were written before the kernel that precedes this one started (weights of a
// model always; a pair list only when another kernel lies between its maker and this call): the launch then carries the
// programmatic-launch attribute and streams its weights while that kernel ends; x and out are touched after it has ended.
Q6K_API int q6k_gemv(const void* x, long long ldx, int tokens, const void* w, const void* w2, int N, int K, const int* pair_expert, int pairs,
                     int pair_div, void* out, long long ldo, int epi, int early, cudaStream_t st) {
    if (tokens == 0 || (pair_expert && pairs == 0)) return 0;
    Q6K_REQUIRE(N > 0 && K > 0 && K % 8 == 0 && ldx % 8 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0 && ((uintptr_t)w2 & 15) == 0,
                "gemv: K=%d and the row pitch %lld must be multiples of 8 and the operands 16-byte aligned", K, ldx);
    Q6K_REQUIRE(epi >= 0 && epi <= 2 && (epi == GEMV_SWIGLU) == (w2 != nullptr), "gemv: epilogue %d with%s a second matrix", epi, w2 ? "" : "out");
    Q6K_REQUIRE(pair_expert ? (pairs > 0 && pairs <= 65535 && pair_div >= 1) : (tokens >= 1 && tokens <= q6k_gemv_max_tokens()),
                "gemv: %d tokens (at most %d) / %d pairs", tokens, q6k_gemv_max_tokens(), pairs);
    const __nv_bfloat16 *xp = (const __nv_bfloat16*)x, *wp = (const __nv_bfloat16*)w, *w2p = (const __nv_bfloat16*)w2;
    const long long es = (long long)N * K;
    const int strides = (K + 255) / 256;                                  // 256-element strides of a row
    const int kw = strides >= 8 ? 8 : strides >= 4 ? 4 : strides >= 2 ? 2 : 1;
    if (pair_expert) {
        if (epi == GEMV_SWIGLU) return gemv_launch_k<1, 2>(early, kw, epi, pairs, st, xp, ldx, wp, w2p, es, pair_expert, pair_div, out, ldo, N, K);
        return gemv_launch_k<1, 4>(early, kw, epi, pairs, st, xp, ldx, wp, w2p, es, pair_expert, pair_div, out, ldo, N, K);
    }
#define GEMV_CASE(TT)                                                                                                               \
    case TT:                                                                                                                        \
        if (epi == GEMV_SWIGLU || TT > 2) return gemv_launch_k<TT, 2>(early, kw, epi, 1, st, xp, ldx, wp, w2p, es, nullptr, 1, out, ldo, N, K); \
        return gemv_launch_k<TT, 4>(early, kw, epi, 1, st, xp, ldx, wp, w2p, es, nullptr, 1, out, ldo, N, K);
    switch (tokens) {
        GEMV_CASE(1)
        GEMV_CASE(2)
        GEMV_CASE(3)
        GEMV_CASE(4)
    }
#undef GEMV_CASE
    return q6k_fail("gemv: %d tokens", tokens);
}
