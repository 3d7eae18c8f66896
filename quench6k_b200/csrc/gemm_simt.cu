// Matrix products on CUDA cores with FP32 fused multiply-adds: the arithmetic of the true 32-bit
// path, and the fallback of the bfloat16 path for shapes the tensor-core kernels refuse.
//
//   out[r, n] (+)= sum_k A[row(r), k] * W_g[n, k]        (W is [N, K], K contiguous, as the
//   reference stores its projection weights: crates/engine/src/flint.rs:293-300)
//
// Rows may be grouped (one weight matrix per group: the experts of a MoE layer, as the reference
// runs them through one grouped kernel, crates/cuda/kernels/moe.cu:142-255) and may be gathered
// through an index.  With two weight matrices the epilogue is SwiGLU: out = silu(A.Wg) * (A.Wu).
//
// Each output element is one accumulator summed over k in ascending order, so its value does not
// depend on which tile or batch the row was in.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16;

enum { EPI_STORE = 0, EPI_ADD = 1, EPI_SWIGLU = 2 };

template <typename T, int EPI>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const T* A, int lda, const int* a_rows, const T* W, const T* W2,
                                                        size_t w_group_stride, void* out_, int ldo, int M, int N, int K,
                                                        const int* tile_group, const int* tile_row0,
                                                        const int* group_offsets, const int* num_tiles) {
    pdl_enter();
    constexpr bool DUAL = EPI == EPI_SWIGLU;
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    __shared__ float Ws2[DUAL ? BK : 1][BN + 4];
    int g = 0, row0 = blockIdx.y * BM, row_end = M;
    if (tile_group) {
        if ((int)blockIdx.y >= *num_tiles) return;
        g = tile_group[blockIdx.y];
        row0 = tile_row0[blockIdx.y];
        row_end = group_offsets[g + 1];
    }
    if (row0 >= row_end) return;
    const int n0 = blockIdx.x * BN;
    const T* Wg = W + (size_t)g * w_group_stride;
    const T* Wg2 = DUAL ? W2 + (size_t)g * w_group_stride : nullptr;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    // loader: this thread brings 4 consecutive k of one tile row of A and of W
    const int lr = tid >> 2, lk = (tid & 3) * 4;
    const int arow_g = row0 + lr;
    const T* a_src = nullptr;
    if (arow_g < row_end) a_src = A + (size_t)(a_rows ? a_rows[arow_g] : arow_g) * lda;
    const T* w_src = (n0 + lr < N) ? Wg + (size_t)(n0 + lr) * K : nullptr;
    const T* w2_src = (DUAL && n0 + lr < N) ? Wg2 + (size_t)(n0 + lr) * K : nullptr;

    float acc[4][4] = {}, acc2[DUAL ? 4 : 1][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + lk + i;
            As[lk + i][lr] = (a_src && k < K) ? to_f32(a_src[k]) : 0.0f;
            Ws[lk + i][lr] = (w_src && k < K) ? to_f32(w_src[k]) : 0.0f;
            if (DUAL) Ws2[lk + i][lr] = (w2_src && k < K) ? to_f32(w2_src[k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[4], b[4], b2[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[k][tx * 4 + j];
            if (DUAL) {
#pragma unroll
                for (int j = 0; j < 4; ++j) b2[j] = Ws2[k][tx * 4 + j];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
                    if (DUAL) acc2[i][j] = fmaf(a[i], b2[j], acc2[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = row0 + ty * 4 + i;
        if (r >= row_end) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            const size_t o = (size_t)r * ldo + n;
            if (EPI == EPI_STORE) {
                ((float*)out_)[o] = acc[i][j];
            } else if (EPI == EPI_ADD) {
                ((float*)out_)[o] += acc[i][j];
            } else {
                const float gte = acc[i][j];
                ((T*)out_)[o] = from_f32<T>(gte / (1.0f + expf(-gte)) * acc2[DUAL ? i : 0][j]);
            }
        }
    }
}

// Row tiles of the groups: for offsets[0..G] the list of (group, first row) of every BM-row tile.
// One block; groups are walked in order so the list is a function of the offsets only.
__global__ void tile_list_kernel(const int* offsets, int G, int bm, int* tile_group, int* tile_row0, int* num_tiles,
                                 int max_tiles) {
    pdl_enter();
    __shared__ int base;
    if (threadIdx.x == 0) base = 0;
    __syncthreads();
    for (int g0 = 0; g0 < G; g0 += blockDim.x) {
        const int g = g0 + threadIdx.x;
        int mine = 0;
        if (g < G) mine = (offsets[g + 1] - offsets[g] + bm - 1) / bm;
        // exclusive scan over the block in group order (serial over warps is fine: G is small)
        __shared__ int scan[1024];
        scan[threadIdx.x] = mine;
        __syncthreads();
        if (threadIdx.x == 0) {
            int run = base;
            for (int i = 0; i < (int)blockDim.x; ++i) {
                const int c = scan[i];
                scan[i] = run;
                run += c;
            }
            base = run;
        }
        __syncthreads();
        if (g < G) {
            const int first = scan[threadIdx.x];
            for (int i = 0; i < mine; ++i)
                if (first + i < max_tiles) {
                    tile_group[first + i] = g;
                    tile_row0[first + i] = offsets[g] + i * bm;
                }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) *num_tiles = base < max_tiles ? base : max_tiles;
}

}  // namespace

Q6K_API int q6k_gemm_tile_rows() { return BM; }

Q6K_API int q6k_tile_list(const int* offsets, int G, int bm, int* tile_group, int* tile_row0, int* num_tiles,
                          int max_tiles, cudaStream_t st) {
    Q6K_REQUIRE(G > 0 && bm > 0 && max_tiles > 0, "tile_list: bad sizes G=%d bm=%d max_tiles=%d", G, bm, max_tiles);
    q6k_launch(tile_list_kernel, 1, 256, 0, st, offsets, G, bm, tile_group, tile_row0, num_tiles, max_tiles);
    return q6k_check_launch("tile_list");
}

// epilogue: 0 store FP32, 1 add into FP32, 2 SwiGLU of (W, W2) stored in the operand dtype.
// Grouped when tile_group != null (max_tiles bounds the tile list; group_offsets has one more entry
// than there are groups); otherwise one group of M rows.
Q6K_API int q6k_gemm_simt(const void* A, int lda, const int* a_rows, const void* W, const void* W2, long long w_group_stride,
                          void* out, int ldo, int M, int N, int K, const int* tile_group, const int* tile_row0,
                          const int* group_offsets, const int* num_tiles, int max_tiles, int epilogue, int dtype,
                          cudaStream_t st) {
    if (M == 0 || N == 0) return 0;
    Q6K_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: bad sizes M=%d N=%d K=%d", M, N, K);
    Q6K_REQUIRE(epilogue >= 0 && epilogue <= 2, "gemm: unknown epilogue %d", epilogue);
    Q6K_REQUIRE(epilogue != EPI_SWIGLU || W2, "gemm: the SwiGLU epilogue needs two weight matrices");
    const int ytiles = tile_group ? max_tiles : (M + BM - 1) / BM;
    Q6K_REQUIRE(ytiles <= 65535, "gemm: %d row tiles exceed the grid limit", ytiles);
    dim3 grid((N + BN - 1) / BN, ytiles);
#define LAUNCH(EPI)                                                                                                     \
    q6k_launch(gemm_simt_kernel<T, EPI>, grid, 256, 0, st, (const T*)A, lda, a_rows, (const T*)W, (const T*)W2,                 \
                                                   (size_t)w_group_stride, out, ldo, M, N, K, tile_group, tile_row0, \
                                                   group_offsets, num_tiles)
    Q6K_DISPATCH(dtype, {
        if (epilogue == EPI_STORE) LAUNCH(EPI_STORE);
        else if (epilogue == EPI_ADD) LAUNCH(EPI_ADD);
        else LAUNCH(EPI_SWIGLU);
    });
#undef LAUNCH
    return q6k_check_launch("gemm_simt");
}
