// Embedding gather, RMSNorm over rows of the FP32 residual stream, and the MoE combine.
// Reference formulas: crates/cuda/kernels/flint.cu:89-95 (embed), :97-122 (rmsnorm),
// :1228-1239 (combine).  Unlike the reference no width is compiled in.
#include "common.cuh"

namespace {

// A token id -(i + 1) stands for fed[i], the i-th token the step before has sampled, which the host
// may not have seen yet (fed: up to n_fed ids on the device).
template <typename T>
__global__ void embed_kernel(const int* tokens, const T* table, float* h, int D, int V, const int* fed, int n_fed) {
    pdl_enter();
    const int t = blockIdx.x;
    int tok = tokens[t];
    if (tok < 0 && fed != nullptr && -tok - 1 < n_fed) tok = fed[-tok - 1];
    tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);      // ids are validated on the host; never read outside the table
    const T* row = table + (size_t)tok * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) h[(size_t)t * D + i] = to_f32(row[i]);
}

// out[r] = T(x[row] * rsqrt(mean(x[row]^2) + eps) * w), row = rows ? rows[r] : r.  Sum of squares,
// rsqrt and the products are FP32; the per-thread partial sums and the block sum run in a fixed order.
// With `add`, x[row] += add[r] first and the sum is written back (the residual add of the block,
// folded in as the reference does, crates/cuda/kernels/flint.cu:97-122).
template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_kernel(float* x, const float* add, const int* rows, const float* w, float eps,
                                                      T* out, int D) {
    pdl_enter();
    __shared__ float red[32];
    const int r = blockIdx.x;
    float* xr = x + (size_t)(rows ? rows[r] : r) * D;
    float ss = 0.0f;
    if (add) {
        const float* ar = add + (size_t)r * D;
        for (int i = threadIdx.x; i < D; i += blockDim.x) {
            const float v = xr[i] + ar[i];
            xr[i] = v;                         // each thread re-reads only what it wrote itself
            ss = fmaf(v, v, ss);
        }
    } else {
        for (int i = threadIdx.x; i < D; i += blockDim.x) ss = fmaf(xr[i], xr[i], ss);
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)D + eps);
    for (int i = threadIdx.x; i < D; i += blockDim.x) out[(size_t)r * D + i] = from_f32<T>(xr[i] * inv * w[i]);
}

// h[t, d] += sum_s w[t, s] * y[pair_row[t*S + s], d], slots in order (so the result does not
// depend on where the permutation put the rows).  pair_row == null: rows are in pair order.
__global__ void combine_kernel(const float* y, const int* pair_row, const float* sel_w, int S, int D, float* h) {
    pdl_enter();
    const int t = blockIdx.x, d = blockIdx.y * blockDim.x + threadIdx.x;
    if (d >= D) return;
    float acc = 0.0f;
    for (int s = 0; s < S; ++s) acc = fmaf(sel_w[t * S + s], y[(size_t)(pair_row ? pair_row[t * S + s] : t * S + s) * D + d], acc);
    h[(size_t)t * D + d] += acc;
}

// The same with the row held in registers (D <= 256 * 4 * V4, D a multiple of 4): one pass over
// the row, 16-byte loads.  `add_splits` > 1: add is [add_splits, R, D] and its slices are summed in
// order first (the split-K partials of the product that feeds the residual add).
// `pair_y`: the routed experts' results come in unsummed, x[t] += sum_s pair_w[t, s] * y[row(t, s)]
// with row(t, s) = pair_row[t*S + s] (or t*S + s), slots in order: the arithmetic of combine4_kernel
// below, which this replaces together with one pass over x.
// NB: loads kept in flight per accumulation (8 for the few rows of a decode step, whose time is
// latency; 2 for many rows, where the registers they cost would halve the blocks per SM).
template <typename T, int V4, int NB>
__global__ void __launch_bounds__(256) rmsnorm_reg_kernel(float* x, const float* add, int add_splits, size_t add_stride, const int* rows,
                                                          const float* w, float eps, T* out, int D, const float* pair_y,
                                                          const int* pair_row, const float* pair_w, int S, int early) {
    // the norm's weight is older than any kernel of the step: it is fetched, and (early != 0) the kernel after this one
    // let start, before the wait for the kernel that makes the rows
    if (early) pdl_launch();
    __shared__ float red[32];
    const int r = blockIdx.x, nv = D >> 2;
    float4 v[V4], g[V4];
#pragma unroll
    for (int i = 0; i < V4; ++i) {
        const int c = threadIdx.x + 256 * i;
        if (c < nv) g[i] = reinterpret_cast<const float4*>(w)[c];
    }
    pdl_wait();
    if (!early) pdl_launch();
    const int t = rows ? rows[r] : r;
    float4* xr = reinterpret_cast<float4*>(x + (size_t)t * D);
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < V4; ++i) {
        const int c = threadIdx.x + 256 * i;
        if (c < nv) {
            v[i] = xr[c];
            if (add) {
                // the slices are fetched eight at a time (independent loads) and added in their order
                const float4* ar = reinterpret_cast<const float4*>(add + (size_t)r * D) + c;
                float4 a = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                for (int s0 = 0; s0 < add_splits; s0 += NB) {
                    float4 b[NB];
#pragma unroll
                    for (int j = 0; j < NB; ++j)
                        if (s0 + j < add_splits) b[j] = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(ar) + (size_t)(s0 + j) * add_stride);
#pragma unroll
                    for (int j = 0; j < NB; ++j)
                        if (s0 + j < add_splits) a.x += b[j].x, a.y += b[j].y, a.z += b[j].z, a.w += b[j].w;
                }
                v[i].x += a.x, v[i].y += a.y, v[i].z += a.z, v[i].w += a.w;
                xr[c] = v[i];
            }
            if (pair_y) {
                float4 a = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                for (int s0 = 0; s0 < S; s0 += NB) {
                    float4 b[NB];
                    float ws[NB];
#pragma unroll
                    for (int j = 0; j < NB; ++j) {
                        if (s0 + j < S) {
                            const int pr = pair_row ? pair_row[t * S + s0 + j] : t * S + s0 + j;
                            ws[j] = pair_w[t * S + s0 + j];
                            b[j] = reinterpret_cast<const float4*>(pair_y + (size_t)pr * D)[c];
                        }
                    }
#pragma unroll
                    for (int j = 0; j < NB; ++j)
                        if (s0 + j < S) a.x = fmaf(ws[j], b[j].x, a.x), a.y = fmaf(ws[j], b[j].y, a.y), a.z = fmaf(ws[j], b[j].z, a.z), a.w = fmaf(ws[j], b[j].w, a.w);
                }
                v[i].x += a.x, v[i].y += a.y, v[i].z += a.z, v[i].w += a.w;
                xr[c] = v[i];
            }
            ss = fmaf(v[i].x, v[i].x, ss), ss = fmaf(v[i].y, v[i].y, ss), ss = fmaf(v[i].z, v[i].z, ss), ss = fmaf(v[i].w, v[i].w, ss);
        }
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)D + eps);
#pragma unroll
    for (int i = 0; i < V4; ++i) {
        const int c = threadIdx.x + 256 * i;
        if (c < nv) {
            T* o = out + (size_t)r * D + 4 * c;
            o[0] = from_f32<T>(v[i].x * inv * g[i].x), o[1] = from_f32<T>(v[i].y * inv * g[i].y);
            o[2] = from_f32<T>(v[i].z * inv * g[i].z), o[3] = from_f32<T>(v[i].w * inv * g[i].w);
        }
    }
}

// The same, four columns per thread with 16-byte loads (D a multiple of 4).
__global__ void combine4_kernel(const float4* y, const int* pair_row, const float* sel_w, int S, int D4, float4* h) {
    pdl_enter();
    const int t = blockIdx.x, d = blockIdx.y * blockDim.x + threadIdx.x;
    if (d >= D4) return;
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int s = 0; s < S; ++s) {
        const float w = sel_w[t * S + s];
        const float4 v = y[(size_t)(pair_row ? pair_row[t * S + s] : t * S + s) * D4 + d];
        acc.x = fmaf(w, v.x, acc.x), acc.y = fmaf(w, v.y, acc.y), acc.z = fmaf(w, v.z, acc.z), acc.w = fmaf(w, v.w, acc.w);
    }
    float4 o = h[(size_t)t * D4 + d];
    o.x += acc.x, o.y += acc.y, o.z += acc.z, o.w += acc.w;
    h[(size_t)t * D4 + d] = o;
}

// act[r, i] = T(silu(g[r, i]) * u[r, i]) for gu = [rows, 2*I] (gate columns first).
template <typename T>
__global__ void swiglu_kernel(const float* gu, T* act, int I, size_t count) {
    pdl_enter();
    const size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (idx >= count) return;
    const size_t r = idx / I;
    const int i = (int)(idx % I);
    const float g = gu[r * 2 * I + i], u = gu[r * 2 * I + I + i];
    act[idx] = from_f32<T>(g / (1.0f + expf(-g)) * u);
}

// out[r, :] = x[idx[r], :] for rows of `bytes` bytes (a multiple of 16), 16 bytes per thread step.
__global__ void gather_rows_kernel(const uint4* x, const int* idx, uint4* out, int vec_per_row) {
    pdl_enter();
    const size_t src = (size_t)idx[blockIdx.x] * vec_per_row, dst = (size_t)blockIdx.x * vec_per_row;
    for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) out[dst + i] = x[src + i];
}

}  // namespace

// Rows of any element type: row_bytes must be a multiple of 16 and both buffers 16-byte aligned.
Q6K_API int q6k_gather_rows(const void* x, const int* idx, void* out, int rows, int row_bytes, cudaStream_t st) {
    if (rows == 0) return 0;
    Q6K_REQUIRE(rows > 0 && row_bytes > 0 && row_bytes % 16 == 0, "gather_rows: rows of %d bytes are not a multiple of 16", row_bytes);
    Q6K_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)out & 15) == 0, "gather_rows: buffers must be 16-byte aligned");
    q6k_launch(gather_rows_kernel, rows, 128, 0, st, (const uint4*)x, idx, (uint4*)out, row_bytes / 16);
    return q6k_check_launch("gather_rows");
}

Q6K_API int q6k_embed(const int* tokens, const void* table, float* h, int T_, int D, int V, int dtype, const int* fed, int n_fed,
                      cudaStream_t st) {
    if (T_ == 0) return 0;
    Q6K_REQUIRE(T_ > 0 && D > 0 && V > 0 && n_fed >= 0, "embed: bad sizes T=%d D=%d V=%d", T_, D, V);
    Q6K_DISPATCH(dtype, q6k_launch(embed_kernel<T>, T_, 256, 0, st, tokens, (const T*)table, h, D, V, fed, n_fed););
    return q6k_check_launch("embed");
}

// add: FP32 [R, D] or null; when given, x[row] += add[r] is stored before normalising (rows must then be null).
// add_splits > 1: add is [add_splits, R, D] (slices add_stride floats apart), summed in order.
// pair_y != null: x[t] += sum_s pair_w[t, s] * pair_y[pair_row ? pair_row[t*S + s] : t*S + s] first (t = rows[r] or r);
// needs the register kernel (D a multiple of 4, at most 4096): q6k_rmsnorm_fuses_pairs tells.
Q6K_API int q6k_rmsnorm_fuses_pairs(int D) { return D % 4 == 0 && D <= 256 * 4 * 4; }

Q6K_API int q6k_rmsnorm(float* x, const float* add, int add_splits, long long add_stride, const int* rows, const float* w, float eps,
                        void* out, int R, int D, int dtype, const float* pair_y, const int* pair_row, const float* pair_w, int S,
                        cudaStream_t st) {
    if (R == 0) return 0;
    Q6K_REQUIRE(R > 0 && D > 0, "rmsnorm: bad sizes R=%d D=%d", R, D);
    Q6K_REQUIRE(!(add && rows), "rmsnorm: the fused add takes no row selection");
    Q6K_REQUIRE(add_splits >= 1, "rmsnorm: bad split count %d", add_splits);
    Q6K_REQUIRE(!pair_y || (pair_w && S > 0), "rmsnorm: weighted rows need their weights");
    const bool vec = D % 4 == 0 && D <= 256 * 4 * 4 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0 && (!add || ((uintptr_t)add & 15) == 0) &&
                     (add_stride % 4 == 0) && (!pair_y || ((uintptr_t)pair_y & 15) == 0);
    if (vec) {
        const int v4 = (D / 4 + 255) / 256;
        // A norm inside the layers may let the kernel after it start, and fetch its first weights, under the kernel before
        // the norm (that kernel reads nothing but weights before its own wait).  Whether that pays depends on the kernel
        // before (measured on B200 at 32,768 cached tokens):
        //  - one or two rows: the kernels around every norm are matrix-vector streams of a few microseconds, and it pays
        //    (1.37 -> 1.31 ms a step at one row, 1.93 -> 1.88 at two);
        //  - up to 16 rows, a norm that adds a product's result (the one between mixer and feed-forward: the o product
        //    before it is a few-token kernel of small blocks, the router's cluster after it finds room beside them):
        //    3.99 -> 3.94 ms a step at eight rows, 2.57 -> 2.55 at four;
        //  - a norm that adds the experts' weighted rows at more than two rows comes after a tensor-core kernel that
        //    fills the SMs, and blocks parked beside it only get in its way (4.03 -> 4.09 ms at eight rows); and the LM
        //    head behind the last norm, parked that early, took twice as long.
        const int early = rows == nullptr && (R <= 2 || (R <= 16 && add != nullptr && pair_y == nullptr));
#define Q6K_NORM_GO(V4_, NB_) q6k_launch_as(early != 0, rmsnorm_reg_kernel<T, V4_, NB_>, R, 256, 0, st, x, add, add_splits, (size_t)add_stride, rows, w, eps, (T*)out, D, pair_y, pair_row, pair_w, S, early)
        Q6K_DISPATCH(dtype, {
            if (R <= 64) {
                if (v4 <= 1) Q6K_NORM_GO(1, 8);
                else if (v4 <= 2) Q6K_NORM_GO(2, 8);
                else Q6K_NORM_GO(4, 8);
            } else {
                if (v4 <= 1) Q6K_NORM_GO(1, 2);
                else if (v4 <= 2) Q6K_NORM_GO(2, 2);
                else Q6K_NORM_GO(4, 2);
            }
        });
#undef Q6K_NORM_GO
        return q6k_check_launch("rmsnorm");
    }
    Q6K_REQUIRE(!pair_y, "rmsnorm: weighted rows need a width that is a multiple of 4 and at most 4096 (got %d)", D);
    Q6K_REQUIRE(add_splits == 1, "rmsnorm: summing split partials needs a width that is a multiple of 4 and at most 4096 (got %d)", D);
    Q6K_DISPATCH(dtype, q6k_launch(rmsnorm_kernel<T>, R, 256, 0, st, x, add, rows, w, eps, (T*)out, D););
    return q6k_check_launch("rmsnorm");
}

Q6K_API int q6k_combine(const float* y, const int* pair_row, const float* sel_w, int T_, int S, int D, float* h,
                        cudaStream_t st) {
    if (T_ == 0) return 0;
    Q6K_REQUIRE(T_ > 0 && S > 0 && D > 0, "combine: bad sizes T=%d S=%d D=%d", T_, S, D);
    if (D % 4 == 0 && ((uintptr_t)y & 15) == 0 && ((uintptr_t)h & 15) == 0)
        q6k_launch(combine4_kernel, dim3(T_, (D / 4 + 255) / 256), 256, 0, st, (const float4*)y, pair_row, sel_w, S, D / 4, (float4*)h);
    else
        q6k_launch(combine_kernel, dim3(T_, (D + 255) / 256), 256, 0, st, y, pair_row, sel_w, S, D, h);
    return q6k_check_launch("combine");
}

Q6K_API int q6k_swiglu(const float* gu, void* act, int rows, int I, int dtype, cudaStream_t st) {
    if (rows == 0) return 0;
    Q6K_REQUIRE(rows > 0 && I > 0, "swiglu: bad sizes rows=%d I=%d", rows, I);
    const size_t count = (size_t)rows * I;
    Q6K_DISPATCH(dtype, q6k_launch(swiglu_kernel<T>, (unsigned)((count + 255) / 256), 256, 0, st, gu, (T*)act, I, count););
    return q6k_check_launch("swiglu");
}
