// Attention over the paged cache for any mix of rows (prompt portions beside decode tokens), any
// head size that is a multiple of 16 up to 256, any number of heads and groups, in FP32 or
// bfloat16 storage with FP32 arithmetic.  This is the kernel of the true 32-bit path and the
// fallback of the bfloat16 path.
//
// Formulas: crates/cuda/kernels/flint.cu:211-529 (query head h reads KV head h / G; score
// q.k/sqrt(hd); key j visible to position p iff j <= p and, with a window W, j > p - W; online
// softmax; probabilities rounded to the storage type before they are summed, :409-415) and
// :531-561 (a sink adds exp(sink_h - m) to the denominator only).
//
// A block takes one (token, KV head); its warps take the G query heads in turn.  Keys are walked
// in tiles of 32 aligned to multiples of 32 of the key index, so the order of the sums for a
// given (position, head) never depends on how the tokens were cut into steps or batched.
#include "common.cuh"

namespace {

constexpr int MAX_HD = 256, DPL = MAX_HD / 32;   // head dims per lane

template <typename T>
__global__ void __launch_bounds__(128) attention_generic_kernel(const T* q, const T* k_pages, const T* v_pages,
                                                                const int* block_table, int max_blocks, int page_size,
                                                                int num_pages, const int* req_of_token, const int* positions, int window,
                                                                const float* sinks, float scale, T* out, int Hq, int Hkv,
                                                                int hd) {
    pdl_enter();
    extern __shared__ float qs[];             // [warps][hd]
    const int t = blockIdx.x, kh = blockIdx.y, G = Hq / Hkv;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int pos = positions[t];
    const int* bt = block_table + (size_t)req_of_token[t] * max_blocks;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    float* qw = qs + warp * hd;
    const size_t head_base = (size_t)kh * num_pages;          // pools are [Hkv, num_pages, page_size, hd]

    for (int g = warp; g < G; g += nwarps) {
        const int h = kh * G + g;
        for (int d = lane; d < hd; d += 32) qw[d] = to_f32(q[((size_t)t * Hq + h) * hd + d]);
        __syncwarp();
        float m = -INFINITY, l = 0.0f, o[DPL];
#pragma unroll
        for (int i = 0; i < DPL; ++i) o[i] = 0.0f;
        for (int j0 = lo & ~31; j0 <= pos; j0 += 32) {
            const int j = j0 + lane;
            const bool ok = j >= lo && j <= pos;
            float s = -INFINITY;
            size_t row = 0;
            if (ok) {
                const int page = bt[j / page_size];
                row = ((head_base + page) * page_size + j % page_size) * hd;
                const T* kr = k_pages + row;
                float acc = 0.0f;
                for (int d = 0; d < hd; ++d) acc = fmaf(qw[d], to_f32(kr[d]), acc);
                s = acc * scale;
            }
            const float mt = warp_max(s);
            const float mn = fmaxf(m, mt);          // finite: the tile holds at least one visible key
            const float corr = m == -INFINITY ? 0.0f : expf(m - mn);
            float p = ok ? round_to<T>(expf(s - mn)) : 0.0f;
            l = l * corr + warp_sum(p);
#pragma unroll
            for (int i = 0; i < DPL; ++i) o[i] *= corr;
            const int nk = min(32, pos - j0 + 1);
            for (int jj = 0; jj < nk; ++jj) {
                const float pj = __shfl_sync(0xffffffffu, p, jj);
                const unsigned long long rj = __shfl_sync(0xffffffffu, (unsigned long long)row, jj);
                if (pj == 0.0f) continue;           // uniform across the warp
                const T* vr = v_pages + rj;
#pragma unroll
                for (int i = 0; i < DPL; ++i) {
                    const int d = lane + 32 * i;
                    if (d < hd) o[i] = fmaf(pj, to_f32(vr[d]), o[i]);
                }
            }
            m = mn;
        }
        float den = l;
        float osc = 1.0f;
        if (sinks) {
            const float sk = sinks[h];
            const float M = fmaxf(m, sk);
            osc = expf(m - M);
            den = l * osc + expf(sk - M);
        }
        const float inv = osc / den;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int d = lane + 32 * i;
            if (d < hd) out[((size_t)t * Hq + h) * hd + d] = from_f32<T>(o[i] * inv);
        }
        __syncwarp();
    }
}

}  // namespace

// q: [T, Hq, hd]; pages: [Hkv, num_pages, page_size, hd]; block_table: [R, max_blocks];
// window 0: every earlier key is visible; sinks: FP32 [Hq] or null; out: [T, Hq*hd].
Q6K_API int q6k_attention_generic(const void* q, const void* k_pages, const void* v_pages, int num_pages, const int* block_table,
                                  int max_blocks, int page_size, const int* req_of_token, const int* positions, int window,
                                  const float* sinks, float scale, void* out, int T_, int Hq, int Hkv, int hd, int dtype,
                                  cudaStream_t st) {
    if (T_ == 0) return 0;
    Q6K_REQUIRE(T_ > 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0, "attention: bad head counts Hq=%d Hkv=%d", Hq, Hkv);
    Q6K_REQUIRE(hd > 0 && hd % 16 == 0 && hd <= MAX_HD, "attention: head_dim %d is not a multiple of 16 in 16..%d", hd, MAX_HD);
    Q6K_REQUIRE(page_size > 0 && max_blocks > 0 && window >= 0, "attention: bad page_size %d / max_blocks %d / window %d",
                page_size, max_blocks, window);
    Q6K_REQUIRE(Hkv <= 65535, "attention: %d KV heads exceed the grid limit", Hkv);
    const int G = Hq / Hkv;
    const int warps = G < 4 ? G : 4;
    dim3 grid(T_, Hkv);
    Q6K_DISPATCH(dtype, q6k_launch(attention_generic_kernel<T>, grid, warps * 32, warps * hd * sizeof(float), st, 
                            (const T*)q, (const T*)k_pages, (const T*)v_pages, block_table, max_blocks, page_size,
                            num_pages, req_of_token, positions, window, sinks, scale, (T*)out, Hq, Hkv, hd););
    return q6k_check_launch("attention_generic");
}
