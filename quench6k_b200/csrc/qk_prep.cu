// Per-head RMSNorm of q and k, rotary position encoding, q into the operand dtype and k, v into
// the pages of the cache.  Reference: crates/cuda/kernels/flint.cu:125-173 (there for one
// sequence, a contiguous cache, head size 128 and theta 10000 compiled in).
//
// The rotation is a parameter: a table inv_freq[rotary_dim / 2] of FP32 inverse frequencies (made
// by the position-encoding part: any base, any scaling of the frequencies), the number of leading
// head dimensions that rotate (rotary_dim <= head_dim; the rest pass through: partial rotary) and
// the pairing: halves (d with d + rotary_dim/2, the reference's) or neighbours (2i with 2i + 1).
// The angle of pair i at position p is float(p) * inv_freq[i], a 32-bit product, as in the reference.
//
// Page layout of one layer's K (and V) plane: [kv_heads, num_pages, page_size, head_dim] (head-major,
// so that pages with consecutive numbers are contiguous for one head and can be fetched as one TMA box).
// The row of position p of request r is page block_table[r][p / page_size], offset p % page_size.
#include "common.cuh"

namespace {

// Grid (T, Hq + Hkv) when the cache is written, (T, Hq) when this layer only reads another
// layer's cache.  One thread per head dimension (blockDim.x >= hd, a multiple of 32).
template <typename T>
__global__ void qk_prep_kernel(const float* qkv, int ld, int splits, size_t split_stride, int Hq, int Hkv, int hd, const float* q_norm, const float* k_norm,
                               float eps, const float* inv_freq, int rd, int neighbours, const int* positions, const int* req_of_token,
                               const int* block_table, int max_blocks, int page_size, int num_pages, T* q_out, T* k_pages, T* v_pages) {
    pdl_enter();
    extern __shared__ float xs[];            // hd floats
    __shared__ float red[32];
    const int t = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
    const bool is_q = h < Hq;
    const int pos = positions[t];
    const bool live = d < hd;
    const float* src = qkv + (size_t)t * ld + (is_q ? h * hd : (Hq + (h - Hq)) * hd);
    float x = 0.0f;
    if (live)
        for (int s = 0; s < splits; ++s) x += src[s * split_stride + d];        // split-K partials, in order
    const float* nw = is_q ? q_norm : k_norm;
    if (nw) {
        const float ss = block_sum(x * x, red);
        if (live) x = x * rsqrtf(ss / (float)hd + eps) * nw[d];
    }
    if (inv_freq) {
        if (live) xs[d] = x;
        __syncthreads();
        if (d < rd) {
            const int half = rd / 2;
            const int i = neighbours ? d >> 1 : (d < half ? d : d - half);
            const bool first = neighbours ? !(d & 1) : d < half;       // the pair's first member: x cos - partner sin
            const int partner = neighbours ? d ^ 1 : (first ? d + half : d - half);
            float sn, cs;
            sincosf((float)pos * inv_freq[i], &sn, &cs);
            x = first ? xs[d] * cs - xs[partner] * sn : xs[d] * cs + xs[partner] * sn;
        }
    }
    if (!live) return;
    if (is_q) {
        q_out[((size_t)t * Hq + h) * hd + d] = from_f32<T>(x);
    } else {
        const int kh = h - Hq;
        const int page = block_table[(size_t)req_of_token[t] * max_blocks + pos / page_size];
        if (page < 0) return;                 // no page behind this position: nothing is written
        const size_t row = (((size_t)kh * num_pages + page) * page_size + pos % page_size) * hd + d;
        k_pages[row] = from_f32<T>(x);
        float v = 0.0f;
        for (int s = 0; s < splits; ++s) v += qkv[s * split_stride + (size_t)t * ld + (size_t)(Hq + Hkv + kh) * hd + d];
        v_pages[row] = from_f32<T>(v);
    }
}

// The same for head sizes that are multiples of 64: one warp per (token, head), each lane holding
// head_dim/32 elements d = lane + 32 i.  Paired by halves with rotary_dim a multiple of 64, both
// members of a pair (d, d + rotary_dim/2) sit in one lane; paired by neighbours, the partner is the
// same element of the lane beside.  Nothing goes through shared memory but the angles' cosines
// and sines.  Block = 8 warps = 8 heads of one token.
template <typename T, int EPL>
__global__ void __launch_bounds__(256) qk_prep_warp_kernel(const float* qkv, int ld, int splits, size_t split_stride, int Hq, int Hkv, const float* q_norm,
                                                           const float* k_norm, float eps, const float* inv_freq, int rd, int neighbours,
                                                           const int* positions, const int* req_of_token, const int* block_table,
                                                           int max_blocks, int page_size, int num_pages, T* q_out, T* k_pages,
                                                           T* v_pages, int heads) {
    pdl_enter();
    constexpr int hd = EPL * 32, half = hd / 2;
    __shared__ float rot_cos[half], rot_sin[half];
    const int t = blockIdx.x, h = blockIdx.y * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    const bool valid = h < heads, is_q = h < Hq;
    const int kh = h - Hq;
    const bool writes_kv = valid && !is_q;
    // everything that does not depend on another load goes out first: the position, the request, this
    // head's slices of q or k and of v; then the page (position and request) and the angles (position)
    const int pos = positions[t];
    const int req = writes_kv ? req_of_token[t] : 0;
    const float* src = qkv + (size_t)t * ld + (size_t)(valid ? h : 0) * hd;           // q heads then k heads are contiguous in a row
    const float* vsrc = qkv + (size_t)t * ld + (size_t)(Hq + Hkv + (writes_kv ? kh : 0)) * hd;
    float x[EPL], v[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        x[i] = valid ? src[lane + 32 * i] : 0.0f;
        v[i] = writes_kv ? vsrc[lane + 32 * i] : 0.0f;
    }
    for (int s = 1; s < splits; ++s) {                                               // split-K partials, in order
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            if (valid) x[i] += src[s * split_stride + lane + 32 * i];
            if (writes_kv) v[i] += vsrc[s * split_stride + lane + 32 * i];
        }
    }
    const int page = writes_kv ? block_table[(size_t)req * max_blocks + pos / page_size] : -1;
    if (inv_freq) {
        // the angles depend on the position and the pair only: once per block, not once per head
        for (int i = threadIdx.x; i < rd / 2; i += blockDim.x) sincosf((float)pos * inv_freq[i], &rot_sin[i], &rot_cos[i]);
        __syncthreads();
    }
    if (!valid) return;
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) ss = fmaf(x[i], x[i], ss);
    const float* nw = is_q ? q_norm : k_norm;
    if (nw) {
        const float inv = rsqrtf(warp_sum(ss) / (float)hd + eps);
#pragma unroll
        for (int i = 0; i < EPL; ++i) x[i] = x[i] * inv * nw[lane + 32 * i];
    }
    if (inv_freq && !neighbours) {
        const int per = rd / 64;                                         // elements of a lane in each half of the rotated part
#pragma unroll
        for (int i = 0; i < EPL / 2; ++i) {
            if (i < per) {
                const int d = lane + 32 * i;                             // d < rd/2; partner d + rd/2 is element i + per
                const float sn = rot_sin[d], cs = rot_cos[d];
                float lo = x[i], hi = 0.0f;
#pragma unroll
                for (int j = 1; j <= EPL / 2; ++j)                       // x[i + per] without indexing registers by a variable
                    if (j == per) hi = x[i + j];
                const float a = lo * cs - hi * sn, b = hi * cs + lo * sn;
                x[i] = a;
#pragma unroll
                for (int j = 1; j <= EPL / 2; ++j)
                    if (j == per) x[i + j] = b;
            }
        }
    } else if (inv_freq) {
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            const int d = lane + 32 * i;
            const float other = __shfl_xor_sync(0xffffffffu, x[i], 1);   // every lane takes part, whether its element rotates or not
            if (d < rd) {
                const float sn = rot_sin[d >> 1], cs = rot_cos[d >> 1];
                x[i] = (d & 1) ? x[i] * cs + other * sn : x[i] * cs - other * sn;
            }
        }
    }
    if (is_q) {
        T* dst = q_out + ((size_t)t * Hq + h) * hd;
#pragma unroll
        for (int i = 0; i < EPL; ++i) dst[lane + 32 * i] = from_f32<T>(x[i]);
    } else {
        if (page < 0) return;
        const size_t row = (((size_t)kh * num_pages + page) * page_size + pos % page_size) * hd;
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            k_pages[row + lane + 32 * i] = from_f32<T>(x[i]);
            v_pages[row + lane + 32 * i] = from_f32<T>(v[i]);
        }
    }
}

}  // namespace

// qkv: FP32 [T, ld] with q heads, then k heads, then v heads in each row.  q_norm/k_norm: FP32 [hd]
// or null (no QK-norm).  inv_freq: FP32 [rotary_dim / 2] or null (no rotation); the first rotary_dim
// dimensions of every q and k head rotate by positions[t] * inv_freq[pair], paired by halves
// (neighbours == 0: d with d + rotary_dim/2) or by neighbours (2i with 2i + 1).
// write_kv == 0: only q is produced (the layer reads a cache another layer wrote).
// splits > 1: qkv is [splits, T, ld] (slices split_stride floats apart) and the slices are summed in order first.
Q6K_API int q6k_qk_prep(const float* qkv, int ld, int splits, long long split_stride, int T_, int Hq, int Hkv, int hd, const float* q_norm, const float* k_norm,
                        float eps, const float* inv_freq, int rotary_dim, int neighbours, const int* positions, const int* req_of_token,
                        const int* block_table, int max_blocks, int page_size, int num_pages, void* q_out, void* k_pages,
                        void* v_pages, int write_kv, int dtype, cudaStream_t st) {
    if (T_ == 0) return 0;
    Q6K_REQUIRE(T_ > 0 && Hq > 0 && Hkv > 0 && hd > 0, "qk_prep: bad sizes T=%d Hq=%d Hkv=%d hd=%d", T_, Hq, Hkv, hd);
    Q6K_REQUIRE(splits >= 1, "qk_prep: bad split count %d", splits);
    Q6K_REQUIRE(hd % 2 == 0 && hd <= 1024, "qk_prep: head_dim %d must be even and at most 1024", hd);
    Q6K_REQUIRE(!inv_freq || (rotary_dim > 0 && rotary_dim % 2 == 0 && rotary_dim <= hd), "qk_prep: %d rotating dimensions of a head of %d", rotary_dim, hd);
    Q6K_REQUIRE(!write_kv || (page_size > 0 && max_blocks > 0), "qk_prep: bad page_size %d / max_blocks %d", page_size, max_blocks);
    const int heads = write_kv ? Hq + Hkv : Hq;
    const int rd = inv_freq ? rotary_dim : 0;
    if ((hd == 64 || hd == 128 || hd == 256) && (!inv_freq || neighbours || rd % 64 == 0)) {
        dim3 wgrid(T_, (heads + 7) / 8);
        Q6K_REQUIRE(wgrid.y <= 65535, "qk_prep: %d heads exceed the grid limit", heads);
#define WARP_LAUNCH(EPL)                                                                                                    \
    q6k_launch(qk_prep_warp_kernel<T, EPL>, wgrid, 256, 0, st, qkv, ld, splits, (size_t)split_stride, Hq, Hkv, q_norm, k_norm, eps, inv_freq, rd, neighbours, positions, req_of_token, \
                                                       block_table, max_blocks, page_size, num_pages, (T*)q_out, (T*)k_pages, (T*)v_pages, heads)
        Q6K_DISPATCH(dtype, {
            if (hd == 64) WARP_LAUNCH(2);
            else if (hd == 128) WARP_LAUNCH(4);
            else WARP_LAUNCH(8);
        });
#undef WARP_LAUNCH
        return q6k_check_launch("qk_prep");
    }
    const int threads = (hd + 31) / 32 * 32;
    dim3 grid(T_, heads);
    Q6K_DISPATCH(dtype, q6k_launch(qk_prep_kernel<T>, grid, threads, hd * sizeof(float), st, 
                            qkv, ld, splits, (size_t)split_stride, Hq, Hkv, hd, q_norm, k_norm, eps, inv_freq, rd, neighbours, positions, req_of_token, block_table,
                            max_blocks, page_size, num_pages, (T*)q_out, (T*)k_pages, (T*)v_pages););
    return q6k_check_launch("qk_prep");
}
