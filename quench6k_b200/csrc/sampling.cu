// Sampling support on the device: per-row argmax (greedy) and an exact top-k candidate pool.
//
// The reference picks greedily with a device argmax, ties to the lower id
// (crates/cuda/kernels/topk.cu:212-303), and samples from a pool of the top candidates that an
// exact device top-k delivers to the host (crates/cli/src/flint.rs:339-353, topk.cu:28-146).
// Both are kept: the pool comes back sorted by (logit descending, id ascending).
#include <cooperative_groups.h>

#include "common.cuh"
#include "no_alloc.h"

namespace {

// Ascending-order-preserving key of a float; NaN sorts lowest; -0 and +0 are the same key, as
// they compare equal.
__device__ __forceinline__ unsigned key_of(float v) {
    if (v != v) return 0u;
    if (v == 0.0f) v = 0.0f;
    const unsigned u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Best (key, index) of a block's candidates; ties go to the lower index.  Result in thread 0.
__device__ __forceinline__ void block_best(unsigned& best, int& best_i, unsigned* bk, int* bi) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned ok = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ok > best || (ok == best && oi < best_i)) best = ok, best_i = oi;
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) bk[warp] = best, bi[warp] = best_i;
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
        best = lane < nw ? bk[lane] : 0u;
        best_i = lane < nw ? bi[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned ok = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ok > best || (ok == best && oi < best_i)) best = ok, best_i = oi;
        }
    }
}

constexpr int ARGMAX_SLICE = 8192;

// Stage 1: block (slice, row) finds the best of its slice of the row.
__global__ void __launch_bounds__(256) argmax_partial_kernel(const float* logits, int V, int slices, unsigned* pk, int* pi) {
    pdl_enter();
    __shared__ unsigned bk[32];
    __shared__ int bi[32];
    const float* row = logits + (size_t)blockIdx.y * V;
    const int lo = blockIdx.x * ARGMAX_SLICE, hi = min(V, lo + ARGMAX_SLICE);
    unsigned best = 0u;
    int best_i = 0x7fffffff;
    // eight loads in flight per thread before the compares
    for (int i0 = lo + threadIdx.x; i0 < hi; i0 += 8 * blockDim.x) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = i0 + u * blockDim.x;
            v[u] = i < hi ? row[i] : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = i0 + u * blockDim.x;
            if (i < hi) {
                const unsigned k = key_of(v[u]);
                if (k > best || (k == best && i < best_i)) best = k, best_i = i;
            }
        }
    }
    block_best(best, best_i, bk, bi);
    if (threadIdx.x == 0) pk[blockIdx.y * slices + blockIdx.x] = best, pi[blockIdx.y * slices + blockIdx.x] = best_i;
}

// Stage 2: one warp per row picks among the slices' winners.
__global__ void argmax_final_kernel(const unsigned* pk, const int* pi, int slices, int* out) {
    pdl_enter();
    unsigned best = 0u;
    int best_i = 0x7fffffff;
    for (int s = threadIdx.x; s < slices; s += 32) {
        const unsigned k = pk[blockIdx.x * slices + s];
        const int i = pi[blockIdx.x * slices + s];
        if (k > best || (k == best && i < best_i)) best = k, best_i = i;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned ok = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ok > best || (ok == best && oi < best_i)) best = ok, best_i = oi;
    }
    if (threadIdx.x == 0) out[blockIdx.x] = best_i;
}

constexpr int POOL_MAX = 256;

// Exact top-K of one row per block (K <= 256): a 4-pass radix select finds the K-th largest key,
// everything above it is taken, ties at it are taken in ascending id order, and the K candidates
// are sorted by (key descending, id ascending) with a bitonic network.
__global__ void __launch_bounds__(1024) topk_pool_kernel(const float* logits, int V, int K, int* out_ids, float* out_vals) {
    pdl_enter();
    __shared__ int hist[256];
    __shared__ unsigned s_prefix;
    __shared__ int s_need, s_count;
    __shared__ unsigned ck[POOL_MAX];
    __shared__ int ci[POOL_MAX];
    __shared__ int seg_eq[1024];
    const float* row = logits + (size_t)blockIdx.x * V;
    const int tid = threadIdx.x, n = blockDim.x;
    if (tid == 0) s_prefix = 0u, s_need = K;
    __syncthreads();
    // radix select, most significant byte first
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        const unsigned himask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        const unsigned prefix = s_prefix;
        for (int i = tid; i < V; i += n) {
            const unsigned k = key_of(row[i]);
            if ((k & himask) == prefix) atomicAdd(&hist[(k >> shift) & 255], 1);
        }
        __syncthreads();
        if (tid == 0) {
            int need = s_need, b = 255;
            for (; b > 0; --b) {
                if (hist[b] >= need) break;
                need -= hist[b];
            }
            s_need = need;                      // how many are wanted from bin b
            s_prefix = prefix | ((unsigned)b << shift);
        }
        __syncthreads();
    }
    const unsigned kth = s_prefix;
    const int need_eq = s_need;                 // ties at the K-th key that are taken
    if (tid == 0) s_count = 0;
    __syncthreads();
    // strictly greater: any order (sorted below)
    for (int i = tid; i < V; i += n) {
        const unsigned k = key_of(row[i]);
        if (k > kth) {
            const int at = atomicAdd(&s_count, 1);
            if (at < POOL_MAX) ck[at] = k, ci[at] = i;
        }
    }
    // equal: the lowest ids.  Thread t owns the contiguous ids [t*seg, (t+1)*seg).
    const int seg = (V + n - 1) / n;
    const int b0 = tid * seg, b1 = min(V, b0 + seg);
    int mine = 0;
    for (int i = b0; i < b1; ++i) mine += key_of(row[i]) == kth;
    seg_eq[tid] = mine;
    __syncthreads();
    const int gt = s_count;
    if (tid == 0) {
        int run = 0;
        for (int i = 0; i < n; ++i) {
            const int c = seg_eq[i];
            seg_eq[i] = run;
            run += c;
        }
    }
    __syncthreads();
    int r = seg_eq[tid];
    for (int i = b0; i < b1 && r < need_eq; ++i)
        if (key_of(row[i]) == kth) {
            if (gt + r < POOL_MAX) ck[gt + r] = kth, ci[gt + r] = i;
            ++r;
        }
    __syncthreads();
    // pad to 256 and sort descending by (key, -id)
    for (int i = tid; i < POOL_MAX; i += n)
        if (i >= K) ck[i] = 0u, ci[i] = 0x7fffffff;
    __syncthreads();
    for (int size = 2; size <= POOL_MAX; size <<= 1)
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            if (tid < POOL_MAX / 2) {
                const int lo = 2 * tid - (tid & (stride - 1));
                const int hi = lo + stride;
                const bool desc = (lo & size) == 0;
                const bool lo_first = ck[lo] > ck[hi] || (ck[lo] == ck[hi] && ci[lo] < ci[hi]);
                if (lo_first != desc) {
                    const unsigned tk = ck[lo]; ck[lo] = ck[hi]; ck[hi] = tk;
                    const int ti = ci[lo]; ci[lo] = ci[hi]; ci[hi] = ti;
                }
            }
            __syncthreads();
        }
    for (int i = tid; i < K; i += n) {
        out_ids[(size_t)blockIdx.x * K + i] = ci[i];
        out_vals[(size_t)blockIdx.x * K + i] = row[ci[i]];
    }
}

// The same selection for long rows by a cluster of eight CTAs: each CTA reads an eighth of the row
// once and keeps its keys in shared memory; the histograms of the radix passes meet in CTA 0's
// shared memory (distributed shared memory: remote atomics and stores), which picks the bin; the
// candidates are written into CTA 0's arrays, ties at the K-th key in ascending id order (the CTAs'
// slices are consecutive id ranges); CTA 0 sorts and stores.  One pass over global memory
// instead of six by one CTA.
// The bin in which the need-th largest key lies, by one warp: lane l owns the 8 bins 255 - 8 l ... 248 - 8 l
// (counted from the top); returns the bin and leaves in `need` how many keys are wanted from it.
__device__ __forceinline__ int select_bin_warp(const int* hist, int& need) {
    const int lane = threadIdx.x & 31, top = 255 - 8 * lane;
    int c[8], mine = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) c[j] = hist[top - j], mine += c[j];
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    const int before = incl - mine;                       // keys in the bins above this lane's
    const bool here = before < need && incl >= need;
    const unsigned who = __ballot_sync(0xffffffffu, here);
    int bin = 0, left = 0;
    if (who == 0u) {                                      // fewer keys than wanted (cannot happen for K <= V): the lowest bin
        bin = 0, left = need;
    } else if (here) {
        left = need - before;
        int j = 0;
        for (; j < 7; ++j) {
            if (c[j] >= left) break;
            left -= c[j];
        }
        bin = top - j;
    }
    const int src = who == 0u ? 0 : __ffs(who) - 1;
    bin = __shfl_sync(0xffffffffu, bin, src), left = __shfl_sync(0xffffffffu, left, src);
    need = left;
    return bin;
}

// Exclusive prefix sum of one value per thread over a block of 1024 threads; `total` gets the sum.
__device__ __forceinline__ int block_exclusive_scan_1024(int v, int* warp_sums, int& total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += u;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        const int w = warp_sums[lane];
        int wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int u = __shfl_up_sync(0xffffffffu, wi, o);
            if (lane >= o) wi += u;
        }
        warp_sums[lane] = wi - w;
        if (lane == 31) warp_sums[32] = wi;
    }
    __syncthreads();
    total = warp_sums[32];
    return warp_sums[warp] + incl - v;
}

constexpr int TOPK_CLUSTER = 8;
constexpr int TOPK_CLUSTER_MIN_V = 8192;                 // shorter rows: one CTA does as well
constexpr int TOPK_CLUSTER_MAX_SLICE = 48 * 1024;        // keys of a slice (192 KB of shared memory)

__global__ void __cluster_dims__(TOPK_CLUSTER, 1, 1) __launch_bounds__(1024, 1)
    topk_pool_cluster_kernel(const float* logits, int V, int K, int slice, int* out_ids, float* out_vals) {
    pdl_enter();
    namespace cg = cooperative_groups;
    extern __shared__ unsigned keys[];
    __shared__ int hist[256];
    __shared__ unsigned s_prefix;
    __shared__ int s_need, s_count;
    __shared__ unsigned ck[POOL_MAX];
    __shared__ int ci[POOL_MAX];
    __shared__ int seg_eq[1024];
    __shared__ int cta_eq[TOPK_CLUSTER];
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank(), tid = threadIdx.x, n = blockDim.x;
    const float* row = logits + (size_t)(blockIdx.x / TOPK_CLUSTER) * V;
    const int i0 = rank * slice, cnt = max(0, min(V, i0 + slice) - i0);
    // CTA 0's copies are the cluster's
    int* l_hist = cluster.map_shared_rank(hist, 0);
    unsigned* l_prefix = cluster.map_shared_rank(&s_prefix, 0);
    int* l_need = cluster.map_shared_rank(&s_need, 0);
    int* l_count = cluster.map_shared_rank(&s_count, 0);
    unsigned* l_ck = cluster.map_shared_rank(ck, 0);
    int* l_ci = cluster.map_shared_rank(ci, 0);
    int* l_cta_eq = cluster.map_shared_rank(cta_eq, 0);

    for (int i = tid; i < cnt; i += n) keys[i] = key_of(row[i0 + i]);
    if (tid == 0) s_prefix = 0u, s_need = K, s_count = 0;
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        const unsigned himask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
        if (tid < 256) hist[tid] = 0;
        cluster.sync();                                  // histograms are empty, the prefix of the pass before is out
        const unsigned prefix = *l_prefix;
        // logits share their leading bits: the lanes of a warp that hit the same bin add once, together
        for (int i0w = 0; i0w < cnt; i0w += n) {
            const int i = i0w + tid;
            int bin = -1;
            if (i < cnt) {
                const unsigned k = keys[i];
                if ((k & himask) == prefix) bin = (int)((k >> shift) & 255);
            }
            const unsigned same = __match_any_sync(0xffffffffu, bin);
            if (bin >= 0 && (tid & 31) == __ffs(same) - 1) atomicAdd(&hist[bin], __popc(same));
        }
        __syncthreads();
        if (rank != 0 && tid < 256 && hist[tid] != 0) atomicAdd(&l_hist[tid], hist[tid]);
        cluster.sync();                                  // CTA 0's histogram holds the whole row
        if (rank == 0 && tid < 32) {
            int need = s_need;
            const int b = select_bin_warp(hist, need);
            if (tid == 0) s_need = need, s_prefix = prefix | ((unsigned)b << shift);
        }
        __syncthreads();                                 // the bin is chosen before the histogram is cleared again
    }
    cluster.sync();
    const unsigned kth = *l_prefix;
    const int need_eq = *l_need;
    // strictly greater: any order (sorted below)
    for (int i = tid; i < cnt; i += n) {
        const unsigned k = keys[i];
        if (k > kth) {
            const int at = atomicAdd(l_count, 1);
            if (at < POOL_MAX) l_ck[at] = k, l_ci[at] = i0 + i;
        }
    }
    // equal: the lowest ids.  Thread t owns a contiguous run of this CTA's slice.
    const int seg = (cnt + n - 1) / n;
    const int b0 = min(cnt, tid * seg), b1 = min(cnt, b0 + seg);
    int mine = 0;
    for (int i = b0; i < b1; ++i) mine += keys[i] == kth;
    int eq_total;
    const int eq_before = block_exclusive_scan_1024(mine, seg_eq, eq_total);
    if (tid == 0) l_cta_eq[rank] = eq_total;
    cluster.sync();                                      // every greater key is in, every CTA's count of equal keys is known
    const int gt = *l_count;
    int r = eq_before;
    for (int c = 0; c < rank; ++c) r += l_cta_eq[c];
    for (int i = b0; i < b1 && r < need_eq; ++i)
        if (keys[i] == kth) {
            if (gt + r < POOL_MAX) l_ck[gt + r] = kth, l_ci[gt + r] = i0 + i;
            ++r;
        }
    cluster.sync();                                      // nothing is written into CTA 0's memory after this
    if (rank != 0) return;
    for (int i = tid; i < POOL_MAX; i += n)
        if (i >= K) ck[i] = 0u, ci[i] = 0x7fffffff;
    __syncthreads();
    for (int size = 2; size <= POOL_MAX; size <<= 1)
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            if (tid < POOL_MAX / 2) {
                const int lo = 2 * tid - (tid & (stride - 1));
                const int hi = lo + stride;
                const bool desc = (lo & size) == 0;
                const bool lo_first = ck[lo] > ck[hi] || (ck[lo] == ck[hi] && ci[lo] < ci[hi]);
                if (lo_first != desc) {
                    const unsigned tk = ck[lo]; ck[lo] = ck[hi]; ck[hi] = tk;
                    const int ti = ci[lo]; ci[lo] = ci[hi]; ci[hi] = ti;
                }
            }
            __syncthreads();
        }
    const size_t out0 = (size_t)(blockIdx.x / TOPK_CLUSTER) * K;
    for (int i = tid; i < K; i += n) {
        out_ids[out0 + i] = ci[i];
        out_vals[out0 + i] = row[ci[i]];
    }
}

}  // namespace

Q6K_API int q6k_argmax_scratch_ints(int rows, int V) { return 2 * rows * ((V + ARGMAX_SLICE - 1) / ARGMAX_SLICE); }

// scratch: q6k_argmax_scratch_ints(rows, V) 32-bit words.
Q6K_API int q6k_argmax(const float* logits, int rows, int V, int* out, void* scratch, cudaStream_t st) {
    if (rows == 0) return 0;
    Q6K_REQUIRE(rows > 0 && V > 0 && rows <= 65535, "argmax: bad sizes rows=%d V=%d", rows, V);
    const int slices = (V + ARGMAX_SLICE - 1) / ARGMAX_SLICE;
    unsigned* pk = (unsigned*)scratch;
    int* pi = (int*)scratch + (size_t)rows * slices;
    q6k_launch(argmax_partial_kernel, dim3(slices, rows), 256, 0, st, logits, V, slices, pk, pi);
    q6k_launch(argmax_final_kernel, rows, 32, 0, st, pk, pi, slices, out);
    return q6k_check_launch("argmax");
}

namespace {
// lse[row] = log(sum_i exp(logits[row, i])) and picked[row] = logits[row, target[row]]: what a perplexity needs of a row
// of logits (reference: the row log-sum-exp of crates/cuda/kernels/topk.cu:181-198).  One block per row; the maximum
// first, then the sum of the exponentials around it, the warps' sums added in warp order.
__global__ void __launch_bounds__(1024) row_lse_kernel(const float* logits, int V, const int* target,
                                                       float* lse, float* picked) {
    pdl_enter();
    __shared__ float red[32];
    const float* row = logits + (size_t)blockIdx.x * V;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, row[i]);
    mx = warp_max(mx);
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = red[0];
    for (int w = 1; w < warps; ++w) mx = fmaxf(mx, red[w]);
    __syncthreads();
    float sum = 0.0f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) sum += expf(row[i] - mx);
    sum = warp_sum(sum);
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.0f;
        for (int w = 0; w < warps; ++w) total += red[w];
        lse[blockIdx.x] = mx + logf(total);
        if (target) picked[blockIdx.x] = row[target[blockIdx.x]];
    }
}
}  // namespace

// logits: FP32 [rows, V]; lse: FP32 [rows]; target (int32 [rows], ids in 0..V-1) and picked (FP32 [rows]) together or both null.
Q6K_API int q6k_row_lse(const float* logits, int rows, int V, const int* target, float* lse, float* picked, cudaStream_t st) {
    if (rows == 0) return 0;
    Q6K_REQUIRE(rows > 0 && V > 0 && (!target == !picked), "row_lse: bad sizes rows=%d V=%d, or only one of target and picked", rows, V);
    q6k_launch(row_lse_kernel, rows, V >= 8192 ? 1024 : 256, 0, st, logits, V, target, lse, picked);
    return q6k_check_launch("row_lse");
}

// ids: int32 [rows, K], vals: FP32 [rows, K], sorted by (logit descending, id ascending).
Q6K_API int q6k_topk_pool(const float* logits, int rows, int V, int K, int* ids, float* vals, cudaStream_t st) {
    if (rows == 0) return 0;
    Q6K_REQUIRE(rows > 0 && V > 0, "topk_pool: bad sizes rows=%d V=%d", rows, V);
    Q6K_REQUIRE(K >= 1 && K <= POOL_MAX && K <= V, "topk_pool: K=%d outside 1..min(%d, V=%d)", K, POOL_MAX, V);
    const int slice = ((V + TOPK_CLUSTER - 1) / TOPK_CLUSTER + 3) & ~3;
    if (V >= TOPK_CLUSTER_MIN_V && slice <= TOPK_CLUSTER_MAX_SLICE && (long long)rows * TOPK_CLUSTER <= 0x7fffffffLL) {
        const size_t smem = (size_t)slice * sizeof(unsigned);
        static bool configured = false;
        if (!configured) {
            if (cudaFuncSetAttribute(topk_pool_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)(TOPK_CLUSTER_MAX_SLICE * sizeof(unsigned))) != cudaSuccess)
                return q6k_check_launch("topk_pool: shared memory attribute");
            configured = true;
        }
        q6k_launch(topk_pool_cluster_kernel, rows * TOPK_CLUSTER, 1024, smem, st, logits, V, K, slice, ids, vals);
        return q6k_check_launch("topk_pool");
    }
    q6k_launch(topk_pool_kernel, rows, 1024, 0, st, logits, V, K, ids, vals);
    return q6k_check_launch("topk_pool");
}

// ---------------------------------------------------------------------------------------------
// The choice of a token from a row's pool on the device, for requests without penalties: the same
// arithmetic as the host's (crates/cli/src/flint.rs:384-431 in the reference; q6k_sample_rows in
// the host library): p_i = exp((l_i - l_0) / temperature) in double precision from a 32-bit quotient,
// p_i < min_p dropped, the shortest prefix whose normalised mass reaches top_p, the CDF inverted with
// u * total by plain running sums.  The pool comes sorted from topk_pool_kernel.  One block per row:
// every thread one exponential, thread 0 the sums.
namespace {

struct SampleRow {                  // 32 bytes per row, written by the host
    int size, top_k;                // candidates to consider (<= 0: leave the row's output alone); 0: the whole pool
    float temperature, top_p, min_p;
    int pad;
    double u;                       // the request's next uniform in [0, 1)
};

__global__ void __launch_bounds__(POOL_MAX) sample_pool_kernel(const int* ids, const float* vals, int stride,
                                                               const SampleRow* rows, int* out) {
    pdl_enter();
    __shared__ double probs[POOL_MAX];
    const int row = blockIdx.x, tid = threadIdx.x;
    const SampleRow r = rows[row];
    const int n = min(r.size, stride);
    if (n <= 0) return;
    ids += (size_t)row * stride, vals += (size_t)row * stride;
    if (r.temperature <= 0.0f || r.top_k == 1 || n == 1) {
        if (tid == 0) out[row] = ids[0];
        return;
    }
    const int keep = r.top_k == 0 ? n : min(r.top_k, n);
    const float top = vals[0];
    if (tid < keep) {
        double q = exp((double)((vals[tid] - top) / r.temperature));
        if (r.min_p > 0.0f && q < (double)r.min_p) q = 0.0;
        probs[tid] = q;
    }
    __syncthreads();
    if (tid != 0) return;
    double total = 0.0;
    for (int i = 0; i < keep; ++i) total += probs[i];
    int cut = keep;
    if (r.top_p < 1.0f) {
        double acc = 0.0;
        for (int i = 0; i < keep; ++i) {
            acc += probs[i] / total;
            if (acc >= (double)r.top_p) {
                cut = i + 1;
                break;
            }
        }
    }
    total = 0.0;
    for (int i = 0; i < cut; ++i) total += probs[i];
    double left = r.u * total;
    int pick = cut - 1;
    for (int i = 0; i < cut; ++i) {
        left -= probs[i];
        if (left <= 0.0) {
            pick = i;
            break;
        }
    }
    out[row] = ids[pick];
}

}  // namespace

// ids / vals: what q6k_topk_pool wrote ([rows, K], sorted); params: [rows] records of 32 bytes on the device
// {int32 size, int32 top_k, float temperature, float top_p, float min_p, int32 unused, double u}; out: int32 [rows].
Q6K_API int q6k_sample_pool(const int* ids, const float* vals, int rows, int K, const void* params, int* out, cudaStream_t st) {
    if (rows == 0) return 0;
    Q6K_REQUIRE(rows > 0 && K >= 1 && K <= POOL_MAX, "sample_pool: bad sizes rows=%d K=%d", rows, K);
    Q6K_REQUIRE(((uintptr_t)params & 7) == 0, "sample_pool: the rows' records must start on 8 bytes");
    static_assert(sizeof(SampleRow) == 32, "the host writes records of 32 bytes");
    q6k_launch(sample_pool_kernel, rows, POOL_MAX, 0, st, ids, vals, K, (const SampleRow*)params, out);
    return q6k_check_launch("sample_pool");
}

// ---------------------------------------------------------------------------------------------
// The variant that allocates nothing (see no_alloc.h).  The scratch of the two-pass argmax sits in
// the library's device image; host code may not use the array's name as a device pointer, so the
// address is fetched once per device and handed to the kernels.
namespace {

constexpr int NOALLOC_SLICES = (Q6K_NOALLOC_MAX_VOCAB + ARGMAX_SLICE - 1) / ARGMAX_SLICE;
static __device__ __align__(256) unsigned g_noalloc_scratch[2 * Q6K_NOALLOC_MAX_ROWS * NOALLOC_SLICES];

constexpr int NOALLOC_MAX_DEVICES = 64;
void* g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {};       // device address of the array, per device, once looked up

}  // namespace

Q6K_API int q6k_argmax_noalloc(const float* logits, int rows, int vocab, int* out, cudaStream_t st) {
    if (rows == 0) return 0;
    Q6K_REQUIRE(rows > 0 && vocab > 0, "argmax_noalloc: bad sizes rows=%d vocab=%d", rows, vocab);
    Q6K_REQUIRE(rows <= Q6K_NOALLOC_MAX_ROWS, "argmax_noalloc: %d rows exceed the built-in scratch for %d rows", rows, Q6K_NOALLOC_MAX_ROWS);
    Q6K_REQUIRE(vocab <= Q6K_NOALLOC_MAX_VOCAB, "argmax_noalloc: vocabulary %d exceeds the built-in scratch for %d", vocab,
                Q6K_NOALLOC_MAX_VOCAB);
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES)
        return q6k_fail("argmax_noalloc: cannot tell the current device (or its index %d is beyond %d)", dev, NOALLOC_MAX_DEVICES - 1);
    if (!g_noalloc_ptr[dev]) {
        // first call on this device: the symbol's address in this device's copy of the image
        void* ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (e != cudaSuccess || !ptr) return q6k_fail("argmax_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        g_noalloc_ptr[dev] = ptr;
    }
    const int slices = (vocab + ARGMAX_SLICE - 1) / ARGMAX_SLICE;
    unsigned* pk = (unsigned*)g_noalloc_ptr[dev];
    int* pi = (int*)g_noalloc_ptr[dev] + (size_t)rows * slices;
    q6k_launch(argmax_partial_kernel, dim3(slices, rows), 256, 0, st, logits, vocab, slices, pk, pi);
    q6k_launch(argmax_final_kernel, rows, 32, 0, st, pk, pi, slices, out);
    return q6k_check_launch("argmax_noalloc");
}
