// Router scoring with top-k selection, and the token -> expert permutation.
//
// Scoring (FP32 throughout): sigmoid per expert, top-k by score, ties to the lower expert index,
// weights divided by (their sum + 1e-20) (crates/cuda/kernels/flint.cu:829-868); or softmax over
// all experts, top-k, divided by the chosen sum (crates/cuda/kernels/moe.cu:19-71).  NaN scores
// count as 0 so that an expert index is never out of range.  Without renormalisation the chosen
// scores are the weights.
//
// Permutation (reference: count/plan/scatter, flint.cu:1163-1209, which ranks with atomics): here
// the row of a (token, slot) pair inside its expert's group is its rank among the pairs of that
// expert in pair order, so the whole permutation is a pure function of the selection.
#include <cooperative_groups.h>

#include <algorithm>

#include "common.cuh"
#include "tma.cuh"

namespace {

// How a round of the selection works, in registers or in shared memory: the scores are not negative, so their
// bits order like signed integers; a lane finds the largest of its own experts (the first of equal ones: its lowest
// index), one warp reduction gives the largest of all, a second the lowest expert index among the lanes that hold
// it (ties go to the lower expert), and that lane marks its entry as taken (bits -1).

// Top-k of one token's scores by one warp, the scores in registers (lane l holds experts l, l + 32, ...; NL of
// them, E <= 32 NL).  Writes the chosen experts and weights (renormalised if asked).  `total` divides softmax scores.
// also_e (or null): a second place for the chosen experts (shared memory of the caller).
//
// One warp runs this alone (and mostly with a cold instruction cache: the code is kept short).  A round: the lane's
// largest entry by a tree of integer maxima, its index by independent compares, two warp reductions, the winner's
// entry marked.  Scores, their sum and the stores wait until the rounds are over (lane r keeps round r's result).
template <int NL>
__device__ __forceinline__ void warp_topk_regs(float (&val)[NL], int E, int k, int sigmoid, int renorm, float total, int* sel_e, float* sel_w,
                                               int* also_e = nullptr) {
    const int lane = threadIdx.x & 31;
    int bits[NL];
#pragma unroll
    for (int i = 0; i < NL; ++i) bits[i] = lane + 32 * i < E ? __float_as_int(val[i]) : -1;      // -1: no expert / taken
    int my_top = -1, my_e = 0;                           // lane r: the bits of the r-th score and its expert (r < 32)
    for (int r = 0; r < k; ++r) {
        int m[NL];
#pragma unroll
        for (int i = 0; i < NL; ++i) m[i] = bits[i];
#pragma unroll
        for (int w = 1; w < NL; w *= 2)
#pragma unroll
            for (int i = 0; i + w < NL; i += 2 * w) m[i] = max(m[i], m[i + w]);
        const int best = m[0];
        int best_i = 0;
#pragma unroll
        for (int i = NL - 1; i >= 0; --i)                // the first of equal ones: the lane's lowest expert
            if (bits[i] == best) best_i = i;
        const int top = __reduce_max_sync(0xffffffffu, best);
        const int idx = __reduce_min_sync(0xffffffffu, best == top ? lane + 32 * best_i : 0x7fffffff);      // ties: the lower expert
        const bool won = (idx & 31) == lane;
#pragma unroll
        for (int i = 0; i < NL; ++i)
            if (won && i == (idx >> 5)) bits[i] = -1;
        if (lane == (r & 31)) {
            if (r >= 32) {                               // the lane's earlier result makes room (more than 32 per token: rare)
                sel_e[r - 32] = my_e, sel_w[r - 32] = __int_as_float(my_top);
                if (also_e) also_e[r - 32] = my_e;
            }
            my_top = top, my_e = idx;
        }
    }
    __syncwarp();
    // the scores and their sum: rounds lane, lane + 32, ... of this lane, the earlier ones from memory
    const int last = ((k - 1 - lane) >> 5) * 32 + lane;  // this lane's last round (negative: none)
    float part = 0.0f, mine = 0.0f;
    for (int r = lane; r < k; r += 32) {
        const float raw = r == last ? __int_as_float(my_top) : sel_w[r];
        const float score = sigmoid ? raw : raw / total;
        part += score;
        if (r == last) mine = score;
        else sel_w[r] = score;
    }
    const float chosen_sum = warp_sum(part);
    const float den = !renorm ? 1.0f : (sigmoid ? chosen_sum + 1e-20f : chosen_sum);
    for (int r = lane; r < k; r += 32) {
        if (r == last) {
            sel_e[r] = my_e, sel_w[r] = mine / den;
            if (also_e) also_e[r] = my_e;
        } else {
            sel_w[r] /= den;
        }
    }
}

// The same for any number of experts, the scores' bits in shared memory bits[0..E) (lane l looks after l, l + 32, ...).
__device__ __forceinline__ void warp_topk_shared(int* bits, int E, int k, int sigmoid, int renorm, float total, int* sel_e, float* sel_w) {
    const int lane = threadIdx.x & 31;
    float chosen_sum = 0.0f, mine = 0.0f;
    for (int r = 0; r < k; ++r) {
        int best = -1, best_e = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const int b = bits[e];
            if (b > best) best = b, best_e = e;
        }
        const int top = __reduce_max_sync(0xffffffffu, best);
        const int idx = __reduce_min_sync(0xffffffffu, best == top ? best_e : 0x7fffffff);
        if ((idx & 31) == lane) bits[idx] = -1;
        const float best_f = __int_as_float(top);
        const float score = sigmoid ? best_f : best_f / total;
        chosen_sum += score;
        if (lane == 0) sel_e[r] = idx;
        if (lane == r) mine = score;                 // lane r keeps the r-th score (r < 32; later ones: below)
        if (r >= 32 && lane == 0) sel_w[r] = score;
    }
    const float den = !renorm ? 1.0f : (sigmoid ? chosen_sum + 1e-20f : chosen_sum);
    __syncwarp();
    if (lane < k && lane < 32) sel_w[lane] = mine / den;
    if (k > 32 && renorm && lane == 0)
        for (int r = 32; r < k; ++r) sel_w[r] /= den;
}

// One token's scores from its logits (sigmoid, or the numerators of the softmax and their sum), then the top-k.
// z: the logits in global memory (written by other blocks of this kernel: read past L1) or, SHARED, in shared memory.
template <int NL, bool SHARED = false>
__device__ __forceinline__ void warp_route_regs(const float* z, int E, int k, int sigmoid, int renorm, int* sel_e, float* sel_w, int* also_e = nullptr) {
    const int lane = threadIdx.x & 31;
    float val[NL];
#pragma unroll
    for (int i = 0; i < NL; ++i) val[i] = lane + 32 * i < E ? (SHARED ? z[lane + 32 * i] : __ldcg(z + lane + 32 * i)) : -INFINITY;
    float total = 1.0f;
    if (sigmoid) {
#pragma unroll
        for (int i = 0; i < NL; ++i) {
            const float s = 1.0f / (1.0f + expf(-val[i]));
            val[i] = s >= 0.0f ? s : 0.0f;
        }
    } else {
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < NL; ++i) mx = fmaxf(mx, val[i]);
        mx = warp_max(mx);
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < NL; ++i) {
            float s = lane + 32 * i < E ? expf(val[i] - mx) : 0.0f;
            s = s >= 0.0f ? s : 0.0f;
            val[i] = s;
            sum += s;
        }
        total = warp_sum(sum);
    }
    warp_topk_regs<NL>(val, E, k, sigmoid, renorm, total, sel_e, sel_w, also_e);
}

// logits: [slices, T, E]; the slices (split-K partial products of the router) are summed in order first.
__global__ void route_kernel(const float* logits, int slices, size_t slice_stride, int T_, int E, int k, int sigmoid, int renorm, int* sel_e,
                             float* sel_w) {
    pdl_enter();
    extern __shared__ float sc[];             // [warps][E]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= T_) return;
    float* v = sc + (size_t)warp * E;
    const float* z = logits + (size_t)t * E;
    for (int e = lane; e < E; e += 32) v[e] = z[e];
    for (int s = 1; s < slices; ++s)                     // slice by slice: a lane's loads of one slice do not wait for one another
        for (int e = lane; e < E; e += 32) v[e] += z[s * slice_stride + e];
    __syncwarp();
    int* se = sel_e + (size_t)t * k;
    float* sw = sel_w + (size_t)t * k;
    if (E <= 256) return warp_route_regs<8, true>(v, E, k, sigmoid, renorm, se, sw);
    if (E <= 704) return warp_route_regs<22, true>(v, E, k, sigmoid, renorm, se, sw);
    float total = 1.0f;
    if (sigmoid) {
        for (int e = lane; e < E; e += 32) {
            float s = 1.0f / (1.0f + expf(-v[e]));
            v[e] = s >= 0.0f ? s : 0.0f;
        }
    } else {
        float mx = -INFINITY;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, v[e]);
        mx = warp_max(mx);
        float sum = 0.0f;
        for (int e = lane; e < E; e += 32) {
            float s = expf(v[e] - mx);
            s = s >= 0.0f ? s : 0.0f;
            v[e] = s;
            sum += s;
        }
        total = warp_sum(sum);
    }
    __syncwarp();
    warp_topk_shared(reinterpret_cast<int*>(v), E, k, sigmoid, renorm, total, se, sw);
}

// Router of a decode step in one launch (reference: router_kernel, crates/cuda/kernels/flint.cu:1002-1055,
// which routes in the block that finishes last).  Here one cluster of eight CTAs does it all and nothing meets
// through global memory:
//
//   1. every CTA owns an eighth of the experts.  It copies their rows of the router matrix into its shared memory
//      (one bulk copy per row, rows padded so that a quarter warp's 16-byte reads fall into different banks) while
//      the kernel launched before this one still runs: the matrix is older than any kernel of the step.
//   2. after the wait its eight warps split D and multiply their stretches of the rows with the step's activations
//      (at most 16 tokens) on mma.sync, experts as the M side, tokens as the N side, both operands read as 16
//      contiguous bytes per lane (the sum over k may be taken in any order both operands agree on); the warps'
//      sums meet in shared memory and are added in warp order.
//   3. the logits go into CTA 0's shared memory (and to global memory for whoever wants them); after a cluster
//      barrier the other CTAs are done, and in CTA 0 a warp per token scores it and picks its top-k.
//   4. CTA 0 sorts the (token, slot) pairs by expert.
// A model with more experts than fit at once (32 rows of D, or 16) walks them in chunks through a few buffers.
namespace cg = cooperative_groups;
constexpr int SMALL_T = 16;
constexpr int RC_CL = 8;                     // CTAs of the cluster
constexpr int RC_WARPS = 8;
constexpr int RC_MAXBUF = 8;
constexpr int RC_PAIRS = 512;                // pairs whose experts fit CTA 0's array
constexpr size_t RC_SMEM = 200 * 1024;       // what a CTA may use of its shared memory

__device__ int g_router_status = 0;

__host__ __device__ inline int rc_stride(int D) { return D * 2 + (64 + 128 - (D * 2) % 128) % 128; }      // bytes; 64 mod 128
__host__ __device__ inline size_t rc_fixed_bytes(int RB, int NB, int E) {                                  // all but the weight buffers
    return (size_t)RC_WARPS * RB * NB * 128 * sizeof(float) + (size_t)NB * 8 * E * sizeof(float) + RC_PAIRS * sizeof(int) + 128;
}

__device__ __forceinline__ void rc_bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar), "l"(policy)
                 : "memory");
}
__device__ __forceinline__ void rc_mma(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NB: blocks of 8 tokens (1 or 2); RB: blocks of 16 experts per chunk (1 or 2); bufs: weight buffers of a chunk each.
template <int NB, int RB>
__global__ void __cluster_dims__(RC_CL, 1, 1) __launch_bounds__(RC_WARPS * 32, 1)
    router_cluster_kernel(const __nv_bfloat16* xn, const __nv_bfloat16* w, int T_, int E, int D, int k, int sigmoid, int renorm, float* logits,
                          int* sel_e, float* sel_w, int* order, int bufs) {
    pdl_launch();
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    constexpr int CR = RB * 16;                                              // experts of a chunk
    extern __shared__ __align__(128) uint8_t rc_smem[];
    const int stride = rc_stride(D);
    uint8_t* wbuf = rc_smem;                                                 // [bufs][CR][stride]
    float* meet = reinterpret_cast<float*>(rc_smem + (size_t)bufs * CR * stride);      // [warps][RB * NB * 128]
    float* lg_all = meet + RC_WARPS * RB * NB * 128;                         // [8 NB][E]: CTA 0's holds every token's logits
    int* pair_e = reinterpret_cast<int*>(lg_all + NB * 8 * E);               // [RC_PAIRS]: the pairs' experts (CTA 0)
    __shared__ __align__(8) uint64_t bars[RC_MAXBUF];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, quad = lane >> 2, pair = lane & 3;
    const int per = (E + RC_CL - 1) / RC_CL, e_begin = min(E, rank * per), n_rows = min(E, e_begin + per) - e_begin;
    const int chunks = (n_rows + CR - 1) / CR;
    if (threadIdx.x == 0) {
        for (int b = 0; b < bufs; ++b) mbar_init(smem_u32(&bars[b]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // chunk c into buffer c % bufs: warp 0, a row per lane (the matrix is read once a step)
    const uint64_t once = l2_evict_first_policy();
    auto stage = [&](int c) {
        const int rows_here = min(CR, n_rows - c * CR), b = c % bufs;
        const uint32_t bar = smem_u32(&bars[b]);
        if (lane == 0) mbar_expect_tx(bar, (uint32_t)rows_here * D * 2);
        __syncwarp();
        for (int r = lane; r < rows_here; r += 32)
            rc_bulk_copy(smem_u32(wbuf + ((size_t)b * CR + r) * stride), w + (size_t)(e_begin + c * CR + r) * D, (uint32_t)D * 2, bar, once);
    };
    if (warp == 0)
        for (int c = 0; c < chunks && c < bufs; ++c) stage(c);
    // another CTA's shared memory may be written once that CTA runs: every CTA says so here, and listens below
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    pdl_wait();                               // the activations, and the outputs' last readers
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    const __nv_bfloat16* xrow[NB];
    bool live[NB];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
        live[nb] = nb * 8 + quad < T_;
        xrow[nb] = xn + (size_t)(live[nb] ? nb * 8 + quad : 0) * D + pair * 8;
    }
    float* lg_zero = cluster.map_shared_rank(lg_all, 0);
    bool ok = true;
    for (int c = 0; c < chunks; ++c) {
        const int b = c % bufs, rows_here = min(CR, n_rows - c * CR);
        if (ok && !mbar_wait(smem_u32(&bars[b]), (c / bufs) & 1)) {
            if (threadIdx.x == 0) atomicExch(&g_router_status, 1);
            ok = false;                       // nothing more is computed; the barriers below are still kept
        }
        float acc[RB][NB][4];
#pragma unroll
        for (int rb = 0; rb < RB; ++rb)
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) acc[rb][nb][0] = acc[rb][nb][1] = acc[rb][nb][2] = acc[rb][nb][3] = 0.0f;
        const uint8_t* wb = wbuf + (size_t)b * CR * stride;
        // a warp's stretches of 128 k, two at a time: all their activations are asked for before the first product
        for (int k0 = warp * 128; ok && k0 < D; k0 += 2 * RC_WARPS * 128) {
            uint4 bx[2][NB][4];
#pragma unroll
            for (int s2 = 0; s2 < 2; ++s2)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int kk = k0 + s2 * RC_WARPS * 128 + j * 32 + pair * 8;      // this lane's eight elements of k
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb) bx[s2][nb][j] = kk < D && live[nb] ? ld_after_wait(xrow[nb] + kk - pair * 8) : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
            for (int s2 = 0; s2 < 2; ++s2) {
                uint4 a[RB][2][4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int kk = k0 + s2 * RC_WARPS * 128 + j * 32 + pair * 8;
#pragma unroll
                    for (int rb = 0; rb < RB; ++rb)
#pragma unroll
                        for (int h = 0; h < 2; ++h)   // rows past the chunk's last hold whatever the buffer held: their sums are dropped;
                                                      // D is a multiple of 8: a lane's 16 bytes are inside or outside as a whole
                            a[rb][h][j] = kk < D ? *reinterpret_cast<const uint4*>(wb + (size_t)(rb * 16 + quad + 8 * h) * stride + kk * 2) : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                    for (int rb = 0; rb < RB; ++rb)
#pragma unroll
                        for (int nb = 0; nb < NB; ++nb) {
                            const uint4 lo = a[rb][0][j], hi = a[rb][1][j], t = bx[s2][nb][j];
                            rc_mma(acc[rb][nb], lo.x, hi.x, lo.y, hi.y, t.x, t.y);
                            rc_mma(acc[rb][nb], lo.z, hi.z, lo.w, hi.w, t.z, t.w);
                        }
            }
        }
#pragma unroll
        for (int rb = 0; rb < RB; ++rb)
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                for (int i = 0; i < 4; ++i) meet[(size_t)warp * (RB * NB * 128) + ((rb * NB + nb) * 4 + i) * 32 + lane] = acc[rb][nb][i];
        __syncthreads();
        // thread -> (row block, token block, element and lane of the fragment): experts quad (+8), tokens 2 pair (+1)
        for (int idx = threadIdx.x; idx < RB * NB * 128; idx += RC_WARPS * 32) {
            const int ln = idx & 31, i = (idx >> 5) & 3, nb = (idx >> 7) % NB, rb = (idx >> 7) / NB;
            const int row = rb * 16 + (ln >> 2) + 8 * (i >> 1), t = nb * 8 + 2 * (ln & 3) + (i & 1);
            if (row >= rows_here || t >= T_) continue;
            float z = 0.0f;
#pragma unroll
            for (int q = 0; q < RC_WARPS; ++q) z += meet[(size_t)q * (RB * NB * 128) + idx];      // warps in order: a fixed sum
            const int e = e_begin + c * CR + row;
            logits[(size_t)t * E + e] = z;
            lg_zero[t * E + e] = z;
        }
        __syncthreads();                      // meet and the buffer are free again
        if (warp == 0 && c + bufs < chunks) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");          // the reads above, before the copy overwrites them
            stage(c + bufs);
        }
    }
    cluster.sync();                           // every token's logits are in CTA 0; nothing is written into its memory after this
    if (rank != 0) return;
    for (int t = warp; t < T_; t += RC_WARPS) {
        const float* z = lg_all + (size_t)t * E;
        if (E <= 256) warp_route_regs<8, true>(z, E, k, sigmoid, renorm, sel_e + (size_t)t * k, sel_w + (size_t)t * k, pair_e + t * k);
        else warp_route_regs<22, true>(z, E, k, sigmoid, renorm, sel_e + (size_t)t * k, sel_w + (size_t)t * k, pair_e + t * k);
    }
    if (T_ == 1 && k <= 32) {
        // one token: its warp sorts the pairs by itself (a pair's place is the number of pairs with a lower expert)
        if (warp != 0) return;
        __syncwarp();
        if (lane < k) {
            const int e = pair_e[lane];
            int rnk = 0;
            for (int q = 0; q < k; ++q) rnk += pair_e[q] < e;                // a token's experts differ
            order[rnk] = lane;
        }
        return;
    }
    __syncthreads();
    // pairs sorted by expert (stable): tiles of one expert run side by side and share its weights in L2.  A pair's
    // place is the number of pairs with a lower expert, or the same expert and a lower index.  `share` lanes count
    // for one pair, each over its part of the pairs.
    const int pairs = T_ * k;
    int share = 1;
    while (share < 32 && pairs * share * 2 <= (int)blockDim.x) share *= 2;
    for (int base = 0; base < pairs; base += blockDim.x / share) {
        const int p = base + threadIdx.x / share, sub = threadIdx.x % share;
        int rnk = 0;
        if (p < pairs) {
            const int e = pair_e[p];
            for (int q = sub; q < pairs; q += share) {
                const int eq = pair_e[q];
                rnk += (eq < e) || (eq == e && q < p);
            }
        }
        for (int o = share >> 1; o > 0; o >>= 1) rnk += __shfl_xor_sync(0xffffffffu, rnk, o);
        if (p < pairs && sub == 0) order[rnk] = p;
    }
}

constexpr int PERM_CHUNK = 1024;           // pairs per chunk of the permutation kernels

// One warp per (expert, chunk of pairs): how many pairs of the chunk chose the expert.
__global__ void count_kernel(const int* sel_e, int pairs, int E, int* counts) {
    pdl_enter();
    const int lane = threadIdx.x & 31;
    const int e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), c = blockIdx.y;
    if (e >= E) return;
    const int lo = c * PERM_CHUNK, hi = min(pairs, lo + PERM_CHUNK);
    int n = 0;
    for (int p0 = lo; p0 < hi; p0 += 32) {
        const int p = p0 + lane;
        n += __popc(__ballot_sync(0xffffffffu, p < hi && sel_e[p] == e));
    }
    if (lane == 0) counts[c * E + e] = n;
}

// The same counts by one block per chunk, a thread per pair, with each pair's rank among the earlier pairs of its
// chunk that chose the same expert (local[p]; the order is the order of the pairs, so the permutation stays the
// deterministic one): lanes with the same expert find one another with match.any, the warps' counts per expert
// stand in shared memory ([32][E] bytes, a warp has at most 32 pairs), a pair adds those of the warps before its own.
constexpr int COUNT_RANK_MAX_E = 1024;
__global__ void __launch_bounds__(PERM_CHUNK) count_rank_kernel(const int* sel_e, int pairs, int E, int* counts,
                                                                int* local) {
    pdl_enter();
    extern __shared__ unsigned char warp_cnt[];          // [32][E]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, c = blockIdx.x;
    for (int i = tid; i < 8 * E; i += PERM_CHUNK) reinterpret_cast<unsigned*>(warp_cnt)[i] = 0u;      // 32 E bytes
    __syncthreads();
    const int p = c * PERM_CHUNK + tid;
    const int e = p < pairs ? sel_e[p] : -1;
    const unsigned same = __match_any_sync(0xffffffffu, e);
    const int in_warp = __popc(same & ((1u << lane) - 1u));
    if (e >= 0 && in_warp == 0) warp_cnt[warp * E + e] = (unsigned char)__popc(same);
    __syncthreads();
    if (e >= 0) {
        int before = in_warp;
        for (int w = 0; w < warp; ++w) before += warp_cnt[w * E + e];
        local[p] = before;
    }
    for (int x = tid; x < E; x += PERM_CHUNK) {
        int n = 0;
#pragma unroll 8
        for (int w = 0; w < 32; ++w) n += warp_cnt[w * E + x];
        counts[c * E + x] = n;
    }
}

// out[r, :] = x[idx[r], :] (rows of vec_per_row 16-byte words), for the path with more experts than count_rank_kernel takes.
__global__ void gather_pairs_kernel(const uint4* x, const int* idx, uint4* out, int vec_per_row) {
    pdl_enter();
    const size_t src = (size_t)idx[blockIdx.x] * vec_per_row, dst = (size_t)blockIdx.x * vec_per_row;
    for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) out[dst + i] = x[src + i];
}

// After the offsets: a pair's row is its expert's offset plus its chunk's first row within the expert plus its
// rank within the chunk (which stands in pair_row); row_token[row] = pair / k.
__global__ void finish_rank_kernel(const int* sel_e, const int* chunk_base, const int* offsets,
                                   int pairs, int k, int E, int* pair_row, int* row_token) {
    pdl_enter();
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= pairs) return;
    const int e = sel_e[p];
    const int row = offsets[e] + chunk_base[(p / PERM_CHUNK) * E + e] + pair_row[p];
    pair_row[p] = row;
    row_token[row] = p / k;
}

// The same with the copy of the pair's input row: out[row, :] = x[pair / k, :] (rows of vec_per_row 16-byte words), a
// block per pair.
__global__ void finish_rank_gather_kernel(const int* sel_e, const int* chunk_base, const int* offsets,
                                          int k, int E, int* pair_row, int* row_token, const uint4* x,
                                          uint4* out, int vec_per_row) {
    pdl_enter();
    const int p = blockIdx.x;
    const int e = sel_e[p];
    const int row = offsets[e] + chunk_base[(p / PERM_CHUNK) * E + e] + pair_row[p];
    __syncthreads();                                     // every thread has read the rank before thread 0 replaces it
    if (threadIdx.x == 0) pair_row[p] = row, row_token[row] = p / k;
    const size_t src = (size_t)(p / k) * vec_per_row, dst = (size_t)row * vec_per_row;
    for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) out[dst + i] = x[src + i];
}

// counts[c, e] -> the chunk's first row within its expert (in place), and offsets = exclusive
// scan over the experts of their totals (E + 1 entries).  One block.
__device__ void tiles_in_block(const int* offsets, int G, int bm, int* tile_group, int* tile_row0, int* num_tiles, int max_tiles);

__global__ void offsets_kernel(int* counts, int chunks, int E, int* offsets, int bm, int* tile_group, int* tile_row0, int* num_tiles,
                               int max_tiles) {
    pdl_enter();
    __shared__ int part[1024];
    const int tid = threadIdx.x, n = blockDim.x;
    const int per = (E + n - 1) / n;
    int sum = 0;
    for (int i = 0; i < per; ++i) {
        const int e = tid * per + i;
        if (e >= E) break;
        int run = 0;
        for (int c0 = 0; c0 < chunks; c0 += 8) {         // eight loads on the way at a time
            int v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = c0 + j < chunks ? counts[(c0 + j) * E + e] : 0;
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (c0 + j < chunks) {
                    counts[(c0 + j) * E + e] = run;
                    run += v[j];
                }
        }
        offsets[e] = run;                      // the expert's total, replaced by its offset below
        sum += run;
    }
    part[tid] = sum;
    __syncthreads();
    if (tid == 0) {
        int run = 0;
        for (int i = 0; i < n; ++i) {
            const int c = part[i];
            part[i] = run;
            run += c;
        }
        offsets[E] = run;
    }
    __syncthreads();
    int run = part[tid];
    for (int i = 0; i < per; ++i) {
        const int e = tid * per + i;
        if (e >= E) break;
        const int total = offsets[e];
        offsets[e] = run;
        run += total;
    }
    if (tile_group != nullptr) {
        __syncthreads();                       // this block's offsets are complete and visible to it
        tiles_in_block(offsets, E, bm, tile_group, tile_row0, num_tiles, max_tiles);
    }
}

// One warp per (expert, chunk): the row of each of its pairs is the expert's offset plus the
// number of earlier pairs of the same expert; row_token[row] = pair / k.
__global__ void rank_kernel(const int* sel_e, const int* chunk_base, const int* offsets, int pairs, int k, int E, int* pair_row,
                            int* row_token) {
    pdl_enter();
    const int lane = threadIdx.x & 31;
    const int e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), c = blockIdx.y;
    if (e >= E) return;
    const int lo = c * PERM_CHUNK, hi = min(pairs, lo + PERM_CHUNK);
    int base = offsets[e] + chunk_base[c * E + e];
    for (int p0 = lo; p0 < hi; p0 += 32) {
        const int p = p0 + lane;
        const bool hit = p < hi && sel_e[p] == e;
        const unsigned mask = __ballot_sync(0xffffffffu, hit);
        if (hit) {
            const int row = base + __popc(mask & ((1u << lane) - 1u));
            pair_row[p] = row;
            row_token[row] = p / k;
        }
        base += __popc(mask);
    }
}

// The list of row tiles of `bm` rows of the groups, made by the block that has just made the offsets
// (the arithmetic of tile_list_kernel of the CUDA-core product file).
__device__ void tiles_in_block(const int* offsets, int G, int bm, int* tile_group, int* tile_row0, int* num_tiles, int max_tiles) {
    __shared__ int base;
    __shared__ int scan[256];
    if (threadIdx.x == 0) base = 0;
    __syncthreads();
    for (int g0 = 0; g0 < G; g0 += blockDim.x) {
        const int g = g0 + threadIdx.x;
        int mine = 0;
        if (g < G) mine = (offsets[g + 1] - offsets[g] + bm - 1) / bm;
        scan[threadIdx.x] = mine;
        __syncthreads();
        if (threadIdx.x == 0) {
            int run = base;
            for (int i = 0; i < (int)blockDim.x; ++i) {
                const int cnt = scan[i];
                scan[i] = run;
                run += cnt;
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

// logits: FP32 [slices, T, E] (slices >= 1: split-K partial products, summed in order).
Q6K_API int q6k_route(const float* logits, int slices, int T_, int E, int k, int sigmoid, int renorm, int* sel_e, float* sel_w,
                      cudaStream_t st) {
    if (T_ == 0) return 0;
    Q6K_REQUIRE(T_ > 0 && E > 0 && k > 0 && k <= E && slices >= 1, "route: bad sizes T=%d E=%d k=%d slices=%d", T_, E, k, slices);
    Q6K_REQUIRE(E <= 8192, "route: %d experts exceed the supported 8192", E);
    const int warps = E <= 2048 ? 4 : 1;
    const size_t smem = (size_t)warps * E * sizeof(float);
    q6k_launch(route_kernel, (T_ + warps - 1) / warps, warps * 32, smem, st, logits, slices, (size_t)T_ * E, T_, E, k, sigmoid, renorm, sel_e,
               sel_w);
    return q6k_check_launch("route");
}

// How the cluster router lays out a step: blocks of 16 experts per chunk (2 where 32 rows of D fit a CTA's shared
// memory beside the rest, else 1, else 0: not supported) and the number of chunk buffers.
static int router_layout(int T_, int E, int D, int* bufs) {
    const int NB = T_ <= 8 ? 1 : 2, per = (E + RC_CL - 1) / RC_CL;
    for (int RB = 2; RB >= 1; --RB) {
        const size_t chunk = (size_t)RB * 16 * rc_stride(D), fixed = rc_fixed_bytes(RB, NB, E);
        if (fixed + chunk > RC_SMEM) continue;
        if (RB == 2 && per <= 16) continue;                                  // an eighth of the experts fits one block of 16
        const int chunks = (per + RB * 16 - 1) / (RB * 16);
        *bufs = (int)std::min<size_t>(std::min(chunks, RC_MAXBUF), (RC_SMEM - fixed) / chunk);
        return RB;
    }
    return 0;
}

// Whether the one-launch decode router takes a step of T tokens with E experts of width D (k of them per token).
Q6K_API int q6k_router_small_supported(int T_, int E, int D, int k) {
    int bufs = 0;
    return T_ > 0 && T_ <= SMALL_T && E > 0 && E <= 704 && k > 0 && k <= E && T_ * k <= RC_PAIRS && D > 0 && D % 8 == 0 &&
           router_layout(T_, E, D, &bufs) > 0;
}

Q6K_API int q6k_router_status() {
    int v = -1;
    if (cudaMemcpyFromSymbol(&v, g_router_status, sizeof v) != cudaSuccess) return -1;
    return v;
}

// xn: bfloat16 [T, D], T <= 16, D a multiple of 8; w: bfloat16 [E, D]; logits: FP32 [T, E] (the router logits, for
// whoever wants them); order: int32 [T*k], the pairs (token * k + slot) sorted by expert, ties in pair order.
Q6K_API int q6k_router_small(const void* xn, const void* w, int T_, int E, int D, int k, int sigmoid, int renorm, float* logits,
                             int* sel_e, float* sel_w, int* order, cudaStream_t st) {
    if (T_ == 0) return 0;
    Q6K_REQUIRE(q6k_router_small_supported(T_, E, D, k), "router_small: %d tokens, %d experts of width %d, %d per token (at most %d tokens, 704 experts, %d pairs)",
                T_, E, D, k, SMALL_T, RC_PAIRS);
    Q6K_REQUIRE(((uintptr_t)xn & 15) == 0 && ((uintptr_t)w & 15) == 0, "router_small: D=%d must be a multiple of 8 and the operands 16-byte aligned", D);
    int bufs = 0;
    const int RB = router_layout(T_, E, D, &bufs), NB = T_ <= 8 ? 1 : 2;
    const size_t smem = (size_t)bufs * RB * 16 * rc_stride(D) + rc_fixed_bytes(RB, NB, E);
#define ROUTER_LAUNCH(NB_, RB_)                                                                                                       \
    do {                                                                                                                              \
        static bool configured = false;                                                                                               \
        if (!configured) {                                                                                                            \
            if (cudaFuncSetAttribute(router_cluster_kernel<NB_, RB_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)RC_SMEM) != cudaSuccess) \
                return q6k_check_launch("router_small: shared memory attribute");                                                     \
            configured = true;                                                                                                        \
        }                                                                                                                             \
        q6k_launch_as(true, router_cluster_kernel<NB_, RB_>, RC_CL, RC_WARPS * 32, smem, st, (const __nv_bfloat16*)xn, (const __nv_bfloat16*)w, T_, E, D, k, \
                      sigmoid, renorm, logits, sel_e, sel_w, order, bufs);                                                            \
    } while (0)
    if (NB == 1 && RB == 1) ROUTER_LAUNCH(1, 1);
    else if (NB == 1) ROUTER_LAUNCH(1, 2);
    else if (RB == 1) ROUTER_LAUNCH(2, 1);
    else ROUTER_LAUNCH(2, 2);
#undef ROUTER_LAUNCH
    return q6k_check_launch("router_small");
}

Q6K_API int q6k_moe_permute_scratch_ints(int pairs, int E) { return ((pairs + PERM_CHUNK - 1) / PERM_CHUNK) * E; }

// scratch: q6k_moe_permute_scratch_ints(pairs, E) ints; offsets: [E+1], pair_row: [pairs], row_token: [pairs]; all int32.
Q6K_API int q6k_moe_permute(const int* sel_e, int pairs, int k, int E, int* scratch, int* offsets, int* pair_row, int* row_token,
                            cudaStream_t st) {
    if (pairs == 0) return 0;
    Q6K_REQUIRE(pairs > 0 && k > 0 && E > 0, "moe_permute: bad sizes pairs=%d k=%d E=%d", pairs, k, E);
    const int chunks = (pairs + PERM_CHUNK - 1) / PERM_CHUNK;
    Q6K_REQUIRE(chunks <= 65535, "moe_permute: %d pairs exceed the grid limit", pairs);
    const dim3 grid((E + 7) / 8, chunks);
    q6k_launch(count_kernel, grid, 256, 0, st, sel_e, pairs, E, scratch);
    q6k_launch(offsets_kernel, 1, 256, 0, st, scratch, chunks, E, offsets, 0, (int*)nullptr, (int*)nullptr, (int*)nullptr, 0);
    q6k_launch(rank_kernel, grid, 256, 0, st, sel_e, scratch, offsets, pairs, k, E, pair_row, row_token);
    return q6k_check_launch("moe_permute");
}

// The permutation and the list of row tiles of bm rows (tile_group, tile_row0: max_tiles entries; num_tiles: 1) in
// three launches (the block that makes the offsets also makes the tile list).
// x != null: the pairs' input rows (row_bytes bytes each, a multiple of 16; x: [pairs / k rows]) are copied into
// gathered[row] by the launch that finishes the ranks.
Q6K_API int q6k_moe_plan(const int* sel_e, int pairs, int k, int E, int* scratch, int* offsets, int* pair_row, int* row_token, int bm,
                         int* tile_group, int* tile_row0, int* num_tiles, int max_tiles, const void* x, void* gathered, int row_bytes,
                         cudaStream_t st) {
    if (pairs == 0) return 0;
    Q6K_REQUIRE(pairs > 0 && k > 0 && E > 0 && bm > 0 && max_tiles > 0, "moe_plan: bad sizes pairs=%d k=%d E=%d bm=%d", pairs, k, E, bm);
    const int chunks = (pairs + PERM_CHUNK - 1) / PERM_CHUNK;
    Q6K_REQUIRE(chunks <= 65535, "moe_plan: %d pairs exceed the grid limit", pairs);
    Q6K_REQUIRE(!x || (gathered && row_bytes > 0 && row_bytes % 16 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)gathered & 15) == 0),
                "moe_plan: rows of %d bytes cannot be gathered (multiples of 16 bytes, 16-byte aligned buffers)", row_bytes);
    if (E <= COUNT_RANK_MAX_E) {
        q6k_launch(count_rank_kernel, chunks, PERM_CHUNK, (size_t)32 * E, st, sel_e, pairs, E, scratch, pair_row);
        q6k_launch(offsets_kernel, 1, 256, 0, st, scratch, chunks, E, offsets, bm, tile_group, tile_row0, num_tiles, max_tiles);
        if (x)
            q6k_launch(finish_rank_gather_kernel, pairs, 128, 0, st, sel_e, scratch, offsets, k, E, pair_row, row_token, (const uint4*)x,
                       (uint4*)gathered, row_bytes / 16);
        else
            q6k_launch(finish_rank_kernel, (pairs + 255) / 256, 256, 0, st, sel_e, scratch, offsets, pairs, k, E, pair_row, row_token);
        return q6k_check_launch("moe_plan");
    }
    const dim3 grid((E + 7) / 8, chunks);
    q6k_launch(count_kernel, grid, 256, 0, st, sel_e, pairs, E, scratch);
    q6k_launch(offsets_kernel, 1, 256, 0, st, scratch, chunks, E, offsets, bm, tile_group, tile_row0, num_tiles, max_tiles);
    q6k_launch(rank_kernel, grid, 256, 0, st, sel_e, scratch, offsets, pairs, k, E, pair_row, row_token);
    if (x) {
        q6k_launch(gather_pairs_kernel, pairs, 128, 0, st, (const uint4*)x, row_token, (uint4*)gathered, row_bytes / 16);
    }
    return q6k_check_launch("moe_plan");
}
