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
#include "common.cuh"

namespace {

// How a round of the selection works, in registers or in shared memory: the scores are not negative, so their
// bits order like signed integers; a lane finds the largest of its own experts (the first of equal ones: its lowest
// index), one warp reduction gives the largest of all, a second the lowest expert index among the lanes that hold
// it (ties go to the lower expert), and that lane marks its entry as taken (bits -1).

// Top-k of one token's scores by one warp, the scores in registers (lane l holds experts l, l + 32, ...; NL of
// them, E <= 32 NL).  Writes the chosen experts and weights (renormalised if asked).  `total` divides softmax scores.
template <int NL>
__device__ __forceinline__ void warp_topk_regs(float (&val)[NL], int E, int k, int sigmoid, int renorm, float total, int* sel_e, float* sel_w) {
    const int lane = threadIdx.x & 31;
    int bits[NL];
#pragma unroll
    for (int i = 0; i < NL; ++i) bits[i] = lane + 32 * i < E ? __float_as_int(val[i]) : -1;      // -1: no expert / taken
    float chosen_sum = 0.0f, mine = 0.0f;
    for (int r = 0; r < k; ++r) {
        int best = -1, best_i = 0;
#pragma unroll
        for (int i = 0; i < NL; ++i)
            if (bits[i] > best) best = bits[i], best_i = i;
        const int top = __reduce_max_sync(0xffffffffu, best);
        const int idx = __reduce_min_sync(0xffffffffu, best == top ? lane + 32 * best_i : 0x7fffffff);      // ties: the lower expert
        if ((idx & 31) == lane) {
#pragma unroll
            for (int i = 0; i < NL; ++i)
                if (i == (idx >> 5)) bits[i] = -1;
        }
        const float best_f = __int_as_float(top);
        const float score = sigmoid ? best_f : best_f / total;
        chosen_sum += score;
        if (lane == 0) sel_e[r] = idx;
        if (lane == r) mine = score;                 // lane r keeps the r-th score (r < 32; later ones: below)
        if (r >= 32 && lane == 0) sel_w[r] = score;
    }
    const float den = !renorm ? 1.0f : (sigmoid ? chosen_sum + 1e-20f : chosen_sum);
    if (lane < k && lane < 32) sel_w[lane] = mine / den;
    if (k > 32 && renorm && lane == 0)
        for (int r = 32; r < k; ++r) sel_w[r] /= den;
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
__device__ __forceinline__ void warp_route_regs(const float* z, int E, int k, int sigmoid, int renorm, int* sel_e, float* sel_w) {
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
    warp_topk_regs<NL>(val, E, k, sigmoid, renorm, total, sel_e, sel_w);
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
// which also routes in its last block).  The logits are a matrix-vector product of at most 16 tokens with the
// [E, D] router matrix: a block of eight warps takes four experts, its warps split D between them (16 bytes per
// lane and row: with D = 2,048 every load of the kernel is in flight at once), each lane multiplies its eight
// weights of four experts with its eight activations of every token, and the 4 x T sums of a warp are brought
// together by a transposing reduction (the lanes halve the set of sums they carry while they double the set of
// lanes summed over: 31 shuffles for 32 sums where one reduction per sum would take 160).  The warps' sums meet
// in shared memory and are added in warp order.  The block that finishes last (atomic ticket, no waiting) scores
// every token, picks its top-k and sorts the (token, slot) pairs by expert.
constexpr int SMALL_T = 16;
constexpr int ROUTER_ROWS = 4;              // experts of a block

// v[0..NV) of every lane -> lane L holds the warp's sum of v[index(L)]; NV a power of two <= 32.  index(L) takes
// its bits from the lane's high bits: for NV = 32 it is L itself, for NV = 8 it is L >> 2 (lanes 0, 4, 8, ... hold sums 0..7).
template <int NV>
__device__ __forceinline__ float transpose_reduce(float (&v)[NV]) {
    const int lane = threadIdx.x & 31;
    int off = 16;
#pragma unroll
    for (int n = NV; n > 1; n >>= 1, off >>= 1) {
        const bool upper = lane & off;
#pragma unroll
        for (int i = 0; i < n / 2; ++i) {
            const float keep = upper ? v[i + n / 2] : v[i], give = upper ? v[i] : v[i + n / 2];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, give, off);
        }
    }
    float r = v[0];
    for (; off > 0; off >>= 1) r += __shfl_xor_sync(0xffffffffu, r, off);
    return r;
}

// TP: the token count rounded up to a power of two (1, 2, 4, 8, 16).
template <int TP>
__global__ void __launch_bounds__(256) router_small_kernel(const __nv_bfloat16* xn, const __nv_bfloat16* __restrict__ w, int T_, int E,
                                                           int D, int k, int sigmoid, int renorm, float* logits, int* sel_e, float* sel_w,
                                                           int* order, unsigned* ticket) {
    // the router matrix is older than any kernel of the step: its rows are asked for while the kernel launched before this
    // one still runs (programmatic dependent launch); the activations wait for that kernel
    pdl_launch();
    bool waited = false;
    constexpr int NV = ROUTER_ROWS * TP;                                  // sums of a warp: index = row * TP + token
    constexpr int PASS = NV > 32 ? 32 : NV;                               // reduced 32 at a time
    __shared__ float meet[8][NV];
    __shared__ int pair_e[SMALL_T * 8 * 4];                               // the last block: the pairs' experts (up to 512 pairs)
    __shared__ int is_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int e0 = blockIdx.x * ROUTER_ROWS;
    {
        float acc[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) acc[i] = 0.0f;
        for (int d0 = (warp * 32 + lane) * 8; d0 < D; d0 += 8 * 256) {
            float wf[ROUTER_ROWS][8];
#pragma unroll
            for (int r = 0; r < ROUTER_ROWS; ++r) {
                const int e = e0 + r < E ? e0 + r : E - 1;                // a ragged last block reads a valid row and drops the sum
                const uint4 wv = *reinterpret_cast<const uint4*>(w + (size_t)e * D + d0);
                const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __bfloat1622float2(w2[i]);
                    wf[r][2 * i] = f.x, wf[r][2 * i + 1] = f.y;
                }
            }
            if (!waited) {
                pdl_wait();
                waited = true;
            }
#pragma unroll
            for (int t = 0; t < TP; ++t) {
                if (t < T_) {
                    const uint4 xv = ld_after_wait(xn + (size_t)t * D + d0);
                    const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 f = __bfloat1622float2(x2[i]);
#pragma unroll
                        for (int r = 0; r < ROUTER_ROWS; ++r) {
                            acc[r * TP + t] = fmaf(f.x, wf[r][2 * i], acc[r * TP + t]);
                            acc[r * TP + t] = fmaf(f.y, wf[r][2 * i + 1], acc[r * TP + t]);
                        }
                    }
                }
            }
        }
        if (!waited) pdl_wait();                                          // a warp without a stride of its own
#pragma unroll
        for (int p0 = 0; p0 < NV; p0 += PASS) {
            float part[PASS];
#pragma unroll
            for (int i = 0; i < PASS; ++i) part[i] = acc[p0 + i];
            const float total = transpose_reduce<PASS>(part);
            constexpr int STEP = 32 / PASS;                               // lanes 0, STEP, 2 STEP, ... hold sums 0, 1, 2, ...
            if (lane % STEP == 0) meet[warp][p0 + lane / STEP] = total;
        }
        __syncthreads();
        if (threadIdx.x < NV) {
            const int r = threadIdx.x / TP, t = threadIdx.x % TP;
            if (t < T_ && e0 + r < E) {
                float z = 0.0f;
#pragma unroll
                for (int wi = 0; wi < 8; ++wi) z += meet[wi][threadIdx.x];       // warps in order: a fixed sum
                logits[(size_t)t * E + e0 + r] = z;
            }
        }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) is_last = atomicAdd(ticket, 1u) == gridDim.x - 1;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    const int pairs = T_ * k;
    const bool sort_here = pairs <= SMALL_T * 8 * 4;          // the pairs' experts fit the shared array: they are sorted from there
    for (int t = warp; t < T_; t += 8) {         // a warp per token, its scores in registers
        const float* z = logits + (size_t)t * E;
        if (E <= 256) warp_route_regs<8>(z, E, k, sigmoid, renorm, sel_e + (size_t)t * k, sel_w + (size_t)t * k);
        else warp_route_regs<22>(z, E, k, sigmoid, renorm, sel_e + (size_t)t * k, sel_w + (size_t)t * k);
        __syncwarp();
        if (sort_here)
            for (int r = lane; r < k; r += 32) pair_e[t * k + r] = sel_e[(size_t)t * k + r];      // this warp's own stores, read back
    }
    // pairs sorted by expert (stable): tiles of one expert run side by side and share its weights in L2.  A pair's
    // place is the number of pairs with a lower expert, or the same expert and a lower index.
    __syncthreads();
    if (sort_here) {
        // `share` lanes count for one pair, each over its part of the pairs
        int share = 1;
        while (share < 32 && pairs * share * 2 <= (int)blockDim.x) share *= 2;
        for (int base = 0; base < pairs; base += blockDim.x / share) {
            const int p = base + threadIdx.x / share, sub = threadIdx.x % share;
            int rank = 0;
            if (p < pairs) {
                const int e = pair_e[p];
                for (int q = sub; q < pairs; q += share) {
                    const int eq = pair_e[q];
                    rank += (eq < e) || (eq == e && q < p);
                }
            }
            for (int o = share >> 1; o > 0; o >>= 1) rank += __shfl_xor_sync(0xffffffffu, rank, o);
            if (p < pairs && sub == 0) order[rank] = p;
        }
    } else {
        for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
            const int e = sel_e[p];
            int rank = 0;
            for (int q = 0; q < pairs; ++q) {
                const int eq = sel_e[q];
                rank += (eq < e) || (eq == e && q < p);
            }
            order[rank] = p;
        }
    }
    if (threadIdx.x == 0) *ticket = 0;          // ready for the next launch
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

// Whether the one-launch decode router takes a step of T tokens with E experts of width D (k of them per token).
Q6K_API int q6k_router_small_supported(int T_, int E, int D, int k) {
    return T_ > 0 && T_ <= SMALL_T && E > 0 && E <= 704 && k > 0 && k <= E && D > 0 && D % 8 == 0;
}

// xn: bfloat16 [T, D], T <= 16, D a multiple of 8; w: bfloat16 [E, D]; logits: FP32 [T, E] scratch;
// ticket: one zeroed 32-bit word that the kernel leaves zeroed.
// order: int32 [T*k], the pairs (token * k + slot) sorted by expert, ties in pair order.
Q6K_API int q6k_router_small(const void* xn, const void* w, int T_, int E, int D, int k, int sigmoid, int renorm, float* logits,
                             int* sel_e, float* sel_w, int* order, unsigned* ticket, cudaStream_t st) {
    if (T_ == 0) return 0;
    Q6K_REQUIRE(q6k_router_small_supported(T_, E, D, k), "router_small: %d tokens, %d experts of width %d, %d per token (at most %d tokens, 704 experts)",
                T_, E, D, k, SMALL_T);
    Q6K_REQUIRE(((uintptr_t)xn & 15) == 0 && ((uintptr_t)w & 15) == 0, "router_small: D=%d must be a multiple of 8 and the operands 16-byte aligned", D);
    const int blocks = (E + ROUTER_ROWS - 1) / ROUTER_ROWS;
#define ROUTER_LAUNCH(TP)                                                                                                            \
    q6k_launch_as(true, router_small_kernel<TP>, blocks, 256, 0, st, (const __nv_bfloat16*)xn, (const __nv_bfloat16*)w, T_, E, D, k, sigmoid, renorm, \
               logits, sel_e, sel_w, order, ticket)
    if (T_ == 1) ROUTER_LAUNCH(1);
    else if (T_ == 2) ROUTER_LAUNCH(2);
    else if (T_ <= 4) ROUTER_LAUNCH(4);
    else if (T_ <= 8) ROUTER_LAUNCH(8);
    else ROUTER_LAUNCH(16);
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
