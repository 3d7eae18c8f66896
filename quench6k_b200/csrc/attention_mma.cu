// bfloat16 attention over the paged cache on tensor cores, for decode rows and prompt portions in
// one launch, with the key range split over CTAs and merged afterwards.
//
// Arithmetic as the reference's attn_kernel / attn_merge_kernel (crates/cuda/kernels/flint.cu:211-561):
// scores in base 2 (scale * log2 e folded in), causal and window mask per row, online softmax per
// key tile, probabilities rounded to bfloat16 before they are summed, sinks in the merge's
// denominator only.  Differences: keys and values come from pages through the block table; a
// launch covers rows of many requests through a tile list; head size and group size are
// parameters (head size 64 or 128 here; other sizes run on the generic kernel).
//
// A tile is up to ROWS = 16 (narrow) or 128 (wide) query rows of one request and one KV head:
// row = token_in_tile * G + head_in_group.  Key tiles hold 64 keys, aligned to multiples of 64 of
// the key index.  Narrow tiles (decode): the 4 warps share the 16 rows and split each key tile
// (16 keys each), then merge their partial softmax states through shared memory.  Wide tiles
// (prompt portions): 8 warps, each owning 16 rows and walking all 64 keys of a tile.
// K and V tiles travel through a ring of shared-memory stages.  With pages of 8 rows or a multiple
// (the usual case) a producer warp brings each page's [rows x 64] boxes in by TMA (tensor maps over
// a layer's K and V pool, 128-byte swizzle, zero fill for keys that have no page; when the pages of
// a key tile have consecutive numbers, which the head-major pool makes contiguous, one box of 64
// keys per half replaces the boxes per page: far fewer TMA operations) and signals
// the four consumer warps through mbarriers (full: transaction bytes; empty: one arrival per
// warp); every wait is bounded and records a code in a status word when it runs out.  With other
// page sizes the consumer warps copy the rows themselves with 16-byte cp.async into two stages.
// Either way the 16-byte chunks are XOR-swizzled by the row, so ldmatrix reads are conflict-free.
#include <climits>
#include <map>
#include <tuple>

#include "common.cuh"
#include "tma.cuh"

namespace {

constexpr int KT = 64;                       // keys per tile
constexpr float LOG2E = 1.4426950408889634f;

struct AttnParams {
    const __nv_bfloat16* q;                  // [T, Hq, HD]
    const __nv_bfloat16* k_pages;            // [Hkv, pages, page_size, HD]
    const __nv_bfloat16* v_pages;
    const int* block_table;                  // [R, max_blocks]
    const float* sinks;                      // [Hq] or null
    __nv_bfloat16* out;                      // [T, Hq*HD]
    float* part_o;                           // [work items, Hkv, rows of a tile, HD]: what each CTA of a split tile found
    float* part_ml;                          // [work items, Hkv, rows of a tile, 2]: its maximum and sum
    const int* work;                         // [n_work, 8] from attention_plan_kernel: one record per CTA column
    const int* tile_plan;                    // [n_tiles, 4]: first row, tokens, splits, first work item
    int n_work;
    int max_blocks, page_size, window, Hq, Hkv, G;
    float scale_log2;
    int pool_rows;                           // rows of the [Hkv * pages * page_size, HD] view of a pool (TMA path)
    int num_pages;                           // pages of a pool (per KV head)
};

__device__ int g_attn_status = 0;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;            // 0 source bytes: the 16 destination bytes become zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t* r, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// ---------------------------------------------------------------------------------------------
// The plan of a launch: which CTA walks which key tiles.  Made on the device from the positions the
// step really has (so a step replayed from a CUDA graph is balanced for its own contexts), once per
// step and window; every layer's launch reads it.
//
// Tile i sees n_i key tiles.  With a budget of n_work CTAs per KV head, every CTA should walk about
// per = sum(n_i) / n_work of them: tile i is split into n_i / per parts (at least one), each of
// ceil(n_i / parts) key tiles.  If the parts do not fit the budget, per grows until they do
// (n_work >= n_tiles, so one part per tile always fits).
// work[w] = {first row, tokens, first position, request, part, parts, first work item, key tiles per part};
// first row -1: no work.  tile_plan[i] = {first row, tokens, parts, first work item}.
constexpr int PLAN_THREADS = 256;

__device__ __forceinline__ int plan_block_sum(int v, int* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();                          // red may still be read from the call before
    if (lane == 0) red[warp] = v;
    __syncthreads();
    int t = 0;
#pragma unroll
    for (int w = 0; w < PLAN_THREADS / 32; ++w) t += red[w];
    return t;
}

__global__ void __launch_bounds__(PLAN_THREADS) attention_plan_kernel(const int* __restrict__ positions, const int* __restrict__ req_of_token,
                                                                       const int* __restrict__ tile_tok0, const int* __restrict__ tile_ntok,
                                                                       int n_tiles, int window, int n_work, int min_per, int* __restrict__ work,
                                                                       int* __restrict__ tile_plan) {
    pdl_enter();
    __shared__ int red[PLAN_THREADS / 32];
    __shared__ int scan[PLAN_THREADS];
    const int tid = threadIdx.x;
    const int chunk = (n_tiles + PLAN_THREADS - 1) / PLAN_THREADS, i0 = tid * chunk, i1 = min(n_tiles, i0 + chunk);
    auto key_tiles = [&](int i) {
        const int tok0 = tile_tok0[i], first = positions[tok0], last = first + tile_ntok[i] - 1;
        const int k_lo = window > 0 ? max(0, first - window + 1) : 0;
        return last / KT + 1 - k_lo / KT;
    };
    long long mine = 0;
    for (int i = i0; i < i1; ++i) mine += key_tiles(i);
    const int total = plan_block_sum((int)min(mine, (long long)(INT_MAX / PLAN_THREADS)), red);      // clamped: the block's sum cannot overflow
    int per = max(max(1, min_per), (total + n_work - 1) / n_work);
    for (int round = 0; round < 64; ++round) {
        int parts = 0;
        for (int i = i0; i < i1; ++i) parts += max(1, key_tiles(i) / per);
        if (plan_block_sum(parts, red) <= n_work) break;
        per = round < 62 ? per + per / 4 + 1 : INT_MAX / 2;      // in the end one part per tile, which fits
    }
    int parts_mine = 0;
    for (int i = i0; i < i1; ++i) parts_mine += max(1, key_tiles(i) / per);
    __syncthreads();
    scan[tid] = parts_mine;
    __syncthreads();
    for (int o = 1; o < PLAN_THREADS; o <<= 1) {                  // inclusive scan over the threads' chunks
        const int v = tid >= o ? scan[tid - o] : 0;
        __syncthreads();
        scan[tid] += v;
        __syncthreads();
    }
    int at = scan[tid] - parts_mine;
    const int used = scan[PLAN_THREADS - 1];
    for (int i = i0; i < i1; ++i) {
        const int n = key_tiles(i), room = max(1, n / per);
        const int each = (n + room - 1) / room, parts = (n + each - 1) / each;       // parts <= room
        const int tok0 = tile_tok0[i], ntok = tile_ntok[i];
        reinterpret_cast<int4*>(tile_plan)[i] = make_int4(tok0, ntok, parts, at);
        const int first = positions[tok0], req = req_of_token[tok0];
        for (int s = 0; s < room; ++s) {
            int4* w = reinterpret_cast<int4*>(work) + 2 * (size_t)(at + s);
            w[0] = make_int4(s < parts ? tok0 : -1, ntok, first, req);
            w[1] = make_int4(s, parts, at, each);
        }
        at += room;
    }
    for (int w = used + tid; w < n_work; w += PLAN_THREADS) {
        reinterpret_cast<int4*>(work)[2 * (size_t)w] = make_int4(-1, 0, 0, 0);
        reinterpret_cast<int4*>(work)[2 * (size_t)w + 1] = make_int4(0, 1, 0, 1);
    }
}

// Byte offset of 16-byte chunk c of row r in a swizzled [rows][HD] bf16 tile (the Q tile).
template <int HD> __device__ __forceinline__ uint32_t sw(int r, int c) { return (uint32_t)(r * HD * 2 + ((c ^ (r & 7)) << 4)); }
// Byte offset of chunk c of key r in a K or V tile: [HD/64 column halves][64 keys][128 bytes], the
// layout TMA's 128-byte swizzle produces for boxes that start on multiples of 8 keys.
__device__ __forceinline__ uint32_t swk(int r, int c) { return (uint32_t)((c >> 3) * (KT * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4)); }

template <int HD, bool WIDE, bool TMA>
__global__ void __launch_bounds__((WIDE ? 8 : 4) * 32 + (TMA ? 32 : 0)) attention_mma_kernel(const __grid_constant__ CUtensorMap tm_k,
                                                                        const __grid_constant__ CUtensorMap tm_v,
                                                                        const __grid_constant__ CUtensorMap tm_k_run,
                                                                        const __grid_constant__ CUtensorMap tm_v_run, const AttnParams p) {
    pdl_enter();
    constexpr int CW = WIDE ? 8 : 4;         // consumer warps
    constexpr int CT = CW * 32;              // consumer threads
    constexpr int ROWS = WIDE ? 128 : 16;
    constexpr int CH = HD / 8;               // 16-byte chunks per row
    constexpr int KW = WIDE ? KT : 16;       // keys of a tile this warp handles
    constexpr int NB = KW / 8;               // score n-blocks per warp
    constexpr int DB = HD / 8;               // output n-blocks
    constexpr uint32_t TILE_BYTES = KT * HD * 2;
    constexpr int STAGES = TMA ? (HD == 128 ? 3 : 4) : 2;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    // [K stage 0 .. S-1][V stage 0 .. S-1][Q: ROWS x HD]; stages start on 1024 bytes (swizzle pattern)
    const uint32_t k_s = smem_u32(smem), v_s = k_s + STAGES * TILE_BYTES, q_s = v_s + STAGES * TILE_BYTES;
    __shared__ __align__(8) uint64_t bars[8];
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[4]);

    const int kh = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g8 = lane >> 2, t4 = lane & 3;
    const int G = p.G;
    // this CTA's record of the plan: everything about its tile in one load
    const int4 wa = reinterpret_cast<const int4*>(p.work)[2 * (size_t)blockIdx.x];
    const int4 wb = reinterpret_cast<const int4*>(p.work)[2 * (size_t)blockIdx.x + 1];
    const int tok0 = wa.x, ntok = wa.y, pos_first = wa.z, split = wb.x, se = wb.y, per = wb.w;
    if (tok0 < 0) return;
    const int pos_last = pos_first + ntok - 1;
    const int* bt = p.block_table + (size_t)wa.w * p.max_blocks;
    const int k_lo = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
    const int first_tile = k_lo / KT, end_tile = pos_last / KT + 1;
    const int t_begin = first_tile + split * per, t_end = min(end_tile, t_begin + per);
    // where this CTA's partial results go: [work item][KV head][row of the tile]
    const size_t part_row0 = ((size_t)blockIdx.x * p.Hkv + kh) * ROWS;

    // ---- the producer (one thread) brings every tile of this CTA's key range into the ring
    auto issue = [&](int i) {
        const int ps = p.page_size, box = ps < KT ? ps : KT;            // keys per TMA box
        const int s2 = i % STAGES;
        const uint32_t fb = full0 + 8 * s2;
        mbar_expect_tx(fb, 2 * TILE_BYTES);
        const int j0 = (t_begin + i) * KT;
        // pages with consecutive numbers are contiguous for one head: when the tile's pages form
        // such a run, each half comes in as one box of 64 keys instead of one box per page
        bool run = ps < KT && j0 >= k_lo && j0 / ps + KT / ps <= p.max_blocks;
        int first = -1;
        if (run) {
            first = bt[j0 / ps];
            run = first >= 0;
            for (int b = 1; b < KT / ps && run; ++b) run = bt[j0 / ps + b] == first + b;
        }
        if (run) {
            const int y = (kh * p.num_pages + first) * ps;
#pragma unroll
            for (int h = 0; h < HD / 64; ++h) {
                const uint32_t off = s2 * TILE_BYTES + h * (KT * 128);
                tma_load_2d(k_s + off, &tm_k_run, h * 64, y, fb);
                tma_load_2d(v_s + off, &tm_v_run, h * 64, y, fb);
            }
            return;
        }
        for (int b = 0; b < KT / box; ++b) {
            const int j = j0 + b * box;
            int y = p.pool_rows;                                         // out of range: the box is filled with zeros
            if (j + box > k_lo && j <= pos_last) {
                const int page = bt[j / ps];
                if (page >= 0) y = (kh * p.num_pages + page) * ps + j % ps;
            }
#pragma unroll
            for (int h = 0; h < HD / 64; ++h) {
                const uint32_t off = s2 * TILE_BYTES + h * (KT * 128) + b * box * 128;
                tma_load_2d(k_s + off, &tm_k, h * 64, y, fb);
                tma_load_2d(v_s + off, &tm_v, h * 64, y, fb);
            }
        }
    };
    if (TMA && tid == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_k) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_v) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_k_run) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_v_run) : "memory");
    }
    if (TMA && tid == CW * 32) {
        // the first tiles are on their way while the consumers still fetch Q
        for (int s2 = 0; s2 < STAGES; ++s2) {
            mbar_init(full0 + 8 * s2, 1);
            mbar_init(empty0 + 8 * s2, CW);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        for (int i = 0; i < STAGES && i < t_end - t_begin; ++i) issue(i);
    }
    // ---- Q tile into shared memory (zero rows past the tile's tokens)
    if (warp < CW) {
        for (int idx = tid; idx < ROWS * CH; idx += CT) {
            const int r = idx / CH, c = idx % CH, tt = r / G, hg = r % G;
            const bool valid = tt < ntok;
            const __nv_bfloat16* src = p.q + ((size_t)(tok0 + (valid ? tt : 0)) * p.Hq + kh * G + hg) * HD + c * 8;
            cp_async16(q_s + sw<HD>(r, c), src, valid);
        }
    }
    auto load_kv = [&](int stage, int kt) {      // the cp.async path: every consumer thread copies its chunks
        for (int idx = tid; idx < KT * CH; idx += CT) {
            const int r = idx / CH, c = idx % CH, j = kt * KT + r;
            const bool in = j >= k_lo && j <= pos_last;
            int page = in ? bt[j / p.page_size] : -1;
            const bool valid = page >= 0;
            const size_t off = valid ? (((size_t)kh * p.num_pages + page) * p.page_size + j % p.page_size) * HD + c * 8 : 0;
            cp_async16(k_s + stage * TILE_BYTES + swk(r, c), p.k_pages + off, valid);
            cp_async16(v_s + stage * TILE_BYTES + swk(r, c), p.v_pages + off, valid);
        }
    };
    if (!TMA) load_kv(0, t_begin);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();

    if (TMA && warp == CW) {
        if (lane == 0) {
            for (int i = STAGES; i < t_end - t_begin; ++i) {
                if (!mbar_wait(empty0 + 8 * (i % STAGES), ((i / STAGES) & 1) ^ 1)) {
                    atomicExch(&g_attn_status, 1);
                    break;
                }
                issue(i);
            }
        }
        return;
    }

    // this thread's two rows (g8 and g8 + 8 of the warp's 16) and their key limits
    const int rbase = WIDE ? warp * 16 : 0, koff = WIDE ? 0 : warp * 16;
    int lim_hi[2], lim_lo[2];
#pragma unroll
    for (int hr = 0; hr < 2; ++hr) {
        const int r = rbase + g8 + hr * 8, tt = r / G;
        const int pos = pos_first + tt;
        lim_hi[hr] = tt < ntok ? pos : -1;
        lim_lo[hr] = p.window > 0 ? pos - p.window + 1 : 0;
    }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
    float o[DB][4];
#pragma unroll
    for (int n = 0; n < DB; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;

    uint32_t qa[HD / 16][4];
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) ldmatrix_x4(qa[ks], q_s + sw<HD>(rbase + (lane & 15), ks * 2 + (lane >> 4)));

    for (int kt = t_begin; kt < t_end; ++kt) {
        const int it = kt - t_begin, stage = it % STAGES;
        if (TMA) {
            if (!mbar_wait(full0 + 8 * stage, (it / STAGES) & 1)) {
                if (lane == 0) atomicExch(&g_attn_status, 2);
                break;
            }
            if (kt == end_tile - 1 && (pos_last + 1) % KT != 0) {
                // the last page came in whole: rows past the last key hold whatever the page held
                // before (masked scores ignore K, but 0 * V must not meet a stale NaN): clear them
                const int r0 = pos_last + 1 - kt * KT;
                for (int idx = r0 * CH + tid; idx < KT * CH; idx += CT)
                    *reinterpret_cast<uint4*>(smem + (v_s - k_s) + stage * TILE_BYTES + swk(idx / CH, idx % CH)) = make_uint4(0, 0, 0, 0);
                asm volatile("bar.sync 1, %0;" ::"n"(CT) : "memory");
            }
        } else {
            if (kt + 1 < t_end) load_kv(stage ^ 1, kt + 1);
            cp_async_commit();
        }
        const uint32_t kb = k_s + stage * TILE_BYTES, vb = v_s + stage * TILE_BYTES;
        const int j0 = kt * KT + koff;
        // ---- S = Q K^T for this warp's keys
        float s[NB][4];
#pragma unroll
        for (int n = 0; n < NB; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
            for (int nj = 0; nj < NB / 2; ++nj) {
                uint32_t b[4];
                const int key = koff + nj * 16 + ((lane >> 4) << 3) + (lane & 7);
                ldmatrix_x4(b, kb + swk(key, ks * 2 + ((lane >> 3) & 1)));
                mma_bf16(s[2 * nj], qa[ks], b[0], b[1]);
                mma_bf16(s[2 * nj + 1], qa[ks], b[2], b[3]);
            }
        }
        // ---- mask, online softmax
        float mx[2] = {m[0], m[1]};
#pragma unroll
        for (int n = 0; n < NB; ++n)
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const int hr = x >> 1, j = j0 + n * 8 + 2 * t4 + (x & 1);
                const bool ok = j <= lim_hi[hr] && j >= lim_lo[hr];
                s[n][x] = ok ? s[n][x] * p.scale_log2 : -INFINITY;
                mx[hr] = fmaxf(mx[hr], s[n][x]);
            }
        float corr[2];
#pragma unroll
        for (int hr = 0; hr < 2; ++hr) {
            mx[hr] = fmaxf(mx[hr], __shfl_xor_sync(0xffffffffu, mx[hr], 1));
            mx[hr] = fmaxf(mx[hr], __shfl_xor_sync(0xffffffffu, mx[hr], 2));
            corr[hr] = mx[hr] == -INFINITY ? 1.0f : exp2f(m[hr] - mx[hr]);
            m[hr] = mx[hr];
            l[hr] *= corr[hr];
        }
#pragma unroll
        for (int n = 0; n < DB; ++n) o[n][0] *= corr[0], o[n][1] *= corr[0], o[n][2] *= corr[1], o[n][3] *= corr[1];
        uint32_t pa[KW / 16][4];
#pragma unroll
        for (int n = 0; n < NB; ++n) {
            float pr[4];
#pragma unroll
            for (int x = 0; x < 4; ++x) pr[x] = m[x >> 1] == -INFINITY ? 0.0f : exp2f(s[n][x] - m[x >> 1]);
            // rounded to bfloat16 before summing, so that l matches the P that multiplies V
            const __nv_bfloat162 lo2 = __floats2bfloat162_rn(pr[0], pr[1]), hi2 = __floats2bfloat162_rn(pr[2], pr[3]);
            const float2 flo = __bfloat1622float2(lo2), fhi = __bfloat1622float2(hi2);
            l[0] += flo.x + flo.y;
            l[1] += fhi.x + fhi.y;
            pa[n / 2][(n % 2) * 2 + 0] = *reinterpret_cast<const uint32_t*>(&lo2);
            pa[n / 2][(n % 2) * 2 + 1] = *reinterpret_cast<const uint32_t*>(&hi2);
        }
        // ---- O += P V
#pragma unroll
        for (int ks = 0; ks < KW / 16; ++ks) {
#pragma unroll
            for (int dj = 0; dj < DB / 2; ++dj) {
                uint32_t b[4];
                const int key = koff + ks * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
                ldmatrix_x4_trans(b, vb + swk(key, dj * 2 + (lane >> 4)));
                mma_bf16(o[2 * dj], pa[ks], b[0], b[1]);
                mma_bf16(o[2 * dj + 1], pa[ks], b[2], b[3]);
            }
        }
        if (TMA) {
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * stage);
        } else {
            cp_async_wait<0>();
            asm volatile("bar.sync 1, %0;" ::"n"(CT) : "memory");
        }
    }
    // row sums live per thread: add the quad's
#pragma unroll
    for (int hr = 0; hr < 2; ++hr) {
        l[hr] += __shfl_xor_sync(0xffffffffu, l[hr], 1);
        l[hr] += __shfl_xor_sync(0xffffffffu, l[hr], 2);
    }

    // ---- results: (m, l, o) per row; narrow tiles first merge the 4 warps' key subsets
    float* red = reinterpret_cast<float*>(smem);             // reuse the tile ring (all loads have landed, all reads are done)
    if (!WIDE) {
        asm volatile("bar.sync 1, 128;" ::: "memory");         // every consumer warp is past its last tile
        // red: [4 warps][16 rows][HD + 2]
        constexpr int LD = HD + 2;
#pragma unroll
        for (int hr = 0; hr < 2; ++hr) {
            float* dst = red + ((size_t)warp * 16 + g8 + hr * 8) * LD;
            if (t4 == 0) dst[HD] = m[hr], dst[HD + 1] = l[hr];
#pragma unroll
            for (int n = 0; n < DB; ++n) {
                dst[n * 8 + 2 * t4] = o[n][hr * 2];
                dst[n * 8 + 2 * t4 + 1] = o[n][hr * 2 + 1];
            }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        // 128 threads: row = tid / 8, 8 threads share a row's HD values
        const int r = tid >> 3, sub = tid & 7, tt = r / G, hg = r % G;
        if (tt >= ntok) return;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, red[((size_t)w * 16 + r) * LD + HD]);
        float wgt[4], L = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = red[((size_t)w * 16 + r) * LD + HD];
            wgt[w] = mw == -INFINITY ? 0.0f : exp2f(mw - M);
            L += wgt[w] * red[((size_t)w * 16 + r) * LD + HD + 1];
        }
        const size_t row = (size_t)(tok0 + tt) * p.Hq + kh * G + hg;
        float osc = 1.0f, den = L;
        if (se == 1 && p.sinks) {
            const float sk = p.sinks[kh * G + hg] * LOG2E, Mx = fmaxf(M, sk);
            osc = exp2f(M - Mx);
            den = L * osc + exp2f(sk - Mx);
        }
        for (int d = sub; d < HD; d += 8) {
            float acc = 0.0f;
#pragma unroll
            for (int w = 0; w < 4; ++w) acc += wgt[w] * red[((size_t)w * 16 + r) * LD + d];
            if (se == 1) p.out[row * HD + d] = __float2bfloat16_rn(acc * osc / den);
            else p.part_o[(part_row0 + r) * HD + d] = acc;
        }
        if (se > 1 && sub == 0) {
            p.part_ml[(part_row0 + r) * 2] = M;
            p.part_ml[(part_row0 + r) * 2 + 1] = L;
        }
    } else {
#pragma unroll
        for (int hr = 0; hr < 2; ++hr) {
            const int r = rbase + g8 + hr * 8, tt = r / G, hg = r % G;
            if (tt >= ntok) continue;
            const size_t row = (size_t)(tok0 + tt) * p.Hq + kh * G + hg;
            if (se == 1) {
                float osc = 1.0f, den = l[hr];
                if (p.sinks) {
                    const float sk = p.sinks[kh * G + hg] * LOG2E, Mx = fmaxf(m[hr], sk);
                    osc = exp2f(m[hr] - Mx);
                    den = l[hr] * osc + exp2f(sk - Mx);
                }
                const float inv = osc / den;
#pragma unroll
                for (int n = 0; n < DB; ++n)
                    *reinterpret_cast<uint32_t*>(p.out + row * HD + n * 8 + 2 * t4) = pack_bf16(o[n][hr * 2] * inv, o[n][hr * 2 + 1] * inv);
            } else {
                float* po = p.part_o + (part_row0 + r) * HD;
#pragma unroll
                for (int n = 0; n < DB; ++n) *reinterpret_cast<float2*>(po + n * 8 + 2 * t4) = make_float2(o[n][hr * 2], o[n][hr * 2 + 1]);
                if (t4 == 0) {
                    p.part_ml[(part_row0 + r) * 2] = m[hr];
                    p.part_ml[(part_row0 + r) * 2 + 1] = l[hr];
                }
            }
        }
    }
}

// out[row] = sum_s 2^(m_s - M) o_s / (sum_s 2^(m_s - M) l_s + 2^(sink - M)); one block per (tile, KV head, row of
// the tile).  A thread owns four head dimensions of every GROUPS-th split, so that the many splits
// of a long context at a small batch are fetched side by side; the groups' sums meet in shared
// memory and are added in group order (a fixed order for a given number of splits).
constexpr int MERGE_THREADS = 256;
template <int HD>
__global__ void __launch_bounds__(MERGE_THREADS) attention_merge_kernel(const AttnParams p) {
    pdl_enter();
    constexpr int LPR = HD / 4;                   // threads that cover one row of HD values
    constexpr int GROUPS = MERGE_THREADS / LPR;
    __shared__ float red[32];
    __shared__ float4 acc_s[GROUPS][LPR];
    __shared__ float den_s[GROUPS];
    const int tile = blockIdx.x, kh = blockIdx.y, r = blockIdx.z, G = p.G;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int4 tp = reinterpret_cast<const int4*>(p.tile_plan)[tile];
    const int tok0 = tp.x, ntok = tp.y, se = tp.z;
    const int tt = r / G, hg = r % G;
    if (tt >= ntok || se == 1) return;        // one part: the attention kernel wrote the output itself
    const size_t row = (size_t)(tok0 + tt) * p.Hq + kh * G + hg;
    // the parts of a tile are consecutive work items: from one part to the next it is a whole [Hkv, rows] block
    const size_t rows_t = gridDim.z, first = ((size_t)tp.w * p.Hkv + kh) * rows_t + r;
    const size_t ml_step = (size_t)p.Hkv * rows_t * 2, po_step = (size_t)p.Hkv * rows_t * HD;
    const float* ml = p.part_ml + first * 2;
    const float* po = p.part_o + first * HD;
    const float sk = p.sinks ? p.sinks[kh * G + hg] * LOG2E : -INFINITY;
    // every load of the first round goes out before the maximum is known: the values and the
    // (m, l) pairs do not depend on it
    constexpr int U = 4;
    const int g = tid / LPR, c = tid % LPR;
    float2 v0[U];
    float4 o0[U];
#pragma unroll
    for (int j = 0; j < U; ++j) {
        const int s = g + j * GROUPS;
        if (s < se) {
            v0[j] = *reinterpret_cast<const float2*>(ml + s * ml_step);
            o0[j] = *reinterpret_cast<const float4*>(po + s * po_step + c * 4);
        }
    }
    float M = sk;
    for (int s = tid; s < se; s += MERGE_THREADS) M = fmaxf(M, ml[s * ml_step]);
    M = warp_max(M);
    if (lane == 0) red[warp] = M;
    __syncthreads();
#pragma unroll
    for (int w = 0; w < MERGE_THREADS / 32; ++w) M = fmaxf(M, red[w]);
    float4 num = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float den = 0.0f;
    auto take = [&](const float2 v, const float4 o) {
        const float w = v.x == -INFINITY ? 0.0f : exp2f(v.x - M);
        den = fmaf(w, v.x == -INFINITY ? 0.0f : v.y, den);
        num.x = fmaf(w, o.x, num.x), num.y = fmaf(w, o.y, num.y), num.z = fmaf(w, o.z, num.z), num.w = fmaf(w, o.w, num.w);
    };
#pragma unroll
    for (int j = 0; j < U; ++j)
        if (g + j * GROUPS < se) take(v0[j], o0[j]);
    for (int s0 = g + U * GROUPS; s0 < se; s0 += U * GROUPS) {
        float2 v[U];
        float4 o[U];
#pragma unroll
        for (int j = 0; j < U; ++j) {
            const int s = s0 + j * GROUPS;
            if (s < se) {
                v[j] = *reinterpret_cast<const float2*>(ml + s * ml_step);
                o[j] = *reinterpret_cast<const float4*>(po + s * po_step + c * 4);
            }
        }
#pragma unroll
        for (int j = 0; j < U; ++j)
            if (s0 + j * GROUPS < se) take(v[j], o[j]);
    }
    acc_s[g][c] = num;
    if (c == 0) den_s[g] = den;
    __syncthreads();
    if (tid < LPR) {
        float4 t = acc_s[0][tid];
        float d = (p.sinks ? exp2f(sk - M) : 0.0f) + den_s[0];
#pragma unroll
        for (int q = 1; q < GROUPS; ++q) {
            const float4 u = acc_s[q][tid];
            t.x += u.x, t.y += u.y, t.z += u.z, t.w += u.w;
            d += den_s[q];
        }
        const float inv = 1.0f / d;
        __nv_bfloat162 lo = __floats2bfloat162_rn(t.x * inv, t.y * inv), hi = __floats2bfloat162_rn(t.z * inv, t.w * inv);
        uint2 pk;
        pk.x = *reinterpret_cast<uint32_t*>(&lo), pk.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p.out + row * HD + tid * 4) = pk;
    }
}

// Tensor maps over the K and V pools of a layer do not change: keep them by (address, rows, box).
std::mutex g_pool_mutex;
std::map<std::tuple<const void*, long long, int, int>, CUtensorMap> g_pool_maps;

int pool_map(CUtensorMap* out, const void* base, long long rows, int hd, int box_rows) {
    std::lock_guard<std::mutex> lock(g_pool_mutex);
    auto key = std::make_tuple(base, rows, hd, box_rows);
    auto it = g_pool_maps.find(key);
    if (it == g_pool_maps.end()) {
        CUtensorMap m;
        if (int rc = make_bf16_map(&m, base, rows, hd, hd, box_rows, true, "attention_mma")) return rc;
        it = g_pool_maps.emplace(key, m).first;
    }
    *out = it->second;
    return 0;
}

template <int HD, bool WIDE, bool TMA>
int launch(const AttnParams& p, const CUtensorMap* maps, int n_tiles, cudaStream_t st) {
    constexpr int ROWS = WIDE ? 128 : 16;
    constexpr int STAGES = TMA ? (HD == 128 ? 3 : 4) : 2;
    const size_t ring = 2 * STAGES * KT * HD * 2 + ROWS * HD * 2;
    const size_t red = WIDE ? 0 : 4 * 16 * (HD + 2) * sizeof(float);
    const size_t smem = (ring > red ? ring : red) + 1024;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attention_mma_kernel<HD, WIDE, TMA>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return q6k_check_launch("attention_mma: shared memory attribute");
        configured = true;
    }
    q6k_launch(attention_mma_kernel<HD, WIDE, TMA>, dim3(p.n_work, p.Hkv), (WIDE ? 8 : 4) * 32 + (TMA ? 32 : 0), smem, st, maps[0], maps[1], maps[2], maps[3], p);
    if (int rc = q6k_check_launch("attention_mma")) return rc;
    if (p.n_work > n_tiles) {                 // some tile may have more than one part
        q6k_launch(attention_merge_kernel<HD>, dim3(n_tiles, p.Hkv, ROWS), MERGE_THREADS, 0, st, p);
        return q6k_check_launch("attention_merge");
    }
    return 0;
}

template <int HD>
int launch_hd(const AttnParams& p, const CUtensorMap* maps, bool wide, bool tma, int n_tiles, cudaStream_t st) {
    if (tma) return wide ? launch<HD, true, true>(p, maps, n_tiles, st) : launch<HD, false, true>(p, maps, n_tiles, st);
    return wide ? launch<HD, true, false>(p, maps, n_tiles, st) : launch<HD, false, false>(p, maps, n_tiles, st);
}

}  // namespace

// Rows per tile for a group size: 16 (narrow) or 128 (wide) query rows hold rows/G tokens.
Q6K_API int q6k_attention_mma_supported(int hd, int G, int wide) { return (hd == 64 || hd == 128) && G >= 1 && G <= (wide ? 128 : 16); }

Q6K_API int q6k_attention_status() {
    int v = -1;
    if (cudaMemcpyFromSymbol(&v, g_attn_status, sizeof v) != cudaSuccess) return -1;
    return v;
}

// The plan of a step's launches for one tile list and window: tiles are tile_tok0/tile_ntok [n_tiles] (first row and
// token count, consecutive positions of one request); work: int32 [n_work, 8], tile_plan: int32 [n_tiles, 4], both
// 16-byte aligned; n_work >= n_tiles CTAs per KV head share the key tiles, none walking fewer than min_per unless
// its tile has no more.
Q6K_API int q6k_attention_plan(const int* positions, const int* req_of_token, const int* tile_tok0, const int* tile_ntok, int n_tiles,
                               int window, int n_work, int min_per, int* work, int* tile_plan, cudaStream_t st) {
    if (n_tiles == 0) return 0;
    Q6K_REQUIRE(n_work >= n_tiles && window >= 0 && min_per >= 1, "attention_plan: %d work items for %d tiles (window %d, at least %d key tiles each)",
                n_work, n_tiles, window, min_per);
    Q6K_REQUIRE(((uintptr_t)work & 15) == 0 && ((uintptr_t)tile_plan & 15) == 0, "attention_plan: the plan's arrays must start on 16 bytes");
    q6k_launch(attention_plan_kernel, 1, PLAN_THREADS, 0, st, positions, req_of_token, tile_tok0, tile_ntok, n_tiles, window, n_work, min_per,
               work, tile_plan);
    return q6k_check_launch("attention_plan");
}

// q: bfloat16 [T, Hq, hd]; pages: bfloat16 [Hkv, num_pages, page_size, hd] (num_pages: pages in each pool; the TMA path
// addresses a pool as one [Hkv * num_pages * page_size, hd] matrix); work / tile_plan: what q6k_attention_plan made for
// these tiles (of at most (wide ? 128 : 16) / G tokens each) and this window; part_o: FP32 [n_work * Hkv * rows * hd],
// part_ml: FP32 [n_work * Hkv * rows * 2] with rows = wide ? 128 : 16 (unused when n_work == n_tiles).
Q6K_API int q6k_attention_mma(const void* q, const void* k_pages, const void* v_pages, long long num_pages, const int* block_table,
                              int max_blocks, int page_size, const int* work, const int* tile_plan, int n_work, int n_tiles, int wide,
                              int window, const float* sinks, float scale, void* out, float* part_o, float* part_ml, int Hq, int Hkv,
                              int hd, cudaStream_t st) {
    if (n_tiles == 0) return 0;
    Q6K_REQUIRE(Hq > 0 && Hkv > 0 && Hq % Hkv == 0, "attention_mma: bad head counts Hq=%d Hkv=%d", Hq, Hkv);
    const int G = Hq / Hkv;
    Q6K_REQUIRE(q6k_attention_mma_supported(hd, G, wide), "attention_mma: head_dim %d / group size %d is not covered by the tensor-core kernel", hd, G);
    Q6K_REQUIRE(page_size > 0 && max_blocks > 0 && window >= 0 && n_work >= n_tiles && work && tile_plan,
                "attention_mma: bad page_size %d / max_blocks %d / window %d / %d work items for %d tiles", page_size, max_blocks, window, n_work, n_tiles);
    Q6K_REQUIRE(n_work == n_tiles || (part_o && part_ml), "attention_mma: splitting the keys needs the partial buffers");
    Q6K_REQUIRE(Hkv <= 65535 && n_tiles <= 65535, "attention_mma: grid limit exceeded (Hkv=%d, tiles=%d)", Hkv, n_tiles);
    AttnParams p{};
    p.q = (const __nv_bfloat16*)q, p.k_pages = (const __nv_bfloat16*)k_pages, p.v_pages = (const __nv_bfloat16*)v_pages;
    p.block_table = block_table, p.sinks = sinks, p.out = (__nv_bfloat16*)out;
    p.work = work, p.tile_plan = tile_plan, p.n_work = n_work;
    p.part_o = part_o, p.part_ml = part_ml;
    p.max_blocks = max_blocks, p.page_size = page_size, p.window = window, p.Hq = Hq, p.Hkv = Hkv, p.G = G;
    p.scale_log2 = scale * LOG2E;
    // pages of 8, 16, 32, 64 keys (or whole multiples of 64) are boxes TMA can place on the swizzle pattern
    p.num_pages = (int)num_pages;
    const long long pool_rows = num_pages * Hkv * page_size;
    const bool tma = page_size % 8 == 0 && (KT % page_size == 0 || page_size % KT == 0) && pool_rows < (1LL << 31) &&
                     ((uintptr_t)k_pages & 15) == 0 && ((uintptr_t)v_pages & 15) == 0;
    CUtensorMap maps[4] = {};                  // K and V by the page, K and V by the run of 64 keys
    if (tma) {
        const int box = page_size < KT ? page_size : KT;
        p.pool_rows = (int)pool_rows;
        if (int rc = pool_map(&maps[0], k_pages, pool_rows, hd, box)) return rc;
        if (int rc = pool_map(&maps[1], v_pages, pool_rows, hd, box)) return rc;
        if (int rc = pool_map(&maps[2], k_pages, pool_rows, hd, KT)) return rc;
        if (int rc = pool_map(&maps[3], v_pages, pool_rows, hd, KT)) return rc;
    }
    return hd == 128 ? launch_hd<128>(p, maps, wide, tma, n_tiles, st) : launch_hd<64>(p, maps, wide, tma, n_tiles, st);
}
