// bfloat16 attention over the paged cache on tensor cores (mma.sync), for decode rows and prompt
// portions in one launch, with the key range split over CTAs and merged afterwards.
//
// The arithmetic is the reference's (crates/cuda/kernels/flint.cu:211-561 computes the same
// quantities): scores in base 2 (scale * log2 e folded in), causal and window mask per row, online
// softmax per key tile, probabilities rounded to bfloat16 before they are summed, sinks in the
// last denominator only.  How it is computed is this file's own: keys and values come from pages
// through the block table; a launch covers rows of many requests through a tile list and a plan
// made on the device; the keys are the M side of both products (see the kernel's comment); head
// size and group size are parameters (head size 64 or 128 here; other sizes run on the generic
// kernel).
//
// A tile is up to 8 or 16 (narrow) or 128 (wide) query rows of one request and one KV head:
// row = token_in_tile * G + head_in_group.  Key tiles hold 64 keys, aligned to multiples of 64 of
// the key index, and travel through a ring of shared-memory stages that a producer warp fills.
// With pages of 8 keys or a multiple (the usual case) it brings each page's [keys x 64] boxes in by
// TMA (tensor maps over a layer's K and V pool, 128-byte swizzle, zero fill for keys that have no
// page; when the pages of a key tile have consecutive numbers, which the head-major pool makes
// contiguous, one box of 64 keys per half replaces the boxes per page: far fewer TMA operations);
// with other page sizes its lanes copy 16-byte chunks with cp.async into the same XOR-swizzled
// layout.  Either way a stage is handed over through mbarriers (full: transaction bytes or the
// copies' arrivals; empty: one arrival per warp that read it); every wait is bounded and records
// a code in a status word when it runs out.
#include <climits>
#include <map>
#include <tuple>

#include "common.cuh"
#include "tma.cuh"

namespace {

constexpr int KT = 64;                       // keys per tile
constexpr int PREP_TOKENS = 8;               // tokens of a tile whose q and keys the kernel can make itself
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
    int early;                               // the plan, the block tables and every key before a tile's first position are older than the
                                             // kernel launched before this one: key tiles may be fetched before the wait for it
    int pool_rows;                           // rows of the [Hkv * pages * page_size, HD] view of a pool (TMA path)
    int num_pages;                           // pages of a pool (per KV head)
    // Narrow tiles may prepare q and the new keys themselves (qkv != null; q is then unused): what the kernel in
    // qk_prep.cu does, folded in.  qkv: FP32 [qkv_splits, T, qkv_ld], q heads | k heads | v heads in a row; the slices
    // (split-K partial products, qkv_split_stride floats apart) are summed in order.
    const float* qkv;
    long long qkv_split_stride;
    int qkv_splits;
    const float* q_norm;                     // [HD] or null
    const float* k_norm;
    const float* inv_freq;                   // [rd / 2] or null: pairs by halves, rd a multiple of 64
    float eps;
    int qkv_ld, rd;
    int write_kv;                            // the new keys and values are made here and written to the pages
};

__device__ int g_attn_status = 0;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;            // 0 source bytes: the 16 destination bytes become zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

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

__global__ void __launch_bounds__(PLAN_THREADS) attention_plan_kernel(const int* positions, const int* req_of_token,
                                                                       const int* tile_tok0, const int* tile_ntok,
                                                                       int n_tiles, int window, int n_work, int min_per, int* work,
                                                                       int* tile_plan) {
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

// Byte offset of chunk c (16 bytes: 8 head dimensions) of key r in a K or V stage: [HD/64 column halves][64 keys][128 bytes],
// the layout TMA's 128-byte swizzle produces for boxes that start on multiples of 8 keys.
__device__ __forceinline__ uint32_t swk(int r, int c) { return (uint32_t)((c >> 3) * (KT * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4)); }

// Transpose of an 8x8 matrix of 16-bit values held one row per four lanes (the mma fragment layout).
__device__ __forceinline__ uint32_t transpose_8x8(uint32_t v) {
    uint32_t r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
    return r;
}

// ---------------------------------------------------------------------------------------------
// The attention kernel.  Keys are the M side of the tensor-core products, query rows the N side:
//
//   S^T [64 keys x NQ rows]  = K [64 x HD] . Q^T [HD x NQ]        (mma.m16n8k16: four key blocks of 16, NQ/8 row blocks)
//   O^T [HD x NQ]           += V^T [HD x 64] . P^T [64 x NQ]      (HD/16 blocks of head dimensions, the same row blocks)
//
// so a decode step's handful of rows (one token of a group of 8 query heads: NQ = 8) fills the
// narrow side of the instruction exactly and nothing is padded to 16 rows, and K and V are the
// operands that come straight from shared memory by ldmatrix (V transposed on the way).  The
// softmax runs down the key axis: a thread holds, of every key block, two keys for two rows; a
// row's maximum over the tile takes three shuffles over the lanes that hold the other keys.  The
// probabilities leave the first product as an accumulator fragment [keys x rows] and enter the
// second as its B operand [keys x rows] in the other fragment layout: movmatrix transposes the 8x8
// blocks in registers, nothing goes through shared memory.
//
// One warp runs a whole [64 keys x NQ rows] tile by itself with its own running maximum, sum and O^T.
// Narrow tiles (NQ rows of one request and KV head: decode): the four consumer warps take the key
// tiles of the CTA's range in turn (tile i belongs to warp i mod 4) and never wait for one another
// for a tile's arithmetic until the end, where their four states are combined through the then idle ring.  Wide tiles
// (128 rows: prompt portions): eight consumer warps own 16 rows each and all walk every key tile.
// A producer warp keeps the ring of K/V stages full: by TMA (one elected lane; pages of 8 keys or
// a multiple) or, for other page sizes, with 16-byte cp.async copies by all its lanes that arrive
// on the same full barriers (cp.async.mbarrier.arrive), so the consumers are the same either way.
template <int HD, int NQ, bool WIDE, bool TMA>
__global__ void __launch_bounds__((WIDE ? 8 : 4) * 32 + 32, WIDE ? 1 : 2) attention_mma_kernel(const __grid_constant__ CUtensorMap tm_k,
                                                                                 const __grid_constant__ CUtensorMap tm_v,
                                                                                 const __grid_constant__ CUtensorMap tm_k_run,
                                                                                 const __grid_constant__ CUtensorMap tm_v_run, const AttnParams p) {
    // Narrow tiles hold all the tokens a request brings to the step, so every key before the tile's first position was
    // written by an earlier step: the producer fetches those key tiles while the kernel launched before this one (the
    // one that writes this step's keys and q) still runs, and only then waits for it (programmatic dependent launch;
    // the plan and the block tables are older than that kernel too).  Wide tiles wait first, like any other kernel.
    const bool EARLY = !WIDE && p.early != 0;
    if (EARLY) pdl_launch();
    else pdl_enter();
    constexpr int CW = WIDE ? 8 : 4;         // consumer warps
    constexpr int ROWS = WIDE ? 128 : NQ;    // query rows of the CTA's tile
    constexpr int NB = NQ / 8;               // row blocks (n = 8) of a warp
    constexpr int KB = KT / 16;              // key blocks (m = 16) of a key tile
    constexpr int DB = HD / 16;              // blocks of head dimensions (k = 16 of the first product, m = 16 of the second)
    constexpr int CH = HD / 8;               // 16-byte chunks per key
    constexpr uint32_t TILE_BYTES = KT * HD * 2;
    constexpr int STAGES = HD == 128 ? 3 : 4;
    static_assert(NQ == 8 || NQ == 16, "a warp's tile has 8 or 16 query rows");
    static_assert(!WIDE || NQ == 16, "wide tiles are eight warps of 16 rows");
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    // [K stage 0 .. S-1][V stage 0 .. S-1]; stages start on 1024 bytes (swizzle pattern)
    const uint32_t k_s = smem_u32(smem), v_s = k_s + STAGES * TILE_BYTES;
    __shared__ __align__(8) uint64_t bars[8];
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[4]);

    const int kh = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = p.G;
    // this CTA's record of the plan: everything about its tile in one load
    const int4 wa = reinterpret_cast<const int4*>(p.work)[2 * (size_t)blockIdx.x];
    const int4 wb = reinterpret_cast<const int4*>(p.work)[2 * (size_t)blockIdx.x + 1];
    const int tok0 = wa.x, ntok = wa.y, pos_first = wa.z, part = wb.x, parts = wb.y, per = wb.w;
    if (tok0 < 0) return;
    const int pos_last = pos_first + ntok - 1;
    const int* bt = p.block_table + (size_t)wa.w * p.max_blocks;
    const int k_lo = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;        // first key any row of the tile sees
    const int first_tile = k_lo / KT, end_tile = pos_last / KT + 1;
    const int t_begin = first_tile + part * per, n_mine = max(0, min(end_tile, t_begin + per) - t_begin);

    // ------------------------------------------------------------------ the producer warp
    if (warp == CW) {
        if (lane == 0) {
            for (int s = 0; s < STAGES; ++s) {
                mbar_init(full0 + 8 * s, TMA ? 1 : 32);
                mbar_init(empty0 + 8 * s, CW);
            }
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
    }
    __syncthreads();                          // the only block-wide barrier before the warps part ways
    if (warp == CW) {
        const int ps = p.page_size;
        if (TMA && lane != 0) return;         // one elected lane issues the TMA loads; the copies of the other path take all 32
        bool waited = !EARLY;
        // a launch that makes the new keys itself finds only keys of earlier steps in the pages: nothing there is the
        // work of the kernel before this one (the rows of this step's positions are replaced in shared memory)
        const bool makes_kv = !WIDE && p.qkv != nullptr && p.write_kv;
        const uint64_t once = l2_evict_first_policy();                       // a step reads a key once
        // The boxes of the key tile that starts at key j0: emit(K map, V map, x, y, byte offset in a stage) for each.
        // Pages with consecutive numbers are contiguous for one head: when the tile's pages form such a run, each
        // half comes in as one box of 64 keys instead of one box per page.
        auto boxes = [&](int j0, auto&& emit) {
            const int box = ps < KT ? ps : KT;                                   // keys per box of the per-page maps
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
                for (int h = 0; h < HD / 64; ++h) emit(&tm_k_run, &tm_v_run, h * 64, y, (uint32_t)(h * (KT * 128)));
                return;
            }
            for (int b = 0; b < KT / box; ++b) {
                const int j = j0 + b * box;
                int y = p.pool_rows;                                             // out of range: the box is filled with zeros
                if (j + box > k_lo && j <= pos_last) {
                    const int page = bt[j / ps];
                    if (page >= 0) y = (kh * p.num_pages + page) * ps + j % ps;
                }
#pragma unroll
                for (int h = 0; h < HD / 64; ++h) emit(&tm_k, &tm_v, h * 64, y, (uint32_t)(h * (KT * 128) + b * box * 128));
            }
        };
        for (int i = 0; i < n_mine; ++i) {
            const int st = i % STAGES;
            // the first tiles of the ring need no free stage; of those, the ones that end before this step's first key need no wait
            if (!waited && (i >= STAGES || (!makes_kv && (t_begin + i + 1) * KT > pos_first))) {
                pdl_wait();
                waited = true;
            }
            if (i >= STAGES && !mbar_wait(empty0 + 8 * st, ((i / STAGES) & 1) ^ 1)) {
                if (lane == 0) atomicExch(&g_attn_status, 1);
                return;
            }
            const uint32_t fb = full0 + 8 * st;
            const int j0 = (t_begin + i) * KT;
            if (TMA) {
                mbar_expect_tx(fb, 2 * TILE_BYTES);
                boxes(j0, [&](const CUtensorMap* mk, const CUtensorMap* mv, int x, int y, uint32_t off) {
                    tma_load_2d_once(k_s + st * TILE_BYTES + off, mk, x, y, fb, once);
                    tma_load_2d_once(v_s + st * TILE_BYTES + off, mv, x, y, fb, once);
                });
            } else {
                // every lane copies its share of the tile's chunks; keys outside the tile's range or without a page become zeros
                for (int idx = lane; idx < KT * CH; idx += 32) {
                    const int r = idx / CH, c = idx % CH, j = j0 + r;
                    const int page = (j >= k_lo && j <= pos_last) ? bt[j / ps] : -1;
                    const bool valid = page >= 0;
                    const size_t off = valid ? (((size_t)kh * p.num_pages + page) * ps + j % ps) * HD + c * 8 : 0;
                    cp_async16(k_s + st * TILE_BYTES + swk(r, c), p.k_pages + off, valid);
                    cp_async16(v_s + st * TILE_BYTES + swk(r, c), p.v_pages + off, valid);
                }
                asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(fb) : "memory");
            }
        }
        if (!TMA) cp_async_wait_all();        // nothing of this warp's is in flight when it leaves
        return;
    }

    // ------------------------------------------------------------------ the consumer warps
    // A thread of the fragment layout: quad = lane / 4 names a key (first product's rows) or a head
    // dimension (second product's rows), pair = lane % 4 names two neighbouring query rows.
    const int quad = lane >> 2, pair = lane & 3;
    const int row0 = WIDE ? warp * NQ : 0;                                   // first row of the CTA's tile this warp works on
    const bool prepares = !WIDE && p.qkv != nullptr;                         // q and the new keys are made here
    __nv_bfloat16* stash = reinterpret_cast<__nv_bfloat16*>(smem + 2 * STAGES * TILE_BYTES);      // [PREP_TOKENS][K, V][HD]
    float2* turn = reinterpret_cast<float2*>(stash + PREP_TOKENS * 2 * HD);                       // [PREP_TOKENS][HD / 2]: cosine, sine
    if (prepares && p.inv_freq) {
        // the rotations of the tile's tokens depend on their positions only: made while the kernel before this one still runs
        const int half = p.rd / 2;
        for (int idx = tid; idx < ntok * half; idx += CW * 32) {
            const int tt = idx / half, i = idx % half;
            float sn, cs;
            sincosf((float)(pos_first + tt) * p.inv_freq[i], &sn, &cs);
            turn[tt * (HD / 2) + i] = make_float2(cs, sn);
        }
        asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
    }
    if (EARLY) pdl_wait();                    // q (or the q/k/v product) is the work of the kernel before this one
    // the rows this thread holds in the accumulator fragments: block nb, rows nb*8 + 2*pair + {0, 1}
    int see_to[NB][2], see_from[NB][2];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const int tt = (row0 + nb * 8 + 2 * pair + c) / G, pos = pos_first + tt;
            see_to[nb][c] = tt < ntok ? pos : -1;                            // a row past the tile's tokens sees nothing
            see_from[nb][c] = p.window > 0 ? pos - p.window + 1 : 0;
        }
    // Q^T as the first product's B operand: this thread's row is nb*8 + quad, its head dimensions
    // 16 ks + 2 pair + {0, 1} and + 8
    uint32_t qf[DB][NB][2];
    bool has_new = false;                      // some of the tile's new keys lie in this CTA's key tiles (the same for all its warps)
    if (prepares) {
        // ---- q, and the keys and values of the tile's tokens, from the FP32 product [q | k | v]: per-head RMSNorm,
        // rotation by position * inv_freq (pairs d, d + rd/2), rounding to bfloat16: the arithmetic of qk_prep.cu.
        // Everything a stretch needs is asked of memory at once: one round trip, then arithmetic.
        const int t_end = t_begin + n_mine;
        has_new = p.write_kv && n_mine > 0 && pos_last / KT >= t_begin && pos_first / KT < t_end;
        if (has_new) {
            // a warp per token: lane l holds head dimensions l + 32 i, so both members of a rotating pair sit in one lane
            constexpr int EPL = HD / 32;
            for (int tt = warp; tt < ntok; tt += CW) {
                const int pos = pos_first + tt;
                if (pos / KT < t_begin || pos / KT >= t_end) continue;       // another part's key tile: that CTA makes it
                const int page = bt[pos / p.page_size];
                const float* ksrc = p.qkv + (size_t)(tok0 + tt) * p.qkv_ld + (size_t)(p.Hq + kh) * HD;
                const float* vsrc = ksrc + (size_t)p.Hkv * HD;
                float x[EPL], v[EPL], w[EPL];
#pragma unroll
                for (int i = 0; i < EPL; ++i) x[i] = ksrc[lane + 32 * i], v[i] = vsrc[lane + 32 * i], w[i] = p.k_norm ? p.k_norm[lane + 32 * i] : 1.0f;
                for (int sp = 1; sp < p.qkv_splits; ++sp)
#pragma unroll
                    for (int i = 0; i < EPL; ++i) x[i] += ksrc[sp * p.qkv_split_stride + lane + 32 * i], v[i] += vsrc[sp * p.qkv_split_stride + lane + 32 * i];
                if (p.k_norm) {
                    float ss = 0.0f;
#pragma unroll
                    for (int i = 0; i < EPL; ++i) ss = fmaf(x[i], x[i], ss);
                    const float inv = rsqrtf(warp_sum(ss) / (float)HD + p.eps);
#pragma unroll
                    for (int i = 0; i < EPL; ++i) x[i] = x[i] * inv * w[i];
                }
                if (p.inv_freq) {
                    const int per = p.rd / 64;                               // elements of a lane in each half of the rotated part
#pragma unroll
                    for (int i = 0; i < EPL / 2; ++i)
                        if (i < per) {
                            const float2 cs = turn[tt * (HD / 2) + lane + 32 * i];
                            float lo = x[i], hi = 0.0f;
#pragma unroll
                            for (int j = 1; j <= EPL / 2; ++j)               // x[i + per] without indexing registers by a variable
                                if (j == per) hi = x[i + j];
                            const float a = lo * cs.x - hi * cs.y, b = hi * cs.x + lo * cs.y;
                            x[i] = a;
#pragma unroll
                            for (int j = 1; j <= EPL / 2; ++j)
                                if (j == per) x[i + j] = b;
                        }
                }
                __nv_bfloat16* sk = stash + (size_t)tt * 2 * HD;
                __nv_bfloat16* kdst = const_cast<__nv_bfloat16*>(p.k_pages) + (((size_t)kh * p.num_pages + max(page, 0)) * p.page_size + pos % p.page_size) * HD;
                __nv_bfloat16* vdst = const_cast<__nv_bfloat16*>(p.v_pages) + (kdst - p.k_pages);
#pragma unroll
                for (int i = 0; i < EPL; ++i) {
                    // a position without a page has no key: zeros, as the pages' loader gives them
                    const __nv_bfloat16 kb16 = __float2bfloat16(page >= 0 ? x[i] : 0.0f), vb16 = __float2bfloat16(page >= 0 ? v[i] : 0.0f);
                    sk[lane + 32 * i] = kb16, sk[HD + lane + 32 * i] = vb16;
                    if (page >= 0) kdst[lane + 32 * i] = kb16, vdst[lane + 32 * i] = vb16;
                }
            }
        }
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            const int r = nb * 8 + quad, tt = r / G, hg = r % G;
            const bool live = tt < ntok;
            const float* src = p.qkv + (size_t)(tok0 + (live ? tt : 0)) * p.qkv_ld + (size_t)(kh * G + hg) * HD + 2 * pair;
            float x[DB][4], w[DB][4];          // slot s of block ks: head dimension 16 ks + 2 pair + (s & 1) + 8 (s >> 1)
#pragma unroll
            for (int ks = 0; ks < DB; ++ks) {
                const float2 a = *reinterpret_cast<const float2*>(src + ks * 16), b = *reinterpret_cast<const float2*>(src + ks * 16 + 8);
                x[ks][0] = a.x, x[ks][1] = a.y, x[ks][2] = b.x, x[ks][3] = b.y;
                if (p.q_norm) {
                    const float2 c = *reinterpret_cast<const float2*>(p.q_norm + ks * 16 + 2 * pair), d = *reinterpret_cast<const float2*>(p.q_norm + ks * 16 + 8 + 2 * pair);
                    w[ks][0] = c.x, w[ks][1] = c.y, w[ks][2] = d.x, w[ks][3] = d.y;
                }
            }
            for (int sp = 1; sp < p.qkv_splits; ++sp)
#pragma unroll
                for (int ks = 0; ks < DB; ++ks) {
                    const float2 a = *reinterpret_cast<const float2*>(src + sp * p.qkv_split_stride + ks * 16), b = *reinterpret_cast<const float2*>(src + sp * p.qkv_split_stride + ks * 16 + 8);
                    x[ks][0] += a.x, x[ks][1] += a.y, x[ks][2] += b.x, x[ks][3] += b.y;
                }
            if (p.q_norm) {
                float ss = 0.0f;
#pragma unroll
                for (int ks = 0; ks < DB; ++ks)
#pragma unroll
                    for (int s = 0; s < 4; ++s) ss = fmaf(x[ks][s], x[ks][s], ss);
                ss += __shfl_xor_sync(0xffffffffu, ss, 1);                   // the four lanes of a quad hold the row's HD values between them
                ss += __shfl_xor_sync(0xffffffffu, ss, 2);
                const float inv = rsqrtf(ss / (float)HD + p.eps);
#pragma unroll
                for (int ks = 0; ks < DB; ++ks)
#pragma unroll
                    for (int s = 0; s < 4; ++s) x[ks][s] = x[ks][s] * inv * w[ks][s];
            }
            if (p.inv_freq) {
                const int per = p.rd / 32;                                   // blocks of 16 dimensions in each half of the rotated part
                const float2* trow = turn + (live ? tt : 0) * (HD / 2) + 2 * pair;
#pragma unroll
                for (int ks = 0; ks < DB / 2; ++ks)
                    if (ks < per) {
#pragma unroll
                        for (int s = 0; s < 4; ++s) {
                            const float2 cs = trow[ks * 16 + (s & 1) + 8 * (s >> 1)];
                            float lo = x[ks][s], hi = 0.0f;
#pragma unroll
                            for (int j = 1; j <= DB / 2; ++j)
                                if (j == per) hi = x[ks + j][s];
                            const float a = lo * cs.x - hi * cs.y, b = hi * cs.x + lo * cs.y;
                            x[ks][s] = a;
#pragma unroll
                            for (int j = 1; j <= DB / 2; ++j)
                                if (j == per) x[ks + j][s] = b;
                        }
                    }
            }
#pragma unroll
            for (int ks = 0; ks < DB; ++ks) {
                qf[ks][nb][0] = live ? pack_bf16(x[ks][0], x[ks][1]) : 0u;
                qf[ks][nb][1] = live ? pack_bf16(x[ks][2], x[ks][3]) : 0u;
            }
        }
        if (has_new) asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");          // the stash is whole before any warp copies from it
    } else {
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            const int r = row0 + nb * 8 + quad, tt = r / G, hg = r % G;
            const bool live = tt < ntok;
            const uint32_t* src = reinterpret_cast<const uint32_t*>(p.q + ((size_t)(tok0 + (live ? tt : 0)) * p.Hq + kh * G + hg) * HD) + pair;
#pragma unroll
            for (int ks = 0; ks < DB; ++ks) {
                qf[ks][nb][0] = live ? src[ks * 8] : 0u;
                qf[ks][nb][1] = live ? src[ks * 8 + 4] : 0u;
            }
        }
    }
    float top[NB][2], sum[NB][2];              // running maximum (base-2 logits) and sum of the probabilities of this thread's keys
    float acc[DB][NB][4];                      // O^T: head dimensions 16 db + quad (+ 8 for [2], [3]), rows as above
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
        top[nb][0] = top[nb][1] = -INFINITY;
        sum[nb][0] = sum[nb][1] = 0.0f;
#pragma unroll
        for (int db = 0; db < DB; ++db) acc[db][nb][0] = acc[db][nb][1] = acc[db][nb][2] = acc[db][nb][3] = 0.0f;
    }

    // Every consumer warp passes every stage's barriers in order, also for the tiles it leaves to the others (it
    // lets go of those at once): a phase bit tells a phase only from its neighbours, so nobody may skip one.
    for (int i = 0; i < n_mine; ++i) {
        const int st = i % STAGES, kt = t_begin + i;
        if (!mbar_wait(full0 + 8 * st, (i / STAGES) & 1)) {
            if (lane == 0) atomicExch(&g_attn_status, 2);
            break;
        }
        if (!WIDE && i % CW != warp) {
            if (lane == 0) mbar_arrive(empty0 + 8 * st);
            continue;
        }
        const uint32_t kb = k_s + st * TILE_BYTES, vb = v_s + st * TILE_BYTES;
        if (!WIDE && has_new && kt >= pos_first / KT) {
            // the rows of this step's positions: from the stash, in place of what the pages held there
            for (int tt = 0; tt < ntok; ++tt) {
                const int pos = pos_first + tt;
                if (pos / KT != kt) continue;
                for (int idx = lane; idx < 2 * CH; idx += 32) {
                    const int which = idx / CH, c = idx % CH;
                    const uint4 val = *reinterpret_cast<const uint4*>(stash + ((size_t)tt * 2 + which) * HD + c * 8);
                    *reinterpret_cast<uint4*>(smem + (which ? v_s - k_s : 0) + st * TILE_BYTES + swk(pos - kt * KT, c)) = val;
                }
            }
            __syncwarp();
        }
        if (TMA && kt == end_tile - 1 && (pos_last + 1) % KT != 0) {
            // the last page came in whole: the keys past the last position hold whatever the page held
            // before.  Their scores are masked, but 0 * V must not meet a stale NaN: clear those V rows.
            const int r0 = pos_last + 1 - kt * KT;
            if (WIDE) {
                for (int idx = r0 * CH + tid; idx < KT * CH; idx += CW * 32)
                    *reinterpret_cast<uint4*>(smem + (v_s - k_s) + st * TILE_BYTES + swk(idx / CH, idx % CH)) = make_uint4(0, 0, 0, 0);
                asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");          // all eight warps read this stage
            } else {
                for (int idx = r0 * CH + lane; idx < KT * CH; idx += 32)
                    *reinterpret_cast<uint4*>(smem + (v_s - k_s) + st * TILE_BYTES + swk(idx / CH, idx % CH)) = make_uint4(0, 0, 0, 0);
                __syncwarp();
            }
        }
        // ---- S^T = K Q^T
        float sc[KB][NB][4];
#pragma unroll
        for (int mb = 0; mb < KB; ++mb) {
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) sc[mb][nb][0] = sc[mb][nb][1] = sc[mb][nb][2] = sc[mb][nb][3] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < DB; ++ks) {
                uint32_t a[4];                 // keys 16 mb + {0..7, 8..15} x head dimensions 16 ks + {0..7, 8..15}
                ldmatrix_x4(a, kb + swk(mb * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)));
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) mma_bf16(sc[mb][nb], a, qf[ks][nb][0], qf[ks][nb][1]);
            }
        }
        // ---- scale, mask, the rows' maxima over the tile
        const int j0 = kt * KT + quad;
        float hi[NB][2];
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            hi[nb][0] = top[nb][0], hi[nb][1] = top[nb][1];
#pragma unroll
            for (int mb = 0; mb < KB; ++mb)
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    const int c = x & 1, j = j0 + mb * 16 + (x >> 1) * 8;
                    const float v = (j <= see_to[nb][c] && j >= see_from[nb][c]) ? sc[mb][nb][x] * p.scale_log2 : -INFINITY;
                    sc[mb][nb][x] = v;
                    hi[nb][c] = fmaxf(hi[nb][c], v);
                }
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                float v = hi[nb][c];
                v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
                v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
                v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
                const float shrink = v == -INFINITY ? 1.0f : exp2f(top[nb][c] - v);      // nothing seen yet: nothing to rescale
                top[nb][c] = v;
                sum[nb][c] *= shrink;
#pragma unroll
                for (int db = 0; db < DB; ++db) acc[db][nb][c] *= shrink, acc[db][nb][2 + c] *= shrink;
            }
        }
        // ---- P^T = 2^(S^T - max), rounded to bfloat16 before it is summed (the sum then matches the
        // P that multiplies V), and turned into the second product's B fragments
        uint32_t pf[KB][NB][2];
#pragma unroll
        for (int mb = 0; mb < KB; ++mb)
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                float e[4];
#pragma unroll
                for (int x = 0; x < 4; ++x) e[x] = top[nb][x & 1] == -INFINITY ? 0.0f : exp2f(sc[mb][nb][x] - top[nb][x & 1]);
                const __nv_bfloat162 lo = __floats2bfloat162_rn(e[0], e[1]), up = __floats2bfloat162_rn(e[2], e[3]);
                sum[nb][0] += __low2float(lo) + __low2float(up);
                sum[nb][1] += __high2float(lo) + __high2float(up);
                pf[mb][nb][0] = transpose_8x8(*reinterpret_cast<const uint32_t*>(&lo));
                pf[mb][nb][1] = transpose_8x8(*reinterpret_cast<const uint32_t*>(&up));
            }
        // ---- O^T += V^T P^T
#pragma unroll
        for (int mb = 0; mb < KB; ++mb)
#pragma unroll
            for (int db = 0; db < DB; ++db) {
                uint32_t a[4];                 // head dimensions 16 db + {0..7, 8..15} x keys 16 mb + {0..7, 8..15}, transposed on load
                ldmatrix_x4_trans(a, vb + swk(mb * 16 + (lane & 7) + ((lane >> 4) << 3), db * 2 + ((lane >> 3) & 1)));
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) mma_bf16(acc[db][nb], a, pf[mb][nb][0], pf[mb][nb][1]);
            }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + 8 * st);
    }
    // a row's sum is spread over the eight lanes that hold its keys
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            float v = sum[nb][c];
            v += __shfl_xor_sync(0xffffffffu, v, 4);
            v += __shfl_xor_sync(0xffffffffu, v, 8);
            v += __shfl_xor_sync(0xffffffffu, v, 16);
            sum[nb][c] = v;
        }

    const size_t part_row0 = ((size_t)blockIdx.x * p.Hkv + kh) * ROWS;       // where this CTA's partial results go
    if (WIDE) {
        // ---- every warp owns its 16 rows: straight to the output (one part) or to the partial buffers
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            if (parts == 1) {
                // the output row of the lane after the transposition below: row nb*8 + quad
                const int r = row0 + nb * 8 + quad, tt = r / G, hg = r % G;
                float scale[2];
#pragma unroll
                for (int c = 0; c < 2; ++c) {                                // this thread's own rows: 1 / denominator, with the sink
                    const int rr = row0 + nb * 8 + 2 * pair + c;
                    float shrink = 1.0f, den = sum[nb][c];
                    if (p.sinks && rr / G < ntok) {
                        const float sk = p.sinks[kh * G + rr % G] * LOG2E, both = fmaxf(top[nb][c], sk);
                        shrink = exp2f(top[nb][c] - both);
                        den = den * shrink + exp2f(sk - both);
                    }
                    scale[c] = shrink / den;
                }
                __nv_bfloat16* dst = p.out + ((size_t)(tok0 + tt) * p.Hq + kh * G + hg) * HD + 2 * pair;
#pragma unroll
                for (int db = 0; db < DB; ++db)
#pragma unroll
                    for (int h = 0; h < 2; ++h) {                            // head dimensions 16 db + 8 h + quad of rows 2 pair + {0, 1} ...
                        const uint32_t v = transpose_8x8(pack_bf16(acc[db][nb][2 * h] * scale[0], acc[db][nb][2 * h + 1] * scale[1]));
                        if (tt < ntok) *reinterpret_cast<uint32_t*>(dst + db * 16 + h * 8) = v;      // ... become dimensions 2 pair + {0, 1} of row quad
                    }
            } else {
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int r = row0 + nb * 8 + 2 * pair + c;
                    if (r / G >= ntok) continue;
                    float* po = p.part_o + (part_row0 + r) * HD + quad;
#pragma unroll
                    for (int db = 0; db < DB; ++db) po[db * 16] = acc[db][nb][c], po[db * 16 + 8] = acc[db][nb][2 + c];
                    if (quad == 0) {
                        p.part_ml[(part_row0 + r) * 2] = top[nb][c];
                        p.part_ml[(part_row0 + r) * 2 + 1] = sum[nb][c];
                    }
                }
            }
        }
        return;
    }
    // ---- narrow tiles: the four warps hold the same rows over different keys.  Their maxima and sums meet in shared
    // memory first; every warp brings its O^T to the common maximum and writes it to a slab of its own; then all 128
    // threads add the four slabs in warp order.  The ring is idle by now: every tile has been waited for and read.
    constexpr int LD = HD + 4;                 // row pitch of a slab in floats (the padding spreads a fragment's stores over the banks)
    float* slab = reinterpret_cast<float*>(smem);                            // [CW][NQ][LD]
    float* stat = slab + CW * NQ * LD;                                       // [CW][NQ][2]: maximum, sum
    asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
    if (quad == 0)
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                float* s2 = stat + ((size_t)warp * NQ + nb * 8 + 2 * pair + c) * 2;
                s2[0] = top[nb][c], s2[1] = sum[nb][c];
            }
    asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const int r = nb * 8 + 2 * pair + c;
            float all = -INFINITY;
#pragma unroll
            for (int w = 0; w < CW; ++w) all = fmaxf(all, stat[((size_t)w * NQ + r) * 2]);
            const float mine = top[nb][c] == -INFINITY ? 0.0f : exp2f(top[nb][c] - all);
            float* dst = slab + ((size_t)warp * NQ + r) * LD + quad;
#pragma unroll
            for (int db = 0; db < DB; ++db) dst[db * 16] = acc[db][nb][c] * mine, dst[db * 16 + 8] = acc[db][nb][2 + c] * mine;
        }
    asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
    // thread -> (row, a stretch of head dimensions): 128 threads over NQ rows
    constexpr int TPR = CW * 32 / NQ, DPT = HD / TPR;                        // threads per row, dimensions per thread
    const int r = tid / TPR, d0 = (tid % TPR) * DPT, tt = r / G, hg = r % G;
    if (tt >= ntok) return;
    float all = -INFINITY, den = 0.0f;
#pragma unroll
    for (int w = 0; w < CW; ++w) all = fmaxf(all, stat[((size_t)w * NQ + r) * 2]);
#pragma unroll
    for (int w = 0; w < CW; ++w) {
        const float mw = stat[((size_t)w * NQ + r) * 2];
        den += mw == -INFINITY ? 0.0f : exp2f(mw - all) * stat[((size_t)w * NQ + r) * 2 + 1];
    }
    float o[DPT];
#pragma unroll
    for (int d = 0; d < DPT; ++d) {
        o[d] = 0.0f;
#pragma unroll
        for (int w = 0; w < CW; ++w) o[d] += slab[((size_t)w * NQ + r) * LD + d0 + d];
    }
    if (parts == 1) {
        float shrink = 1.0f;
        if (p.sinks) {
            const float sk = p.sinks[kh * G + hg] * LOG2E, both = fmaxf(all, sk);
            shrink = exp2f(all - both);
            den = den * shrink + exp2f(sk - both);
        }
        const float inv = shrink / den;
        __nv_bfloat16* dst = p.out + ((size_t)(tok0 + tt) * p.Hq + kh * G + hg) * HD + d0;
#pragma unroll
        for (int d = 0; d < DPT; d += 2) *reinterpret_cast<uint32_t*>(dst + d) = pack_bf16(o[d] * inv, o[d + 1] * inv);
    } else {
        float* po = p.part_o + (part_row0 + r) * HD + d0;
#pragma unroll
        for (int d = 0; d < DPT; ++d) po[d] = o[d];
        if (tid % TPR == 0) {
            p.part_ml[(part_row0 + r) * 2] = all;
            p.part_ml[(part_row0 + r) * 2 + 1] = den;
        }
    }
}

// out[row] = sum_s 2^(m_s - M) o_s / (sum_s 2^(m_s - M) l_s + 2^(sink - M)); one block per (tile, KV head, row of
// the tile).  A thread owns four head dimensions of every GROUPS-th split, so that the many splits
// of a long context at a small batch are fetched side by side; the groups' sums meet in shared
// memory and are added in group order (a fixed order for a given number of splits).
constexpr int MERGE_THREADS = 256;
// U: parts a thread has in flight at once.  Few tiles with many parts each (a batch of one or two deep in their
// contexts): 10, so that a round of 80 parts (head size 128) is one trip to memory; many tiles: 4, which leaves
// registers for three blocks per SM.
template <int HD, int U>
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

template <int HD, int NQ, bool WIDE, bool TMA>
constexpr size_t attention_smem() {
    constexpr int STAGES = HD == 128 ? 3 : 4;
    constexpr size_t ring = 2 * STAGES * KT * HD * 2;
    constexpr size_t meet = WIDE ? 0 : 4 * NQ * (HD + 4 + 2) * sizeof(float);       // the narrow tiles' slabs and statistics: in the ring, idle by then
    static_assert(ring >= meet, "the slabs lie in the ring");
    // behind the ring of a narrow tile: the new keys and values of its tokens (bfloat16) and their rotations (cosine, sine)
    constexpr size_t stash = WIDE ? 0 : (size_t)PREP_TOKENS * (2 * HD * 2 + HD / 2 * 8);
    return ring + stash + 1024;
}

template <int HD, int NQ, bool WIDE, bool TMA>
int launch(const AttnParams& p, const CUtensorMap* maps, int n_tiles, cudaStream_t st) {
    constexpr int ROWS = WIDE ? 128 : NQ;
    constexpr size_t smem = attention_smem<HD, NQ, WIDE, TMA>();
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attention_mma_kernel<HD, NQ, WIDE, TMA>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return q6k_check_launch("attention_mma: shared memory attribute");
        configured = true;
    }
    q6k_launch_as(!WIDE && p.early != 0, attention_mma_kernel<HD, NQ, WIDE, TMA>, dim3(p.n_work, p.Hkv), (WIDE ? 8 : 4) * 32 + 32, smem, st, maps[0], maps[1], maps[2], maps[3], p);
    if (int rc = q6k_check_launch("attention_mma")) return rc;
    if (p.n_work > n_tiles) {                 // some tile may have more than one part
        if (p.n_work >= 32 * n_tiles) q6k_launch(attention_merge_kernel<HD, 10>, dim3(n_tiles, p.Hkv, ROWS), MERGE_THREADS, 0, st, p);
        else q6k_launch(attention_merge_kernel<HD, 4>, dim3(n_tiles, p.Hkv, ROWS), MERGE_THREADS, 0, st, p);
        return q6k_check_launch("attention_merge");
    }
    return 0;
}

template <int HD>
int launch_hd(const AttnParams& p, const CUtensorMap* maps, int rows, bool tma, int n_tiles, cudaStream_t st) {
    if (rows == 128) return tma ? launch<HD, 16, true, true>(p, maps, n_tiles, st) : launch<HD, 16, true, false>(p, maps, n_tiles, st);
    if (rows == 16) return tma ? launch<HD, 16, false, true>(p, maps, n_tiles, st) : launch<HD, 16, false, false>(p, maps, n_tiles, st);
    return tma ? launch<HD, 8, false, true>(p, maps, n_tiles, st) : launch<HD, 8, false, false>(p, maps, n_tiles, st);
}

// CTAs of the kernel that one SM holds at once (what shared memory and registers allow).
template <int HD, int NQ, bool WIDE>
int resident_per_sm() {
    int n = 0;
    constexpr size_t smem = attention_smem<HD, NQ, WIDE, true>();
    if (cudaFuncSetAttribute(attention_mma_kernel<HD, NQ, WIDE, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attention_mma_kernel<HD, NQ, WIDE, true>, (WIDE ? 8 : 4) * 32 + 32, smem) != cudaSuccess) return 0;
    return n;
}

}  // namespace

// The head sizes and group sizes the kernel takes.  A tile holds the query rows of consecutive tokens of one
// request for one KV head (row = token * G + head of the group): 8 or 16 rows (narrow: decode and the like) or 128
// (wide: prompt portions).
Q6K_API int q6k_attention_mma_supported(int hd, int G, int wide) { return (hd == 64 || hd == 128) && G >= 1 && G <= (wide ? 128 : 16); }

// Rows of the tiles to use when the requests of a step bring at most max_tokens tokens each: the smallest
// tile that holds them (8, 16 or 128), or 0 when this kernel does not take the head and group size.
Q6K_API int q6k_attention_mma_tile_rows(int hd, int G, int max_tokens) {
    if (!q6k_attention_mma_supported(hd, G, 1)) return 0;
    if ((long long)G * max_tokens <= 8) return 8;
    if ((long long)G * max_tokens <= 16) return 16;
    return 128;
}

// CTAs of the kernel for tiles of `rows` rows that the current device holds at once: the plan of a launch splits the
// keys over exactly this many, so that one wave does all the work.  0 on an error or an unsupported shape.
Q6K_API int q6k_attention_mma_resident_ctas(int hd, int rows) {
    int dev = 0, sms = 0, per = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    if (hd == 128) per = rows == 128 ? resident_per_sm<128, 16, true>() : rows == 16 ? resident_per_sm<128, 16, false>() : resident_per_sm<128, 8, false>();
    else if (hd == 64) per = rows == 128 ? resident_per_sm<64, 16, true>() : rows == 16 ? resident_per_sm<64, 16, false>() : resident_per_sm<64, 8, false>();
    return per * sms;
}

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
// these tiles (of at most rows / G tokens each; rows: 8, 16 or 128) and this window; part_o: FP32 [n_work * Hkv * rows * hd],
// part_ml: FP32 [n_work * Hkv * rows * 2] (unused when n_work == n_tiles).
// early != 0 (tiles of 8 or 16 rows only): the caller's word that the plan and the block table were made before the kernel
// launched before this one started, and that this kernel writes this step's keys; key tiles older than a tile's first
// position are then fetched while it still runs.
// qkv != null (tiles of 8 or 16 rows only; q is then unused): FP32 [qkv_splits, T, qkv_ld] rows of q heads | k heads | v heads
// (slices qkv_split_stride floats apart, summed in order: split-K partial products), which the
// kernel itself normalises per head (q_norm, k_norm: FP32 [hd] or null; eps), rotates (inv_freq: FP32 [rotary_dim / 2] or
// null; pairs d, d + rotary_dim / 2; rotary_dim a multiple of 64) and rounds; write_kv != 0: the tiles' keys and values
// are made the same way and written to the pages (which nothing else may read or write meanwhile).  With early != 0 the
// kernel launched before this one must then have been launched early itself or be the only writer of qkv.
Q6K_API int q6k_attention_mma_prepares(int hd, int G, int rows, int rotary_dim, int neighbours) {
    return (hd == 64 || hd == 128) && (rows == 8 || rows == 16) && G >= 1 && rows / G <= PREP_TOKENS &&
           (rotary_dim == 0 || (!neighbours && rotary_dim % 64 == 0 && rotary_dim <= hd));
}

Q6K_API int q6k_attention_mma(const void* q, const void* k_pages, const void* v_pages, long long num_pages, const int* block_table,
                              int max_blocks, int page_size, const int* work, const int* tile_plan, int n_work, int n_tiles, int rows,
                              int window, const float* sinks, float scale, void* out, float* part_o, float* part_ml, int Hq, int Hkv,
                              int hd, int early, const float* qkv, int qkv_ld, int qkv_splits, long long qkv_split_stride, const float* q_norm, const float* k_norm, float eps,
                              const float* inv_freq, int rotary_dim, int write_kv, cudaStream_t st) {
    if (n_tiles == 0) return 0;
    Q6K_REQUIRE(Hq > 0 && Hkv > 0 && Hq % Hkv == 0, "attention_mma: bad head counts Hq=%d Hkv=%d", Hq, Hkv);
    const int G = Hq / Hkv;
    Q6K_REQUIRE(rows == 8 || rows == 16 || rows == 128, "attention_mma: tiles of %d rows (8, 16 or 128 are built)", rows);
    Q6K_REQUIRE(q6k_attention_mma_supported(hd, G, rows == 128) && G <= rows, "attention_mma: head_dim %d / group size %d is not covered by tiles of %d rows", hd, G, rows);
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
    p.early = early;
    if (qkv) {
        Q6K_REQUIRE(q6k_attention_mma_prepares(hd, G, rows, inv_freq ? rotary_dim : 0, 0), "attention_mma: tiles of %d rows of heads of %d (groups of %d) do not prepare q and k with %d rotating dimensions",
                    rows, hd, G, rotary_dim);
        Q6K_REQUIRE(qkv_ld >= (write_kv ? Hq + 2 * Hkv : Hq) * hd && qkv_ld % 2 == 0 && ((uintptr_t)qkv & 7) == 0, "attention_mma: qkv rows of %d values for %d + 2 x %d heads of %d", qkv_ld, Hq, Hkv, hd);
        Q6K_REQUIRE(qkv_splits >= 1 && qkv_split_stride % 2 == 0, "attention_mma: %d slices of qkv, %lld values apart", qkv_splits, qkv_split_stride);
        p.qkv_splits = qkv_splits, p.qkv_split_stride = qkv_split_stride;
        p.qkv = qkv, p.qkv_ld = qkv_ld, p.q_norm = q_norm, p.k_norm = k_norm, p.eps = eps, p.write_kv = write_kv;
        p.inv_freq = inv_freq, p.rd = inv_freq ? rotary_dim : 0;
    } else {
        Q6K_REQUIRE(q != nullptr, "attention_mma: neither q nor qkv%s", "");
    }
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
    return hd == 128 ? launch_hd<128>(p, maps, rows, tma, n_tiles, st) : launch_hd<64>(p, maps, rows, tma, n_tiles, st);
}
