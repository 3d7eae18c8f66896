// bfloat16 matrix products on the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor
// memory), operands brought into shared memory by TMA.  sm_100a only.
//
//   out[r, n] (+)= sum_k A[r, k] * W_g[n, k]       A: [rows, K], W: [groups, N, K], K contiguous
//
// The reference runs every projection and every expert through one grouped kernel with mma.sync
// tiles of 64 rows (crates/cuda/kernels/moe.cu:142-255) and single-token products through
// CUDA-core GEMVs (crates/cuda/kernels/flint.cu:589-824).  Here one kernel serves both regimes by
// swapping the operands: a tile of 128 WEIGHT rows is the M side of the MMA and the tokens are the
// N side (16 to 256 of them), so a decode step of a few tokens still fills the tensor core's M
// and simply streams the weights through a deep TMA pipeline, while a prefill tile reuses each
// weight tile over up to 256 tokens.
//
// A persistent CTA per SM walks tiles of [128 weights x BT tokens] (optionally one slice of K each):
//   warp 0     producer: waits for a free stage, arms its mbarrier with the byte count, issues the
//              TMA loads of the weight tile(s) [128 x 64] and the token tile [BT x 64] (128-byte swizzle)
//   warp 1     allocates tensor memory (two accumulator buffers); one thread issues 4 tcgen05.mma
//              (K = 16 each) per stage and commits the stage's "empty" barrier; after a tile's last
//              stage it commits "accumulator full" and turns to the other buffer
//   warps 2-5  epilogue: tcgen05.ld of their 32 accumulator lanes (one lane = one weight row, one
//              column = one token) and the store: plain, added into the FP32 stream, SwiGLU of two
//              accumulators, or a split-K partial; they hand a buffer back ("accumulator empty") as soon
//              as its values are in registers, so the next tile's MMAs overlap the stores
// Every wait on an mbarrier is bounded; a wait that runs out records a code in a status word that
// q6k_tc_status() returns, the roles fall through to the common exit, and tensor memory is freed.
#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"
#include "tma.cuh"

namespace {

constexpr int BK = 64;                 // bf16 per k-block: one 128-byte swizzle row
constexpr int WM = 128;                // weight rows per tile (UMMA M)
constexpr int MAX_STAGES = 12;

enum { EPI_STORE = 0, EPI_ADD = 1, EPI_SWIGLU = 2, EPI_PARTIAL = 3 };

__device__ int g_tc_status = 0;

struct Params {
    void* out;
    float* partial;                    // split-K partials [splits, rows_total, N]
    const int* tile_group;             // grouped: per row tile its group and first row
    const int* tile_row0;
    const int* group_offsets;
    const int* num_tiles;
    const int* pair_order;             // pair mode: tile y works on pair pair_order[y] (null: pair y)
    unsigned* tickets;                 // pair mode with K slices: one arrival counter per (pair, n-tile), zero between launches
    int rows_total, N, K, ldo;
    int epilogue, stages, kb_per_split;
    int pair_div;                      // > 0: one tile per (token, slot) pair, see q6k_gemm_tc_pairs
    int lists_old;                     // the pair list was written before the kernel launched before this one started: weights may be fetched before the wait
    int n_y, n_z;                      // row tiles (or pairs; an upper bound when num_tiles is given) and K slices
    int w_once;                        // every weight tile is fetched by one CTA only (or by a few side by side): its lines may leave the L2 cache first
};

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 bf16) with the
// 128-byte swizzle, 8-row groups 1024 bytes apart; version 1 (sm_100).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}

// Instruction descriptor: D FP32, A and B bfloat16, both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t umma_idesc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(WM >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

__host__ __device__ constexpr int tmem_cols(int want) { return want <= 32 ? 32 : want <= 64 ? 64 : want <= 128 ? 128 : want <= 256 ? 256 : 512; }

// One tile of the persistent schedule: which weights, which token rows, which slice of K.
struct Tile {
    int g, n0, row0, row_end, out0, kb0, nkb, z;
};

// Tile t of the launch: n-tiles fastest (neighbouring CTAs share the token tile), then row tiles
// (or pairs, or the grouped tile list), then K slices.  Every role of a CTA decodes the same
// sequence t = blockIdx.x, blockIdx.x + gridDim.x, ...
template <int BT>
__device__ __forceinline__ bool decode_tile(const Params& p, int t, int n_x, int n_y, Tile& o) {
    const int x = t % n_x, y = (t / n_x) % n_y;
    o.z = t / (n_x * n_y);
    o.n0 = x * WM;
    o.g = 0;
    if (p.pair_div > 0) {
        // tile y is pair y: its expert's weights, the single input row y / pair_div, the output row y
        const int pair = p.pair_order ? p.pair_order[y] : y;
        o.g = p.tile_group[pair];
        o.row0 = pair / p.pair_div;
        o.row_end = o.row0 + 1;
        o.out0 = pair;
    } else if (p.tile_group) {
        o.g = p.tile_group[y];
        o.row0 = p.tile_row0[y];
        o.row_end = p.group_offsets[o.g + 1];
        o.out0 = o.row0;
    } else {
        o.row0 = y * BT;
        o.row_end = p.rows_total;
        o.out0 = o.row0;
    }
    const int kb_total = (p.K + BK - 1) / BK;
    o.kb0 = o.z * p.kb_per_split;
    o.nkb = min(p.kb_per_split, kb_total - o.kb0);
    return o.row0 < o.row_end && o.nkb > 0;
}

// Persistent: one CTA per SM walks the tiles.  The producer runs ahead through the shared-memory
// ring across tile boundaries; the MMA thread alternates between two accumulators in tensor
// memory, so the epilogue warps drain one tile while the next one is being multiplied.
template <int BT, bool DUAL>
__global__ void __launch_bounds__(192) gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_w2,
                                                       const __grid_constant__ CUtensorMap tm_a, const Params p) {
    // Dense tiles follow from the launch alone, so their weights can be on the way before the kernel
    // that makes the activations has ended; tile lists and pair lists come from earlier kernels, and
    // only a caller who knows that another kernel lies between their maker and this one says so.
    const bool early = p.tile_group == nullptr || p.lists_old != 0;
    if (!early) pdl_wait();
    const int n_x = (p.N + WM - 1) / WM;
    const int n_y = p.pair_div > 0 ? p.n_y : (p.tile_group ? *p.num_tiles : p.n_y);
    const int total = n_x * n_y * p.n_z;
    if ((int)blockIdx.x >= total) return;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    constexpr uint32_t W_BYTES = WM * BK * 2, A_BYTES = BT * BK * 2;
    constexpr uint32_t STAGE_BYTES = W_BYTES * (DUAL ? 2 : 1) + A_BYTES;
    constexpr int ACC_COLS = DUAL ? 2 * BT : BT;           // columns of one accumulator buffer
    constexpr int COLS = tmem_cols(2 * ACC_COLS);
    __shared__ __align__(8) uint64_t bars[2 * MAX_STAGES + 4];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int fix_last;
    const int stages = p.stages;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[MAX_STAGES]);
    const uint32_t acc_full0 = smem_u32(&bars[2 * MAX_STAGES]), acc_empty0 = smem_u32(&bars[2 * MAX_STAGES + 2]);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full0 + 8 * b, 1);
            mbar_init(acc_empty0 + 8 * b, 4);              // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_a) : "memory");
        if (DUAL) asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_w2) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    pdl_launch();                                          // this block holds its tensor memory: a successor may come

    if (warp == 0) {
        if (lane == 0) {
            int pre = 0;                                   // k-blocks whose weights went out before the wait
            const uint64_t once = l2_evict_first_policy();
            auto load_w = [&](uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
                if (p.w_once) tma_load_2d_once(dst, map, x, y, bar, once);
                else tma_load_2d(dst, map, x, y, bar);
            };
            if (early) {
                for (int t = blockIdx.x; t < total && pre < stages; t += gridDim.x) {
                    Tile tl;
                    if (!decode_tile<BT>(p, t, n_x, n_y, tl)) continue;
                    const int wy = tl.g * p.N + tl.n0;
                    for (int i = 0; i < tl.nkb && pre < stages; ++i, ++pre) {
                        const uint32_t st = smem_u32(smem + (size_t)pre * STAGE_BYTES);
                        const uint32_t fb = full0 + 8 * pre;
                        mbar_expect_tx(fb, STAGE_BYTES);
                        const int kx = (tl.kb0 + i) * BK;
                        load_w(st, &tm_w, kx, wy, fb);
                        if (DUAL) load_w(st + W_BYTES, &tm_w2, kx, wy, fb);
                    }
                }
                pdl_wait();
            }
            int it = 0;                                    // k-blocks issued so far, over all tiles
            bool ok = true;
            for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
                Tile tl;
                if (!decode_tile<BT>(p, t, n_x, n_y, tl)) continue;
                const int wy = tl.g * p.N + tl.n0;
                for (int i = 0; i < tl.nkb; ++i, ++it) {
                    const int s = it % stages;
                    const uint32_t st = smem_u32(smem + (size_t)s * STAGE_BYTES);
                    const uint32_t fb = full0 + 8 * s;
                    const int kx = (tl.kb0 + i) * BK;
                    if (it >= pre) {
                        if (!mbar_wait(empty0 + 8 * s, ((it / stages) & 1) ^ 1)) {
                            atomicExch(&g_tc_status, 1);
                            ok = false;
                            break;
                        }
                        mbar_expect_tx(fb, STAGE_BYTES);
                        load_w(st, &tm_w, kx, wy, fb);
                        if (DUAL) load_w(st + W_BYTES, &tm_w2, kx, wy, fb);
                    }
                    tma_load_2d(st + W_BYTES * (DUAL ? 2 : 1), &tm_a, kx, tl.row0, fb);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(BT);
            int it = 0, nt = 0;                            // k-blocks and tiles consumed so far
            bool ok = true;
            for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
                Tile tl;
                if (!decode_tile<BT>(p, t, n_x, n_y, tl)) continue;
                const int buf = nt & 1;
                if (!mbar_wait(acc_empty0 + 8 * buf, ((nt >> 1) & 1) ^ 1)) {      // the epilogue has drained this buffer
                    atomicExch(&g_tc_status, 4);
                    break;
                }
                tc_fence_after();
                const uint32_t acc_addr = tmem_base + buf * ACC_COLS;
                for (int i = 0; i < tl.nkb; ++i, ++it) {
                    const int s = it % stages;
                    if (!mbar_wait(full0 + 8 * s, (it / stages) & 1)) {
                        atomicExch(&g_tc_status, 2);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t st = smem_u32(smem + (size_t)s * STAGE_BYTES);
                    const uint64_t dw = umma_desc_sw128(st), dw2 = umma_desc_sw128(st + W_BYTES);
                    const uint64_t da = umma_desc_sw128(st + W_BYTES * (DUAL ? 2 : 1));
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint32_t acc = (i | k) != 0;
                        umma_bf16(acc_addr, dw + 2 * k, da + 2 * k, idesc, acc);          // + 32 bytes of K per step
                        if (DUAL) umma_bf16(acc_addr + BT, dw2 + 2 * k, da + 2 * k, idesc, acc);
                    }
                    umma_commit(empty0 + 8 * s);
                }
                if (!ok) break;
                umma_commit(acc_full0 + 8 * buf);          // arrives when every MMA issued so far has finished
                ++nt;
            }
        }
    } else {
        // epilogue: this warp owns accumulator lanes 32*(warp%4) .. +31
        const int quarter = warp & 3;
        const int n_local = quarter * 32 + lane;
        int nt = 0;
        if (early) pdl_wait();                             // the output may still be in use by the kernel before
        for (int t = blockIdx.x; t < total; t += gridDim.x) {
            Tile tl;
            if (!decode_tile<BT>(p, t, n_x, n_y, tl)) continue;
            const int buf = nt & 1;
            if (!mbar_wait(acc_full0 + 8 * buf, (nt >> 1) & 1)) {
                if (lane == 0) atomicExch(&g_tc_status, 3);
                break;
            }
            tc_fence_after();
            const int n = tl.n0 + n_local;
            const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * ACC_COLS;
            const int valid = min(BT, tl.row_end - tl.row0);
            if (p.pair_div > 0 && p.n_z > 1) {
                // A pair's K slices run in different CTAs.  Each leaves its slice's sums in global
                // memory and takes a ticket; the one that comes last adds the slices in their order
                // (whoever it is: the result does not depend on the arrival order) and finishes the tile.
                float v[16], u[16];
                tmem_ld16(lane_addr, v);
                if (DUAL) tmem_ld16(lane_addr + BT, u);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);
                constexpr int PARTS = DUAL ? 2 : 1;
                const size_t slice = (size_t)p.n_y * PARTS * p.N;          // floats per K slice
                float* mine = p.partial + (size_t)tl.out0 * PARTS * p.N;
                if (n < p.N) {
                    __stcg(mine + tl.z * slice + n, v[0]);
                    if (DUAL) __stcg(mine + tl.z * slice + p.N + n, u[0]);
                }
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (threadIdx.x == 64) {
                    unsigned* tk = p.tickets + (size_t)tl.out0 * n_x + tl.n0 / WM;
                    const int last = atomicAdd(tk, 1u) == (unsigned)(p.n_z - 1);
                    if (last) *tk = 0;                                    // nobody else comes: ready for the next launch
                    fix_last = last;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const int last = fix_last;
                asm volatile("bar.sync 1, 128;" ::: "memory");             // fix_last may be rewritten for the next tile
                if (last && n < p.N) {
                    __threadfence();
                    float a = 0.0f, b = 0.0f;
                    for (int z = 0; z < p.n_z; ++z) {
                        a += __ldcg(mine + z * slice + n);
                        if (DUAL) b += __ldcg(mine + z * slice + p.N + n);
                    }
                    const size_t row = (size_t)tl.out0;
                    if (p.epilogue == EPI_SWIGLU) ((__nv_bfloat16*)p.out)[row * p.ldo + n] = __float2bfloat16_rn(a / (1.0f + expf(-a)) * b);
                    else ((float*)p.out)[row * p.ldo + n] = a;
                }
                ++nt;
                continue;
            }
#pragma unroll 1
            for (int c0 = 0; c0 < valid; c0 += 16) {
                float v[16], u[16];
                tmem_ld16(lane_addr + c0, v);
                if (DUAL) tmem_ld16(lane_addr + BT + c0, u);
                if (c0 + 16 >= valid) {
                    // everything this warp needs of the buffer is in registers: hand it back
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);
                }
                if (n < p.N) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int tt = c0 + j;
                        if (tt >= valid) break;
                        const size_t row = (size_t)(tl.out0 + tt);
                        if (p.epilogue == EPI_STORE) {
                            ((float*)p.out)[row * p.ldo + n] = v[j];
                        } else if (p.epilogue == EPI_ADD) {
                            ((float*)p.out)[row * p.ldo + n] += v[j];
                        } else if (p.epilogue == EPI_SWIGLU) {
                            const float gte = v[j];
                            ((__nv_bfloat16*)p.out)[row * p.ldo + n] = __float2bfloat16_rn(gte / (1.0f + expf(-gte)) * u[DUAL ? j : 0]);
                        } else {
                            p.partial[((size_t)tl.z * p.rows_total + row) * p.N + n] = v[j];
                        }
                    }
                }
            }
            ++nt;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(COLS) : "memory");
    }
}

// ------------------------------------------------------------------------- a pair of CTAs per tile
// Dense products with many rows: two CTAs of a cluster work on one tile of [256 weights x BT2 tokens]
// with tcgen05.mma.cta_group::2.  Each CTA brings its 128 weight rows and its half of the token tile
// into its own shared memory, the leader (rank 0) issues the MMAs, which read both CTAs' shared
// memory and write each CTA's half of the accumulator (its 128 weight rows x BT2 tokens) into that
// CTA's tensor memory.  Per MMA and SM that is half the token-tile traffic of the one-CTA kernel,
// whose MMAs wait for shared memory.  Barriers: both CTAs' TMA loads count their bytes on the
// leader's "full" barrier (the .cta_group::2 form of the copy takes a barrier of the pair's other
// CTA); the leader's tcgen05.commit arrives on "empty" and "accumulator full" in both CTAs; the
// epilogue warps of both arrive on the leader's "accumulator empty".
constexpr uint32_t PEER_MASK = 0xFEFFFFFFu;    // a shared-memory address of either CTA of a pair -> the same offset in the even one

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(bar & PEER_MASK)
        : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8, %9, %10, %11, %12}, p;\n\t}" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {          // arrives at this offset in both CTAs
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
                 "h"((uint16_t)3)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive_leader(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar & PEER_MASK) : "memory");
}
// D FP32, A and B bfloat16, both K-major, M = 256 over the pair, N = n.
__host__ __device__ constexpr uint32_t umma_idesc_pair(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

template <int BT2>
__global__ void __launch_bounds__(192) gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_a,
                                                           const Params p) {
    // The tiles follow from the launch alone: the pair sets itself up and sends for the weights of its first ring of
    // k-blocks before it waits for the kernel that makes the activations (and whose reader may still use the output).
    const uint32_t rank = cluster_ctarank();
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int n_x = (p.N + 2 * WM - 1) / (2 * WM), total = n_x * p.n_y;
    const int kb_total = (p.K + BK - 1) / BK;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    constexpr uint32_t W_BYTES = WM * BK * 2, A_BYTES = (BT2 / 2) * BK * 2, STAGE_BYTES = W_BYTES + A_BYTES;
    constexpr int ACC_COLS = BT2;
    __shared__ __align__(8) uint64_t bars[2 * MAX_STAGES + 4];
    __shared__ uint32_t tmem_base_slot;
    const int stages = p.stages;
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[MAX_STAGES]);
    const uint32_t acc_full0 = smem_u32(&bars[2 * MAX_STAGES]), acc_empty0 = smem_u32(&bars[2 * MAX_STAGES + 2]);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(full0 + 8 * s, 1);                   // the leader's: its producer's arrival with both CTAs' bytes
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full0 + 8 * b, 1);
            mbar_init(acc_empty0 + 8 * b, 8);              // the leader's: four epilogue warps of each CTA
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_a) : "memory");
    }
    if (warp == 1) {                                       // the same warp of both CTAs allocates for the pair
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                    // both CTAs' barriers exist before either signals the other
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    pdl_launch();

    if (warp == 0) {
        if (lane == 0) {
            int pre = 0;                                   // k-blocks whose weights went out before the wait
            for (int t = pair; t < total && pre < stages; t += n_pairs) {
                const int n0 = (t % n_x) * 2 * WM + (int)rank * WM;
                for (int i = 0; i < kb_total && pre < stages; ++i, ++pre) {
                    const uint32_t st = smem_u32(smem + (size_t)pre * STAGE_BYTES), fb = full0 + 8 * pre;
                    if (rank == 0) mbar_expect_tx(fb, 2 * STAGE_BYTES);
                    tma_load_2d_pair(st, &tm_w, i * BK, n0, fb);
                }
            }
            pdl_wait();
            int it = 0;
            bool ok = true;
            for (int t = pair; t < total && ok; t += n_pairs) {
                const int n0 = (t % n_x) * 2 * WM + (int)rank * WM, row0 = (t / n_x) * BT2 + (int)rank * (BT2 / 2);
                for (int i = 0; i < kb_total; ++i, ++it) {
                    const int s = it % stages;
                    const uint32_t st = smem_u32(smem + (size_t)s * STAGE_BYTES), fb = full0 + 8 * s;
                    if (it >= pre) {                       // the first ring's stages are fresh and their weights on the way
                        if (!mbar_wait(empty0 + 8 * s, ((it / stages) & 1) ^ 1)) {
                            atomicExch(&g_tc_status, 11);
                            ok = false;
                            break;
                        }
                        if (rank == 0) mbar_expect_tx(fb, 2 * STAGE_BYTES);
                        tma_load_2d_pair(st, &tm_w, i * BK, n0, fb);
                    }
                    tma_load_2d_pair(st + W_BYTES, &tm_a, i * BK, row0, fb);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = umma_idesc_pair(BT2);
            int it = 0, nt = 0;
            bool ok = true;
            for (int t = pair; t < total && ok; t += n_pairs, ++nt) {
                const int buf = nt & 1;
                if (!mbar_wait(acc_empty0 + 8 * buf, ((nt >> 1) & 1) ^ 1)) {
                    atomicExch(&g_tc_status, 14);
                    break;
                }
                tc_fence_after();
                const uint32_t acc_addr = tmem_base + buf * ACC_COLS;
                for (int i = 0; i < kb_total; ++i, ++it) {
                    const int s = it % stages;
                    if (!mbar_wait(full0 + 8 * s, (it / stages) & 1)) {
                        atomicExch(&g_tc_status, 12);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t st = smem_u32(smem + (size_t)s * STAGE_BYTES);
                    const uint64_t dw = umma_desc_sw128(st), da = umma_desc_sw128(st + W_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) umma_bf16_pair(acc_addr, dw + 2 * k, da + 2 * k, idesc, (i | k) != 0);
                    umma_commit_pair(empty0 + 8 * s);
                }
                if (!ok) break;
                umma_commit_pair(acc_full0 + 8 * buf);
            }
        }
    } else {
        const int quarter = warp & 3;
        int nt = 0;
        pdl_wait();                                        // the output may still be in use by the kernel before
        for (int t = pair; t < total; t += n_pairs, ++nt) {
            const int buf = nt & 1;
            if (!mbar_wait(acc_full0 + 8 * buf, (nt >> 1) & 1)) {
                if (lane == 0) atomicExch(&g_tc_status, 13);
                break;
            }
            tc_fence_after();
            const int n = (t % n_x) * 2 * WM + (int)rank * WM + quarter * 32 + lane, tok0 = (t / n_x) * BT2;
            const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * ACC_COLS;
            const int valid = min(BT2, p.rows_total - tok0);
#pragma unroll 1
            for (int c0 = 0; c0 < valid; c0 += 16) {
                float v[16];
                tmem_ld16(lane_addr + c0, v);
                if (c0 + 16 >= valid) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_leader(acc_empty0 + 8 * buf);
                }
                if (n < p.N) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (c0 + j >= valid) break;
                        float* o = (float*)p.out + (size_t)(tok0 + c0 + j) * p.ldo + n;
                        *o = p.epilogue == EPI_ADD ? *o + v[j] : v[j];
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                    // the peer has no MMA, copy or arrival of ours in flight
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

// out[r, n] (=|+=) sum_s partial[s, r, n], s ascending.
__global__ void splitk_reduce_kernel(const float* partial, int splits, size_t count, float* out, int N, int ldo, int add) {
    pdl_enter();
    const size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (i >= count) return;
    float acc = 0.0f;
    for (int s = 0; s < splits; ++s) acc += partial[(size_t)s * count + i];
    const size_t o = (i / N) * ldo + i % N;
    out[o] = add ? out[o] + acc : acc;
}

// ---------------------------------------------------------------------------------------- host
int make_map(CUtensorMap* map, const void* base, long long rows, int K, long long pitch, int box_rows, bool weights) {
    return make_bf16_map(map, base, rows, K, pitch, box_rows, weights, "gemm_tc");
}

// Weight maps do not change between calls: keep them by (address, rows, K).
std::mutex g_map_mutex;
std::map<std::tuple<const void*, long long, int>, CUtensorMap> g_weight_maps;

int weight_map(CUtensorMap* out, const void* base, long long rows, int K) {
    std::lock_guard<std::mutex> lock(g_map_mutex);
    auto key = std::make_tuple(base, rows, K);
    auto it = g_weight_maps.find(key);
    if (it == g_weight_maps.end()) {
        CUtensorMap m;
        if (int rc = make_map(&m, base, rows, K, K, WM, true)) return rc;
        it = g_weight_maps.emplace(key, m).first;
    }
    *out = it->second;
    return 0;
}

int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

// n_y: row tiles, pairs, or the tile list's capacity; n_z: K slices.
template <int BT, bool DUAL>
int launch(const CUtensorMap& tw, const CUtensorMap& tw2, const CUtensorMap& ta, Params p, int n_y, int n_z, cudaStream_t st) {
    constexpr int stage = WM * BK * 2 * (DUAL ? 2 : 1) + BT * BK * 2;
    // narrow token tiles (weight streaming): two CTAs per SM, each with half of the shared memory;
    // wide ones: one CTA per SM whose ring takes all of it
    int per_sm = BT <= 64 ? (220 * 1024) / (stage * 3) : 1;
    per_sm = per_sm < 1 ? 1 : (per_sm > 4 ? 4 : per_sm);
    const long long total = (long long)((p.N + WM - 1) / WM) * n_y * n_z;
    // fewer tiles than that: the CTAs an SM really gets share its memory, so a lone CTA has a ring
    // deep enough to have its whole K slice on the way at once
    const int need = (int)((total + sm_count() - 1) / sm_count());
    if (need < per_sm) per_sm = need < 1 ? 1 : need;
    int stages = ((220 / per_sm) * 1024) / stage;
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    p.stages = stages;
    p.n_y = n_y, p.n_z = n_z;
    const size_t smem = (size_t)stages * stage + 1024;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_tc_kernel<BT, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 1024) != cudaSuccess)
            return q6k_check_launch("gemm_tc: shared memory attribute");
        configured = true;
    }
    const int slots = sm_count() * per_sm;
    const int grid = (int)(total < slots ? total : slots);
    q6k_launch_as(p.tile_group == nullptr || p.lists_old != 0, gemm_tc_kernel<BT, DUAL>, grid, 192, smem, st, tw, tw2, ta, p);
    return q6k_check_launch("gemm_tc");
}

// The CTA-pair kernel: tiles of [256 weights x BT2 tokens], one cluster of two CTAs per SM pair.
template <int BT2>
int launch_pair(const CUtensorMap& tw, const CUtensorMap& ta, Params p, cudaStream_t st) {
    constexpr int stage = WM * BK * 2 + (BT2 / 2) * BK * 2;
    int stages = (200 * 1024) / stage;
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    p.stages = stages;
    p.n_y = (p.rows_total + BT2 - 1) / BT2;
    const size_t smem = (size_t)stages * stage + 1024;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_tc_pair_kernel<BT2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 1024) != cudaSuccess)
            return q6k_check_launch("gemm_tc pair: shared memory attribute");
        configured = true;
    }
    const long long total = (long long)((p.N + 2 * WM - 1) / (2 * WM)) * p.n_y;
    const int pairs = sm_count() / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (unsigned)(total < pairs ? total : pairs)), cfg.blockDim = dim3(192), cfg.dynamicSmemBytes = smem, cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;      // the weights of the first ring are fetched under the kernel before
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr, cfg.numAttrs = q6k_pdl_mode() != 0 ? 2 : 1;
    cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<BT2>, tw, ta, p);
    return q6k_check_launch("gemm_tc pair");
}

// Token tile of the pair kernel for (rows, N), or 0 when the one-CTA kernel serves the product:
// plain dense products with at least 512 rows and 256 weight rows.  Q6K_TC_PAIR=0 switches it off.
static int pair_plan(int rows, int N, int K) {
    static const bool off = [] {
        const char* v = getenv("Q6K_TC_PAIR");
        return v && v[0] == '0';
    }();
    if (off || rows < 512 || N < 2 * WM || K % 8 != 0) return 0;
    const long long n_x = (N + 2 * WM - 1) / (2 * WM), pairs = sm_count() / 2;
    if (n_x * ((rows + 255) / 256) * 2 < pairs) return 0;   // too few tiles for the pairs: the one-CTA kernel narrows its tile
    const long long r256 = (n_x * ((rows + 255) / 256) + pairs - 1) / pairs, r192 = (n_x * ((rows + 191) / 192) + pairs - 1) / pairs;
    return r192 * 192 < r256 * 256 ? 192 : 256;            // the tile that ends the last round earlier
}

}  // namespace

Q6K_API int q6k_tc_status() {
    int v = -1;
    if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof v) != cudaSuccess) return -1;
    return v;
}

Q6K_API int q6k_tc_token_tile(int rows, int dual) {
    const int cap = dual ? 128 : 256;
    for (int bt = 16; bt < cap; bt *= 2)
        if (rows <= bt) return bt;
    return cap;
}

// Bytes of split-K workspace the dense call below may use for (rows, N, K); 0 if it will not split.
static int splits_for(int rows, int N, int K, int bt) {
    const int n_tiles = (N + WM - 1) / WM, row_tiles = (rows + bt - 1) / bt, kb = (K + BK - 1) / BK;
    const int ctas = n_tiles * row_tiles;
    if (ctas * 2 > sm_count() || kb < 4) return 1;
    int s = sm_count() / ctas;                 // fill one wave of the persistent CTAs
    if (s > kb / 2) s = kb / 2;
    if (s < 1) s = 1;
    const int per = (kb + s - 1) / s;          // k-blocks per slice; the slices that are not empty:
    return (kb + per - 1) / per;
}

// Token tile and K slices of a dense product: the widest token tile that holds the rows, narrowed
// while many rows meet so few weight tiles that half of the SMs would idle (the router at prefill);
// K is sliced only when even that leaves most SMs without a tile (a few rows: decode).
static void dense_plan(int rows, int N, int K, bool dual, int* bt, int* splits) {
    int b = q6k_tc_token_tile(rows, dual);
    const int n_tiles = (N + WM - 1) / WM;
    if (!dual && rows >= 512 && n_tiles * ((rows + 127) / 128) * 2 < sm_count()) {
        // many rows on few weight tiles (the router of a prompt portion): tiles of 128 tokens with K sliced over the
        // idle SMs keep the MMAs wide; narrow tiles with the whole K in a row per CTA took 18 us for 2 GFLOP
        const int s = splits_for(rows, N, K, 128);
        if (s > 1) {
            *bt = 128, *splits = s;
            return;
        }
    }
    while (b > 32 && rows > b && n_tiles * ((rows + b - 1) / b) * 2 < sm_count()) b /= 2;
    if (b == 256 && !dual && rows > 256) {
        // the persistent CTAs work in rounds of one tile each: a tile of 192 tokens can need the same
        // number of rounds as one of 256 (q/k/v at 2,048 tokens: 440 tiles against 320, three rounds
        // either way) and then ends a quarter earlier; its narrower MMAs are taken as a tenth dearer
        const long long r256 = ((long long)n_tiles * ((rows + 255) / 256) + sm_count() - 1) / sm_count();
        const long long r192 = ((long long)n_tiles * ((rows + 191) / 192) + sm_count() - 1) / sm_count();
        if (r192 * 192 * 11 < r256 * 256 * 10) b = 192;
    }
    *bt = b;
    *splits = dual ? 1 : splits_for(rows, N, K, b);
}

// Number of K slices the dense call below uses for (rows, N, K).
Q6K_API int q6k_gemm_tc_splits(int rows, int N, int K) {
    int bt, s;
    dense_plan(rows, N, K, false, &bt, &s);
    return s;
}

Q6K_API long long q6k_gemm_tc_workspace(int rows, int N, int K) {
    const int s = q6k_gemm_tc_splits(rows, N, K);
    return s > 1 ? (long long)s * rows * N * 4 : 0;
}

// A: bfloat16 [rows_total, K] with row pitch lda (elements).  W (and W2 for the SwiGLU epilogue):
// bfloat16 [groups, N, K] contiguous.  epilogue: 0 store FP32, 1 add into FP32, 2 SwiGLU -> bfloat16.
// Grouped when tile_group != null: bt is the token tile the tile list was made for.  Dense calls
// may split K over CTAs when the output has too few tiles to fill the GPU; they then need
// `workspace` of q6k_gemm_tc_workspace bytes.  keep_partials != 0: when K is split, the partial
// products stay in the workspace as FP32 [q6k_gemm_tc_splits, rows, N] for the caller's next
// kernel to sum (in slice order) and `out` is not written.
Q6K_API int q6k_gemm_tc(const void* A, long long lda, int rows_total, const void* W, const void* W2, int groups, int N, int K,
                        void* out, int ldo, int epilogue, const int* tile_group, const int* tile_row0,
                        const int* group_offsets, const int* num_tiles, int max_tiles, int bt, float* workspace,
                        long long workspace_bytes, int keep_partials, cudaStream_t st) {
    if (rows_total == 0 || N == 0) return 0;
    Q6K_REQUIRE(rows_total > 0 && N > 0 && K > 0 && groups > 0, "gemm_tc: bad sizes rows=%d N=%d K=%d groups=%d", rows_total, N, K, groups);
    Q6K_REQUIRE(K % 8 == 0 && lda % 8 == 0, "gemm_tc: K=%d and the row pitch %lld must be multiples of 8 (TMA rows start on 16 bytes)", K, lda);
    Q6K_REQUIRE(((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0 && (!W2 || ((uintptr_t)W2 & 15) == 0),
                "gemm_tc: operands must be 16-byte aligned");
    Q6K_REQUIRE(epilogue >= 0 && epilogue <= 2, "gemm_tc: unknown epilogue %d", epilogue);
    const bool dual = epilogue == EPI_SWIGLU;
    Q6K_REQUIRE(!dual || W2, "gemm_tc: the SwiGLU epilogue needs two weight matrices");
    const bool grouped = tile_group != nullptr;
    int planned_splits = 1;
    if (!grouped) dense_plan(rows_total, N, K, dual, &bt, &planned_splits);
    Q6K_REQUIRE(bt == 16 || bt == 32 || bt == 64 || bt == 128 || ((bt == 192 || bt == 256) && !dual), "gemm_tc: token tile %d is not supported", bt);
    Q6K_REQUIRE((long long)groups * N < (1LL << 31), "gemm_tc: weight rows exceed the TMA coordinate range");

    CUtensorMap tw, tw2, ta;
    if (int rc = weight_map(&tw, W, (long long)groups * N, K)) return rc;
    tw2 = tw;
    if (dual)
        if (int rc = weight_map(&tw2, W2, (long long)groups * N, K)) return rc;
    if (!grouped && !dual && planned_splits == 1) {
        if (const int bt2 = pair_plan(rows_total, N, K)) {
            if (int rc = make_map(&ta, A, rows_total, K, lda, bt2 / 2, false)) return rc;
            Params pp{};
            pp.out = out, pp.rows_total = rows_total, pp.N = N, pp.K = K, pp.ldo = ldo, pp.epilogue = epilogue;
            return bt2 == 192 ? launch_pair<192>(tw, ta, pp, st) : launch_pair<256>(tw, ta, pp, st);
        }
    }
    if (int rc = make_map(&ta, A, rows_total, K, lda, bt, false)) return rc;

    Params p{};
    p.out = out;
    p.tile_group = tile_group, p.tile_row0 = tile_row0, p.group_offsets = group_offsets, p.num_tiles = num_tiles;
    p.rows_total = rows_total, p.N = N, p.K = K, p.ldo = ldo, p.epilogue = epilogue;
    // one row tile (dense), or groups of about one row tile each (experts with a prompt portion's rows): every
    // weight tile is fetched once, or by the few row tiles of its group, which lie side by side
    p.w_once = grouped ? (long long)rows_total <= 2LL * groups * bt : rows_total <= 128;
    const int kb = (K + BK - 1) / BK;
    int splits = 1;
    if (!grouped && !dual) {
        splits = planned_splits;
        if (splits > 1 && (!workspace || workspace_bytes < (long long)splits * rows_total * N * 4)) splits = 1;
    }
    p.kb_per_split = (kb + splits - 1) / splits;
    splits = (kb + p.kb_per_split - 1) / p.kb_per_split;
    if (splits > 1) {
        p.partial = workspace;
        p.epilogue = EPI_PARTIAL;
    }
    const int ytiles = grouped ? max_tiles : (rows_total + bt - 1) / bt;
    int rc;
#define GO(BT_)                                                                               \
    case BT_:                                                                                 \
        rc = dual ? launch<(BT_ > 128 ? 128 : BT_), true>(tw, tw2, ta, p, ytiles, splits, st) \
                  : launch<BT_, false>(tw, tw2, ta, p, ytiles, splits, st);                   \
        break;
    switch (bt) {
        GO(16) GO(32) GO(64) GO(128) GO(192) GO(256)
        default: return q6k_fail("gemm_tc: token tile %d", bt);
    }
#undef GO
    if (rc) return rc;
    if (splits > 1 && !keep_partials) {
        const size_t count = (size_t)rows_total * N;
        q6k_launch(splitk_reduce_kernel, (unsigned)((count + 255) / 256), 256, 0, st, workspace, splits, count, (float*)out, N, ldo,
                                                                             epilogue == EPI_ADD);
        return q6k_check_launch("gemm_tc split-K reduce");
    }
    return 0;
}

// Few tokens (decode): one tile per (token, slot) pair instead of a permutation.  pair_expert:
// int32 [pairs] (the router's selection, flattened); pair y multiplies input row y / pair_div of A
// (pair_div = slots per token for the gate/up product, 1 for the down product, whose input rows
// are already per pair) with the weights of expert pair_expert[y] and writes output row y.
// pair_order (int32 [pairs] or null): the order in which the pairs are worked on; sorted by expert
// it lets the tiles of one expert run side by side and find its weights in L2.
// epilogue: 0 store FP32, 2 SwiGLU -> bfloat16.
// K slices of a pair product: only when the pairs are so few that most SMs would have no tile.
static int pair_splits(int pairs, int N, int K) {
    const int tiles = pairs * ((N + WM - 1) / WM), kb = (K + BK - 1) / BK;
    if (tiles * 2 > sm_count() || kb < 8) return 1;
    int s = sm_count() / tiles;
    if (s > kb / 4) s = kb / 4;
    if (s > 8) s = 8;
    if (s < 1) s = 1;
    const int per = (kb + s - 1) / s;
    return (kb + per - 1) / per;
}

// Scratch the pair product below needs when it slices K: floats for the slices' sums and counters
// (which must be zero before the first call; the kernel leaves them zero).
Q6K_API int q6k_gemm_tc_pairs_scratch(int pairs, int N, int K, int dual, long long* floats, int* counters) {
    const int s = pair_splits(pairs, N, K);
    *floats = s > 1 ? (long long)s * pairs * (dual ? 2 : 1) * N : 0;
    *counters = s > 1 ? pairs * ((N + WM - 1) / WM) : 0;
    return 0;
}

Q6K_API int q6k_gemm_tc_pairs(const void* A, long long lda, int a_rows, const void* W, const void* W2, int groups, int N, int K,
                              void* out, int ldo, int epilogue, const int* pair_expert, const int* pair_order, int pairs, int pair_div,
                              float* partial, long long partial_floats, unsigned* tickets, int n_tickets, int lists_old, cudaStream_t st) {
    if (pairs == 0 || N == 0) return 0;
    Q6K_REQUIRE(a_rows > 0 && N > 0 && K > 0 && groups > 0 && pairs > 0 && pair_div > 0, "gemm_tc_pairs: bad sizes rows=%d N=%d K=%d pairs=%d", a_rows, N, K, pairs);
    Q6K_REQUIRE(K % 8 == 0 && lda % 8 == 0, "gemm_tc_pairs: K=%d and the row pitch %lld must be multiples of 8", K, lda);
    Q6K_REQUIRE(((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0 && (!W2 || ((uintptr_t)W2 & 15) == 0), "gemm_tc_pairs: operands must be 16-byte aligned");
    Q6K_REQUIRE(epilogue == EPI_STORE || epilogue == EPI_SWIGLU, "gemm_tc_pairs: unknown epilogue %d", epilogue);
    const bool dual = epilogue == EPI_SWIGLU;
    Q6K_REQUIRE(!dual || W2, "gemm_tc_pairs: the SwiGLU epilogue needs two weight matrices");
    Q6K_REQUIRE((long long)groups * N < (1LL << 31), "gemm_tc_pairs: too many weight rows");
    CUtensorMap tw, tw2, ta;
    if (int rc = weight_map(&tw, W, (long long)groups * N, K)) return rc;
    tw2 = tw;
    if (dual)
        if (int rc = weight_map(&tw2, W2, (long long)groups * N, K)) return rc;
    if (int rc = make_map(&ta, A, a_rows, K, lda, 16, false)) return rc;
    Params p{};
    p.out = out, p.tile_group = pair_expert, p.rows_total = a_rows, p.N = N, p.K = K, p.ldo = ldo, p.epilogue = epilogue;
    const int kb = (K + BK - 1) / BK;
    int splits = pair_splits(pairs, N, K);
    if (splits > 1) {
        long long need_f;
        int need_c;
        q6k_gemm_tc_pairs_scratch(pairs, N, K, dual, &need_f, &need_c);
        if (!partial || !tickets || partial_floats < need_f || n_tickets < need_c) splits = 1;      // no scratch given: whole K per tile
    }
    p.kb_per_split = (kb + splits - 1) / splits;
    p.partial = partial, p.tickets = tickets;
    p.pair_div = pair_div;
    p.pair_order = pair_order;
    p.lists_old = lists_old;
    p.w_once = 1;                          // a pair's weight tile is shared with the few pairs of the same expert, which run side by side
    return dual ? launch<16, true>(tw, tw2, ta, p, pairs, splits, st) : launch<16, false>(tw, tw2, ta, p, pairs, splits, st);
}
