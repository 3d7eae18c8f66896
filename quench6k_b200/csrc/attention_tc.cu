// bfloat16 attention for prompt portions on the 5th-generation tensor cores: both products of
// every key tile (S = Q K^T and O += P V) are tcgen05.mma with their accumulators in tensor
// memory; K and V pages come in by TMA.  sm_100a only; head size 128.
//
// Arithmetic as the reference's attn_kernel (crates/cuda/kernels/flint.cu:211-529): scores in base 2
// with scale * log2 e folded in, causal and window mask per row, online softmax per key tile,
// probabilities rounded to bfloat16 before they are summed, the sink added to the denominator at
// the end (:505-526).  The reference computes it with mma.sync tiles of 64 or 128 rows; here:
//
// A CTA takes up to 256 query rows of one request and one KV head as two halves of 128 (row =
// token_in_half * G + head_in_group) and walks key tiles of 128 keys, which both halves share.
//   warp 0      producers: one lane brings the K tiles, another the V tiles, as TMA boxes
//               [page rows x 64] into rings of three and two tiles ([2 column halves][128 keys]
//               [128 bytes], 128-byte swizzle; keys without a page are zero-filled through an
//               out-of-range coordinate)
//   warp 1      one thread issues the MMAs, for each half in turn: S_h = Q_h K_i^T (8 x K=16, both
//               operands K-major in shared memory) and, when P_h is in tensor memory, O_h += P_h V_i
//               (8 x K=16, P as the operand from tensor memory, V as an MN-major operand)
//   warps 2-5   softmax of half 0, warps 6-9 of half 1: one thread per query row reads its row of S
//               from tensor memory (tcgen05.ld, no shuffles), keeps the running max and sum, rescales
//               O in tensor memory when the max has grown by more than 2^8, writes P as bfloat16
//               into tensor memory over the scores (tcgen05.st), and finally normalises O.  While one
//               half's softmax runs, the other half's products keep the tensor pipe busy.
// Tensor memory: S_0 (and P_0) at columns 0..127, S_1 at 128..255, O_0 at 256..383, O_1 at 384..511.
// Every wait on an mbarrier is bounded and records a code in a status word when it runs out.
#include <map>
#include <tuple>

#include "common.cuh"
#include "tma.cuh"

namespace {

constexpr int HD = 128;                      // head size
constexpr int BM = 128;                      // query rows per tile
constexpr int BN = 128;                      // keys per key tile
constexpr float LOG2E = 1.4426950408889634f;
constexpr uint32_t HALF_BYTES = 128 * 128;   // one 64-column half of a [128 x 128] bf16 tile
constexpr uint32_t TILE_BYTES = 2 * HALF_BYTES;
constexpr int KS = 3, VS = 2;                // stages of the K and of the V ring

struct TcAttnParams {
    const __nv_bfloat16* q;                  // [T, Hq, HD]
    const int* block_table;                  // [R, max_blocks]
    const int* req_of_token;
    const int* positions;
    const int* tile_tok0;
    const int* tile_ntok;
    const float* sinks;                      // [Hq] or null
    __nv_bfloat16* out;                      // [T, Hq*HD]
    int max_blocks, page_size, window, Hq, Hkv, G, pool_rows, num_pages;
    float scale_log2;
};

__device__ int g_attn_tc_status = 0;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}

// K-major operand, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
// MN-major operand (V: for one key the head dimensions are contiguous), 128-byte swizzle: 64
// elements of N per 128-byte row, the next 64 elements of N HALF_BYTES further (leading offset),
// 8-key groups 1024 bytes apart (stride offset).
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(HALF_BYTES >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
// D FP32, A and B bfloat16, M = 128, N = 128; b_mn: B is MN-major.
__host__ __device__ constexpr uint32_t idesc_128x128(bool b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
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

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, "
        "%20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// The same without the wait: several loads may be in flight; tmem_ld_wait() before any value is used.
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, float* v) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, "
        "%20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, "
        "%20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
        "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
        "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
        "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 2^x by the special-function unit: 2^-inf = 0, no range fix-ups (arguments here are <= 8).
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 2^x on the FMA pipe for x <= 8: round(x) goes into the exponent, a cubic gives 2^f on [-0.5, 0.5]
// (relative error 7.5e-5, far below the bfloat16 rounding that follows).  x below -126 counts as
// -126 (2^-126 instead of 0: nothing a sum or a product can see).  A quarter of a tile's
// exponentials go this way so that the special-function unit is not the only one that works.
__device__ __forceinline__ float ex2_poly(float x) {
    x = fmaxf(x, -126.0f);
    const float t = x + 12582912.0f;              // 1.5 * 2^23: the integer nearest to x in the low mantissa bits
    const float f = x - (t - 12582912.0f);
    float q = fmaf(0.05517157f, f, 0.24261111f);
    q = fmaf(q, f, 0.69326103f);
    q = fmaf(q, f, 0.99992806f);
    return __int_as_float(__float_as_int(q) + (__float_as_int(t) << 23));
}

// Byte offset of 16-byte chunk c (0..15) of row r in a [2 halves][128 rows][128 bytes] swizzled tile.
__device__ __forceinline__ uint32_t swz(int r, int c) { return (uint32_t)((c >> 3) * HALF_BYTES + r * 128 + (((c & 7) ^ (r & 7)) << 4)); }

// O += P V with P read from tensor memory (lanes = query rows, two keys per 32-bit column).
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t}" ::"r"(tmem_d),
        "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]),
        "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}

constexpr int TC_THREADS = 320;

__global__ void __launch_bounds__(TC_THREADS) attention_tc_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                                                                  const __grid_constant__ CUtensorMap tm_k_run,
                                                                  const __grid_constant__ CUtensorMap tm_v_run, const TcAttnParams p) {
    pdl_enter();
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    // [Q of half 0][Q of half 1][K0][K1][K2][V0][V1], each a [2][128][128 B] tile of 32 KB
    const uint32_t q_s = smem_u32(smem), k_s = q_s + 2 * TILE_BYTES, v_s = k_s + KS * TILE_BYTES;
    __shared__ __align__(8) uint64_t bars[22];
    __shared__ uint32_t tmem_slot;
    const uint32_t k_full0 = smem_u32(&bars[0]), k_empty0 = smem_u32(&bars[3]), v_full0 = smem_u32(&bars[6]), v_empty0 = smem_u32(&bars[8]);
    const uint32_t s_full0 = smem_u32(&bars[10]), p_full0 = smem_u32(&bars[12]), pv_done0 = smem_u32(&bars[14]), q_full0 = smem_u32(&bars[16]), p_full1 = smem_u32(&bars[18]);

    // the KV heads of a tile side by side, the tiles in the order of the list (the host puts those with the
    // most keys first, so that the long ones of every head start in the first wave of CTAs)
    const int tile = blockIdx.y, kh = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = p.G;
    // the two halves: two tiles of one request (their tokens, positions and ranges of key tiles);
    // the second may be empty.  The K/V stream covers the union of the ranges.
    const int tok_h0 = p.tile_tok0[2 * tile], tok_h1 = p.tile_tok0[2 * tile + 1];
    int nt_h[2] = {p.tile_ntok[2 * tile], p.tile_ntok[2 * tile + 1]}, pf[2], pl[2], first_h[2], end_h[2], lo_h[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        pf[h] = nt_h[h] > 0 ? p.positions[h == 0 ? tok_h0 : tok_h1] : 0;
        pl[h] = pf[h] + nt_h[h] - 1;
        lo_h[h] = p.window > 0 ? max(0, pf[h] - p.window + 1) : 0;
        first_h[h] = nt_h[h] > 0 ? lo_h[h] / BN : 0;
        end_h[h] = nt_h[h] > 0 ? pl[h] / BN + 1 : 0;
    }
    const int* bt = p.block_table + (size_t)p.req_of_token[tok_h0] * p.max_blocks;
    const bool two = nt_h[1] > 0;
    const int pos_last = two ? max(pl[0], pl[1]) : pl[0];
    const int k_lo = two ? min(lo_h[0], lo_h[1]) : lo_h[0];
    const int u_first = two ? min(first_h[0], first_h[1]) : first_h[0], u_end = max(end_h[0], end_h[1]), n_union = u_end - u_first;
    auto active = [&](int h, int i) { return i >= first_h[h] && i < end_h[h]; };

    if (tid == 0) {
        for (int s = 0; s < KS; ++s) {
            mbar_init(k_full0 + 8 * s, 1);
            mbar_init(k_empty0 + 8 * s, 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(v_full0 + 8 * s, 1);
            mbar_init(v_empty0 + 8 * s, 1);
            mbar_init(s_full0 + 8 * s, 1);
            mbar_init(p_full0 + 8 * s, 128);
            mbar_init(p_full1 + 8 * s, 128);
            mbar_init(pv_done0 + 8 * s, 1);
            mbar_init(q_full0 + 8 * s, 128);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_k) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_v) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_k_run) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_v_run) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;

    if (warp == 0) {
        // ---- producers: lane 0 brings the K tiles, lane 1 the V tiles (each at its ring's pace)
        if (lane < 2) {
            const bool is_k = lane == 0;
            const int ps = p.page_size, ring = is_k ? KS : VS;
            const uint32_t full0 = is_k ? k_full0 : v_full0, empty0 = is_k ? k_empty0 : v_empty0, base = is_k ? k_s : v_s;
            const CUtensorMap* map = is_k ? &tm_k : &tm_v;
            const CUtensorMap* map_run = is_k ? &tm_k_run : &tm_v_run;
            constexpr int RUN = 64;                                      // keys per run box
            for (int i = 0; i < n_union; ++i) {
                const int s = i % ring;
                if (!mbar_wait(empty0 + 8 * s, ((i / ring) & 1) ^ 1)) {
                    atomicExch(&g_attn_tc_status, 1);
                    break;
                }
                const uint32_t fb = full0 + 8 * s;
                mbar_expect_tx(fb, TILE_BYTES);
                const int j0 = (u_first + i) * BN;
                const uint32_t dst = base + s * TILE_BYTES;
                // pages with consecutive numbers are contiguous for one head (head-major pools): where the
                // pages of 64 keys form such a run, each half comes in as one box instead of one per page
                for (int r = 0; r < BN / RUN; ++r) {
                    const int jr = j0 + r * RUN;
                    bool run = ps < RUN && jr >= k_lo && jr / ps + RUN / ps <= p.max_blocks;
                    int first = -1;
                    if (run) {
                        first = bt[jr / ps];
                        run = first >= 0;
                        for (int b = 1; b < RUN / ps && run; ++b) run = bt[jr / ps + b] == first + b;
                    }
                    if (run) {
                        const int y = (kh * p.num_pages + first) * ps;
#pragma unroll
                        for (int h = 0; h < 2; ++h) tma_load_2d(dst + h * HALF_BYTES + r * RUN * 128, map_run, h * 64, y, fb);
                        continue;
                    }
                    const int per = ps < RUN ? RUN / ps : 1, bx = ps < RUN ? ps : RUN;      // boxes of this 64-key part
                    for (int b = 0; b < per; ++b) {
                        const int j = jr + b * bx;
                        int y = p.pool_rows;                             // out of range: zeros
                        if (j + bx > k_lo && j <= pos_last) {
                            const int page = bt[j / ps];
                            if (page >= 0) y = (kh * p.num_pages + page) * ps + j % ps;
                        }
#pragma unroll
                        for (int h = 0; h < 2; ++h) tma_load_2d(dst + h * HALF_BYTES + (r * RUN + b * bx) * 128, map, h * 64, y, fb);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer.  For key tile r: O_h += P_h V_r as soon as half h's probabilities are in
        // tensor memory, then at once S_h = Q_h K_(r+1)^T into the columns P_h has just been read
        // from (the tensor pipe runs its instructions in the order of issue), half 0 and half 1 in
        // turn: while one half's softmax runs, the other half's products do.
        if (lane == 0) {
            constexpr uint32_t idesc_s = idesc_128x128(false), idesc_o = idesc_128x128(true);
            int pv_cnt[2] = {0, 0};
            bool q_ready[2] = {false, false}, ok = true;
            auto issue_qk = [&](int h, int r) {
                if (!q_ready[h]) {
                    if (!mbar_wait(q_full0 + 8 * h, 0)) {
                        atomicExch(&g_attn_tc_status, 2);
                        ok = false;
                        return;
                    }
                    q_ready[h] = true;
                    tc_fence_after();
                }
                const uint32_t k_src = k_s + (r % KS) * TILE_BYTES, q_src = q_s + h * TILE_BYTES;
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint32_t off = (k >> 2) * HALF_BYTES + (k & 3) * 32;
                    umma(tmem + h * BN, desc_k_major(q_src + off), desc_k_major(k_src + off), idesc_s, k != 0);
                }
                umma_commit(s_full0 + 8 * h);
            };
            if (n_union > 0) {
                if (!mbar_wait(k_full0, 0)) {
                    atomicExch(&g_attn_tc_status, 3);
                    ok = false;
                }
                tc_fence_after();
                for (int h = 0; h < 2 && ok; ++h)
                    if (active(h, u_first)) issue_qk(h, 0);
                if (ok) umma_commit(k_empty0);
            }
            for (int r = 0; r < n_union && ok; ++r) {
                const int i = u_first + r, vs = r % VS;
                const bool next = r + 1 < n_union;
                if (!mbar_wait(v_full0 + 8 * vs, (r / VS) & 1) || (next && !mbar_wait(k_full0 + 8 * ((r + 1) % KS), ((r + 1) / KS) & 1))) {
                    atomicExch(&g_attn_tc_status, 3);
                    break;
                }
                tc_fence_after();
                const uint32_t v_src = v_s + vs * TILE_BYTES;
                for (int h = 0; h < 2 && ok; ++h) {
                    if (active(h, i)) {
                        if (!mbar_wait(p_full0 + 8 * h, pv_cnt[h] & 1)) {
                            atomicExch(&g_attn_tc_status, 4);
                            ok = false;
                            break;
                        }
                        tc_fence_after();
#pragma unroll
                        for (int k = 0; k < BN / 32; ++k)     // A: 16 keys = 8 columns of P; B: V, MN-major, 16 keys = 2048 bytes
                            umma_ts(tmem + 256 + h * HD, tmem + h * BN + k * 8, desc_mn_major(v_src + k * 2048), idesc_o, (pv_cnt[h] | k) != 0);
                        if (!mbar_wait(p_full1 + 8 * h, pv_cnt[h] & 1)) {      // the second 64 keys
                            atomicExch(&g_attn_tc_status, 4);
                            ok = false;
                            break;
                        }
                        tc_fence_after();
#pragma unroll
                        for (int k = BN / 32; k < BN / 16; ++k)
                            umma_ts(tmem + 256 + h * HD, tmem + h * BN + k * 8, desc_mn_major(v_src + k * 2048), idesc_o, 1u);
                        umma_commit(pv_done0 + 8 * h);
                        ++pv_cnt[h];
                    }
                    if (next && active(h, i + 1)) issue_qk(h, r + 1);
                }
                if (!ok) break;
                umma_commit(v_empty0 + 8 * vs);
                if (next) umma_commit(k_empty0 + 8 * ((r + 1) % KS));
            }
        }
    } else {
        // ---- softmax, correction, epilogue: two warpgroups, one per half; thread = query row
        const int h = (warp - 2) >> 2;
        const int quarter = warp & 3, row = quarter * 32 + lane, st = tid - 64 - 128 * h;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const uint32_t s_addr = tmem + lane_base + h * BN, o_addr = tmem + lane_base + 256 + h * HD;
        const int ntk = nt_h[h], tokh = h == 0 ? tok_h0 : tok_h1, tok0 = tok_h0;
        // Q of this half (zero rows past its tokens), by cp.async into the swizzled layout
        for (int idx = st; idx < BM * 16; idx += 128) {
            const int r = idx >> 4, c = idx & 15, tt = r / G, hg = r % G;
            const bool valid = tt < ntk;
            const __nv_bfloat16* src = p.q + ((size_t)(valid ? tokh + tt : tok0) * p.Hq + kh * G + hg) * HD + c * 8;
            cp_async16(q_s + h * TILE_BYTES + swz(r, c), src, valid);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive(q_full0 + 8 * h);

        const int tt = row / G, hg = row % G;
        const bool row_valid = tt < ntk;
        const int pos = pf[h] + tt;
        const int lim_hi = row_valid ? pos : -1, lim_lo = p.window > 0 ? pos - p.window + 1 : 0;
        const int n_mine = end_h[h] - first_h[h];
        float m = -INFINITY, l = 0.0f;
        bool ok = true;
        for (int t = 0; t < n_mine; ++t) {
            const int i = first_h[h] + t, j0 = i * BN;
            // S of this tile exists; the commit that says so came after every earlier product of the
            // issuer, so O holds the previous tile's sum and the previous P has been read
            if (!mbar_wait(s_full0 + 8 * h, t & 1)) {
                if (lane == 0) atomicExch(&g_attn_tc_status, 5);
                ok = false;
                break;
            }
            tc_fence_after();
            // tiles that every row of the half sees whole (below the diagonal, inside the window) need no mask
            const bool whole = j0 + BN - 1 <= pf[h] && (p.window == 0 || j0 >= pl[h] - p.window + 1);
            // the row's 128 scores come into registers with one wait; masked ones become -inf
            float v[BN];
#pragma unroll
            for (int c = 0; c < BN / 32; ++c) tmem_ld32_issue(s_addr + c * 32, v + c * 32);
            tmem_ld_wait();
            if (!whole) {
#pragma unroll
                for (int x = 0; x < BN; ++x) {
                    const int j = j0 + x;
                    v[x] = (j <= lim_hi && j >= lim_lo) ? v[x] : -INFINITY;
                }
            }
            float mx16[16];                              // sixteen independent chains, then a tree
#pragma unroll
            for (int x = 0; x < 16; ++x) mx16[x] = fmaxf(v[x], v[x + 16]);
#pragma unroll
            for (int y = 32; y < BN; y += 16) {
#pragma unroll
                for (int x = 0; x < 16; ++x) mx16[x] = fmaxf(mx16[x], v[y + x]);
            }
#pragma unroll
            for (int w = 8; w >= 1; w >>= 1) {
#pragma unroll
                for (int x = 0; x < w; ++x) mx16[x] = fmaxf(mx16[x], mx16[x + w]);
            }
            float mx = mx16[0];
            mx *= p.scale_log2;                          // the scale is positive: max commutes with it
            // The reference point of the exponentials follows the running maximum lazily: it moves
            // only when the maximum has grown by more than 2^8, so O in tensor memory is rescaled
            // rarely; probabilities then reach at most 256, which bfloat16 and the FP32 sums hold.
            float ref = m, corr = 1.0f;
            if (mx > m + 8.0f || m == -INFINITY) {
                ref = fmaxf(m, mx);
                corr = (m == -INFINITY) ? 1.0f : exp2f(m - ref);
            }
            if (t > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll 1
                for (int c = 0; c < HD / 32; ++c) {
                    float o[32];
                    tmem_ld32(o_addr + c * 32, o);
#pragma unroll
                    for (int x = 0; x < 32; ++x) o[x] *= corr;
                    tmem_st32(o_addr + c * 32, o);
                }
            }
            // probabilities p = 2^(s * scale - ref), rounded to bfloat16 before they are summed, into
            // tensor memory over the scores they came from (two keys per column: the 32 keys of chunk c
            // go to columns 16c..16c+15); a masked score is -inf and gives 0; so does a row without
            // any key yet (ref = -inf)
            const float neg_ref = ref == -INFINITY ? 0.0f : -ref;
            const bool last_tile_zero = i == u_end - 1 && (pos_last + 1) % BN != 0;
            auto zero_v_tail = [&]() {
                // the last page came in whole: clear the V rows past the last key (0 * stale NaN); both
                // halves may do so, with the same zeros, before either lets its product start
                const int r = i - u_first;
                if (!mbar_wait(v_full0 + 8 * (r % VS), (r / VS) & 1)) {
                    if (lane == 0) atomicExch(&g_attn_tc_status, 7);
                    ok = false;
                    return;
                }
                const uint32_t v_off = (v_s - q_s) + (r % VS) * TILE_BYTES;
                const int r0 = pos_last + 1 - j0;
                for (int idx = r0 * 16 + st; idx < BN * 16; idx += 128)
                    *reinterpret_cast<uint4*>(smem + v_off + swz(idx >> 4, idx & 15)) = make_uint4(0, 0, 0, 0);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            };
            float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t packed[16];
#pragma unroll
                for (int x = 0; x < 32; x += 2) {
                    const float x0 = fmaf(v[c * 32 + x], p.scale_log2, neg_ref), x1 = fmaf(v[c * 32 + x + 1], p.scale_log2, neg_ref);
                    const bool poly = ((x >> 1) & 3) == 3;          // known at compile time: the loop is unrolled
                    const float p0 = poly ? ex2_poly(x0) : ex2_approx(x0), p1 = poly ? ex2_poly(x1) : ex2_approx(x1);
                    const __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
                    const uint32_t bits = *reinterpret_cast<const uint32_t*>(&pb);
                    sum4[(x >> 1) & 1] += __uint_as_float(bits << 16);
                    sum4[2 + ((x >> 1) & 1)] += __uint_as_float(bits & 0xffff0000u);
                    packed[x >> 1] = bits;
                }
                tmem_st16(s_addr + c * 16, packed);
                if (c == 1) {
                    // the first 64 keys' probabilities are complete: their part of the product may start
                    if (last_tile_zero) {
                        zero_v_tail();
                        if (!ok) break;
                    }
                    tmem_st_wait();
                    tc_fence_before();
                    mbar_arrive(p_full0 + 8 * h);
                }
            }
            if (!ok) break;
            const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            l = l * corr + sum;
            m = ref;
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(p_full1 + 8 * h);
        }
        if (ok && n_mine > 0) {
            if (!mbar_wait(pv_done0 + 8 * h, (n_mine - 1) & 1)) {
                if (lane == 0) atomicExch(&g_attn_tc_status, 8);
                ok = false;
            }
            tc_fence_after();
        }
        if (ok && n_mine > 0) {
            // every lane takes part in the aligned tensor-memory loads; only rows of real tokens store
            float osc = 1.0f, den = l;
            if (p.sinks && row_valid) {
                const float sk = p.sinks[kh * G + hg] * LOG2E, Mx = fmaxf(m, sk);
                osc = exp2f(m - Mx);
                den = l * osc + exp2f(sk - Mx);
            }
            const float inv = row_valid ? osc / den : 0.0f;
            __nv_bfloat16* dst = p.out + ((size_t)(row_valid ? tokh + tt : tok0) * p.Hq + kh * G + hg) * HD;
#pragma unroll 1
            for (int c = 0; c < HD / 32; ++c) {
                float o[32];
                tmem_ld32(o_addr + c * 32, o);
                uint32_t packed[16];
#pragma unroll
                for (int x = 0; x < 32; x += 2) {
                    const __nv_bfloat162 pb = __floats2bfloat162_rn(o[x] * inv, o[x + 1] * inv);
                    packed[x >> 1] = *reinterpret_cast<const uint32_t*>(&pb);
                }
                if (row_valid) {
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4)
                        *reinterpret_cast<uint4*>(dst + c * 32 + q4 * 8) = make_uint4(packed[q4 * 4], packed[q4 * 4 + 1], packed[q4 * 4 + 2], packed[q4 * 4 + 3]);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}

std::mutex g_tc_pool_mutex;
std::map<std::tuple<const void*, long long, int>, CUtensorMap> g_tc_pool_maps;

int tc_pool_map(CUtensorMap* out, const void* base, long long rows, int box_rows) {
    std::lock_guard<std::mutex> lock(g_tc_pool_mutex);
    auto key = std::make_tuple(base, rows, box_rows);
    auto it = g_tc_pool_maps.find(key);
    if (it == g_tc_pool_maps.end()) {
        CUtensorMap m;
        if (int rc = make_bf16_map(&m, base, rows, HD, HD, box_rows, true, "attention_tc")) return rc;
        it = g_tc_pool_maps.emplace(key, m).first;
    }
    *out = it->second;
    return 0;
}

}  // namespace

Q6K_API int q6k_attention_tc_status() {
    int v = -1;
    if (cudaMemcpyFromSymbol(&v, g_attn_tc_status, sizeof v) != cudaSuccess) return -1;
    return v;
}

// Tokens one half of a CTA may hold: 128 // G (128 query rows).
Q6K_API int q6k_attention_tc_tile_tokens(int G) { return G >= 1 && G <= BM ? BM / G : 0; }

// Whether the kernel covers these sizes: head size 128, up to 128 rows per half (G <= 128), pages
// of 8, 16, 32, 64 or 128 keys.
Q6K_API int q6k_attention_tc_supported(int hd, int G, int page_size) {
    return hd == HD && G >= 1 && G <= BM && page_size >= 8 && page_size <= BN && BN % page_size == 0;
}

// q: bfloat16 [T, Hq, 128]; pages: bfloat16 [Hkv, num_pages, page_size, 128]; tile_tok0 / tile_ntok:
// [n_tiles, 2], for each CTA two tiles of one request, each of at most q6k_attention_tc_tile_tokens(G)
// tokens at consecutive positions (the second may have no tokens); tiles whose key ranges overlap
// share the K/V stream (for causal attention without a window: a late tile with an early one); out: bfloat16 [T, Hq*128].  Every tile reads its whole
// key range (no key splits): the kernel for prompt portions.
Q6K_API int q6k_attention_tc(const void* q, const void* k_pages, const void* v_pages, long long num_pages, const int* block_table,
                             int max_blocks, int page_size, const int* req_of_token, const int* positions, const int* tile_tok0,
                             const int* tile_ntok, int n_tiles, int window, const float* sinks, float scale, void* out, int Hq, int Hkv,
                             int hd, cudaStream_t st) {
    if (n_tiles == 0) return 0;
    Q6K_REQUIRE(Hq > 0 && Hkv > 0 && Hq % Hkv == 0, "attention_tc: bad head counts Hq=%d Hkv=%d", Hq, Hkv);
    const int G = Hq / Hkv;
    Q6K_REQUIRE(q6k_attention_tc_supported(hd, G, page_size), "attention_tc: head_dim %d / group size %d / page size %d is not covered", hd, G, page_size);
    Q6K_REQUIRE(max_blocks > 0 && window >= 0 && n_tiles <= 65535, "attention_tc: bad max_blocks %d / window %d / %d tiles", max_blocks, window, n_tiles);
    const long long pool_rows = num_pages * Hkv * page_size;
    Q6K_REQUIRE(pool_rows < (1LL << 31) && ((uintptr_t)k_pages & 15) == 0 && ((uintptr_t)v_pages & 15) == 0 && ((uintptr_t)q & 15) == 0 &&
                    ((uintptr_t)out & 15) == 0,
                "attention_tc: pools too large for TMA coordinates or operands not 16-byte aligned");
    TcAttnParams p{};
    p.q = (const __nv_bfloat16*)q, p.block_table = block_table, p.req_of_token = req_of_token, p.positions = positions;
    p.tile_tok0 = tile_tok0, p.tile_ntok = tile_ntok, p.sinks = sinks, p.out = (__nv_bfloat16*)out;
    p.max_blocks = max_blocks, p.page_size = page_size, p.window = window, p.Hq = Hq, p.Hkv = Hkv, p.G = G;
    p.pool_rows = (int)pool_rows, p.num_pages = (int)num_pages, p.scale_log2 = scale * LOG2E;
    CUtensorMap tk, tv, tk_run, tv_run;
    const int box = page_size < 64 ? page_size : 64;       // pages of 128 keys are fetched as two boxes of 64
    if (int rc = tc_pool_map(&tk, k_pages, pool_rows, box)) return rc;
    if (int rc = tc_pool_map(&tv, v_pages, pool_rows, box)) return rc;
    if (int rc = tc_pool_map(&tk_run, k_pages, pool_rows, 64)) return rc;
    if (int rc = tc_pool_map(&tv_run, v_pages, pool_rows, 64)) return rc;
    const size_t smem = (2 + KS + VS) * TILE_BYTES + 1024;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return q6k_check_launch("attention_tc: shared memory attribute");
        configured = true;
    }
    q6k_launch(attention_tc_kernel, dim3(Hkv, n_tiles), TC_THREADS, smem, st, tk, tv, tk_run, tv_run, p);
    return q6k_check_launch("attention_tc");
}
