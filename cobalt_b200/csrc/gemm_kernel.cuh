// Prefill GEMM: Y[m, k] = sum_j bf16(W[k, j]) * X[m, j] with tcgen05.mma, accumulators in
// tensor memory.
//
// One CTA owns 128 weight rows and up to 512 tokens.  Per 64-column stage it forms
//   D0[128 x n0] += A[128 x 64] * B0[n0 x 64]^T      D1[128 x n1] += A * B1[n1 x 64]^T
// (n0, n1 <= 256 tokens; bf16 operands, fp32 accumulators in 2 x 256 TMEM columns), so a weight
// tile is dequantised once per 512 tokens.  Both operands are K-major in shared memory with the
// 128-byte swizzle.
//
//   warps 0-7  decode: two groups of four warps take alternate stages; thread r of a group owns
//              weight row r.  It reads the row's bitmask words and code bits straight from the
//              tile image in global memory (next stage prefetched into registers), expands the 64
//              columns of the stage to bf16 (decode_core.cuh) and writes eight swizzled 16-byte
//              chunks into the A stage.  After the main loop the same warps drain TMEM (warp w
//              reads lanes 32*(w%4).., accumulator w/4) and store the outputs.
//   warp 8     one elected lane issues the TMA loads of the activation stage (2-D tensor map,
//              box 64 columns x 256 tokens, 128-byte swizzle, rows beyond M zero-filled).
//   warp 9     one elected lane issues tcgen05.mma and tcgen05.commit.
//
// Generic-proxy writes to A stages are published with fence.proxy.async before the mbarrier
// arrive.  Every wait is bounded: on expiry the kernel records a status code, stops issuing
// work, frees its tensor memory and returns.  With split-K (small grids) every CTA writes its
// fp32 tile to scratch and the last CTA of a tile adds the splits in order.
//
// Behaviour replaced: cbk::gemm_tile (mma.sync m16n8k16, per-fragment bf16x2 dequantisation,
// src/cobaltkernel/csrc/cobalt_gemm.cuh:243-609) driven by gemm_phase
// (src/cobaltkernel/csrc/prefill_kernel.cu:103-150).
#pragma once
#include <cuda.h>
#include "common.cuh"
#include "gemv_kernel.cuh"   // finish_output

namespace cb {

constexpr int GEMM_ROWS = 128;            // UMMA M
constexpr int GEMM_NT = 256;              // UMMA N (tokens per accumulator)
constexpr int GEMM_ACCS = 2;              // accumulators per CTA -> 512 tokens
constexpr int GEMM_TOKENS = GEMM_NT * GEMM_ACCS;
constexpr int GEMM_KS = 64;               // columns per stage = one 128-byte swizzle row of bf16
constexpr int GEMM_RB = GEMM_ROWS / TILE_ROWS;   // 8 row blocks per CTA
constexpr int GEMM_LUT_COPIES = 8;
constexpr int GEMM_A_STAGES = 3;
constexpr int GEMM_B_STAGES = 2;
constexpr int GEMM_DECODE_THREADS = 256;
constexpr int GEMM_THREADS = GEMM_DECODE_THREADS + 64;
constexpr uint32_t GEMM_LUT_BYTES = LUT_ENTRIES * GEMM_LUT_COPIES * 8;   // 16 KB
constexpr uint32_t GEMM_A_BYTES = GEMM_ROWS * GEMM_KS * 2;               // 16 KB
constexpr uint32_t GEMM_BHALF_BYTES = GEMM_NT * GEMM_KS * 2;             // 32 KB
constexpr uint32_t GEMM_B_BYTES = GEMM_BHALF_BYTES * GEMM_ACCS;          // 64 KB
constexpr uint32_t GEMM_BAR_BYTES = 256;
constexpr uint32_t GEMM_SMEM_BYTES = GEMM_A_STAGES * GEMM_A_BYTES + GEMM_B_STAGES * GEMM_B_BYTES + GEMM_LUT_BYTES +
                                     GEMM_BAR_BYTES + 1024;

struct GemmParams {
    MatView W;
    uint16_t* y; int64_t ldy;
    float* y32;                 // when set, raw fp32 sums go here instead (no bias, no rounding)
    const uint16_t* bias;
    int M;
    int tok_per_cta;            // tokens per CTA: 512, or less (multiple of 16) to spread a small problem over more SMs
    int splits;                 // split-K factor (column tiles are divided among blockIdx.z)
    float* partials;            // [tile][split][GEMM_TOKENS][GEMM_ROWS] fp32 (splits > 1)
    uint32_t* counters;         // [tile]
    uint32_t* status;
};

// ---- tcgen05 / TMA wrappers
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// 2-D tiled TMA load (no multicast): box of the tensor map at (x = column, y = token) -> shared
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}

// K-major, 128-byte swizzle, 8-row groups 1024 B apart; descriptor version 1 (sm_100)
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);        // start address
    d |= (uint64_t)1 << 16;                               // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                     // stride byte offset
    d |= (uint64_t)1 << 46;                               // version
    d |= (uint64_t)2 << 61;                               // SWIZZLE_128B
    return d;
}
// D = f32, A = B = bf16, both K-major, M = 128, N = n
__device__ __forceinline__ uint32_t umma_idesc(uint32_t n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((GEMM_ROWS >> 4) << 24);
}

// Nibble window (128 bits, first survivor in bits 0..3 of w0) of the 32-column word whose first
// survivor has rank `rank` in the tile's code stream `codes` (global memory, 4-byte aligned).
template <int BITS>
__device__ __forceinline__ void fetch_window(const uint32_t* codes, uint32_t rank, uint32_t (&raw)[5]) {
    const uint32_t bitpos = rank * (uint32_t)BITS;
    const uint32_t* p = codes + (bitpos >> 5);
    constexpr int NW = BITS == 4 ? 5 : (BITS == 3 ? 4 : 3);
#pragma unroll
    for (int i = 0; i < 5; ++i) raw[i] = i < NW ? __ldg(p + i) : 0u;
}
template <int BITS>
__device__ __forceinline__ void align_window(const uint32_t (&raw)[5], uint32_t rank, uint32_t& w0, uint32_t& w1,
                                             uint32_t& w2, uint32_t& w3) {
    const uint32_t o = (rank * (uint32_t)BITS) & 31u;
    const uint32_t a0 = funnel_r(raw[0], raw[1], o), a1 = funnel_r(raw[1], raw[2], o);
    const uint32_t a2 = funnel_r(raw[2], raw[3], o), a3 = funnel_r(raw[3], raw[4], o);
    if (BITS == 4) {
        w0 = a0; w1 = a1; w2 = a2; w3 = a3;
    } else if (BITS == 3) {                     // 96 bits = four 24-bit chunks of 8 codes
        w0 = spread3(a0 & 0x00FFFFFFu);
        w1 = spread3(funnel_r(a0, a1, 24) & 0x00FFFFFFu);
        w2 = spread3(funnel_r(a1, a2, 16) & 0x00FFFFFFu);
        w3 = spread3(a2 >> 8);
    } else {                                    // 64 bits = four 16-bit chunks of 8 codes
        w0 = spread2(a0); w1 = spread2(a0 >> 16); w2 = spread2(a1); w3 = spread2(a1 >> 16);
    }
}

template <int BITS>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_tcgen05_kernel(const GemmParams P,
                                                                       const __grid_constant__ CUtensorMap xmap) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const MatView& W = P.W;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full_mask = 0xFFFFFFFFu;

    // ---- shared memory carve-up (operand stages 1024-byte aligned)
    const uint32_t s_raw = smem_u32(smem);
    const uint32_t s0 = (s_raw + 1023u) & ~1023u;                         // the allocation carries 1 KB of slack
    uint8_t* const sm = smem + (s0 - s_raw);
    const uint32_t a_base = s0;
    const uint32_t b_base = a_base + GEMM_A_STAGES * GEMM_A_BYTES;
    const uint32_t lut_addr = b_base + GEMM_B_STAGES * GEMM_B_BYTES;
    const uint32_t bar_base = lut_addr + GEMM_LUT_BYTES;
    auto bar_afull = [&](int s) { return bar_base + 8u * s; };             // 3
    auto bar_aempty = [&](int s) { return bar_base + 24u + 8u * s; };      // 3
    auto bar_bfull = [&](int s) { return bar_base + 48u + 8u * s; };       // 2
    auto bar_bempty = [&](int s) { return bar_base + 64u + 8u * s; };      // 2
    const uint32_t bar_acc = bar_base + 80u;
    const uint32_t tmem_slot = bar_base + 96u;

    const int row_tile = blockIdx.x;
    const int m0 = blockIdx.y * P.tok_per_cta;
    int n_tok = P.M - m0;
    if (n_tok > P.tok_per_cta) n_tok = P.tok_per_cta;
    const int n_half0 = n_tok < GEMM_NT ? n_tok : GEMM_NT;
    const int n_half1 = n_tok - n_half0;
    const uint32_t n_mma0 = (uint32_t)((n_half0 + 15) & ~15), n_mma1 = (uint32_t)((n_half1 + 15) & ~15);
    const int rb0 = row_tile * GEMM_RB;
    int n_rb = W.RB - rb0;
    if (n_rb > GEMM_RB) n_rb = GEMM_RB;
    // column tiles of this split
    const int split = blockIdx.z;
    const int ct_per = (W.CT + P.splits - 1) / P.splits;
    const int ct_begin = split * ct_per;
    int ct_end = ct_begin + ct_per;
    if (ct_end > W.CT) ct_end = W.CT;
    int my_stages = 0;
    for (int ct = ct_begin; ct < ct_end; ++ct) my_stages += 2 * tile_width(W, ct);

    if (threadIdx.x == 0) {
        for (int s = 0; s < GEMM_A_STAGES; ++s) { mbar_init(bar_afull(s), 128); mbar_init(bar_aempty(s), 1); }
        for (int s = 0; s < GEMM_B_STAGES; ++s) { mbar_init(bar_bfull(s), 1); mbar_init(bar_bempty(s), 1); }
        mbar_init(bar_acc, 1);
        mbar_fence_init();
        fence_proxy_async();
    }
    {   // expansion table replicas
        LutEntry* lut_s = reinterpret_cast<LutEntry*>(sm + (lut_addr - s0));
        for (int i = threadIdx.x; i < LUT_ENTRIES * GEMM_LUT_COPIES; i += GEMM_THREADS) lut_s[i] = g_lut.e[i / GEMM_LUT_COPIES];
    }
    if (warp == 9) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = lds32(tmem_slot);

    if (warp < 8) {
        // =========================================================== decode + epilogue
        const int group = warp >> 2;                      // takes stages with (q & 1) == group
        const int r = threadIdx.x & 127;                  // weight row within the CTA tile
        const int rbl = r >> 4, rr = r & 15;
        const bool have_rb = rbl < n_rb;
        const uint32_t lut_lane = lut_addr + (uint32_t)(lane & (GEMM_LUT_COPIES - 1)) * 8u;
        const LutEntry* lut_lane_ptr = reinterpret_cast<const LutEntry*>(sm + (lut_addr - s0)) + (lane & (GEMM_LUT_COPIES - 1));
        auto lut = [lut_lane](uint32_t idx) {
            const uint2 e = lds64(lut_lane + idx * (GEMM_LUT_COPIES * 8u));
            return LutEntry{e.x, e.y};
        };
        bool healthy = true;
        int q = 0;                                        // stage counter of this CTA (both groups count every stage)
        // Weight bytes are read by per-thread loads whose addresses depend on each other (tile offset -> masks -> code
        // windows).  One thread per row block asks the L2 for whole tiles two column tiles ahead, so that those loads
        // find their lines in the cache instead of paying a DRAM round trip each.
        auto prefetch_tile = [&](int ct) {
            if (have_rb && rr == 0 && group == 0 && ct < ct_end) {
                const uint32_t* to = W.tile_off + (size_t)(rb0 + rbl) * W.CT + ct;
                const uint32_t o0 = __ldg(to), o1 = __ldg(to + 1);
                asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(W.tiles + (size_t)o0 * 16), "r"((o1 - o0) * 16u) : "memory");
            }
        };
        prefetch_tile(ct_begin);
        prefetch_tile(ct_begin + 1);
        for (int ct = ct_begin; ct < ct_end && healthy; ++ct) {
            const int w = tile_width(W, ct);
            prefetch_tile(ct + 2);
            // this row's segments, and where its codes start inside the tile
            uint4 mk[TILE_GROUPS];
            uint32_t szv[TILE_GROUPS];
            uint32_t cnt = 0;
            const uint32_t* codes = nullptr;
            if (have_rb) {
                const uint8_t* tile = W.tiles + (size_t)__ldg(W.tile_off + (size_t)(rb0 + rbl) * W.CT + ct) * 16;
                codes = reinterpret_cast<const uint32_t*>(tile + TILE_ROWS * w * 20);
#pragma unroll
                for (int gi = 0; gi < TILE_GROUPS; ++gi) {
                    mk[gi] = make_uint4(0, 0, 0, 0);
                    szv[gi] = 0;
                    if (gi < w) {
                        mk[gi] = __ldg(reinterpret_cast<const uint4*>(tile) + rr * w + gi);
                        szv[gi] = __ldg(reinterpret_cast<const uint32_t*>(tile + TILE_ROWS * w * 16) + rr * w + gi);
                        cnt += __popc(mk[gi].x) + __popc(mk[gi].y) + __popc(mk[gi].z) + __popc(mk[gi].w);
                    }
                }
            } else {
#pragma unroll
                for (int gi = 0; gi < TILE_GROUPS; ++gi) { mk[gi] = make_uint4(0, 0, 0, 0); szv[gi] = 0; }
            }
            uint32_t inc = cnt;
#pragma unroll
            for (int d = 1; d < 16; d <<= 1) {
                const uint32_t up = __shfl_up_sync(full_mask, inc, d, 16);
                if ((lane & 15) >= d) inc += up;
            }
            uint32_t off = inc - cnt;                      // rank of this row's first survivor within the tile

            const int nks = 2 * w;                         // 64-column stages in this column tile
            for (int ks = 0; ks < nks; ++ks, ++q) {
                const uint32_t m0w = (ks & 1) ? mk[0].z : mk[0].x;
                const uint32_t m1w = (ks & 1) ? mk[0].w : mk[0].y;
                const uint32_t sz_cur = szv[0];
                const uint32_t off0 = off, off1 = off + __popc(m0w);
                off = off1 + __popc(m1w);
                if (ks & 1) {                              // group finished: rotate the next one into slot 0
#pragma unroll
                    for (int k2 = 0; k2 + 1 < TILE_GROUPS; ++k2) { mk[k2] = mk[k2 + 1]; szv[k2] = szv[k2 + 1]; }
                }
                if ((q & 1) != group) continue;            // the other group's stage
                uint32_t raw0[5] = {0, 0, 0, 0, 0}, raw1[5] = {0, 0, 0, 0, 0};
                if (have_rb) {
                    fetch_window<BITS>(codes, off0, raw0);
                    fetch_window<BITS>(codes, off1, raw1);
                }
                const SegParams sp = make_seg_params(sz_cur, BITS, W.col_scale != nullptr);
                uint32_t e0[16], e1[16];
                uint32_t w0, w1, w2, w3;
                const int col = (ct * TILE_GROUPS + (ks >> 1)) * GROUP + (ks & 1) * 64;
                if (sp.fast) {
                    align_window<BITS>(raw0, off0, w0, w1, w2, w3);
                    decode32_fast(m0w, w0, w1, w2, w3, sp, lut, e0);
                    align_window<BITS>(raw1, off1, w0, w1, w2, w3);
                    decode32_fast(m1w, w0, w1, w2, w3, sp, lut, e1);
                } else {
                    float cs[32];
                    const float* csp = nullptr;
                    if (W.col_scale != nullptr) {
                        for (int i = 0; i < 32; ++i) cs[i] = half_bits_to_float(W.col_scale[col + i]);
                        csp = cs;
                    }
                    align_window<BITS>(raw0, off0, w0, w1, w2, w3);
                    decode32<GEMM_LUT_COPIES>(m0w, w0, w1, w2, w3, sp, lut_lane_ptr, csp, e0);
                    if (W.col_scale != nullptr)
                        for (int i = 0; i < 32; ++i) cs[i] = half_bits_to_float(W.col_scale[col + 32 + i]);
                    align_window<BITS>(raw1, off1, w0, w1, w2, w3);
                    decode32<GEMM_LUT_COPIES>(m1w, w0, w1, w2, w3, sp, lut_lane_ptr, csp, e1);
                }
                const int s = q % GEMM_A_STAGES;
                healthy = __all_sync(full_mask, mbar_wait_bounded(bar_aempty(s), (((uint32_t)(q / GEMM_A_STAGES)) & 1u) ^ 1u,
                                                                  P.status, DEV_TIMEOUT_EMPTY));
                if (!healthy) break;
                const uint32_t rowaddr = a_base + s * GEMM_A_BYTES + (uint32_t)(r >> 3) * 1024u + (uint32_t)(r & 7) * 128u;
                const uint32_t x7 = (uint32_t)(r & 7);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    sts128(rowaddr + (((uint32_t)c ^ x7) << 4), e0[4 * c], e0[4 * c + 1], e0[4 * c + 2], e0[4 * c + 3]);
                    sts128(rowaddr + (((uint32_t)(c + 4) ^ x7) << 4), e1[4 * c], e1[4 * c + 1], e1[4 * c + 2], e1[4 * c + 3]);
                }
                fence_proxy_async();
                mbar_arrive(bar_afull(s));
            }
        }
        // ---- epilogue: TMEM lane = weight row; warp w drains accumulator w/4
        if (healthy && my_stages > 0) healthy = __all_sync(full_mask, mbar_wait_bounded(bar_acc, 0u, P.status, DEV_TIMEOUT_ACC));
        tc_fence_after();
        const int row = row_tile * GEMM_ROWS + r;
        const int acc_id = group;
        const int ntok_acc = acc_id ? n_half1 : n_half0;
        const uint32_t nmma_acc = acc_id ? n_mma1 : n_mma0;
        const int tok_base = m0 + acc_id * GEMM_NT;
        const uint32_t tile_id = blockIdx.y * gridDim.x + blockIdx.x;
        float* part = P.partials ? P.partials + ((size_t)tile_id * P.splits + split) * ((size_t)GEMM_TOKENS * GEMM_ROWS) : nullptr;
        if (healthy) {
            for (uint32_t c0 = 0; c0 < nmma_acc; c0 += 32) {
                uint32_t v[32];
                if (my_stages > 0) {
                    tmem_ld32(tmem_d + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(acc_id * GEMM_NT) + c0, v);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = 0u;
                }
                if (P.splits == 1) {
                    if (row < W.K) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int tk = (int)c0 + i;
                            if (tk < ntok_acc) {
                                if (P.y32) P.y32[(size_t)(tok_base + tk) * P.ldy + row] = __uint_as_float(v[i]);
                                else P.y[(size_t)(tok_base + tk) * P.ldy + row] = finish_output(__uint_as_float(v[i]), P.bias, row);
                            }
                        }
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int tk = (int)c0 + i;
                        if (tk < ntok_acc) part[(size_t)(acc_id * GEMM_NT + tk) * GEMM_ROWS + r] = __uint_as_float(v[i]);
                    }
                }
            }
        }
        tc_fence_before();
        if (P.splits > 1) {
            // the last split to arrive adds all splits in order and writes the outputs
            __threadfence();
            asm volatile("bar.sync 1, 256;" ::: "memory");            // the 8 decode warps only
            if (threadIdx.x == 0) sts32(bar_base + 104u, atomicAdd(&P.counters[tile_id], 1u));
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (lds32(bar_base + 104u) == (uint32_t)(P.splits - 1) && healthy) {
                __threadfence();
                const float* base = P.partials + (size_t)tile_id * P.splits * ((size_t)GEMM_TOKENS * GEMM_ROWS);
                if (row < W.K) {
                    // eight tokens x four splits of loads in flight per thread: one thread per row walks up to 256 tokens,
                    // and a token at a time would be one L2 latency per token (the whole cost of a small-M launch)
                    constexpr int TU = 8, KU = 4;
                    const size_t split_stride = (size_t)GEMM_TOKENS * GEMM_ROWS;
                    for (int tk0 = 0; tk0 < ntok_acc; tk0 += TU) {
                        float sum[TU];
#pragma unroll
                        for (int j = 0; j < TU; ++j) sum[j] = 0.0f;
                        for (int k0 = 0; k0 < P.splits; k0 += KU) {
                            float v[KU][TU];
#pragma unroll
                            for (int kk = 0; kk < KU; ++kk)
#pragma unroll
                                for (int j = 0; j < TU; ++j) {
                                    const int tk = tk0 + j < ntok_acc ? tk0 + j : ntok_acc - 1;
                                    v[kk][j] = k0 + kk < P.splits
                                        ? __ldcg(base + (size_t)(k0 + kk) * split_stride + (size_t)(acc_id * GEMM_NT + tk) * GEMM_ROWS + r) : 0.0f;
                                }
#pragma unroll
                            for (int kk = 0; kk < KU; ++kk)             // splits in order: the sum does not depend on the grid
#pragma unroll
                                for (int j = 0; j < TU; ++j)
                                    if (k0 + kk < P.splits) sum[j] += v[kk][j];
                        }
#pragma unroll
                        for (int j = 0; j < TU; ++j) {
                            const int tk = tk0 + j;
                            if (tk < ntok_acc) {
                                if (P.y32) P.y32[(size_t)(tok_base + tk) * P.ldy + row] = sum[j];
                                else P.y[(size_t)(tok_base + tk) * P.ldy + row] = finish_output(sum[j], P.bias, row);
                            }
                        }
                    }
                }
                if (threadIdx.x == 0) P.counters[tile_id] = 0u;
            }
        }
    } else if (warp == 8) {
        // =========================================================== activation loader (TMA)
        if (lane == 0) {
            bool healthy = true;
            int q = 0;
            const uint32_t bytes = (uint32_t)GEMM_BHALF_BYTES * (n_half1 > 0 ? 2u : 1u);
            for (int ct = ct_begin; ct < ct_end && healthy; ++ct) {
                const int w = tile_width(W, ct);
                for (int ks = 0; ks < 2 * w; ++ks, ++q) {
                    const int s = q % GEMM_B_STAGES;
                    healthy = mbar_wait_bounded(bar_bempty(s), (((uint32_t)(q / GEMM_B_STAGES)) & 1u) ^ 1u, P.status, DEV_TIMEOUT_EMPTY);
                    if (!healthy) break;
                    const int col = ct * TILE_GROUPS * GROUP + ks * GEMM_KS;
                    mbar_arrive_expect_tx(bar_bfull(s), bytes);
                    tma_load_2d(b_base + s * GEMM_B_BYTES, &xmap, col, m0, bar_bfull(s));
                    if (n_half1 > 0) tma_load_2d(b_base + s * GEMM_B_BYTES + GEMM_BHALF_BYTES, &xmap, col, m0 + GEMM_NT, bar_bfull(s));
                }
            }
        }
        __syncwarp();
    } else {
        // =========================================================== MMA issuer
        if (lane == 0) {
            const uint32_t idesc0 = umma_idesc(n_mma0), idesc1 = umma_idesc(n_mma1 ? n_mma1 : 16);
            bool healthy = true;
            for (int q = 0; q < my_stages && healthy; ++q) {
                const int sa = q % GEMM_A_STAGES, sb = q % GEMM_B_STAGES;
                healthy = mbar_wait_bounded(bar_afull(sa), ((uint32_t)(q / GEMM_A_STAGES)) & 1u, P.status, DEV_TIMEOUT_FULL);
                if (healthy) healthy = mbar_wait_bounded(bar_bfull(sb), ((uint32_t)(q / GEMM_B_STAGES)) & 1u, P.status, DEV_TIMEOUT_STAGE);
                if (!healthy) break;
                tc_fence_after();
                const uint64_t ad = umma_smem_desc(a_base + sa * GEMM_A_BYTES);
                const uint64_t bd0 = umma_smem_desc(b_base + sb * GEMM_B_BYTES);
                const uint64_t bd1 = umma_smem_desc(b_base + sb * GEMM_B_BYTES + GEMM_BHALF_BYTES);
#pragma unroll
                for (int k = 0; k < GEMM_KS / 16; ++k)
                    umma_bf16(tmem_d, ad + (uint64_t)(2 * k), bd0 + (uint64_t)(2 * k), idesc0, (q > 0 || k > 0) ? 1u : 0u);
                if (n_mma1) {
#pragma unroll
                    for (int k = 0; k < GEMM_KS / 16; ++k)
                        umma_bf16(tmem_d + GEMM_NT, ad + (uint64_t)(2 * k), bd1 + (uint64_t)(2 * k), idesc1, (q > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(bar_aempty(sa));
                umma_commit(bar_bempty(sb));
            }
            if (healthy && my_stages > 0) umma_commit(bar_acc);
        }
        __syncwarp();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) { tc_fence_after(); tmem_dealloc(tmem_d, 512); }
}

}  // namespace cb
