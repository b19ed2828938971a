// Prefill GEMM: Y[m, k] = sum_j bf16(W[k, j]) * X[m, j] with tcgen05.mma, accumulators in
// tensor memory.
//
// One CTA owns 128 weight rows (8 row blocks of the tile image) and up to 256 tokens:
//   D[128 rows x n tokens] (TMEM, fp32)  +=  A[128 x 64] (bf16, decoded weights)  *  B[n x 64]^T (bf16, x)
// per 64-column stage, both operands K-major in shared memory with the 128-byte swizzle.
//
//   warps 0-3  decode: thread r owns weight row r.  It expands the row's bitmask + codes for the
//              64 columns of the stage into 64 bf16 and writes them as eight swizzled 16-byte
//              chunks.  After the main loop the same warps drain TMEM (warp q reads lanes 32q..)
//              and store bf16 outputs.
//   warps 4-7  load the activation stage (16-byte vector loads, swizzled stores) and keep the
//              compressed-tile ring fed with bulk async copies (8 tiles per 512-column tile).
//   warp 8     one elected lane issues tcgen05.mma and tcgen05.commit.
//
// Generic-proxy writes to operand stages are published with fence.proxy.async before the
// mbarrier arrive; the MMA thread orders itself with tcgen05.fence::after_thread_sync.  Every
// wait is bounded: on expiry the kernel records a status code, stops issuing work, lets its
// outstanding copies land (bounded), frees its tensor memory and returns.
//
// Behaviour replaced: cbk::gemm_tile (mma.sync m16n8k16, per-fragment bf16x2 dequantisation,
// src/cobaltkernel/csrc/cobalt_gemm.cuh:243-609) driven by gemm_phase
// (src/cobaltkernel/csrc/prefill_kernel.cu:103-150).
#pragma once
#include "common.cuh"
#include "gemv_kernel.cuh"   // load_window, finish_output

namespace cb {

constexpr int GEMM_ROWS = 128;            // UMMA M
constexpr int GEMM_MAX_NT = 256;          // UMMA N (tokens per CTA)
constexpr int GEMM_KS = 64;               // columns per stage = one 128-byte swizzle row of bf16
constexpr int GEMM_RB = GEMM_ROWS / TILE_ROWS;   // 8 row blocks per CTA
constexpr int GEMM_LUT_COPIES = 8;
constexpr int GEMM_THREADS = 288;
constexpr uint32_t GEMM_LUT_BYTES = LUT_ENTRIES * GEMM_LUT_COPIES * 8;   // 16 KB
constexpr uint32_t GEMM_A_BYTES = GEMM_ROWS * GEMM_KS * 2;               // 16 KB
constexpr uint32_t GEMM_B_BYTES = GEMM_MAX_NT * GEMM_KS * 2;             // 32 KB
constexpr uint32_t GEMM_BAR_BYTES = 256;

struct GemmParams {
    MatView W;
    const uint16_t* x; int64_t ldx;
    uint16_t* y; int64_t ldy;
    const uint16_t* bias;
    int M;
    int stages;                 // operand stages (2..4)
    uint32_t slot_bytes;        // one compressed tile slot
    uint32_t nib_bytes;         // per-slot nibble buffer (bits < 4), else 0
    uint32_t* status;
};

// ---- tcgen05 wrappers
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

template <int BITS>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_tcgen05_kernel(const GemmParams P) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const MatView& W = P.W;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full_mask = 0xFFFFFFFFu;

    // ---- shared memory carve-up (all operand stages 1024-byte aligned)
    const uint32_t s0 = smem_u32(smem);
    const uint32_t a_base = s0;                                          // stages x 16 KB
    const uint32_t b_base = a_base + P.stages * GEMM_A_BYTES;            // stages x 32 KB
    const uint32_t lut_addr = b_base + P.stages * GEMM_B_BYTES;          // 16 KB
    const uint32_t bar_base = lut_addr + GEMM_LUT_BYTES;                 // barriers + tmem pointer
    const uint32_t ring_base = bar_base + GEMM_BAR_BYTES;                // 2 x 8 x (slot + nib)
    const uint32_t per_slot = P.slot_bytes + P.nib_bytes;
    // barrier map (8 bytes each): full[4] empty[4] cfull[2] cempty[2] acc  | tmem pointer at +120
    auto bar_full = [&](int s) { return bar_base + 8u * s; };
    auto bar_empty = [&](int s) { return bar_base + 32u + 8u * s; };
    auto bar_cfull = [&](int b) { return bar_base + 64u + 8u * b; };
    auto bar_cempty = [&](int b) { return bar_base + 80u + 8u * b; };
    const uint32_t bar_acc = bar_base + 96u;
    const uint32_t tmem_slot = bar_base + 120u;

    const int row_tile = blockIdx.x;                     // 128 rows
    const int m0 = blockIdx.y * GEMM_MAX_NT;             // first token
    int n_tok = P.M - m0;
    if (n_tok > GEMM_MAX_NT) n_tok = GEMM_MAX_NT;
    const uint32_t n_mma = (uint32_t)((n_tok + 15) & ~15);
    const int rb0 = row_tile * GEMM_RB;
    int n_rb = W.RB - rb0;
    if (n_rb > GEMM_RB) n_rb = GEMM_RB;
    const int total_stages = 2 * W.G;                    // 64-column stages over N

    if (threadIdx.x == 0) {
        for (int s = 0; s < P.stages; ++s) { mbar_init(bar_full(s), 256); mbar_init(bar_empty(s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(bar_cfull(b), 1); mbar_init(bar_cempty(b), 128); }
        mbar_init(bar_acc, 1);
        mbar_fence_init();
        fence_proxy_async();
    }
    {   // expansion table replicas
        LutEntry* lut_s = reinterpret_cast<LutEntry*>(smem + (lut_addr - s0));
        for (int i = threadIdx.x; i < LUT_ENTRIES * GEMM_LUT_COPIES; i += GEMM_THREADS) lut_s[i] = g_lut.e[i / GEMM_LUT_COPIES];
    }
    if (warp == 8) { tmem_alloc(tmem_slot, 256); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = lds32(tmem_slot);

    if (warp < 4) {
        // =========================================================== decode + epilogue
        const int r = threadIdx.x;                        // weight row within the CTA tile
        const int rbl = r >> 4, rr = r & 15;
        const bool have_rb = rbl < n_rb;
        const LutEntry* lut_lane = reinterpret_cast<const LutEntry*>(smem + (lut_addr - s0)) + (lane & (GEMM_LUT_COPIES - 1));
        const uint32_t half_mask = (lane < 16) ? 0x0000FFFFu : 0xFFFF0000u;
        bool healthy = true;
        int q = 0;                                        // global stage counter
        for (int ct = 0; ct < W.CT && healthy; ++ct) {
            const int buf = ct & 1;
            const int w = tile_width(W, ct);
            healthy = __all_sync(full_mask, mbar_wait_bounded(bar_cfull(buf), (uint32_t)(ct >> 1) & 1u, P.status, DEV_TIMEOUT_STAGE));
            if (!healthy) break;
            const uint32_t slot = ring_base + (uint32_t)(buf * GEMM_RB + rbl) * per_slot;
            // this row's segments and where its codes start
            uint4 mk[TILE_GROUPS];
            uint32_t szv[TILE_GROUPS];
            uint32_t cnt = 0;
#pragma unroll
            for (int gi = 0; gi < TILE_GROUPS; ++gi) {
                mk[gi] = make_uint4(0, 0, 0, 0);
                szv[gi] = 0;
                if (have_rb && gi < w) {
                    mk[gi] = lds128(slot + (rr * w + gi) * 16);
                    szv[gi] = lds32(slot + TILE_ROWS * w * 16 + (rr * w + gi) * 4);
                    cnt += __popc(mk[gi].x) + __popc(mk[gi].y) + __popc(mk[gi].z) + __popc(mk[gi].w);
                }
            }
            uint32_t inc = cnt;
#pragma unroll
            for (int d = 1; d < 16; d <<= 1) {
                const uint32_t up = __shfl_up_sync(full_mask, inc, d, 16);
                if ((lane & 15) >= d) inc += up;
            }
            uint32_t off = inc - cnt;                      // first survivor of this row within the tile
            uint32_t cbase = slot + TILE_ROWS * w * 20;
            if (BITS < 4) {
                const uint32_t total = __shfl_sync(full_mask, inc, 15, 16);
                const uint32_t nchunks = (total + 7u) >> 3;
                const uint32_t nibb = slot + P.slot_bytes;
                if (have_rb) {
                    for (uint32_t c = (uint32_t)(lane & 15); c < nchunks; c += 16) {
                        uint32_t outv;
                        if (BITS == 3) {
                            const uint32_t bo = 3u * c, a = cbase + (bo & ~3u);
                            outv = spread3(funnel_r(lds32(a), lds32(a + 4), (bo & 3u) * 8u) & 0x00FFFFFFu);
                        } else {
                            outv = spread2(lds32(cbase + (c >> 1) * 4u) >> (16u * (c & 1u)));
                        }
                        sts32(nibb + c * 4u, outv);
                    }
                }
                __syncwarp(half_mask);
                cbase = nibb;
            }
            const int nks = 2 * w;                         // 64-column stages in this column tile
            for (int ks = 0; ks < nks; ++ks, ++q) {
                const int gi = ks >> 1;
                uint32_t m0w, m1w;
                {
                    const uint4 mm = mk[0];                // rotate so that index 0 is the current group
                    m0w = (ks & 1) ? mm.z : mm.x;
                    m1w = (ks & 1) ? mm.w : mm.y;
                }
                const SegParams sp = make_seg_params(szv[0], BITS, W.col_scale != nullptr);
                uint32_t e0[16], e1[16];
                float cs[32];
                const float* csp = nullptr;
                const int col = (ct * TILE_GROUPS + gi) * GROUP + (ks & 1) * 64;
                uint32_t w0, w1, w2, w3;
                if (W.col_scale != nullptr) {
                    for (int i = 0; i < 32; ++i) cs[i] = half_bits_to_float(W.col_scale[col + i]);
                    csp = cs;
                }
                load_window(cbase, off, w0, w1, w2, w3);
                decode32<GEMM_LUT_COPIES>(m0w, w0, w1, w2, w3, sp, lut_lane, csp, e0);
                off += __popc(m0w);
                if (W.col_scale != nullptr)
                    for (int i = 0; i < 32; ++i) cs[i] = half_bits_to_float(W.col_scale[col + 32 + i]);
                load_window(cbase, off, w0, w1, w2, w3);
                decode32<GEMM_LUT_COPIES>(m1w, w0, w1, w2, w3, sp, lut_lane, csp, e1);
                off += __popc(m1w);
                if (ks & 1) {                              // group finished: rotate the next one into slot 0
#pragma unroll
                    for (int k2 = 0; k2 + 1 < TILE_GROUPS; ++k2) { mk[k2] = mk[k2 + 1]; szv[k2] = szv[k2 + 1]; }
                }
                const int s = q % P.stages;
                healthy = __all_sync(full_mask, mbar_wait_bounded(bar_empty(s), (((uint32_t)(q / P.stages)) & 1u) ^ 1u,
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
                mbar_arrive(bar_full(s));
            }
            if (healthy) mbar_arrive(bar_cempty(buf));
        }
        // ---- epilogue: TMEM lane = weight row
        if (healthy) healthy = __all_sync(full_mask, mbar_wait_bounded(bar_acc, 0u, P.status, DEV_TIMEOUT_ACC));
        tc_fence_after();
        if (healthy) {
            const int row = row_tile * GEMM_ROWS + r;
            for (uint32_t c0 = 0; c0 < n_mma; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem_d + ((uint32_t)(warp * 32) << 16) + c0, v);
                tmem_ld_wait();
                if (row < W.K) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int tok = m0 + (int)c0 + i;
                        if (tok < P.M) P.y[(size_t)tok * P.ldy + row] = finish_output(__uint_as_float(v[i]), P.bias, row);
                    }
                }
            }
        }
        tc_fence_before();
    } else if (warp < 8) {
        // =========================================================== activation + compressed-tile loader
        const int li = threadIdx.x - 128;                 // 0..127
        bool healthy = true;
        auto issue_ctile = [&](int ct) {                  // one thread: 8 bulk copies for column tile ct
            const int buf = ct & 1;
            uint32_t total = 0;
            uint32_t o0[GEMM_RB], o1[GEMM_RB];
            for (int b = 0; b < n_rb; ++b) {
                o0[b] = W.tile_off[(rb0 + b) * W.CT + ct];
                o1[b] = W.tile_off[(rb0 + b) * W.CT + ct + 1];
                total += (o1[b] - o0[b]) * 16u;
            }
            fence_proxy_async();
            mbar_arrive_expect_tx(bar_cfull(buf), total);
            for (int b = 0; b < n_rb; ++b)
                bulk_g2s(ring_base + (uint32_t)(buf * GEMM_RB + b) * per_slot, W.tiles + (size_t)o0[b] * 16,
                         (o1[b] - o0[b]) * 16u, bar_cfull(buf));
        };
        if (li == 0) { issue_ctile(0); if (W.CT > 1) issue_ctile(1); }
        int q = 0;
        const int chunks = (int)n_mma * 8;                // 16-byte chunks per stage
        for (int ct = 0; ct < W.CT && healthy; ++ct) {
            const int w = tile_width(W, ct);
            for (int ks = 0; ks < 2 * w && healthy; ++ks, ++q) {
                const int col = ct * TILE_GROUPS * GROUP + ks * GEMM_KS;
                const int s = q % P.stages;
                uint4 v[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int idx = li + 128 * i;
                    v[i] = make_uint4(0, 0, 0, 0);
                    if (idx < chunks) {
                        const int row = idx >> 3, ch = idx & 7;
                        if (m0 + row < P.M)
                            v[i] = __ldg(reinterpret_cast<const uint4*>(P.x + (size_t)(m0 + row) * P.ldx + col + ch * 8));
                    }
                }
                healthy = mbar_wait_bounded(bar_empty(s), (((uint32_t)(q / P.stages)) & 1u) ^ 1u, P.status, DEV_TIMEOUT_EMPTY);
                if (!healthy) break;
                const uint32_t bs = b_base + s * GEMM_B_BYTES;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int idx = li + 128 * i;
                    if (idx < chunks) {
                        const uint32_t row = (uint32_t)idx >> 3, ch = (uint32_t)idx & 7u;
                        sts128(bs + (row >> 3) * 1024u + (row & 7u) * 128u + ((ch ^ (row & 7u)) << 4), v[i].x, v[i].y, v[i].z, v[i].w);
                    }
                }
                fence_proxy_async();
                mbar_arrive(bar_full(s));
            }
            // refill the compressed ring two column tiles ahead once the decoders released this buffer
            if (li == 0 && healthy && ct + 2 < W.CT) {
                healthy = mbar_wait_bounded(bar_cempty(ct & 1), (uint32_t)(ct >> 1) & 1u, P.status, DEV_TIMEOUT_STAGE);
                if (healthy) issue_ctile(ct + 2);
            }
            healthy = __all_sync(full_mask, healthy);
        }
    } else {
        // =========================================================== MMA issuer
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(n_mma);
            bool healthy = true;
            for (int q = 0; q < total_stages && healthy; ++q) {
                const int s = q % P.stages;
                healthy = mbar_wait_bounded(bar_full(s), ((uint32_t)(q / P.stages)) & 1u, P.status, DEV_TIMEOUT_FULL);
                if (!healthy) break;
                tc_fence_after();
                const uint64_t ad = umma_smem_desc(a_base + s * GEMM_A_BYTES);
                const uint64_t bd = umma_smem_desc(b_base + s * GEMM_B_BYTES);
#pragma unroll
                for (int k = 0; k < GEMM_KS / 16; ++k)
                    umma_bf16(tmem_d, ad + (uint64_t)(2 * k), bd + (uint64_t)(2 * k), idesc, (q > 0 || k > 0) ? 1u : 0u);
                umma_commit(bar_empty(s));
            }
            if (healthy) umma_commit(bar_acc);
        }
        __syncwarp();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) { tc_fence_after(); tmem_dealloc(tmem_d, 256); }
}

}  // namespace cb
