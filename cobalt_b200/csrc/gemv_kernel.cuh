// Decode GEMV for M <= 16 tokens.
//
// Persistent kernel, one CTA per SM.  The tiles of the matrix (row-block-major) are cut into
// one contiguous range per warp, balanced to +-1 tile over all warps of the grid, so every SM
// gets the same share whatever the matrix shape.  Each warp pulls its tiles with 1-D bulk async
// copies into a private shared-memory ring (mbarrier completion), locates every segment's
// survivor codes with a popcount prefix sum over the warp, expands them to dense bf16 weights
// in registers (decode_core.cuh) and contracts them against the activations with mma.sync
// m16n8k16 (A = 16 rows x 16 columns of weights, B = 16 columns x 8 tokens).  Lane
// (g = lane/4, t = lane%4) owns rows g and g+8 of the row block and group t of the tile; in
// MMA step s it supplies columns 4s..4s+3 of that group, so the 16 k-slots of one MMA are 4
// consecutive columns from each of the tile's 4 groups and the B fragment of the lane is
// simply 8 contiguous bytes of x.
//
// A row block that is covered by several warps is finished in two deterministic stages.  The
// parts held by one CTA meet in shared memory: the last of its warps to arrive adds the fp32
// fragments in range order.  If the block straddles CTAs, that subtotal goes to global scratch and
// the last CTA to arrive adds the subtotals in CTA order (fence + atomic + L2 round trips,
// microseconds).  Warps whose range ends in a block that continues into the next CTA walk their
// range backwards, so that this slow exchange happens at the start of both neighbours' work
// instead of at the very end of the kernel.
//
// Behaviour replaced: cbk::gemv_sparse / gemv_sparse_expand, one warp per row with a 32-lane
// prefix scan per 1024-column window (src/cobaltkernel/csrc/cobalt_gemv.cuh:216-393).
#pragma once
#include "common.cuh"

namespace cb {

constexpr int GEMV_WARPS = 16;
constexpr int GEMV_THREADS = GEMV_WARPS * 32;
constexpr int GEMV_MAX_STAGES = 4;
constexpr uint32_t GEMV_LUT_BYTES = LUT_ENTRIES * LUT_COPIES * 8;      // 32 KB
constexpr uint32_t GEMV_BAR_BYTES = GEMV_WARPS * GEMV_MAX_STAGES * 8;  // 512 B
constexpr uint32_t GEMV_REDCNT_BYTES = 128;                            // in-CTA arrival counters: one per first owner + one
// in-CTA reduction fragments: [warp][head|tail][4 * MT * 32] floats
constexpr uint32_t gemv_red_bytes(int mt) { return GEMV_WARPS * 2 * 4 * mt * 32 * 4; }

constexpr int GEMV_MAX_MATS = 4;

// one matrix of a (possibly fused) launch; all matrices of a launch share x, N and the bit width
struct GemvMat {
    const uint8_t* tiles;
    const uint32_t* tile_off;
    uint16_t* y;                         // bf16 output [M, K] ...
    float* y32;                          // ... or, when set, raw fp32 sums (no bias, no rounding)
    const uint16_t* bias;
    int64_t ldy;
    int K;
    int rb_start;                        // first row block of this matrix in the launch's row-block space
};

struct GemvParams {
    GemvMat mat[GEMV_MAX_MATS];
    int n_mats;
    int N, G, CT, RB;                    // shared geometry; RB = row blocks of all matrices together
    const uint16_t* col_scale;           // single-matrix launches only
    const uint16_t* x; int64_t ldx;
    int M;
    int stages;
    uint32_t slot_bytes, nib_bytes;
    uint32_t total_warps;                // grid * GEMV_WARPS
    float* partials;                     // [total_warps][2][4 * MT * 32]
    uint32_t* counters;                  // [row blocks]
    uint32_t* status;
};

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// bf16( bf16(acc) + bias ): the reference rounds the matmul result first and adds the bias after
__device__ __forceinline__ uint16_t finish_output(float acc, const uint16_t* bias, int row) {
    uint16_t r = float_to_bf16(acc);
    if (bias) r = float_to_bf16(bf16_to_float(r) + bf16_to_float(bias[row]));
    return r;
}

// Read-only 16-byte load kept in program order with the shared-memory loads of the decoder, so
// that it is issued before the decode of the word it belongs to and its latency hides behind it.
__device__ __forceinline__ uint4 ldg_nc_early(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// nibble stream window of one 32-column word: 128 bits starting at nibble `nib_off`
__device__ __forceinline__ void load_window(uint32_t cbase, uint32_t nib_off, uint32_t& w0, uint32_t& w1,
                                            uint32_t& w2, uint32_t& w3) {
    const uint32_t bitpos = nib_off * 4u;
    const uint32_t a = cbase + (bitpos >> 5) * 4u;
    const uint32_t r0 = lds32(a), r1 = lds32(a + 4), r2 = lds32(a + 8), r3 = lds32(a + 12), r4 = lds32(a + 16);
    const uint32_t o = bitpos & 31u;
    w0 = funnel_r(r0, r1, o); w1 = funnel_r(r1, r2, o); w2 = funnel_r(r2, r3, o); w3 = funnel_r(r3, r4, o);
}

// first tile of warp gw / warp that owns tile tau, for the balanced contiguous partition
__device__ __forceinline__ uint32_t range_start(uint32_t gw, uint32_t T, uint32_t Wt) { return (uint32_t)(((uint64_t)gw * T) / Wt); }
__device__ __forceinline__ uint32_t tile_owner(uint32_t tau, uint32_t T, uint32_t Wt) { return ((tau + 1u) * Wt - 1u) / T; }

template <int BITS, int MT>
__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_mma_kernel(const GemvParams P) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t full = 0xFFFFFFFFu;
    auto mat_of = [&](int rbg) {                                       // matrix that owns row block rbg of the launch
        int m = 0;
#pragma unroll
        for (int k = 1; k < GEMV_MAX_MATS; ++k)
            if (k < P.n_mats && rbg >= P.mat[k].rb_start) m = k;
        return m;
    };

    // ---- block set-up: barriers first, so that the first tiles are in flight while the
    //      expansion table replicas are being written
    LutEntry* lut_s = reinterpret_cast<LutEntry*>(smem);
    const uint32_t bar0 = smem_u32(smem + GEMV_LUT_BYTES) + warp * GEMV_MAX_STAGES * 8;
    if (lane == 0)
        for (int s = 0; s < P.stages; ++s) mbar_init(bar0 + 8 * s, 1);
    constexpr int FR = 4 * MT * 32;                                    // floats of one accumulator fragment set
    uint32_t* red_cnt = reinterpret_cast<uint32_t*>(smem + GEMV_LUT_BYTES + GEMV_BAR_BYTES);
    float* red = reinterpret_cast<float*>(smem + GEMV_LUT_BYTES + GEMV_BAR_BYTES + GEMV_REDCNT_BYTES);
    if (threadIdx.x <= GEMV_WARPS) red_cnt[threadIdx.x] = 0u;
    mbar_fence_init();
    fence_proxy_async();
    __syncthreads();

    const int M = P.M, CT = P.CT;
    const uint32_t T = (uint32_t)P.RB * (uint32_t)P.CT, Wt = P.total_warps;
    const uint32_t gw = blockIdx.x * GEMV_WARPS + warp;
    const uint32_t t0 = range_start(gw, T, Wt), t1 = range_start(gw + 1, T, Wt);
    const int n = (int)(t1 - t0);

    const uint32_t per_warp = P.stages * P.slot_bytes + P.nib_bytes;
    const uint32_t ring = smem_u32(smem + GEMV_LUT_BYTES + GEMV_BAR_BYTES + GEMV_REDCNT_BYTES + gemv_red_bytes(MT)) + warp * per_warp;
    const uint32_t cta_t0 = range_start(blockIdx.x * GEMV_WARPS, T, Wt), cta_t1 = range_start((blockIdx.x + 1) * GEMV_WARPS, T, Wt);
    // A warp whose range ends in the row block that continues into the next CTA walks backwards: that block's
    // exchange through global scratch then starts early in both CTAs instead of ending the kernel.
    const bool rev = n > 0 && ((t1 - 1u) / (uint32_t)P.CT + 1u) * (uint32_t)P.CT > cta_t1;
    auto tile_at = [&](int i) { return rev ? t1 - 1u - (uint32_t)i : t0 + (uint32_t)i; };
    const uint32_t nib = ring + P.stages * P.slot_bytes;
    const uint32_t lut_lane = smem_u32(smem) + (uint32_t)(lane & (LUT_COPIES - 1)) * 8u;
    const LutEntry* lut_lane_ptr = lut_s + (lane & (LUT_COPIES - 1));

    // address and size of the i-th tile of the walk, looked up by lane i for the first 32 tiles
    auto tile_src = [&](uint32_t tau, const uint8_t*& src, uint32_t& bytes) {
        const int rbg = (int)(tau / (uint32_t)P.CT);
        const GemvMat& mt = P.mat[mat_of(rbg)];
        const uint32_t local = tau - (uint32_t)mt.rb_start * (uint32_t)P.CT;
        const uint32_t o0 = mt.tile_off[local], o1 = mt.tile_off[local + 1];
        src = mt.tiles + (size_t)o0 * 16;
        bytes = (o1 - o0) * 16u;
    };
    const uint8_t* my_src = nullptr;
    uint32_t my_bytes = 0;
    if (lane < n) tile_src(tile_at(lane), my_src, my_bytes);

    auto issue = [&](int i, int slot_idx) {                            // all lanes call; lane 0 acts
        const uint8_t* src;
        uint32_t bytes;
        if (i < 32) {
            const unsigned long long a = __shfl_sync(full, (unsigned long long)my_src, i);
            src = (const uint8_t*)a;
            bytes = __shfl_sync(full, my_bytes, i);
        } else {
            tile_src(tile_at(i), src, bytes);
        }
        if (lane == 0) {
            const uint32_t bar = bar0 + 8 * slot_idx;
            fence_proxy_async();
            mbar_arrive_expect_tx(bar, bytes);
            bulk_g2s(ring + slot_idx * P.slot_bytes, src, bytes, bar);
        }
    };

    int issued = n < P.stages ? n : P.stages;
    for (int i = 0; i < issued; ++i) issue(i, i);

    for (int i = threadIdx.x; i < LUT_ENTRIES * LUT_COPIES; i += GEMV_THREADS) lut_s[i] = g_lut.e[i / LUT_COPIES];
    __syncthreads();
    // Programmatic dependent launch: everything above touched only the weights and this CTA's shared
    // memory.  From here on the activations and the scratch of the previous kernel in the stream are used.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (n == 0) return;

    float acc[MT][4];
#pragma unroll
    for (int b = 0; b < MT; ++b) { acc[b][0] = acc[b][1] = acc[b][2] = acc[b][3] = 0.0f; }

    // ---- finish one row block: direct store, or deterministic reduction by the last arriver
    auto flush = [&](int rb) {
        const uint32_t first = (uint32_t)rb * P.CT, last = first + P.CT - 1;
        const GemvMat& mt = P.mat[mat_of(rb)];
        const int row0 = (rb - mt.rb_start) * TILE_ROWS + g, row1 = row0 + 8;
        const bool whole = (t0 <= first) && (t1 > last);
        if (!whole) {
            // ---- stage 1, shared memory: the parts held by this CTA's warps, added in range order by the last of them
            const uint32_t o_first = tile_owner(first, T, Wt), o_last = tile_owner(last, T, Wt);
            const uint32_t cta_lo = blockIdx.x * GEMV_WARPS;
            const uint32_t lo_t = first > cta_t0 ? first : cta_t0, hi_t = last < cta_t1 - 1u ? last : cta_t1 - 1u;   // tiles of the block in this CTA
            const uint32_t o_lo = o_first > cta_lo ? o_first : cta_lo;
            const uint32_t o_hi = o_last < cta_lo + GEMV_WARPS - 1u ? o_last : cta_lo + GEMV_WARPS - 1u;
            const uint32_t nlocal = (T < Wt) ? hi_t - lo_t + 1u : o_hi - o_lo + 1u;      // at most one tile per warp when T < Wt
            if (nlocal > 1u) {
                float* mine = red + (warp * 2 + (t0 >= first ? 0 : 1)) * FR;
#pragma unroll
                for (int b = 0; b < MT; ++b)
#pragma unroll
                    for (int r = 0; r < 4; ++r) mine[(b * 4 + r) * 32 + lane] = acc[b][r];
                __threadfence_block();
                __syncwarp();
                // counter: keyed by the first owner inside the CTA; the block that began in an earlier CTA has its own
                const uint32_t key = o_first < cta_lo ? (uint32_t)GEMV_WARPS : o_first - cta_lo;
                uint32_t old = 0;
                if (lane == 0) old = atomicAdd(&red_cnt[key], 1u);
                old = __shfl_sync(full, old, 0);
                if (old != nlocal - 1u) return;
                __threadfence_block();
#pragma unroll
                for (int b = 0; b < MT; ++b) { acc[b][0] = acc[b][1] = acc[b][2] = acc[b][3] = 0.0f; }
                if (T < Wt) {                                          // one tile per owner, owners not consecutive
                    for (uint32_t tau = lo_t; tau <= hi_t; ++tau) {
                        const volatile float* src = red + (tile_owner(tau, T, Wt) - cta_lo) * 2u * FR;
#pragma unroll
                        for (int b = 0; b < MT; ++b)
#pragma unroll
                            for (int r = 0; r < 4; ++r) acc[b][r] += src[(b * 4 + r) * 32 + lane];
                    }
                } else {                                               // consecutive owners; only the block's first owner can hold it as a tail
                    for (uint32_t o = o_lo; o <= o_hi; ++o) {
                        const uint32_t tail = (o == o_first && range_start(o, T, Wt) < first) ? 1u : 0u;
                        const volatile float* src = red + ((o - cta_lo) * 2u + tail) * FR;
#pragma unroll
                        for (int b = 0; b < MT; ++b)
#pragma unroll
                            for (int r = 0; r < 4; ++r) acc[b][r] += src[(b * 4 + r) * 32 + lane];
                    }
                }
            }
            // ---- stage 2, global scratch: one subtotal per CTA, added in CTA order by the last CTA to arrive
            const uint32_t c_first = o_first / GEMV_WARPS, c_last = o_last / GEMV_WARPS;
            if (c_first != c_last) {
                float* mine = P.partials + (size_t)(blockIdx.x * 2u + (cta_t0 >= first ? 0u : 1u)) * FR;
#pragma unroll
                for (int b = 0; b < MT; ++b)
#pragma unroll
                    for (int r = 0; r < 4; ++r) mine[(b * 4 + r) * 32 + lane] = acc[b][r];
                fence_acq_rel_gpu();
                __syncwarp();
                uint32_t old = 0;
                if (lane == 0) old = atomicAdd(&P.counters[rb], 1u);
                old = __shfl_sync(full, old, 0);
                if (old != c_last - c_first) return;
                fence_acq_rel_gpu();
#pragma unroll
                for (int b = 0; b < MT; ++b) { acc[b][0] = acc[b][1] = acc[b][2] = acc[b][3] = 0.0f; }
                for (uint32_t c = c_first; c <= c_last; ++c) {         // only the first CTA can hold the block as a tail
                    const uint32_t tail = (c == c_first && range_start(c * GEMV_WARPS, T, Wt) < first) ? 1u : 0u;
                    const float* src = P.partials + (size_t)(c * 2u + tail) * FR;
#pragma unroll
                    for (int b = 0; b < MT; ++b)
#pragma unroll
                        for (int r = 0; r < 4; ++r) acc[b][r] += __ldcg(src + (b * 4 + r) * 32 + lane);
                }
                if (lane == 0) P.counters[rb] = 0u;
            }
        }
#pragma unroll
        for (int b = 0; b < MT; ++b) {
            const int tok0 = 8 * b + 2 * t, tok1 = tok0 + 1;
            if (mt.y32) {
                if (row0 < mt.K) {
                    if (tok0 < P.M) mt.y32[(size_t)tok0 * mt.ldy + row0] = acc[b][0];
                    if (tok1 < P.M) mt.y32[(size_t)tok1 * mt.ldy + row0] = acc[b][1];
                }
                if (row1 < mt.K) {
                    if (tok0 < P.M) mt.y32[(size_t)tok0 * mt.ldy + row1] = acc[b][2];
                    if (tok1 < P.M) mt.y32[(size_t)tok1 * mt.ldy + row1] = acc[b][3];
                }
                continue;
            }
            if (row0 < mt.K) {
                if (tok0 < P.M) mt.y[(size_t)tok0 * mt.ldy + row0] = finish_output(acc[b][0], mt.bias, row0);
                if (tok1 < P.M) mt.y[(size_t)tok1 * mt.ldy + row0] = finish_output(acc[b][1], mt.bias, row0);
            }
            if (row1 < mt.K) {
                if (tok0 < P.M) mt.y[(size_t)tok0 * mt.ldy + row1] = finish_output(acc[b][2], mt.bias, row1);
                if (tok1 < P.M) mt.y[(size_t)tok1 * mt.ldy + row1] = finish_output(acc[b][3], mt.bias, row1);
            }
        }
    };

    bool healthy = true;
    int st = -1;                                                      // ring slot and phase parity of tile i
    uint32_t par = 0;
    const uint32_t tau0 = rev ? t1 - 1u : t0;                           // first tile of the walk
    int cur_rb = (int)(tau0 / (uint32_t)P.CT);
    int rb = cur_rb, ct = (int)(tau0 - (uint32_t)cur_rb * P.CT) + (rev ? 1 : -1);   // stepped at the top of every iteration
    for (int i = 0; i < issued; ++i) {
        if (++st == P.stages) { st = 0; par ^= 1u; }
        const bool ok = mbar_wait_bounded(bar0 + 8 * st, par, P.status, DEV_TIMEOUT_TILE);
        healthy = __all_sync(full, healthy && ok);
        if (!healthy) continue;                                        // drain what is in flight, decode nothing

        if (rev) { if (--ct < 0) { ct = CT - 1; --rb; } }
        else if (++ct == CT) { ct = 0; ++rb; }
        if (rb != cur_rb) {
            flush(cur_rb);
#pragma unroll
            for (int b = 0; b < MT; ++b) { acc[b][0] = acc[b][1] = acc[b][2] = acc[b][3] = 0.0f; }
            cur_rb = rb;
        }
        int w = P.G - TILE_GROUPS * ct;
        if (w > TILE_GROUPS) w = TILE_GROUPS;
        const bool active = t < w;
        const uint32_t slot = ring + st * P.slot_bytes;
        const int segA = g * w + t, segB = (g + 8) * w + t;
        uint4 mA = make_uint4(0, 0, 0, 0), mB = make_uint4(0, 0, 0, 0);
        uint32_t szA = 0, szB = 0;
        if (active) {
            mA = lds128(slot + segA * 16);
            mB = lds128(slot + segB * 16);
            szA = lds32(slot + TILE_ROWS * w * 16 + segA * 4);
            szB = lds32(slot + TILE_ROWS * w * 16 + segB * 4);
        }
        const uint32_t cntA = __popc(mA.x) + __popc(mA.y) + __popc(mA.z) + __popc(mA.w);
        const uint32_t cntB = __popc(mB.x) + __popc(mB.y) + __popc(mB.z) + __popc(mB.w);
        const uint32_t v = cntA | (cntB << 16);
        uint32_t inc = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t up = __shfl_up_sync(full, inc, d);
            if (lane >= d) inc += up;
        }
        const uint32_t tot = __shfl_sync(full, inc, 31);
        const uint32_t exc = inc - v;
        uint32_t offA = exc & 0xFFFFu;                                 // in codes
        uint32_t offB = (tot & 0xFFFFu) + (exc >> 16);

        uint32_t cbase = slot + TILE_ROWS * w * 20;
        if (BITS < 4) {                                                // re-pack the tile's codes as nibbles
            const uint32_t total = (tot & 0xFFFFu) + (tot >> 16);
            const uint32_t nchunks = (total + 7u) >> 3;
            for (uint32_t c = lane; c < nchunks; c += 32) {
                uint32_t outv;
                if (BITS == 3) {
                    const uint32_t bo = 3u * c, a = cbase + (bo & ~3u);
                    outv = spread3(funnel_r(lds32(a), lds32(a + 4), (bo & 3u) * 8u) & 0x00FFFFFFu);
                } else {
                    outv = spread2(lds32(cbase + (c >> 1) * 4u) >> (16u * (c & 1u)));
                }
                sts32(nib + c * 4u, outv);
            }
            __syncwarp();
            cbase = nib;
        }

        const SegParams pA = make_seg_params(szA, BITS, P.col_scale != nullptr);
        const SegParams pB = make_seg_params(szB, BITS, P.col_scale != nullptr);
        const bool all_fast = __all_sync(full, pA.fast && pB.fast);
        const int col0 = (ct * TILE_GROUPS + t) * GROUP;               // first column of this lane's group
        // Tokens beyond M read the last real token (their MMA columns are never stored); lanes beyond a
        // partial tile read column 0 of x, which their all-zero weights cancel.
        const uint16_t* xrow[MT];
#pragma unroll
        for (int b = 0; b < MT; ++b) {
            int tok = g + 8 * b;
            if (tok > M - 1) tok = M - 1;
            xrow[b] = P.x + (size_t)tok * P.ldx + (active ? col0 : 0);
        }
        auto lut = [lut_lane](uint32_t idx) {
            const uint2 e = lds64(lut_lane + idx * (LUT_COPIES * 8u));
            return LutEntry{e.x, e.y};
        };

#pragma unroll 1
        for (int j = 0; j < 4; ++j) {
            const uint32_t mAj = mA.x, mBj = mB.x;                     // rotate instead of indexing registers
            mA.x = mA.y; mA.y = mA.z; mA.z = mA.w;
            mB.x = mB.y; mB.y = mB.z; mB.z = mB.w;
            uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
            load_window(cbase, offA, a0, a1, a2, a3);
            load_window(cbase, offB, b0, b1, b2, b3);
            offA += __popc(mAj);
            offB += __popc(mBj);
            if (all_fast) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {                          // 16 columns at a time keeps fewer registers live
                    uint4 xv[MT][2];
#pragma unroll
                    for (int b = 0; b < MT; ++b) {
                        const uint4* xp = reinterpret_cast<const uint4*>(xrow[b] + 32 * j + 16 * h);
                        xv[b][0] = ldg_nc_early(xp);
                        xv[b][1] = ldg_nc_early(xp + 1);
                    }
                    uint32_t ea[8], eb[8];
                    decode16_fast(h ? (mAj >> 16) : (mAj & 0xFFFFu), a0, a1, a2, a3, pA, lut, ea);
                    decode16_fast(h ? (mBj >> 16) : (mBj & 0xFFFFu), b0, b1, b2, b3, pB, lut, eb);
#pragma unroll
                    for (int b = 0; b < MT; ++b) {
                        mma_bf16_16816(acc[b], ea[0], eb[0], ea[1], eb[1], xv[b][0].x, xv[b][0].y);
                        mma_bf16_16816(acc[b], ea[2], eb[2], ea[3], eb[3], xv[b][0].z, xv[b][0].w);
                        mma_bf16_16816(acc[b], ea[4], eb[4], ea[5], eb[5], xv[b][1].x, xv[b][1].y);
                        mma_bf16_16816(acc[b], ea[6], eb[6], ea[7], eb[7], xv[b][1].z, xv[b][1].w);
                    }
                }
            } else {
                uint32_t ea[16], eb[16];
                float cs[32];
                const float* csp = nullptr;
                if (P.col_scale != nullptr && active) {
#pragma unroll
                    for (int q = 0; q < 32; ++q) cs[q] = half_bits_to_float(P.col_scale[col0 + 32 * j + q]);
                    csp = cs;
                }
                decode32<LUT_COPIES>(mAj, a0, a1, a2, a3, pA, lut_lane_ptr, csp, ea);
                decode32<LUT_COPIES>(mBj, b0, b1, b2, b3, pB, lut_lane_ptr, csp, eb);
#pragma unroll
                for (int b = 0; b < MT; ++b) {
                    const uint4* xp = reinterpret_cast<const uint4*>(xrow[b] + 32 * j);
                    const uint4 x0 = __ldg(xp), x1 = __ldg(xp + 1), x2 = __ldg(xp + 2), x3 = __ldg(xp + 3);
                    mma_bf16_16816(acc[b], ea[0], eb[0], ea[1], eb[1], x0.x, x0.y);
                    mma_bf16_16816(acc[b], ea[2], eb[2], ea[3], eb[3], x0.z, x0.w);
                    mma_bf16_16816(acc[b], ea[4], eb[4], ea[5], eb[5], x1.x, x1.y);
                    mma_bf16_16816(acc[b], ea[6], eb[6], ea[7], eb[7], x1.z, x1.w);
                    mma_bf16_16816(acc[b], ea[8], eb[8], ea[9], eb[9], x2.x, x2.y);
                    mma_bf16_16816(acc[b], ea[10], eb[10], ea[11], eb[11], x2.z, x2.w);
                    mma_bf16_16816(acc[b], ea[12], eb[12], ea[13], eb[13], x3.x, x3.y);
                    mma_bf16_16816(acc[b], ea[14], eb[14], ea[15], eb[15], x3.z, x3.w);
                }
            }
        }

        __syncwarp();
        if (issued < n) { issue(issued, st); ++issued; }       // tile i + stages reuses the slot just drained
    }
    if (!healthy) return;
    flush(cur_rb);
}

}  // namespace cb
