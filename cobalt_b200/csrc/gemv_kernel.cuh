// Decode GEMV for M <= 16 tokens.
//
// Persistent kernel, one CTA per SM.  The matrix is a sequence of tiles (row-block-major); a tile is four
// "words" of 32 columns x 4 groups x 16 rows.  The words of the launch are cut into one contiguous range
// per warp: either every CTA takes whole row blocks (no partial sums cross CTAs) or the words are balanced to
// +-1 over all warps of the grid; the host picks the cheaper one per launch (cost model in words per warp,
// gemv_config() in cobalt_abi.cu).  Each warp pulls the tiles its
// range touches with 1-D bulk async copies into a private shared-memory ring (mbarrier completion), locates
// every segment's survivor codes with a popcount prefix sum over the warp, expands them to dense bf16 weights
// in registers (decode_core.cuh) and contracts them against the activations with mma.sync m16n8k16
// (A = 16 rows x 16 columns of weights, B = 16 columns x 8 tokens).  Lane (g = lane/4, t = lane%4) owns rows g
// and g+8 of the row block and group t of the tile; in MMA step s it supplies columns 4s..4s+3 of that group,
// so the 16 k-slots of one MMA are 4 consecutive columns from each of the tile's 4 groups and the B fragment
// of the lane is simply 8 contiguous bytes of x.
//
// The inner loop works in units of 16 columns (two mask bytes per row).  Everything a unit needs from shared
// memory - three words of the code stream at the unit's bit offset, the expansion table entries of its four
// mask bytes, its activations - is requested one unit ahead, so the loads of unit u+1 are in flight while unit
// u is being expanded.  Codes are decoded straight from the 2-, 3- or 4-bit stream (decode8), there is no
// re-pack pass.
//
// Activations: when M * N * 2 bytes fit beside the ring (always for one token), the CTA copies x into shared
// memory once, 16-byte chunks XOR-swizzled so that the 32 lanes of a fragment load hit 8 distinct bank groups
// per quarter warp; otherwise every lane reads its fragment from a fragment-ordered copy of x in global memory
// (x_permute_kernel: 512 contiguous bytes per warp and fragment), also one unit ahead.  A second instantiation
// of the kernel (gemv_mma_special_kernel) can compute the staged rows itself - residual add + RMSNorm, the gated
// activation, the sum of tensor-parallel partial sums - and can push its own fp32 sums into peer buffers.
//
// Row blocks covered by several warps.  Every warp holds at most two partial sums: of the row block its range
// starts in and of the one it ends in.  They are combined deterministically, in warp order:
//   * a block whose words all belong to this CTA: each warp parks its fp32 fragments in shared memory, tagged
//     with the row block; after one CTA barrier at the end of the walk the first holder of every tag adds the
//     fragments in warp order and stores the rows;
//   * a block that straddles CTAs: its holders in this CTA meet early through a shared-memory arrival counter
//     (the last of them adds the fragments in warp order), that subtotal goes to global scratch and the last
//     CTA to arrive adds the subtotals in CTA order (fence + atomic + L2 round trips, microseconds).  Warps
//     whose range ends in a block that continues into the next CTA walk their tiles backwards, so that this slow
//     exchange happens at the start of both neighbours' work instead of at the very end of the kernel.
//
// Behaviour replaced: cbk::gemv_sparse / gemv_sparse_expand, one warp per row with a 32-lane
// prefix scan per 1024-column window (src/cobaltkernel/csrc/cobalt_gemv.cuh:216-393).
#pragma once
#include "common.cuh"
#include "staged_input.cuh"

namespace cb {

constexpr int GEMV_WARPS = 16;
constexpr int GEMV_THREADS = GEMV_WARPS * 32;
constexpr int GEMV_MAX_STAGES = 4;
constexpr int TILE_WORDS = 4;                                              // 32-column words per tile
// expansion table in shared memory: 16-byte entries, 8 replicas.  A 128-bit shared load is served one
// quarter warp at a time, so 8 replicas (lane & 7) make every lookup conflict-free.
constexpr int GEMV_LUT_COPIES = 8;
constexpr uint32_t GEMV_LUT_BYTES = LUT_ENTRIES * GEMV_LUT_COPIES * 16;    // 32 KB; the staged activations follow
constexpr uint32_t GEMV_BAR_BYTES = (GEMV_WARPS * GEMV_MAX_STAGES + 2) * 8;   // tile barriers + the "activations staged" barrier
// in-CTA bookkeeping: arrival counters of the straddling blocks (one per first owner + one), then the
// row-block tags of the parked fragments [warp][head|tail]
constexpr uint32_t GEMV_REDCNT_BYTES = 128 + GEMV_WARPS * 2 * 4;
// in-CTA reduction fragments: [warp][head|tail][4 * MT * 32] floats
constexpr uint32_t gemv_red_bytes(int mt) { return GEMV_WARPS * 2 * 4 * mt * 32 * 4; }

constexpr int GEMV_MAX_MATS = 4;
static_assert(GEMV_WARPS * 2 == 32, "the end-of-walk reduction keeps one parked-fragment tag per lane");

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
    const uint4* xperm;                  // activations in fragment order (see x_permute_kernel), used when x is not staged
    int M;
    int mode;                            // in_kind | GEMV_MODE_PUSH | GEMV_MODE_SUMMED: the one word the common path tests; the
                                         // fields of the special modes sit at the end, in parameter lines it never touches
    int stages;
    uint32_t slot_bytes;
    uint32_t xs_bytes;                   // shared-memory bytes reserved for staged activations (0: read x from global)
    uint32_t total_warps;                // grid * GEMV_WARPS
    int aligned;                         // CTAs hold whole row blocks (no exchange between CTAs)
    uint32_t part_q, part_r;             // partition quotient and remainder, see cta_range_start()
    float* partials;                     // [grid][2][4 * MT * 32]: CTA subtotals of straddling row blocks
    uint32_t* counters;                  // [row blocks]
    uint32_t* status;
    // Activations computed while they are staged (staged launches only; 0: x is read as it is).
    //   GEMV_IN_GLU:     x = bf16( bf16(act(in_a)) * in_b ), in_flavor 0 SiLU / 1 tanh-GELU
    //   GEMV_IN_ADDNORM: h' = bf16(in_a + delta'), x = RMSNorm(h') * in_w; in_b = delta or null, in_wb = Gemma's
    //                    branch-norm weight or null, in_flavor 0 Llama / 1 Gemma; CTA 0 writes h' to in_hout
    int in_kind, in_flavor;
    const uint16_t* in_a; const uint16_t* in_b; int64_t in_ld;
    const uint16_t* in_w; const uint16_t* in_wb; uint16_t* in_hout; float in_eps;
    // GEMV_IN_ADDNORM whose delta is the sum over ranks of the partials pushed into this rank's peer buffer
    // (in_world > 0; in_b unused): the staging waits for every rank's flag of the current epoch, then adds the rows
    int in_world;
    const uint8_t* in_slots; unsigned long long in_stride; const uint32_t* in_flags;
    // Row-parallel output (raw fp32 sums, written to mat[0].y32 = the local staging area) copied by the last CTA of the
    // launch into row `push_rank` of the epoch's slot in EVERY rank's peer buffer and published to all ranks
    // (push_world > 0; single-matrix launches)
    int push_world, push_rank;
    unsigned long long push_base[PEER_MAX_RANKS];
    unsigned long long push_stride, push_flags_off;
    uint32_t* push_flags;                // this rank's flag block (local address)
    uint32_t* push_done;                 // CTA arrival counter in the launch's scratch, zero between launches
};
constexpr int GEMV_IN_GLU = 1, GEMV_IN_ADDNORM = 2, GEMV_MODE_IN_MASK = 3, GEMV_MODE_PUSH = 4, GEMV_MODE_SUMMED = 8;

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// bf16( bf16(acc) + bias ): the reference rounds the matmul result first and adds the bias after
__device__ __forceinline__ uint16_t finish_output(float acc, const uint16_t* bias, int row) {
    uint16_t r = float_to_bf16(acc);
    if (bias) r = float_to_bf16(bf16_to_float(r) + bf16_to_float(bias[row]));
    return r;
}

// Partition of the U words of a launch over G CTAs.  The host passes q = X / G and r = X % G, where X is the
// number of row blocks (`aligned`: every CTA holds whole row blocks, none is shared between CTAs) or the number
// of words (balanced ranges); CTA c starts at unit c*q + min(c, r), i.e. the first r CTAs hold one unit more.
// Warp w of a CTA gets [w*L/16, (w+1)*L/16) of the CTA's L words.  No division on the kernel's start-up path.
__device__ __forceinline__ uint32_t cta_range_start(uint32_t c, uint32_t q, uint32_t r, uint32_t WPB, bool aligned) {
    const uint32_t unit = c * q + (c < r ? c : r);
    return aligned ? unit * WPB : unit;
}
__device__ __forceinline__ uint32_t cta_of_word(uint32_t u, uint32_t q, uint32_t r) {      // balanced ranges only
    const uint32_t thr = r * (q + 1u);
    return u < thr ? u / (q + 1u) : r + (u - thr) / q;
}
__device__ __forceinline__ uint32_t warp_range_start(uint32_t cta_u0, uint32_t L, uint32_t w) { return cta_u0 + ((w * L) / GEMV_WARPS); }

__device__ __forceinline__ uint32_t atom_add_acq_rel_cta_shared(uint32_t* p, uint32_t v) {
    uint32_t old;
    asm volatile("atom.acq_rel.cta.shared::cta.add.u32 %0, [%1], %2;" : "=r"(old) : "r"(smem_u32(p)), "r"(v) : "memory");
    return old;
}
__device__ __forceinline__ uint32_t atom_add_acq_rel_gpu(uint32_t* p, uint32_t v) {
    uint32_t old;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
    return old;
}
// L2 eviction policies: the weight stream is read once (evict first), the small tile-offset tables are read
// by every launch and should survive the stream (evict last)
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t p; asm("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p)); return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t p; asm("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p)); return p;
}
__device__ __forceinline__ uint32_t ldg_hint(const uint32_t* p, uint64_t pol) {
    uint32_t v; asm volatile("ld.global.L2::cache_hint.u32 %0, [%1], %2;" : "=r"(v) : "l"(p), "l"(pol)); return v;
}
__device__ __forceinline__ void bulk_g2s_hint(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar, uint64_t pol) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(pol) : "memory");
}

// table entry of one mask byte, computed (no global read on the kernel's critical path); same contents as
// make_lut4(build_expand_lut()[mb], bits)
__device__ __forceinline__ uint4 gemv_lut_entry(uint32_t mb, int bits) {
    uint32_t s[8];
    uint32_t rank = 0;
#pragma unroll
    for (int p = 0; p < 8; ++p) {
        const uint32_t kept = (mb >> p) & 1u;
        const uint32_t sel = (rank & 1u) ? 4u + (rank >> 1) : (rank >> 1);
        s[p] = kept ? sel : 7u;
        rank += kept;
    }
    return make_uint4(s[0] | (s[2] << 4) | (s[1] << 8) | (s[3] << 12), s[4] | (s[6] << 4) | (s[5] << 8) | (s[7] << 12),
                      rank == 8u ? 0x3210u : 0x4210u, rank * (uint32_t)bits);
}

// Activations in fragment order, for launches whose x does not fit into shared memory: chunk (ct, c, b, lane) holds the
// 8 columns [512*ct + 128*t + 8*c, +8) of token min(g + 8*b, M-1), lane = 4*g + t, so that the 32 lanes of a warp read
// 512 contiguous bytes per fragment load instead of 32 separate lines (the read-only path serves one line per cycle).
// One thread per 16-byte chunk; columns beyond N (partial last tile) are zero.
__global__ void x_permute_kernel(const uint16_t* __restrict__ x, int64_t ldx, int M, int N, int CT, int MT, uint4* __restrict__ out) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int total = CT * 16 * MT * 32;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int lane = i & 31, b = (i >> 5) % MT, c = ((i >> 5) / MT) & 15, ct = (i >> 5) / MT / 16;
        const int g = lane >> 2, t = lane & 3;
        int tok = g + 8 * b;
        if (tok > M - 1) tok = M - 1;
        const int col = 512 * ct + 128 * t + 8 * c;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (col < N) v = __ldg(reinterpret_cast<const uint4*>(x + (size_t)tok * ldx + col));
        out[i] = v;
    }
}

// ---- activations computed while they are staged (out of line: these are the less common launches)
__device__ __forceinline__ void gemv_stage_chunk(uint8_t* xs, int chunks_per_row, int m, int c, const uint4& v) {
    const int pc = c ^ (((c >> 4) & 3) | ((m & 1) << 2));
    *reinterpret_cast<uint4*>(xs + ((size_t)m * chunks_per_row + pc) * 16) = v;
}

__device__ __noinline__ void gemv_stage_glu(const GemvParams& P, uint8_t* xs) {
    constexpr int XPRE = 2;
    const int chunks_per_row = P.N / 8, x_total = chunks_per_row * P.M;
    auto stage_chunk = [&](int m, int c, const uint4& v) { gemv_stage_chunk(xs, chunks_per_row, m, c, v); };
    // gated activation of the two halves of the previous projection, applied while staging
    // (the reference closes it in the gate|up epilogue: src/cobaltkernel/csrc/megakernel.cu:1805-1892)
    auto ld_a = [&](int m, int c) { return __ldg(reinterpret_cast<const uint4*>(P.in_a + (size_t)m * P.in_ld) + c); };
    auto ld_b = [&](int m, int c) { return __ldg(reinterpret_cast<const uint4*>(P.in_b + (size_t)m * P.in_ld) + c); };
    uint4 ga[XPRE], ub[XPRE];
#pragma unroll
    for (int q = 0; q < XPRE; ++q) {
        const int i = threadIdx.x + q * GEMV_THREADS;
        if (i < x_total) { const int m = i / chunks_per_row, c = i - m * chunks_per_row; ga[q] = ld_a(m, c); ub[q] = ld_b(m, c); }
    }
#pragma unroll
    for (int q = 0; q < XPRE; ++q) {
        const int i = threadIdx.x + q * GEMV_THREADS;
        if (i < x_total) { const int m = i / chunks_per_row; stage_chunk(m, i - m * chunks_per_row, glu_chunk(ga[q], ub[q], P.in_flavor)); }
    }
    for (int i = threadIdx.x + XPRE * GEMV_THREADS; i < x_total; i += GEMV_THREADS) {
        const int m = i / chunks_per_row, c = i - m * chunks_per_row;
        stage_chunk(m, c, glu_chunk(ld_a(m, c), ld_b(m, c), P.in_flavor));
    }
}

__device__ __noinline__ void gemv_stage_addnorm(const GemvParams& P, uint8_t* xs, float* red) {
    constexpr int XPRE = 2;
    const int lane = threadIdx.x & 31;
    const int chunks_per_row = P.N / 8, x_total = chunks_per_row * P.M;
    auto stage_chunk = [&](int m, int c, const uint4& v) { gemv_stage_chunk(xs, chunks_per_row, m, c, v); };
    // residual add + RMSNorm applied while staging (the reference normalises while it writes its activation
    // copy: write_xprime, src/cobaltkernel/csrc/megakernel.cu:270-288); rows are multiples of 256 values, so the
    // 32 chunks a warp handles in one step belong to one row.  Warp totals live in the (still unused) fragment area.
    float* tot_branch = red;
    float* tot_joined = red + 1024;
    const int groups = chunks_per_row >> 5;
    const bool has_delta = P.in_b != nullptr, norm_branch = (has_delta || (P.mode & GEMV_MODE_SUMMED)) && P.in_wb != nullptr;
    const bool summed = (P.mode & GEMV_MODE_SUMMED) != 0;                            // delta = sum of the ranks' pushed partials
    const bool has_delta2 = has_delta || summed;
    const uint8_t* slot_row0 = nullptr;
    auto ld_h = [&](int m, int c) { return __ldg(reinterpret_cast<const uint4*>(P.in_a + (size_t)m * P.in_ld) + c); };
    auto ld_d = [&](int m, int c) {
        if (summed) return peer_sum_chunk(slot_row0, P.in_stride, P.in_world, (size_t)m * P.N + (size_t)c * 8);
        return __ldg(reinterpret_cast<const uint4*>(P.in_b + (size_t)m * P.in_ld) + c);
    };
    uint4 hq[XPRE], dq[XPRE];
#pragma unroll
    for (int q = 0; q < XPRE; ++q) {
        const int i = threadIdx.x + q * GEMV_THREADS;
        if (i < x_total) { const int m = i / chunks_per_row; hq[q] = ld_h(m, i - m * chunks_per_row); }
    }
    if (summed) {                                                  // bounded wait for every rank's partial of this epoch
        const uint32_t e = *reinterpret_cast<const volatile uint32_t*>(P.in_flags + PEER_EPOCH_INDEX);
        slot_row0 = P.in_slots + (1ull + (unsigned long long)(e & 1u) * P.in_world) * P.in_stride;
        if (!peer_wait_epoch(P.in_flags, P.in_world, e) && threadIdx.x == 0) atomicCAS(P.status, 0u, (uint32_t)DEV_TIMEOUT_PEER);
    }
#pragma unroll
    for (int q = 0; q < XPRE; ++q) {
        const int i = threadIdx.x + q * GEMV_THREADS;
        dq[q] = make_uint4(0, 0, 0, 0);
        if (i < x_total && has_delta2) { const int m = i / chunks_per_row; dq[q] = ld_d(m, i - m * chunks_per_row); }
    }
    if (norm_branch) {                                             // sums of delta^2 per row
        auto branch_total = [&](int i, const uint4& dd) {          // i < x_total is the same for all lanes of a warp
            float d[8];
            chunk_to_floats(dd, d);
            const float s = warp_butterfly_sum(i < x_total ? chunk_sumsq(d) : 0.0f);
            if (lane == 0 && i < x_total) tot_branch[i >> 5] = s;
        };
#pragma unroll
        for (int q = 0; q < XPRE; ++q) branch_total(threadIdx.x + q * GEMV_THREADS, dq[q]);
        for (int i = threadIdx.x + XPRE * GEMV_THREADS; i < x_total; i += GEMV_THREADS) {
            const int m = i / chunks_per_row;
            branch_total(i, ld_d(m, i - m * chunks_per_row));
        }
        __syncthreads();
    }
    auto joined_chunk = [&](int m, int c, const uint4& hh, const uint4& dd, float (&v)[8]) {      // h' of one chunk
        chunk_to_floats(hh, v);
        if (has_delta2) {
            float d[8];
            chunk_to_floats(dd, d);
            if (norm_branch) {
                const float rb = row_rsqrt(tot_branch + m * groups, groups, P.N, P.in_eps);
                float wb[8];
                chunk_to_floats(__ldg(reinterpret_cast<const uint4*>(P.in_wb) + c), wb);
#pragma unroll
                for (int k = 0; k < 8; ++k) d[k] = branch_value(d[k], rb, wb[k]);
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = joined_value(v[k], d[k]);
        }
    };
    const bool writes_h = blockIdx.x == 0 && P.in_hout != nullptr;
    auto joined_total = [&](int i, const float (&v)[8]) {
        const float s = warp_butterfly_sum(i < x_total ? chunk_sumsq(v) : 0.0f);
        if (lane == 0 && i < x_total) tot_joined[i >> 5] = s;
        if (writes_h && i < x_total) {
            const int m = i / chunks_per_row, c = i - m * chunks_per_row;
            reinterpret_cast<uint4*>(P.in_hout + (size_t)m * P.in_ld)[c] = floats_to_chunk(v);
        }
    };
    float vk[XPRE][8];
#pragma unroll
    for (int q = 0; q < XPRE; ++q) {
        const int i = threadIdx.x + q * GEMV_THREADS;
#pragma unroll
        for (int k = 0; k < 8; ++k) vk[q][k] = 0.0f;
        if (i < x_total) { const int m = i / chunks_per_row; joined_chunk(m, i - m * chunks_per_row, hq[q], dq[q], vk[q]); }
        joined_total(i, vk[q]);
    }
    for (int i = threadIdx.x + XPRE * GEMV_THREADS; i < x_total; i += GEMV_THREADS) {
        const int m = i / chunks_per_row, c = i - m * chunks_per_row;
        float v[8];
        joined_chunk(m, c, ld_h(m, c), has_delta2 ? ld_d(m, c) : make_uint4(0, 0, 0, 0), v);
        joined_total(i, v);
    }
    __syncthreads();
    auto normed_chunk = [&](int m, int c, const float (&v)[8]) {
        const float r = row_rsqrt(tot_joined + m * groups, groups, P.N, P.in_eps);
        float wn[8], o[8];
        chunk_to_floats(__ldg(reinterpret_cast<const uint4*>(P.in_w) + c), wn);
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = normed_value(v[k], r, wn[k], P.in_flavor);
        stage_chunk(m, c, floats_to_chunk(o));
    };
#pragma unroll
    for (int q = 0; q < XPRE; ++q) {
        const int i = threadIdx.x + q * GEMV_THREADS;
        if (i < x_total) { const int m = i / chunks_per_row; normed_chunk(m, i - m * chunks_per_row, vk[q]); }
    }
    for (int i = threadIdx.x + XPRE * GEMV_THREADS; i < x_total; i += GEMV_THREADS) {         // the rest is recomputed, not kept
        const int m = i / chunks_per_row, c = i - m * chunks_per_row;
        float v[8];
        joined_chunk(m, c, ld_h(m, c), has_delta2 ? ld_d(m, c) : make_uint4(0, 0, 0, 0), v);
        normed_chunk(m, c, v);
    }
}

// Pushing launches write their fp32 sums into the local staging area like any fp32 launch.  The LAST CTA of the launch
// to get here (arrival counter in scratch) copies the complete partial into row `push_rank` of the epoch's slot in
// every rank's buffer (posted NVLink stores), advances the local epoch and tells every rank that this rank's partial is
// complete - one system-scope fence per launch.  The consumer (the next projection's staging or the summing kernel)
// waits for these flags.  A launch that gave up (status word set) still publishes: its peers then read rows it did
// not finish, which the status word reports, instead of running into their own time-out.
__device__ __noinline__ void gemv_push_publish(const GemvParams& P, uint32_t* s_last) {
    __syncthreads();                                                   // the CTA's stores are ordered before thread 0's fence
    if (threadIdx.x == 0) {
        __threadfence();
        *s_last = atom_add_acq_rel_gpu(P.push_done, 1u) == gridDim.x - 1u ? 1u : 0u;
    }
    __syncthreads();
    if (*reinterpret_cast<volatile uint32_t*>(s_last) == 0u) return;
    __threadfence();
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(P.push_flags + PEER_EPOCH_INDEX) + 1u;
    const unsigned long long row_off = (1ull + (unsigned long long)(epoch & 1u) * P.push_world + P.push_rank) * P.push_stride;
    const float4* src = reinterpret_cast<const float4*>(P.mat[0].y32);
    const uint32_t n4 = (uint32_t)((size_t)P.M * P.mat[0].K / 4);     // K is a multiple of 16
    for (uint32_t i = threadIdx.x; i < n4; i += GEMV_THREADS) {
        const float4 v = __ldcg(src + i);
#pragma unroll
        for (int q = 0; q < PEER_MAX_RANKS; ++q)
            if (q < P.push_world) reinterpret_cast<float4*>(P.push_base[q] + row_off)[i] = v;
    }
    __syncthreads();                                                   // the release below covers every thread's stores
    if (threadIdx.x == 0) {
        *P.push_done = 0u;
        P.push_flags[PEER_EPOCH_INDEX] = epoch;
        __threadfence_system();
#pragma unroll
        for (int q = 0; q < PEER_MAX_RANKS; ++q)
            if (q < P.push_world)
                st_release_sys_u32(reinterpret_cast<uint32_t*>(P.push_base[q] + P.push_flags_off) + P.push_rank, epoch);
    }
}

// what one unit (16 columns of both rows of a lane) reads from memory; requested one unit ahead
template <int MT>
struct GemvUnit {
    uint32_t ra0, ra1, ra2, rb0, rb1, rb2;     // code-stream words at the unit's bit offset, rows A and B
    uint4 ea0, ea1, eb0, eb1;                  // table entries of the unit's mask bytes
    uint4 x[MT][2];                            // activations: 16 columns x token g (+8)
};

// SPECIAL = the launch computes its activations while staging them, adds pushed partial sums, or pushes its own
// (GemvParams::mode != 0).  The common launch is a kernel of its own without any of that code, so that the
// less common modes cost it neither a start-up test nor a register.
template <int BITS, int MT, bool XS, bool SPECIAL>
__device__ __forceinline__ void gemv_mma_body(const GemvParams& P) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t full = 0xFFFFFFFFu;
    // Fields of the matrix that owns row block rbg of the launch.  Selected with compares over the (at most four)
    // parameter slots: indexing the parameter block with a run-time value would turn every access into a load from
    // the constant cache, cold at every launch and on the path to the first tile request.
    auto mat_of = [&](int rbg) {
        int m = 0;
#pragma unroll
        for (int k = 1; k < GEMV_MAX_MATS; ++k)
            if (k < P.n_mats && rbg >= P.mat[k].rb_start) m = k;
        return m;
    };
#define MAT_FIELD(m, f) ((m) == 0 ? P.mat[0].f : (m) == 1 ? P.mat[1].f : (m) == 2 ? P.mat[2].f : P.mat[3].f)

    // ---- shared-memory map: table | staged activations | barriers | in-CTA counters, tags | in-CTA fragments | rings
    uint4* lut_s = reinterpret_cast<uint4*>(smem);
    uint8_t* xs = smem + GEMV_LUT_BYTES;
    uint8_t* after_x = xs + P.xs_bytes;
    const uint32_t bar0 = smem_u32(after_x) + warp * GEMV_MAX_STAGES * 8;
    const uint32_t xbar = smem_u32(after_x) + GEMV_WARPS * GEMV_MAX_STAGES * 8;     // every thread arrives once x and the table are in place
    constexpr int FR = 4 * MT * 32;                                    // floats of one accumulator fragment set
    uint32_t* red_cnt = reinterpret_cast<uint32_t*>(after_x + GEMV_BAR_BYTES);
    int* red_tag = reinterpret_cast<int*>(after_x + GEMV_BAR_BYTES + 128);          // [warp][head|tail] row block or -1
    float* red = reinterpret_cast<float*>(after_x + GEMV_BAR_BYTES + GEMV_REDCNT_BYTES);
    // ---- this warp's share of the launch, and the offsets of its first tiles (their loads fly during the set-up)
    const int M = P.M, CT = P.CT;
    const uint32_t WPB = (uint32_t)TILE_WORDS * (uint32_t)CT;          // words per row block
    const bool aligned = P.aligned != 0;
    const uint32_t cta_u0 = cta_range_start(blockIdx.x, P.part_q, P.part_r, WPB, aligned);
    const uint32_t cta_u1 = cta_range_start(blockIdx.x + 1u, P.part_q, P.part_r, WPB, aligned);
    const uint32_t Lc = cta_u1 - cta_u0;
    const uint32_t u0 = warp_range_start(cta_u0, Lc, (uint32_t)warp), u1 = warp_range_start(cta_u0, Lc, (uint32_t)warp + 1u);
    const bool busy = u1 > u0;
    const uint32_t ta = u0 / TILE_WORDS, tb = busy ? (u1 - 1u) / TILE_WORDS : ta;   // first and last tile the range touches
    const int n = busy ? (int)(tb - ta + 1u) : 0;
    // row blocks of this CTA that it shares with a neighbour (-1: none on that side; never with aligned ranges)
    int blk_left = -1, blk_right = -1;
    bool rev = false;
    if (!aligned && Lc != 0u) {
        if (cta_u0 % WPB != 0u) blk_left = (int)(cta_u0 / WPB);
        if (cta_u1 % WPB != 0u) blk_right = (int)((cta_u1 - 1u) / WPB);
        // A warp whose range ends in the row block that continues into the next CTA walks backwards: that block's
        // exchange through global scratch then starts early in both CTAs instead of ending the kernel.
        rev = busy && blk_right >= 0 && u1 - 1u >= (uint32_t)blk_right * WPB;
    }
    auto tile_at = [&](int i) { return rev ? tb - (uint32_t)i : ta + (uint32_t)i; };
    const uint64_t pol_stream = l2_policy_evict_first(), pol_keep = l2_policy_evict_last();

    // offsets of the i-th tile of the walk, requested by lane i for the first 32 tiles; they are turned into an
    // address and a size only when the copy is issued, so the loads fly during the block set-up
    auto tile_offsets = [&](uint32_t tau, uint32_t& o0, uint32_t& o1, const uint8_t*& base) {
        const int m = mat_of((int)(tau / (uint32_t)P.CT));
        const uint32_t local = tau - (uint32_t)MAT_FIELD(m, rb_start) * (uint32_t)P.CT;
        const uint32_t* toff = MAT_FIELD(m, tile_off);
        base = MAT_FIELD(m, tiles);
        o0 = ldg_hint(toff + local, pol_keep);
        o1 = ldg_hint(toff + local + 1, pol_keep);
    };
    const uint8_t* my_base = nullptr;
    uint32_t my_o0 = 0, my_o1 = 0;
    if (lane < n) tile_offsets(tile_at(lane), my_o0, my_o1, my_base);

    // ---- block set-up: barriers first, so that the first tiles are in flight while the table is being written
    if (lane == 0)
        for (int s = 0; s < P.stages; ++s) mbar_init(bar0 + 8 * s, 1);
    if (threadIdx.x == 0) mbar_init(xbar, GEMV_THREADS);
    if (threadIdx.x < 2) red_cnt[threadIdx.x] = 0u;
    if (threadIdx.x < GEMV_WARPS * 2) red_tag[threadIdx.x] = -1;
    mbar_fence_init();
    fence_proxy_async();
    __syncthreads();

    uint8_t* ring_p = after_x + GEMV_BAR_BYTES + GEMV_REDCNT_BYTES + gemv_red_bytes(MT) + (size_t)warp * P.stages * P.slot_bytes;
    const uint32_t ring = smem_u32(ring_p);
    const uint32_t lut_lane = smem_u32(lut_s) + (uint32_t)(lane & (GEMV_LUT_COPIES - 1)) * 16u;      // this lane's replica
    const uint32_t xs32 = smem_u32(xs);                               // 256-byte aligned: the swizzle is XORed into addresses

    auto issue = [&](int i, int slot_idx, bool drained) {              // all lanes call; lane 0 acts
        const uint8_t* base;
        uint32_t o0, o1;
        if (i < 32) {
            base = (const uint8_t*)__shfl_sync(full, (unsigned long long)my_base, i);
            o0 = __shfl_sync(full, my_o0, i);
            o1 = __shfl_sync(full, my_o1, i);
        } else {
            tile_offsets(tile_at(i), o0, o1, base);
        }
        if (lane == 0) {
            const uint32_t bar = bar0 + 8 * slot_idx;
            const uint32_t bytes = (o1 - o0) * 16u;
            if (drained) fence_proxy_async();                          // the slot was read through the generic proxy before
            mbar_arrive_expect_tx(bar, bytes);
            bulk_g2s_hint(ring + slot_idx * P.slot_bytes, base + (size_t)o0 * 16, bytes, bar, pol_stream);
        }
    };

    int issued = n < P.stages ? n : P.stages;
    if (issued > 0) issue(0, 0, false);                               // the first tile is on its way before anything else
    // Programmatic dependent launch: everything above touched only the weights and this CTA's shared
    // memory.  From here on the activations and the scratch of the previous kernel in the stream are used.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // x -> shared memory, rows of N bf16, 16-byte chunk c of token m stored at chunk c ^ swizzle(group, m).  The
    // first chunks of every thread are requested before the table is built, so that their latency hides behind it.
    constexpr int XPRE = 2;
    const int chunks_per_row = P.N / 8;
    const int x_total = XS ? chunks_per_row * M : 0;
    static_assert(GEMV_THREADS == 2 * LUT_ENTRIES && GEMV_LUT_COPIES == 8, "table fill: one entry and four replicas per thread");
    auto fill_table = [&]() {
        const uint32_t mb = threadIdx.x & (LUT_ENTRIES - 1), half = threadIdx.x / LUT_ENTRIES;
        const uint4 e = gemv_lut_entry(mb, BITS);
        uint4* dst = lut_s + mb * GEMV_LUT_COPIES + half * (GEMV_LUT_COPIES / 2);
#pragma unroll
        for (int c = 0; c < GEMV_LUT_COPIES / 2; ++c) dst[c] = e;
    };
    auto stage_chunk = [&](int m, int c, const uint4& v) {
        const int pc = c ^ (((c >> 4) & 3) | ((m & 1) << 2));
        *reinterpret_cast<uint4*>(xs + ((size_t)m * chunks_per_row + pc) * 16) = v;
    };
    if (!SPECIAL || !XS || (P.mode & GEMV_MODE_IN_MASK) == 0) {
        uint4 xpre[XPRE];
#pragma unroll
        for (int q = 0; q < XPRE; ++q) {
            const int i = threadIdx.x + q * GEMV_THREADS;
            if (i < x_total) {
                const int m = i / chunks_per_row, c = i - m * chunks_per_row;
                xpre[q] = __ldg(reinterpret_cast<const uint4*>(P.x + (size_t)m * P.ldx) + c);
            }
        }
        fill_table();
#pragma unroll
        for (int q = 0; q < XPRE; ++q) {
            const int i = threadIdx.x + q * GEMV_THREADS;
            if (i < x_total) { const int m = i / chunks_per_row; stage_chunk(m, i - m * chunks_per_row, xpre[q]); }
        }
        for (int i = threadIdx.x + XPRE * GEMV_THREADS; i < x_total; i += GEMV_THREADS) {
            const int m = i / chunks_per_row, c = i - m * chunks_per_row;
            stage_chunk(m, c, __ldg(reinterpret_cast<const uint4*>(P.x + (size_t)m * P.ldx) + c));
        }
    } else {
        // special inputs: computed while staged, out of line so that they do not weigh on the common path's code
        fill_table();
        if ((P.mode & GEMV_MODE_IN_MASK) == GEMV_IN_GLU) gemv_stage_glu(P, xs);
        else gemv_stage_addnorm(P, xs, red);
    }
    mbar_arrive(xbar);                                                 // releases this thread's table and x stores
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    for (int i = 1; i < issued; ++i) issue(i, i, false);               // the rest of the ring, off the path to the first decode

    float acc[MT][4];
#pragma unroll
    for (int b = 0; b < MT; ++b) { acc[b][0] = acc[b][1] = acc[b][2] = acc[b][3] = 0.0f; }

    // ---- rows of one finished row block -> y
    auto store_rows = [&](int rb) {
        const int mi = mat_of(rb);
        GemvMat mt;
        mt.y = MAT_FIELD(mi, y); mt.y32 = MAT_FIELD(mi, y32); mt.bias = MAT_FIELD(mi, bias); mt.ldy = MAT_FIELD(mi, ldy);
        mt.K = MAT_FIELD(mi, K); mt.rb_start = MAT_FIELD(mi, rb_start);
        const int row0 = (rb - mt.rb_start) * TILE_ROWS + g, row1 = row0 + 8;
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
    auto park = [&](float* dst) {
#pragma unroll
        for (int b = 0; b < MT; ++b)
#pragma unroll
            for (int r = 0; r < 4; ++r) dst[(b * 4 + r) * 32 + lane] = acc[b][r];
    };
    auto clear_acc = [&]() {
#pragma unroll
        for (int b = 0; b < MT; ++b) { acc[b][0] = acc[b][1] = acc[b][2] = acc[b][3] = 0.0f; }
    };

    // ---- the warp has added its last word of row block rb
    auto finish_block = [&](int rb) {
        const uint32_t first = (uint32_t)rb * WPB, last = first + WPB - 1u;
        if (u0 <= first && u1 > last) { store_rows(rb); return; }      // the whole block was this warp's
        const int side = u0 >= first ? 0 : 1;                          // the block the range starts in / ends in
        float* mine = red + (warp * 2 + side) * FR;
        if (rb != blk_left && rb != blk_right) {                       // all holders are in this CTA: combined after the walk
            park(mine);
            if (lane == 0) red_tag[warp * 2 + side] = rb;
            return;
        }
        // ---- straddling block, stage 1: its holders in this CTA (consecutive warps), added in warp order by the
        //      last of them to arrive.  Lane w < 16 works out warp w's range; two ballots give the holders and which
        //      of them hold the block as the one their range ends in.
        const uint32_t wl0 = warp_range_start(cta_u0, Lc, (uint32_t)(lane & 15)), wl1 = warp_range_start(cta_u0, Lc, (uint32_t)(lane & 15) + 1u);
        const bool holds = lane < GEMV_WARPS && wl1 > wl0 && wl0 <= last && wl1 > first;
        const uint32_t holders = __ballot_sync(full, holds), tails = __ballot_sync(full, holds && wl0 < first);
        const uint32_t nlocal = (uint32_t)__popc(holders);
        if (nlocal > 1u) {
            park(mine);
            __syncwarp();
            uint32_t old = 0;
            if (lane == 0) old = atom_add_acq_rel_cta_shared(&red_cnt[rb == blk_left ? 0 : 1], 1u);
            old = __shfl_sync(full, old, 0);
            if (old != nlocal - 1u) return;
            clear_acc();
            for (uint32_t hm = holders; hm; hm &= hm - 1u) {
                const uint32_t o = (uint32_t)__ffs(hm) - 1u;
                const volatile float* src = red + (o * 2u + ((tails >> o) & 1u)) * FR;
#pragma unroll
                for (int b = 0; b < MT; ++b)
#pragma unroll
                    for (int r = 0; r < 4; ++r) acc[b][r] += src[(b * 4 + r) * 32 + lane];
            }
        }
        // ---- stage 2, global scratch: one subtotal per CTA, added in CTA order by the last CTA to arrive
        const uint32_t c_first = cta_of_word(first, P.part_q, P.part_r), c_last = cta_of_word(last, P.part_q, P.part_r);
        if (c_first != c_last) {
            float* sub = P.partials + (size_t)(blockIdx.x * 2u + (cta_u0 >= first ? 0u : 1u)) * FR;
            park(sub);
            __syncwarp();
            uint32_t old = 0;
            if (lane == 0) old = atom_add_acq_rel_gpu(&P.counters[rb], 1u);
            old = __shfl_sync(full, old, 0);
            if (old != c_last - c_first) return;
            clear_acc();
            for (uint32_t c = c_first; c <= c_last; ++c) {             // only the first CTA can hold the block as a tail
                const uint32_t tail = (c == c_first && cta_range_start(c, P.part_q, P.part_r, WPB, false) < first) ? 1u : 0u;
                const float* src = P.partials + (size_t)(c * 2u + tail) * FR;
#pragma unroll
                for (int b = 0; b < MT; ++b)
#pragma unroll
                    for (int r = 0; r < 4; ++r) acc[b][r] += __ldcg(src + (b * 4 + r) * 32 + lane);
            }
            if (lane == 0) P.counters[rb] = 0u;
        }
        store_rows(rb);
    };

    // tokens of this lane's B fragments: g and g + 8; columns of tokens beyond M are computed from the last
    // real token and never stored
    int tok[MT];
#pragma unroll
    for (int b = 0; b < MT; ++b) { tok[b] = g + 8 * b; if (tok[b] > M - 1) tok[b] = M - 1; }
    const uint32_t x_row_bytes = (uint32_t)P.N * 2u;

    bool healthy = true;
    bool staged = false;                                              // has this warp seen the table and the staged x yet?
    int st = -1;                                                      // ring slot and phase parity of tile i
    uint32_t par = 0;
    const uint32_t tau0 = rev ? tb : ta;                                // first tile of the walk
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
            finish_block(cur_rb);
            clear_acc();
            cur_rb = rb;
        }
        // words of this tile that belong to the range
        const uint32_t tau = tile_at(i);
        const int ja = tau == ta ? (int)(u0 % TILE_WORDS) : 0;
        const int jb = tau == tb ? (int)((u1 - 1u) % TILE_WORDS) + 1 : TILE_WORDS;
        int w = P.G - TILE_GROUPS * ct;
        if (w > TILE_GROUPS) w = TILE_GROUPS;
        const bool active = t < w;
        const uint32_t slot = ring + (uint32_t)st * P.slot_bytes;      // shared-window address of the tile
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
        uint32_t bitA = (exc & 0xFFFFu) * BITS;                        // bit offset of the lane's first code, row A / row B
        uint32_t bitB = ((tot & 0xFFFFu) + (exc >> 16)) * BITS;
        const uint32_t cw = slot + TILE_ROWS * w * 20;                 // code stream of the tile
        for (int r = 0; r < ja; ++r) {                                 // skip the words in front of the range
            bitA += BITS * __popc(mA.x); bitB += BITS * __popc(mB.x);
            mA.x = mA.y; mA.y = mA.z; mA.z = mA.w;
            mB.x = mB.y; mB.y = mB.z; mB.z = mB.w;
        }

        if (!staged) {                                                 // first tile: the table and the staged x must be in place
            healthy = __all_sync(full, mbar_wait_bounded(xbar, 0u, P.status, DEV_TIMEOUT_TILE));
            staged = true;
            if (!healthy) continue;
        }
        const SegParams pA = make_seg_params(szA, BITS, P.col_scale != nullptr);
        const SegParams pB = make_seg_params(szB, BITS, P.col_scale != nullptr);
        const bool all_fast = __all_sync(full, pA.fast && pB.fast);
        const int col0 = active ? (ct * TILE_GROUPS + t) * GROUP : 0;  // first column of this lane's group; lanes beyond a
                                                                       // partial tile read column 0, their zero weights cancel it
        // activations of this lane's group: staged copy (byte offset with the swizzle folded in) or global rows
        uint32_t xs_lane[MT];
        const uint16_t* xrow[MT];
        const uint4* xfrag = P.xperm + (size_t)ct * 16 * MT * 32 + lane;       // this lane's chunks of the tile's columns
#pragma unroll
        for (int b = 0; b < MT; ++b) {
            xs_lane[b] = xs32 + (uint32_t)tok[b] * x_row_bytes + (uint32_t)col0 * 2u + ((uint32_t)((t & 3) | ((tok[b] & 1) << 2)) << 4);
            xrow[b] = P.x + (size_t)tok[b] * P.ldx + col0;
        }

        if (all_fast) {
            // ---- request everything unit `u` (16 columns: half h of mask word j) needs
            auto load_unit = [&](uint32_t m16A, uint32_t m16B, uint32_t bA, uint32_t bB, int j, int h) {
                GemvUnit<MT> Un;
                const uint32_t pa = cw + ((bA >> 5) << 2), pb = cw + ((bB >> 5) << 2);
                Un.ra0 = lds32(pa); Un.ra1 = lds32(pa + 4); Un.ra2 = BITS == 2 ? 0u : lds32(pa + 8);
                Un.rb0 = lds32(pb); Un.rb1 = lds32(pb + 4); Un.rb2 = BITS == 2 ? 0u : lds32(pb + 8);
                Un.ea0 = lds128(lut_lane + (m16A & 0xFFu) * (GEMV_LUT_COPIES * 16u));
                Un.ea1 = lds128(lut_lane + (m16A >> 8) * (GEMV_LUT_COPIES * 16u));
                Un.eb0 = lds128(lut_lane + (m16B & 0xFFu) * (GEMV_LUT_COPIES * 16u));
                Un.eb1 = lds128(lut_lane + (m16B >> 8) * (GEMV_LUT_COPIES * 16u));
#pragma unroll
                for (int b = 0; b < MT; ++b) {
                    if (XS) {
                        const uint32_t jo = (uint32_t)j << 6;
                        Un.x[b][0] = lds128(xs_lane[b] ^ (jo | (uint32_t)(32 * h)));
                        Un.x[b][1] = lds128(xs_lane[b] ^ (jo | (uint32_t)(32 * h + 16)));
                    } else {
                        // fragment-ordered copy: chunk index 4*(j & 3) + 2*h (j == 4 is the unused look-ahead)
                        const uint4* xp = xfrag + ((size_t)(4 * (j & 3) + 2 * h) * MT + b) * 32;
                        Un.x[b][0] = __ldg(xp);
                        Un.x[b][1] = __ldg(xp + MT * 32);
                    }
                }
                return Un;
            };
            // ---- expand one unit and feed the tensor cores
            auto compute_unit = [&](const GemvUnit<MT>& Un, uint32_t bA, uint32_t bB) {
                uint32_t oa[8], ob[8];
                const uint32_t a0 = funnel_r(Un.ra0, Un.ra1, bA);
                const uint32_t a1 = BITS == 2 ? a0 >> Un.ea0.w : funnel_rc(a0, funnel_r(Un.ra1, Un.ra2, bA), Un.ea0.w);
                decode8<BITS>(a0, Un.ea0.x, Un.ea0.y, Un.ea0.z, pA, oa);
                decode8<BITS>(a1, Un.ea1.x, Un.ea1.y, Un.ea1.z, pA, oa + 4);
                const uint32_t b0 = funnel_r(Un.rb0, Un.rb1, bB);
                const uint32_t b1 = BITS == 2 ? b0 >> Un.eb0.w : funnel_rc(b0, funnel_r(Un.rb1, Un.rb2, bB), Un.eb0.w);
                decode8<BITS>(b0, Un.eb0.x, Un.eb0.y, Un.eb0.z, pB, ob);
                decode8<BITS>(b1, Un.eb1.x, Un.eb1.y, Un.eb1.z, pB, ob + 4);
#pragma unroll
                for (int b = 0; b < MT; ++b) {
                    mma_bf16_16816(acc[b], oa[0], ob[0], oa[1], ob[1], Un.x[b][0].x, Un.x[b][0].y);
                    mma_bf16_16816(acc[b], oa[2], ob[2], oa[3], ob[3], Un.x[b][0].z, Un.x[b][0].w);
                    mma_bf16_16816(acc[b], oa[4], ob[4], oa[5], ob[5], Un.x[b][1].x, Un.x[b][1].y);
                    mma_bf16_16816(acc[b], oa[6], ob[6], oa[7], ob[7], Un.x[b][1].z, Un.x[b][1].w);
                }
            };

            // one word (two units) of both rows; `cur` arrives requested, the first unit of the next word leaves requested
            auto do_word = [&](GemvUnit<MT>& cur, uint32_t mAj, uint32_t mBj, uint32_t mAn, uint32_t mBn, int j) {
                const uint32_t bitA1 = bitA + BITS * __popc(mAj & 0xFFFFu), bitB1 = bitB + BITS * __popc(mBj & 0xFFFFu);
                const GemvUnit<MT> nxt = load_unit(mAj >> 16, mBj >> 16, bitA1, bitB1, j, 1);
                compute_unit(cur, bitA, bitB);
                const uint32_t bitA2 = bitA + BITS * __popc(mAj), bitB2 = bitB + BITS * __popc(mBj);
                // after the last word this requests a unit that is never expanded (harmless in-bounds reads)
                cur = load_unit(mAn & 0xFFFFu, mBn & 0xFFFFu, bitA2, bitB2, j + 1, 0);
                compute_unit(nxt, bitA1, bitB1);
                bitA = bitA2; bitB = bitB2;
            };
            GemvUnit<MT> cur = load_unit(mA.x & 0xFFFFu, mB.x & 0xFFFFu, bitA, bitB, ja, 0);
            if (ja == 0 && jb == TILE_WORDS) {                         // whole tile: straight-line code, no register rotation
                do_word(cur, mA.x, mB.x, mA.y, mB.y, 0);
                do_word(cur, mA.y, mB.y, mA.z, mB.z, 1);
                do_word(cur, mA.z, mB.z, mA.w, mB.w, 2);
                do_word(cur, mA.w, mB.w, mA.w, mB.w, 3);
            } else {
#pragma unroll 1
                for (int j = ja; j < jb; ++j) {
                    const uint32_t mAj = mA.x, mBj = mB.x;             // rotate instead of indexing registers
                    mA.x = mA.y; mA.y = mA.z; mA.z = mA.w;
                    mB.x = mB.y; mB.y = mB.z; mB.z = mB.w;
                    do_word(cur, mAj, mBj, mA.x, mB.x, j);
                }
            }
        } else {
            // ---- literal fp32 path (off-grid zero points, column scale): one 32-column word at a time
            auto word_at = [&](uint32_t k) { return lds32(cw + 4u * k); };
#pragma unroll 1
            for (int j = ja; j < jb; ++j) {
                const uint32_t mAj = mA.x, mBj = mB.x;
                mA.x = mA.y; mA.y = mA.z; mA.z = mA.w;
                mB.x = mB.y; mB.y = mB.z; mB.z = mB.w;
                uint32_t ea[16], eb[16];
                float cs[32];
                const float* csp = nullptr;
                if (P.col_scale != nullptr) {
#pragma unroll
                    for (int q = 0; q < 32; ++q) cs[q] = half_bits_to_float(P.col_scale[col0 + 32 * j + q]);
                    csp = cs;
                }
                decode32_slow(mAj, word_at, bitA, BITS, pA, csp, ea);
                decode32_slow(mBj, word_at, bitB, BITS, pB, csp, eb);
                bitA += BITS * __popc(mAj);
                bitB += BITS * __popc(mBj);
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
        if (issued < n) { issue(issued, st, true); ++issued; }       // tile i + stages reuses the slot just drained
    }
    if (healthy && busy) finish_block(cur_rb);

    // ---- row blocks shared by warps of this CTA only: first holder adds the parked fragments in warp order
    __syncthreads();
    if (healthy) {
        const int lane_tag = red_tag[lane];                            // GEMV_WARPS * 2 == 32 slots: one per lane
#pragma unroll 1
        for (int side = 0; side < 2; ++side) {
            const int slot_id = warp * 2 + side;
            const int tag = __shfl_sync(full, lane_tag, slot_id);
            if (tag < 0) continue;
            uint32_t holders = __ballot_sync(full, lane_tag == tag);   // parked fragments of this row block, in warp order
            if ((int)__ffs(holders) - 1 != slot_id) continue;          // only the first holder reduces
            clear_acc();
            while (holders) {
                const int k = __ffs(holders) - 1;
                holders &= holders - 1u;
                const float* src = red + k * FR;
#pragma unroll
                for (int b = 0; b < MT; ++b)
#pragma unroll
                    for (int r = 0; r < 4; ++r) acc[b][r] += src[(b * 4 + r) * 32 + lane];
            }
            store_rows(tag);
        }
    }
    if (SPECIAL && (P.mode & GEMV_MODE_PUSH)) gemv_push_publish(P, red_cnt + 2);
}

template <int BITS, int MT, bool XS>
__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_mma_kernel(const GemvParams P) {
    gemv_mma_body<BITS, MT, XS, false>(P);
}
// parameters in place (their address is handed to the out-of-line staging and push functions)
template <int BITS, int MT, bool XS>
__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_mma_special_kernel(const __grid_constant__ GemvParams P) {
    gemv_mma_body<BITS, MT, XS, true>(P);
}

}  // namespace cb
