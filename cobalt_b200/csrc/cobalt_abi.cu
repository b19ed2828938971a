// C ABI of libcobalt_b200.so: argument validation, launch configuration, kernel launches.
// See include/cobalt_b200.h for the contract of every entry point.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "common.cuh"
#include "walk_kernels.cuh"
#include "gemv_kernel.cuh"
#include "gemm_kernel.cuh"
#include "glue_kernels.cuh"

using namespace cb;

namespace {

constexpr size_t SMEM_LIMIT = 227 * 1024;
constexpr int MAX_DEVICES = 64;

int g_num_sms[MAX_DEVICES];
int g_cc_major[MAX_DEVICES];
bool g_dev_known[MAX_DEVICES];
// Launch heuristics can be overridden for experiments when the library is built with -DCOBALT_TUNING_HOOKS
// (cobalt_set_tuning is then exported); the product build has no such state.
#ifdef COBALT_TUNING_HOOKS
int g_tune_tiles_per_split = 0;     // 0 = heuristic
int g_tune_gemv_stages = 0;
int g_tune_gemm_stages = 0;
int g_tune_gemv_mode = 0;           // 0 = heuristic, 1 = CTAs hold whole row blocks, 2 = balanced words
#else
constexpr int g_tune_tiles_per_split = 0, g_tune_gemv_stages = 0, g_tune_gemm_stages = 0, g_tune_gemv_mode = 0;
#endif

inline size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

int device_info(int* num_sms) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return COBALT_ELAUNCH;
    if (dev < 0 || dev >= MAX_DEVICES) return COBALT_EINVAL;
    if (!g_dev_known[dev]) {
        if (cudaDeviceGetAttribute(&g_num_sms[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return COBALT_ELAUNCH;
        if (cudaDeviceGetAttribute(&g_cc_major[dev], cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return COBALT_ELAUNCH;
        g_dev_known[dev] = true;
    }
    if (g_cc_major[dev] != 10) return COBALT_EARCH;
    *num_sms = g_num_sms[dev];
    return COBALT_OK;
}

int check_mat(const CobaltMat* w) {
    if (!w || !w->tiles || !w->tile_off) return COBALT_EINVAL;
    if (w->K <= 0 || w->N <= 0 || w->N % GROUP != 0 || w->group != GROUP) return COBALT_EINVAL;
    if (w->bits < 2 || w->bits > 4) return COBALT_EINVAL;
    if (w->n_row_blocks != (w->K + TILE_ROWS - 1) / TILE_ROWS) return COBALT_EINVAL;
    if (w->n_col_tiles != (w->N / GROUP + TILE_GROUPS - 1) / TILE_GROUPS) return COBALT_EINVAL;
    if (((uintptr_t)w->tiles & 15) || ((uintptr_t)w->tile_off & 3)) return COBALT_EINVAL;
    if (w->max_tile_bytes < 320 || (w->max_tile_bytes & 15)) return COBALT_EINVAL;
    if (w->max_tile_bytes > TILE_ROWS * TILE_GROUPS * 20 + TILE_ROWS * TILE_GROUPS * GROUP * 4 / 8 + 16) return COBALT_EINVAL;
    if (w->max_tile_nnz > (uint32_t)(TILE_ROWS * TILE_GROUPS * GROUP)) return COBALT_EINVAL;
    if ((size_t)w->max_tile_nnz * w->bits / 8 + 320 > (size_t)w->max_tile_bytes + 16) return COBALT_EINVAL;
    return COBALT_OK;
}

int check_io(const void* x, int64_t ldx, const void* y, int64_t ldy, int M, int K, int N) {
    if (!x || !y || M <= 0) return COBALT_EINVAL;
    if (ldx < N || ldy < K) return COBALT_EINVAL;
    if (((uintptr_t)x & 15) || (ldx & 7)) return COBALT_EINVAL;       // 16-byte vector loads of x
    if ((uintptr_t)y & 1) return COBALT_EINVAL;
    return COBALT_OK;
}

// ----------------------------------------------------------------------------- GEMV configuration
struct GemvCfg {
    int stages, mt, grid;
    bool xs;                           // activations staged in shared memory
    bool aligned;                      // every CTA holds whole row blocks
    uint32_t slot, xs_bytes, total_warps, part_q, part_r;
    size_t smem, counters_off, partials_off, xperm_off, total;
};

// geometry shared by the matrices of one (possibly fused) GEMV launch
struct GemvGeom { int RB, CT, bits; uint32_t max_tile_bytes, max_tile_nnz; };

GemvGeom geom_of(const CobaltMat* w) {
    GemvGeom g;
    g.RB = w->n_row_blocks; g.CT = w->n_col_tiles; g.bits = w->bits;
    g.max_tile_bytes = w->max_tile_bytes; g.max_tile_nnz = w->max_tile_nnz;
    return g;
}

int gemv_config(const GemvGeom& g, int N, int M, int num_sms, GemvCfg* c) {
    const int RB = g.RB, CT = g.CT;
    c->mt = M > 8 ? 2 : 1;
    c->slot = (uint32_t)round_up((size_t)g.max_tile_bytes + 32, 128);
    const size_t fixed = GEMV_LUT_BYTES + GEMV_BAR_BYTES + GEMV_REDCNT_BYTES + gemv_red_bytes(c->mt) + 64;
    // Two ring slots per warp keep one tile in flight behind the one being decoded.  The activations are staged in
    // shared memory when they fit beside such a ring (always for one token); what is left goes to deeper rings.
    const size_t xs_want = c->mt == 1 ? round_up((size_t)M * N * 2 + 64, 256) : 0;
    c->xs = xs_want != 0 && fixed + xs_want + (size_t)GEMV_WARPS * 2 * c->slot <= SMEM_LIMIT;
    c->xs_bytes = c->xs ? (uint32_t)xs_want : 0u;
    // without the staged copy the activations come through L1: a shallower ring leaves it more room
    int stages = g_tune_gemv_stages > 0 ? g_tune_gemv_stages : (c->xs ? 3 : 2);
    if (stages > GEMV_MAX_STAGES) stages = GEMV_MAX_STAGES;
    while (stages > 1 && fixed + c->xs_bytes + (size_t)GEMV_WARPS * stages * c->slot > SMEM_LIMIT) --stages;
    if (fixed + c->xs_bytes + (size_t)GEMV_WARPS * stages * c->slot > SMEM_LIMIT) return COBALT_EINVAL;
    c->stages = stages;
    c->smem = fixed + c->xs_bytes + (size_t)GEMV_WARPS * stages * c->slot;
    // Persistent grid, at most one CTA per SM.  Preferred: every CTA holds whole row blocks, so that no partial sums
    // cross CTAs - the grid is the smallest one that reaches the minimal number of row blocks per CTA.  When that
    // leaves much of the machine idle (few, long row blocks), the words are balanced over all SMs instead and the
    // blocks that straddle CTAs are exchanged through global scratch.
    const long tiles = (long)RB * CT;
    const long per_cta = (RB + num_sms - 1) / num_sms;                  // row blocks of the busiest CTA
    long grid = (RB + per_cta - 1) / per_cta;
    // words per warp either way; the exchange of the straddling blocks costs about as much as five words
    const double words_aligned = (double)per_cta * CT * TILE_WORDS / GEMV_WARPS;
    const double words_balanced = (double)tiles * TILE_WORDS / ((double)num_sms * GEMV_WARPS) + 5.0;
    bool aligned = words_aligned <= words_balanced;
    if (g_tune_gemv_mode == 1) aligned = true;
    if (g_tune_gemv_mode == 2) aligned = false;
    if (!aligned) grid = num_sms;
    if (g_tune_tiles_per_split > 0) { grid = g_tune_tiles_per_split; aligned = false; }   // tuning key 0 overrides the grid size
    if (grid > tiles) grid = tiles;
    if (grid < 1) grid = 1;
    c->grid = (int)grid;
    c->aligned = aligned;
    const unsigned long units = aligned ? (unsigned long)RB : (unsigned long)tiles * TILE_WORDS;
    c->part_q = (uint32_t)(units / (unsigned long)grid);
    c->part_r = (uint32_t)(units % (unsigned long)grid);
    c->total_warps = (uint32_t)(grid * GEMV_WARPS);
    if ((unsigned long long)(tiles + 1) * TILE_WORDS * (unsigned long long)grid >= (1ull << 32)) return COBALT_ETOOBIG;   // 32-bit partition arithmetic
    c->counters_off = SCRATCH_STATUS_BYTES;
    // the counters of both kernels live in the first 64 KB behind the status word and their partial sums behind
    // that, so that one zero-initialised buffer can serve GEMV and GEMM calls in any order (each kernel returns
    // its counters to zero; neither ever sees the other's partial sums where it expects counters)
    c->partials_off = c->counters_off + round_up((size_t)RB * 4, 256);
    if (c->partials_off < SCRATCH_STATUS_BYTES + SCRATCH_COUNTER_BYTES) c->partials_off = SCRATCH_STATUS_BYTES + SCRATCH_COUNTER_BYTES;
    c->xperm_off = c->partials_off + round_up((size_t)grid * 2 * 4 * c->mt * 32 * sizeof(float), 256);    // one subtotal per CTA and side
    // fragment-ordered activations of launches that cannot stage x: [column tiles][16 chunks][mt][32 lanes] x 16 bytes
    c->total = c->xperm_off + (c->xs ? 0 : (size_t)CT * 16 * c->mt * 32 * 16);
    return COBALT_OK;
}

template <int BITS, int MT, bool XS>
int launch_gemv(const GemvParams& P, const GemvCfg& c, cudaStream_t st) {
    // two kernels per shape class: the common launch, and the one that also carries the staged-input and push modes
    const bool special = P.mode != 0;
    void (*kernel)(const GemvParams) = special ? gemv_mma_special_kernel<BITS, MT, XS> : gemv_mma_kernel<BITS, MT, XS>;
    static bool configured[MAX_DEVICES][2];
    int dev = 0;
    cudaGetDevice(&dev);
    if (!configured[dev][special ? 1 : 0]) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_LIMIT) != cudaSuccess)
            return COBALT_ELAUNCH;
        configured[dev][special ? 1 : 0] = true;
    }
    // programmatic stream serialisation: the prologue of this kernel (barrier set-up, table fill, first weight
    // tiles) may overlap the tail of the previous kernel in the stream; the kernel itself waits before it
    // touches activations or scratch
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)c.grid);
    cfg.blockDim = dim3(GEMV_THREADS);
    cfg.dynamicSmemBytes = c.smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, P) == cudaSuccess ? COBALT_OK : COBALT_ELAUNCH;
}

// ----------------------------------------------------------------------------- GEMM configuration
struct GemmCfg {
    int splits, tok_per_cta;
    dim3 grid;
    size_t counters_off, partials_off, total;
};

int gemm_config(const CobaltMat* w, int M, int num_sms, GemmCfg* c) {
    const int row_tiles = (w->n_row_blocks + GEMM_RB - 1) / GEMM_RB;
    // One token tile whenever the tokens fit one (M <= 512): a CTA decodes its 128-row slab of the weights whatever the
    // number of tokens, so cutting the tokens would decode every weight tile several times.  SMs that such a grid
    // leaves idle are filled by splitting the columns instead (split-K over whole column tiles, fp32 partial sums).
    int tpc = 64;
    while (tpc < GEMM_TOKENS && tpc < M) tpc *= 2;
    c->tok_per_cta = tpc;
    const int tok_tiles = (M + tpc - 1) / tpc;
    const long units = (long)row_tiles * tok_tiles;
    long splits = 1;
    if (g_tune_gemm_stages > 0) splits = g_tune_gemm_stages;                 // tuning key 2 overrides the split-K factor
    else if (units < (long)num_sms) splits = num_sms / units;
    if (splits > 16) splits = 16;
    if (splits > w->n_col_tiles) splits = w->n_col_tiles;
    if (splits < 1) splits = 1;
    {   // every split gets at least one column tile: the kernel hands out ceil(CT / splits) tiles per split
        const long per = (w->n_col_tiles + splits - 1) / splits;
        splits = (w->n_col_tiles + per - 1) / per;
    }
    c->splits = (int)splits;
    c->grid = dim3((unsigned)row_tiles, (unsigned)tok_tiles, (unsigned)splits);
    c->counters_off = SCRATCH_STATUS_BYTES;
    c->partials_off = c->counters_off + round_up((size_t)units * 4, 256);
    if (c->partials_off < SCRATCH_STATUS_BYTES + SCRATCH_COUNTER_BYTES) c->partials_off = SCRATCH_STATUS_BYTES + SCRATCH_COUNTER_BYTES;
    c->total = c->partials_off + (splits > 1 ? (size_t)units * splits * GEMM_TOKENS * GEMM_ROWS * sizeof(float) : 0);
    return COBALT_OK;
}

typedef CUresult (*TensorMapEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                      const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                      CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

TensorMapEncodeFn tensor_map_encoder() {
    static TensorMapEncodeFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (TensorMapEncodeFn)p;
    }
    return fn;
}

// activations [M, N] bf16, row stride ldx elements: box = 64 columns x 256 tokens, 128-byte swizzle
int make_x_map(CUtensorMap* map, const void* x, int64_t ldx, int M, int N) {
    TensorMapEncodeFn enc = tensor_map_encoder();
    if (!enc) return COBALT_ELAUNCH;
    cuuint64_t gdim[2] = {(cuuint64_t)N, (cuuint64_t)M};
    cuuint64_t gstride[1] = {(cuuint64_t)ldx * 2};
    cuuint32_t box[2] = {(cuuint32_t)GEMM_KS, (cuuint32_t)GEMM_NT};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), gdim, gstride, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? COBALT_OK : COBALT_EINVAL;
}

template <int BITS>
int launch_gemm(const GemmParams& P, const CUtensorMap& xmap, const GemmCfg& c, cudaStream_t st) {
    static bool configured[MAX_DEVICES];
    int dev = 0;
    cudaGetDevice(&dev);
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(gemm_tcgen05_kernel<BITS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEMM_SMEM_BYTES) != cudaSuccess)
            return COBALT_ELAUNCH;
        configured[dev] = true;
    }
    gemm_tcgen05_kernel<BITS><<<c.grid, GEMM_THREADS, GEMM_SMEM_BYTES, st>>>(P, xmap);
    return cudaGetLastError() == cudaSuccess ? COBALT_OK : COBALT_ELAUNCH;
}

constexpr long STAGED_NORM_MAX_VALUES = 8192, STAGED_GLU_MAX_VALUES = 32768;     // M * in_features a staged input may compute
constexpr size_t SCRATCH_PUSH_DONE_OFF = 128;            // CTA arrival counter of pushing launches, inside the status block

int check_slots(const CobaltPeerSlots* s, size_t floats) {
    if (!s->peer_base || s->world < 1 || s->world > PEER_MAX_RANKS || s->rank < 0 || s->rank >= s->world) return COBALT_EINVAL;
    if (floats == 0 || floats * sizeof(float) > s->slot_stride_bytes) return COBALT_EINVAL;
    if ((s->slot_stride_bytes & 15) || (s->flags_off_bytes & 15) ||
        s->flags_off_bytes < (size_t)(1 + 2 * s->world) * s->slot_stride_bytes) return COBALT_EINVAL;
    for (int q = 0; q < s->world; ++q)
        if (!s->peer_base[q] || (s->peer_base[q] & 15)) return COBALT_EINVAL;
    return COBALT_OK;
}

// shared body of every GEMV entry point: `n` matrices that share x, N and the bit width
struct GemvOut { void* y; int64_t ldy; const void* bias; };

int gemv_launch(int n, const CobaltMat* const* w, const GemvOut* out, const void* x, int64_t ldx, int M, bool fp32_out,
                void* scratch, size_t scratch_bytes, bool clear_counters, void* stream, const CobaltStagedInput* in = nullptr,
                const CobaltPeerSlots* push = nullptr) {
    if (n < 1 || n > GEMV_MAX_MATS || !w || !out) return COBALT_EINVAL;
    if (M <= 0 || M > MAX_GEMV_M) return COBALT_EINVAL;
    if (in) {                                                // activations computed while staged: `a` stands in for x in the checks
        if (in->kind != COBALT_IN_PLAIN && in->kind != COBALT_IN_GLU && in->kind != COBALT_IN_ADDNORM) return COBALT_EINVAL;
        if (in->flavor < 0 || in->flavor > 1 || !in->a) return COBALT_EINVAL;
        if (((uintptr_t)in->b | (uintptr_t)in->w | (uintptr_t)in->w_branch | (uintptr_t)in->h_out) & 15) return COBALT_EINVAL;
        if (in->kind == COBALT_IN_GLU && !in->b) return COBALT_EINVAL;
        if (in->b_slots && (in->kind != COBALT_IN_ADDNORM || in->b)) return COBALT_EINVAL;
        if (in->kind == COBALT_IN_ADDNORM) {
            if (!in->w || in->h_out == in->a) return COBALT_EINVAL;
            if (in->w_branch && (in->flavor != 1 || !(in->b || in->b_slots))) return COBALT_EINVAL;
        }
        if (in->b_slots) {
            int rc = check_slots(in->b_slots, (size_t)M * w[0]->N);
            if (rc) return rc;
        }
        x = in->a;
        ldx = in->ld;
    }
    if (push) {
        if (n != 1 || !fp32_out) return COBALT_EINVAL;
        int rc = check_slots(push, (size_t)M * w[0]->K);
        if (rc) return rc;
    }
    GemvGeom g = {};
    for (int i = 0; i < n; ++i) {
        int rc = check_mat(w[i]);
        if (rc) return rc;
        rc = check_io(x, ldx, push ? x : out[i].y, push ? (int64_t)w[i]->K : out[i].ldy, M, w[i]->K, w[i]->N);
        if (rc) return rc;
        if (i == 0) g = geom_of(w[0]);
        else {
            if (w[i]->N != w[0]->N || w[i]->bits != w[0]->bits || w[i]->col_scale || w[0]->col_scale) return COBALT_EINVAL;
            g.RB += w[i]->n_row_blocks;
            if (w[i]->max_tile_bytes > g.max_tile_bytes) g.max_tile_bytes = w[i]->max_tile_bytes;
            if (w[i]->max_tile_nnz > g.max_tile_nnz) g.max_tile_nnz = w[i]->max_tile_nnz;
        }
    }
    int sms = 0;
    int rc = device_info(&sms);
    if (rc) return rc;
    GemvCfg c;
    rc = gemv_config(g, w[0]->N, M, sms, &c);
    if (rc) return rc;
    // Staged inputs pay one L2 round trip per 512 chunks of 8 values in every CTA: worth it for the one or two tokens of a
    // decode step, not for more (8 tokens of 5376 values measured slower than the norm kernel followed by the GEMV).
    if (in && in->kind != COBALT_IN_PLAIN &&
        (!c.xs || w[0]->col_scale || (in->kind == COBALT_IN_ADDNORM && (w[0]->N % 256 != 0 || (long)M * w[0]->N > STAGED_NORM_MAX_VALUES)) ||
         (in->kind == COBALT_IN_GLU && (long)M * w[0]->N > STAGED_GLU_MAX_VALUES))) return COBALT_EUNSUPPORTED;
    if (!scratch || ((uintptr_t)scratch & 255) || scratch_bytes < c.total) return COBALT_ESCRATCH;
    cudaStream_t st = (cudaStream_t)stream;
    if (clear_counters) {
        // the status word and the per-row-block arrival counters must start at zero; the partial
        // sums behind them are always written before they are read
        if (cudaMemsetAsync(scratch, 0, c.counters_off + round_up((size_t)g.RB * 4, 256), st) != cudaSuccess) return COBALT_ELAUNCH;
    }
    GemvParams P = {};
    P.n_mats = n;
    int rb = 0;
    for (int i = 0; i < n; ++i) {
        P.mat[i].tiles = (const uint8_t*)w[i]->tiles;
        P.mat[i].tile_off = w[i]->tile_off;
        P.mat[i].y = fp32_out ? nullptr : (uint16_t*)out[i].y;
        P.mat[i].y32 = fp32_out ? (float*)out[i].y : nullptr;
        P.mat[i].bias = (const uint16_t*)out[i].bias;
        P.mat[i].ldy = out[i].ldy;
        P.mat[i].K = w[i]->K;
        P.mat[i].rb_start = rb;
        rb += w[i]->n_row_blocks;
    }
    P.N = w[0]->N; P.G = w[0]->N / GROUP; P.CT = g.CT; P.RB = g.RB;
    P.col_scale = (const uint16_t*)w[0]->col_scale;
    P.x = (const uint16_t*)x; P.ldx = ldx;
    P.xperm = (const uint4*)((uint8_t*)scratch + c.xperm_off);
    P.M = M;
    P.stages = c.stages;
    P.slot_bytes = c.slot; P.xs_bytes = c.xs_bytes;
    P.total_warps = c.total_warps;
    P.aligned = c.aligned ? 1 : 0;
    P.part_q = c.part_q; P.part_r = c.part_r;
    P.status = (uint32_t*)scratch;
    P.counters = (uint32_t*)((uint8_t*)scratch + c.counters_off);
    P.partials = (float*)((uint8_t*)scratch + c.partials_off);
    if (push) {
        P.mode |= GEMV_MODE_PUSH;
        P.push_world = push->world; P.push_rank = push->rank;
        for (int q = 0; q < push->world; ++q) P.push_base[q] = push->peer_base[q];
        P.push_stride = push->slot_stride_bytes; P.push_flags_off = push->flags_off_bytes;
        P.push_flags = (uint32_t*)(push->peer_base[push->rank] + push->flags_off_bytes);
        P.push_done = (uint32_t*)((uint8_t*)scratch + SCRATCH_PUSH_DONE_OFF);
        P.mat[0].y32 = (float*)push->peer_base[push->rank];  // the local staging area: [M, K] fp32, dense
        P.mat[0].y = nullptr;
        P.mat[0].ldy = w[0]->K;
    }
    if (in && in->kind != COBALT_IN_PLAIN) {
        if (in->b_slots) {
            const CobaltPeerSlots* sl = in->b_slots;
            P.mode |= GEMV_MODE_SUMMED;
            P.in_world = sl->world;
            P.in_slots = (const uint8_t*)sl->peer_base[sl->rank];
            P.in_stride = sl->slot_stride_bytes;
            P.in_flags = (const uint32_t*)(sl->peer_base[sl->rank] + sl->flags_off_bytes);
        }
        P.in_kind = in->kind == COBALT_IN_GLU ? GEMV_IN_GLU : GEMV_IN_ADDNORM;
        P.mode |= P.in_kind;
        P.in_flavor = in->flavor;
        P.in_a = (const uint16_t*)in->a; P.in_b = (const uint16_t*)in->b; P.in_ld = in->ld;
        P.in_w = (const uint16_t*)in->w; P.in_wb = (const uint16_t*)in->w_branch; P.in_hout = (uint16_t*)in->h_out;
        P.in_eps = in->eps;
    }
    if (!c.xs) {                                             // fragment-ordered copy of x, read by every warp of the GEMV
        const int chunks = g.CT * 16 * c.mt * 32;
        cudaLaunchConfig_t pc = {};
        pc.gridDim = dim3((unsigned)((chunks + 255) / 256 < 4 * sms ? (chunks + 255) / 256 : 4 * sms));
        pc.blockDim = dim3(256);
        pc.stream = st;
        cudaLaunchAttribute pattr[1];
        pattr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        pattr[0].val.programmaticStreamSerializationAllowed = 1;
        pc.attrs = pattr;
        pc.numAttrs = 1;
        if (cudaLaunchKernelEx(&pc, x_permute_kernel, (const uint16_t*)x, ldx, M, w[0]->N, g.CT, c.mt, (uint4*)((uint8_t*)scratch + c.xperm_off)) != cudaSuccess)
            return COBALT_ELAUNCH;
    }
    if (c.mt == 1 && c.xs) {
        switch (g.bits) {
            case 2: return launch_gemv<2, 1, true>(P, c, st);
            case 3: return launch_gemv<3, 1, true>(P, c, st);
            default: return launch_gemv<4, 1, true>(P, c, st);
        }
    }
    if (c.mt == 1) {
        switch (g.bits) {
            case 2: return launch_gemv<2, 1, false>(P, c, st);
            case 3: return launch_gemv<3, 1, false>(P, c, st);
            default: return launch_gemv<4, 1, false>(P, c, st);
        }
    }
    switch (g.bits) {
        case 2: return launch_gemv<2, 2, false>(P, c, st);
        case 3: return launch_gemv<3, 2, false>(P, c, st);
        default: return launch_gemv<4, 2, false>(P, c, st);
    }
}

int gemv_impl(const CobaltMat* w, const void* x, int64_t ldx, void* y, int64_t ldy, const void* bias, int M,
              void* scratch, size_t scratch_bytes, bool clear_counters, void* stream, bool fp32_out = false) {
    GemvOut o = {y, ldy, bias};
    return gemv_launch(1, &w, &o, x, ldx, M, fp32_out, scratch, scratch_bytes, clear_counters, stream);
}

}  // namespace

extern "C" {

int cobalt_version(void) { return (1 << 16) | 0; }

const char* cobalt_strerror(int status) {
    switch (status) {
        case COBALT_OK: return "ok";
        case COBALT_EINVAL: return "invalid argument (null pointer, shape, alignment or bit width)";
        case COBALT_ESCRATCH: return "scratch buffer missing, misaligned or too small";
        case COBALT_ELAUNCH: return "CUDA runtime or launch error";
        case COBALT_EARCH: return "device is not compute capability 10.x (B200)";
        case COBALT_ETIMEOUT: return "a bounded device-side wait expired";
        case COBALT_ETOOBIG: return "size exceeds the stated maximum of this entry point";
        case COBALT_EUNSUPPORTED: return "this shape cannot take the fused path; use the separate entry points";
        default: return "unknown status";
    }
}

#ifdef COBALT_TUNING_HOOKS
// Experiment hook: key 0 = GEMV grid size, 1 = GEMV ring stages, 2 = GEMM split-K factor, 3 = GEMV partition
// (1 = whole row blocks per CTA, 2 = balanced words); value 0 restores the heuristic.
int cobalt_set_tuning(int key, int value) {
    if (value < 0) return COBALT_EINVAL;
    switch (key) {
        case 0: g_tune_tiles_per_split = value; return COBALT_OK;
        case 1: g_tune_gemv_stages = value; return COBALT_OK;
        case 2: g_tune_gemm_stages = value; return COBALT_OK;
        case 3: g_tune_gemv_mode = value; return COBALT_OK;
        default: return COBALT_EINVAL;
    }
}
#endif

size_t cobalt_gemv_scratch_bytes(const CobaltMat* w, int M) {
    int sms = 0;
    if (check_mat(w) != COBALT_OK || M <= 0 || M > MAX_GEMV_M) return 0;
    if (device_info(&sms) != COBALT_OK) return 0;
    GemvCfg c;
    if (gemv_config(geom_of(w), w->N, M, sms, &c) != COBALT_OK) return 0;
    return c.total;
}

int cobalt_gemv(const CobaltMat* w, const void* x, int64_t ldx, void* y, int64_t ldy, const void* bias, int M,
                void* scratch, size_t scratch_bytes, void* stream) {
    return gemv_impl(w, x, ldx, y, ldy, bias, M, scratch, scratch_bytes, /*clear_counters=*/false, stream);
}

// ---- allocation-free variant: scratch lives in a file-scope device array ---------------------
// One array per GPU that loads the library (held until the process exits).  Host code only ever
// sees the array's host-side stand-in, so its device address is looked up once per device with
// cudaGetSymbolAddress while that device is current.
static __device__ __align__(256) unsigned char g_static_scratch[COBALT_STATIC_SCRATCH_BYTES];
static void* g_static_scratch_ptr[MAX_DEVICES];

int cobalt_gemv_static(const CobaltMat* w, const void* x, int64_t ldx, void* y, int64_t ldy, const void* bias, int M,
                       void* stream) {
    int rc = check_mat(w);
    if (rc) return rc;
    if (M <= 0 || M > MAX_GEMV_M) return COBALT_EINVAL;
    int sms = 0;
    rc = device_info(&sms);
    if (rc) return rc;
    GemvCfg c;
    rc = gemv_config(geom_of(w), w->N, M, sms, &c);
    if (rc) return rc;
    if (c.total > (size_t)COBALT_STATIC_SCRATCH_BYTES) return COBALT_ETOOBIG;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return COBALT_ELAUNCH;
    if (!g_static_scratch_ptr[dev]) {                    // first call on this device: resolve the symbol
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || !p) return COBALT_ELAUNCH;
        g_static_scratch_ptr[dev] = p;
    }
    return gemv_impl(w, x, ldx, y, ldy, bias, M, g_static_scratch_ptr[dev], COBALT_STATIC_SCRATCH_BYTES,
                     /*clear_counters=*/true, stream);
}

size_t cobalt_gemv_fused_scratch_bytes(int n_mats, const CobaltMat* const* w, int M) {
    if (n_mats < 1 || n_mats > GEMV_MAX_MATS || !w || M <= 0 || M > MAX_GEMV_M) return 0;
    GemvGeom g = {};
    for (int i = 0; i < n_mats; ++i) {
        if (check_mat(w[i]) != COBALT_OK) return 0;
        if (i == 0) g = geom_of(w[0]);
        else {
            g.RB += w[i]->n_row_blocks;
            if (w[i]->max_tile_bytes > g.max_tile_bytes) g.max_tile_bytes = w[i]->max_tile_bytes;
            if (w[i]->max_tile_nnz > g.max_tile_nnz) g.max_tile_nnz = w[i]->max_tile_nnz;
        }
    }
    int sms = 0;
    if (device_info(&sms) != COBALT_OK) return 0;
    GemvCfg c;
    if (gemv_config(g, w[0]->N, M, sms, &c) != COBALT_OK) return 0;
    return c.total;
}

int cobalt_gemv_fused(int n_mats, const CobaltMat* const* w, const void* x, int64_t ldx, void* const* y, const int64_t* ldy,
                      const void* const* bias, int M, void* scratch, size_t scratch_bytes, void* stream) {
    if (n_mats < 1 || n_mats > GEMV_MAX_MATS || !w || !y || !ldy) return COBALT_EINVAL;
    GemvOut o[GEMV_MAX_MATS];
    for (int i = 0; i < n_mats; ++i) { o[i].y = y[i]; o[i].ldy = ldy[i]; o[i].bias = bias ? bias[i] : nullptr; }
    return gemv_launch(n_mats, w, o, x, ldx, M, false, scratch, scratch_bytes, false, stream);
}

int cobalt_gemv_fused_staged(int n_mats, const CobaltMat* const* w, const CobaltStagedInput* in, void* const* y,
                             const int64_t* ldy, const void* const* bias, int M, int out_fp32,
                             const CobaltPeerSlots* push, void* scratch, size_t scratch_bytes, void* stream) {
    if (n_mats < 1 || n_mats > GEMV_MAX_MATS || !w || !in) return COBALT_EINVAL;
    if (!push && (!y || !ldy)) return COBALT_EINVAL;
    if (out_fp32 && bias) return COBALT_EINVAL;
    GemvOut o[GEMV_MAX_MATS];
    for (int i = 0; i < n_mats; ++i) {
        o[i].y = push ? nullptr : y[i];
        o[i].ldy = push ? 0 : ldy[i];
        o[i].bias = bias ? bias[i] : nullptr;
    }
    return gemv_launch(n_mats, w, o, nullptr, 0, M, out_fp32 != 0, scratch, scratch_bytes, false, stream, in, push);
}

int cobalt_peer_sum(const CobaltPeerSlots* slots, size_t n, void* out, int out_fp32, void* status, void* stream) {
    if (!slots || !out || ((uintptr_t)out & 15) || (n & 7) || n > 0xFFFFFFFFull) return COBALT_EINVAL;
    int rc = check_slots(slots, n);
    if (rc) return rc;
    int sms = 0;
    rc = device_info(&sms);
    if (rc) return rc;
    PeerParams P = {};
    for (int q = 0; q < slots->world; ++q) P.base[q] = slots->peer_base[q];
    P.rank = slots->rank; P.world = slots->world; P.n = (unsigned int)n;
    P.slot_stride = slots->slot_stride_bytes; P.flags_off = slots->flags_off_bytes;
    P.out = out_fp32 ? nullptr : (uint16_t*)out;
    P.out32 = out_fp32 ? (float*)out : nullptr;
    P.status = (uint32_t*)status;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(1024);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, peer_sum_kernel, P) == cudaSuccess ? COBALT_OK : COBALT_ELAUNCH;
}

int cobalt_gemv_rowwalk(const CobaltMat* w, const void* x, int64_t ldx, void* y, int64_t ldy, const void* bias, int M,
                        void* stream) {
    int rc = check_mat(w);
    if (rc) return rc;
    if (M > MAX_GEMV_M) return COBALT_EINVAL;
    rc = check_io(x, ldx, y, ldy, M, w->K, w->N);
    if (rc) return rc;
    int sms = 0;
    rc = device_info(&sms);
    if (rc) return rc;
    MatView V = make_view(w);
    cudaStream_t st = (cudaStream_t)stream;
    if (M <= 1)
        gemv_rowwalk_kernel<1><<<V.RB, 64, 0, st>>>(V, (const uint16_t*)x, ldx, (uint16_t*)y, ldy, (const uint16_t*)bias, M);
    else if (M <= 4)
        gemv_rowwalk_kernel<4><<<V.RB, 64, 0, st>>>(V, (const uint16_t*)x, ldx, (uint16_t*)y, ldy, (const uint16_t*)bias, M);
    else
        gemv_rowwalk_kernel<16><<<V.RB, 64, 0, st>>>(V, (const uint16_t*)x, ldx, (uint16_t*)y, ldy, (const uint16_t*)bias, M);
    return cudaGetLastError() == cudaSuccess ? COBALT_OK : COBALT_ELAUNCH;
}

size_t cobalt_gemm_scratch_bytes(const CobaltMat* w, int M) {
    int sms = 0;
    if (check_mat(w) != COBALT_OK || M <= 0) return 0;
    if (device_info(&sms) != COBALT_OK) return 0;
    GemmCfg c;
    if (gemm_config(w, M, sms, &c) != COBALT_OK) return 0;
    return c.total;
}

static int gemm_impl(const CobaltMat* w, const void* x, int64_t ldx, void* y, int64_t ldy, const void* bias, int M,
                     void* scratch, size_t scratch_bytes, void* stream, bool fp32_out) {
    int rc = check_mat(w);
    if (rc) return rc;
    rc = check_io(x, ldx, y, ldy, M, w->K, w->N);
    if (rc) return rc;
    int sms = 0;
    rc = device_info(&sms);
    if (rc) return rc;
    GemmCfg c;
    rc = gemm_config(w, M, sms, &c);
    if (rc) return rc;
    if (!scratch || ((uintptr_t)scratch & 255) || scratch_bytes < c.total) return COBALT_ESCRATCH;
    CUtensorMap xmap;
    rc = make_x_map(&xmap, x, ldx, M, w->N);
    if (rc) return rc;
    GemmParams P;
    P.W = make_view(w);
    P.y = fp32_out ? nullptr : (uint16_t*)y; P.ldy = ldy;
    P.y32 = fp32_out ? (float*)y : nullptr;
    P.bias = (const uint16_t*)bias;
    P.M = M;
    P.splits = c.splits;
    P.tok_per_cta = c.tok_per_cta;
    P.status = (uint32_t*)scratch;
    P.counters = (uint32_t*)((uint8_t*)scratch + c.counters_off);
    P.partials = c.splits > 1 ? (float*)((uint8_t*)scratch + c.partials_off) : nullptr;
    cudaStream_t st = (cudaStream_t)stream;
    switch (w->bits) {
        case 2: return launch_gemm<2>(P, xmap, c, st);
        case 3: return launch_gemm<3>(P, xmap, c, st);
        default: return launch_gemm<4>(P, xmap, c, st);
    }
}

int cobalt_gemm(const CobaltMat* w, const void* x, int64_t ldx, void* y, int64_t ldy, const void* bias, int M,
                void* scratch, size_t scratch_bytes, void* stream) {
    return gemm_impl(w, x, ldx, y, ldy, bias, M, scratch, scratch_bytes, stream, false);
}

int cobalt_linear_f32(const CobaltMat* w, const void* x, int64_t ldx, float* y, int64_t ldy, int M, void* scratch,
                      size_t scratch_bytes, void* stream) {
    if (M <= MAX_GEMV_M) return gemv_impl(w, x, ldx, y, ldy, nullptr, M, scratch, scratch_bytes, false, stream, true);
    return gemm_impl(w, x, ldx, y, ldy, nullptr, M, scratch, scratch_bytes, stream, true);
}

int cobalt_dequant(const CobaltMat* w, void* w_bf16, void* stream) {
    int rc = check_mat(w);
    if (rc) return rc;
    if (!w_bf16) return COBALT_EINVAL;
    int sms = 0;
    rc = device_info(&sms);
    if (rc) return rc;
    MatView V = make_view(w);
    unpack_kernel<<<dim3(V.CT, V.RB), 64, 0, (cudaStream_t)stream>>>(V, nullptr, nullptr, (uint16_t*)w_bf16);
    return cudaGetLastError() == cudaSuccess ? COBALT_OK : COBALT_ELAUNCH;
}

int cobalt_unpack(const CobaltMat* w, uint8_t* codes, uint8_t* keep, void* stream) {
    int rc = check_mat(w);
    if (rc) return rc;
    if (!codes && !keep) return COBALT_EINVAL;
    int sms = 0;
    rc = device_info(&sms);
    if (rc) return rc;
    MatView V = make_view(w);
    unpack_kernel<<<dim3(V.CT, V.RB), 64, 0, (cudaStream_t)stream>>>(V, codes, keep, nullptr);
    return cudaGetLastError() == cudaSuccess ? COBALT_OK : COBALT_ELAUNCH;
}

int cobalt_linear_host_async(const CobaltMat* w, const void* x_host, void* y_host, const void* bias, int M, void* dev_x,
                             void* dev_y, void* scratch, size_t scratch_bytes, void* stream) {
    int rc = check_mat(w);
    if (rc) return rc;
    if (!x_host || !y_host || !dev_x || !dev_y || M <= 0) return COBALT_EINVAL;
    cudaStream_t st = (cudaStream_t)stream;
    if (cudaMemcpyAsync(dev_x, x_host, (size_t)M * w->N * 2, cudaMemcpyHostToDevice, st) != cudaSuccess) return COBALT_ELAUNCH;
    // both kernels return their arrival counters to zero, so a scratch buffer that was zeroed once stays usable by either
    if (M <= MAX_GEMV_M)
        rc = gemv_impl(w, dev_x, w->N, dev_y, w->K, bias, M, scratch, scratch_bytes, /*clear_counters=*/false, stream);
    else
        rc = cobalt_gemm(w, dev_x, w->N, dev_y, w->K, bias, M, scratch, scratch_bytes, stream);
    if (rc) return rc;
    if (cudaMemcpyAsync(y_host, dev_y, (size_t)M * w->K * 2, cudaMemcpyDeviceToHost, st) != cudaSuccess) return COBALT_ELAUNCH;
    return COBALT_OK;
}

int cobalt_gemv_fused_host_async(int n_mats, const CobaltMat* const* w, const void* x_host, void* const* y_host, int M,
                                 void* dev_x, void* const* dev_y, void* scratch, size_t scratch_bytes, void* stream) {
    if (n_mats < 1 || n_mats > GEMV_MAX_MATS || !w || !x_host || !y_host || !dev_x || !dev_y) return COBALT_EINVAL;
    if (M <= 0 || M > MAX_GEMV_M) return COBALT_EINVAL;
    GemvOut o[GEMV_MAX_MATS];
    for (int i = 0; i < n_mats; ++i) {
        int rc = check_mat(w[i]);
        if (rc) return rc;
        if (!y_host[i] || !dev_y[i]) return COBALT_EINVAL;
        o[i].y = dev_y[i]; o[i].ldy = w[i]->K; o[i].bias = nullptr;
    }
    cudaStream_t st = (cudaStream_t)stream;
    if (cudaMemcpyAsync(dev_x, x_host, (size_t)M * w[0]->N * 2, cudaMemcpyHostToDevice, st) != cudaSuccess) return COBALT_ELAUNCH;
    int rc = gemv_launch(n_mats, w, o, dev_x, w[0]->N, M, false, scratch, scratch_bytes, false, stream);
    if (rc) return rc;
    for (int i = 0; i < n_mats; ++i)
        if (cudaMemcpyAsync(y_host[i], dev_y[i], (size_t)M * w[i]->K * 2, cudaMemcpyDeviceToHost, st) != cudaSuccess) return COBALT_ELAUNCH;
    return COBALT_OK;
}

int cobalt_linear_host(const CobaltMat* w, const void* x_host, void* y_host, const void* bias, int M, void* dev_x,
                       void* dev_y, void* scratch, size_t scratch_bytes, void* stream) {
    int rc = cobalt_linear_host_async(w, x_host, y_host, bias, M, dev_x, dev_y, scratch, scratch_bytes, stream);
    if (rc) return rc;
    return cudaStreamSynchronize((cudaStream_t)stream) == cudaSuccess ? COBALT_OK : COBALT_ELAUNCH;
}

int cobalt_add_rmsnorm(const void* h, const void* delta, const void* w, void* h_out, void* y, int T, int H, float eps,
                       int flavor, const void* w_branch, void* stream) {
    if (!h || !w || !y || T <= 0 || H <= 0 || flavor < 0 || flavor > 1) return COBALT_EINVAL;
    if (w_branch && (flavor != 1 || !delta)) return COBALT_EINVAL;
    int sms = 0;
    int rc = device_info(&sms);
    if (rc) return rc;
    const bool vec = H % 256 == 0 && H <= 256 * ADDNORM_MAX_ITERS * (ADDNORM_THREADS / 32) && !(((uintptr_t)h | (uintptr_t)delta | (uintptr_t)w |
                     (uintptr_t)h_out | (uintptr_t)y | (uintptr_t)w_branch) & 15);
    if (vec)
        add_rmsnorm_kernel<<<T, ADDNORM_THREADS, 0, (cudaStream_t)stream>>>((const uint16_t*)h, (const uint16_t*)delta, (const uint16_t*)w,
                                                                           (uint16_t*)h_out, (uint16_t*)y, H, eps, flavor, (const uint16_t*)w_branch);
    else
        add_rmsnorm_generic_kernel<<<T, 256, 0, (cudaStream_t)stream>>>((const uint16_t*)h, (const uint16_t*)delta, (const uint16_t*)w,
                                                                       (uint16_t*)h_out, (uint16_t*)y, H, eps, flavor, (const uint16_t*)w_branch);
    return cudaGetLastError() == cudaSuccess ? COBALT_OK : COBALT_ELAUNCH;
}

int cobalt_rope_kv(void* q, const void* k, const void* v, const int64_t* positions, const float* inv_freq, void* k_cache,
                   void* v_cache, int T, int n_heads, int n_kv_heads, int head_dim, int max_ctx, const void* q_norm_w,
                   const void* k_norm_w, float eps, int64_t cache_seq_stride, void* stream) {
    if (!q || !k || !v || !positions || !inv_freq || !k_cache || !v_cache) return COBALT_EINVAL;
    if (T <= 0 || n_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0 || (head_dim & 1) || max_ctx <= 0) return COBALT_EINVAL;
    if ((q_norm_w == nullptr) != (k_norm_w == nullptr) || cache_seq_stride < 0) return COBALT_EINVAL;
    int sms = 0;
    int rc = device_info(&sms);
    if (rc) return rc;
    if (q_norm_w) {
        const long long warps = (long long)T * (n_heads + 2 * n_kv_heads);
        rope_kv_norm_kernel<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
            (uint16_t*)q, (const uint16_t*)k, (const uint16_t*)v, (const long long*)positions, inv_freq, (uint16_t*)k_cache,
            (uint16_t*)v_cache, T, n_heads, n_kv_heads, head_dim, max_ctx, (const uint16_t*)q_norm_w, (const uint16_t*)k_norm_w, eps,
            (long long)cache_seq_stride);
        return cudaGetLastError() == cudaSuccess ? COBALT_OK : COBALT_ELAUNCH;
    }
    const long long n = (long long)T * (n_heads + 2 * n_kv_heads) * (head_dim / 2);
    rope_kv_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        (uint16_t*)q, (const uint16_t*)k, (const uint16_t*)v, (const long long*)positions, inv_freq, (uint16_t*)k_cache,
        (uint16_t*)v_cache, T, n_heads, n_kv_heads, head_dim, max_ctx, (long long)cache_seq_stride);
    return cudaGetLastError() == cudaSuccess ? COBALT_OK : COBALT_ELAUNCH;
}

int cobalt_allreduce_peer(const uint64_t* peer_base, int rank, int world, size_t n, size_t slot_stride_bytes,
                          size_t flags_off_bytes, void* out, int out_fp32, void* status, void* stream) {
    if (!peer_base || !out || world < 1 || world > PEER_MAX_RANKS || rank < 0 || rank >= world) return COBALT_EINVAL;
    if (n == 0 || (n & 3) || n * sizeof(float) > slot_stride_bytes || n > 0xFFFFFFFFull) return COBALT_EINVAL;
    if (((uintptr_t)out & 15)) return COBALT_EINVAL;
    if ((slot_stride_bytes & 15) || (flags_off_bytes & 15) || flags_off_bytes < (size_t)(1 + 2 * world) * slot_stride_bytes) return COBALT_EINVAL;
    int sms = 0;
    int rc = device_info(&sms);
    if (rc) return rc;
    PeerParams P = {};
    for (int q = 0; q < world; ++q) {
        if (!peer_base[q] || (peer_base[q] & 15)) return COBALT_EINVAL;
        P.base[q] = peer_base[q];
    }
    P.rank = rank; P.world = world; P.n = (unsigned int)n;
    P.slot_stride = slot_stride_bytes; P.flags_off = flags_off_bytes;
    P.out = out_fp32 ? nullptr : (uint16_t*)out;
    P.out32 = out_fp32 ? (float*)out : nullptr;
    P.status = (uint32_t*)status;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(1024);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, peer_allreduce_kernel, P) == cudaSuccess ? COBALT_OK : COBALT_ELAUNCH;
}

size_t cobalt_attn_decode_scratch_bytes(int n_heads, int head_dim, int max_ctx) {
    if (n_heads <= 0 || head_dim <= 0 || max_ctx <= 0) return 0;
    const size_t chunks = ((size_t)max_ctx + ATTN_CHUNK - 1) / ATTN_CHUNK;
    return round_up((size_t)n_heads * max_ctx * 4, 256) + round_up((size_t)n_heads * chunks * 8, 256) +
           round_up(chunks * n_heads * head_dim * 4, 256);
}

int cobalt_attn_decode(const void* q, const void* k_cache, const void* v_cache, const int64_t* positions, void* scratch,
                       size_t scratch_bytes, void* out, int n_heads, int n_kv_heads, int head_dim, int max_ctx, int window,
                       float scale, int n_seq, int64_t cache_seq_stride, void* stream) {
    if (!q || !k_cache || !v_cache || !positions || !scratch || !out) return COBALT_EINVAL;
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || n_heads / n_kv_heads > ATTN_MAX_REP) return COBALT_EINVAL;
    if (n_seq < 1 || n_seq > 65535 || cache_seq_stride < 0) return COBALT_EINVAL;
    if (head_dim < 64 || head_dim > 256 || head_dim % 64 != 0 || max_ctx <= 0) return COBALT_EINVAL;
    if (((uintptr_t)k_cache & 3) || ((uintptr_t)q & 3) || ((uintptr_t)scratch & 255)) return COBALT_EINVAL;
    const int chunks = (max_ctx + ATTN_CHUNK - 1) / ATTN_CHUNK;
    if (chunks > ATTN_MAX_CHUNKS) return COBALT_ETOOBIG;
    if (scratch_bytes < (size_t)n_seq * cobalt_attn_decode_scratch_bytes(n_heads, head_dim, max_ctx)) return COBALT_ESCRATCH;
    int sms = 0;
    int rc = device_info(&sms);
    if (rc) return rc;
    const int rep = n_heads / n_kv_heads;
    // scratch: scores [n_seq][n_heads][max_ctx], chunk statistics [n_seq][n_heads][chunks][2], partial contexts [n_seq][chunks][n_heads][D]
    float* att = (float*)scratch;
    float* stat = (float*)((uint8_t*)scratch + round_up((size_t)n_seq * n_heads * max_ctx * 4, 256));
    float* part = (float*)((uint8_t*)stat + round_up((size_t)n_seq * n_heads * chunks * 8, 256));
    cudaStream_t st = (cudaStream_t)stream;
    const dim3 grid((unsigned)chunks, (unsigned)n_kv_heads, (unsigned)n_seq);
    attn_scores_kernel<<<grid, ATTN_THREADS, 0, st>>>((const uint16_t*)q, (const uint16_t*)k_cache, (const long long*)positions, att, stat,
                                             rep, head_dim, max_ctx, window, scale, (long long)cache_seq_stride);
    attn_context_kernel<<<grid, ATTN_THREADS, 0, st>>>(att, stat, (const uint16_t*)v_cache, (const long long*)positions, part, rep,
                                              head_dim, max_ctx, window, n_heads, (long long)cache_seq_stride);
    const int n = n_heads * head_dim;
    attn_combine_kernel<<<dim3((unsigned)((n + 255) / 256), (unsigned)n_seq), 256, 0, st>>>(part, (const long long*)positions, (uint16_t*)out, n,
                                                                                          chunks, window);
    return cudaGetLastError() == cudaSuccess ? COBALT_OK : COBALT_ELAUNCH;
}

// one-kernel attention: [status 256 B][counters n_seq * n_kv * 2 u32][chunk statistics][partial contexts]
size_t cobalt_attn_decode_fused_scratch_bytes(int n_heads, int n_kv_heads, int head_dim, int max_ctx, int n_seq) {
    if (n_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0 || max_ctx <= 0 || n_seq <= 0) return 0;
    const size_t chunks = ((size_t)max_ctx + ATTN_CHUNK - 1) / ATTN_CHUNK;
    return SCRATCH_STATUS_BYTES + round_up((size_t)n_seq * n_kv_heads * 8, 256) + round_up((size_t)n_seq * n_heads * chunks * 8, 256) +
           round_up((size_t)n_seq * chunks * n_heads * head_dim * 4, 256);
}

int cobalt_attn_decode_fused(const void* q, const void* k_cache, const void* v_cache, const int64_t* positions, void* scratch,
                             size_t scratch_bytes, void* out, int n_heads, int n_kv_heads, int head_dim, int max_ctx,
                             int window, float scale, int n_seq, int64_t cache_seq_stride, void* stream) {
    if (!q || !k_cache || !v_cache || !positions || !scratch || !out) return COBALT_EINVAL;
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || n_heads / n_kv_heads > ATTN_MAX_REP) return COBALT_EINVAL;
    if (n_seq < 1 || n_seq > 65535 || cache_seq_stride < 0) return COBALT_EINVAL;
    if (head_dim < 64 || head_dim > 256 || head_dim % 64 != 0 || max_ctx <= 0) return COBALT_EINVAL;
    if (((uintptr_t)k_cache & 3) || ((uintptr_t)q & 3) || ((uintptr_t)scratch & 255)) return COBALT_EINVAL;
    const int chunks = (max_ctx + ATTN_CHUNK - 1) / ATTN_CHUNK;
    if (chunks > ATTN_MAX_CHUNKS) return COBALT_ETOOBIG;
    if (scratch_bytes < cobalt_attn_decode_fused_scratch_bytes(n_heads, n_kv_heads, head_dim, max_ctx, n_seq)) return COBALT_ESCRATCH;
    int sms = 0;
    int rc = device_info(&sms);
    if (rc) return rc;
    // every CTA must be resident at once (they wait for each other): otherwise the three-kernel entry point is the way
    static int per_sm[MAX_DEVICES];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return COBALT_ELAUNCH;
    if (per_sm[dev] == 0) {
        int n = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attn_decode_fused_kernel, ATTN_THREADS, 0) != cudaSuccess || n < 1) return COBALT_ELAUNCH;
        per_sm[dev] = n;
    }
    if ((long)chunks * n_kv_heads * n_seq > (long)per_sm[dev] * sms) return COBALT_EUNSUPPORTED;
    int rep = n_heads / n_kv_heads;
    uint32_t* status = (uint32_t*)scratch;
    uint32_t* counters = (uint32_t*)((uint8_t*)scratch + SCRATCH_STATUS_BYTES);
    float* stat = (float*)((uint8_t*)counters + round_up((size_t)n_seq * n_kv_heads * 8, 256));
    float* part = (float*)((uint8_t*)stat + round_up((size_t)n_seq * n_heads * chunks * 8, 256));
    const uint16_t* qp = (const uint16_t*)q; const uint16_t* kp = (const uint16_t*)k_cache; const uint16_t* vp = (const uint16_t*)v_cache;
    const long long* pp = (const long long*)positions;
    uint16_t* op = (uint16_t*)out;
    long long stride = (long long)cache_seq_stride;
    void* args[] = {&qp, &kp, &vp, &pp, &stat, &part, &counters, &status, &op, &rep, &head_dim, &max_ctx, &window, &scale, &stride};
    const dim3 grid((unsigned)chunks, (unsigned)n_kv_heads, (unsigned)n_seq);
    return cudaLaunchCooperativeKernel((const void*)attn_decode_fused_kernel, grid, dim3(ATTN_THREADS), args, 0, (cudaStream_t)stream) == cudaSuccess
               ? COBALT_OK : COBALT_ELAUNCH;
}

int cobalt_swiglu(const void* gate, const void* up, void* out, int64_t n, int act, void* stream) {
    if (!gate || !up || !out || n <= 0 || act < 0 || act > 1) return COBALT_EINVAL;
    int sms = 0;
    int rc = device_info(&sms);
    if (rc) return rc;
    swiglu_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const uint16_t*)gate, (const uint16_t*)up,
                                                                                 (uint16_t*)out, (long long)n, act);
    return cudaGetLastError() == cudaSuccess ? COBALT_OK : COBALT_ELAUNCH;
}

int cobalt_device_status(const void* scratch, void* stream, uint32_t* status_out) {
    if (!status_out) return COBALT_EINVAL;
    if (!scratch) {                                          // the status word of cobalt_gemv_static()'s private array
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess) return COBALT_ELAUNCH;
        if (dev < 0 || dev >= MAX_DEVICES) return COBALT_EINVAL;
        if (!g_static_scratch_ptr[dev]) { *status_out = 0; return COBALT_OK; }      // never used on this device: nothing to report
        scratch = g_static_scratch_ptr[dev];
    }
    cudaStream_t st = (cudaStream_t)stream;
    if (cudaMemcpyAsync(status_out, scratch, 4, cudaMemcpyDeviceToHost, st) != cudaSuccess) return COBALT_ELAUNCH;
    if (cudaStreamSynchronize(st) != cudaSuccess) return COBALT_ELAUNCH;
    return *status_out == 0 ? COBALT_OK : COBALT_ETIMEOUT;
}

}  // extern "C"
