/*
 * cobalt_b200.h -- C ABI of libcobalt_b200.so
 *
 * Sparse low-bit compressed linear layer for NVIDIA B200 (sm_100a): activations times a
 * weight stored as a per-row occupancy bitmask, 2/3/4-bit codes for the surviving
 * positions and one fp16 scale + fp16 zero point per 128-wide group.
 *
 * Conventions
 *   - W is [K, N] = [out_features, in_features]; groups run along N; N % 128 == 0.
 *   - Every pointer is a DEVICE pointer unless the name says "host".  The caller owns all
 *     buffers; the library allocates nothing.
 *   - `stream` is a cudaStream_t passed as void*.  Calls are stream-ordered and never
 *     synchronise (except cobalt_linear_host() and cobalt_device_status(), which say so).
 *   - Return value: 0 on success, a negative COBALT_E* code otherwise.  Arguments are
 *     validated on the host; nothing traps or aborts.
 *   - Activations and outputs are bf16 (uint16 storage), row-major with a leading
 *     dimension in elements.
 *
 * Tile image (what `tiles` / `tile_off` point at), produced by cobalt_b200/format.py:
 *   row block rb = 16 rows, column tile ct = up to 4 groups (512 columns); tiles are stored
 *   row-block-major, tile index = rb * n_col_tiles + ct, each padded to 16 bytes:
 *     mask   16*w segments x 16 B : segment (r, gi) at index r*w + gi, 4 u32 words,
 *                                   bit b of word j = column 128*(4*ct+gi) + 32*j + b
 *     sz     16*w x 4 B           : { fp16 scale, fp16 zero }
 *     codes  little-endian stream of `bits`-wide survivor codes, segment order, ascending column
 *   w = min(4, N/128 - 4*ct).  tile_off[i] is the start of tile i in 16-byte units.
 */
#ifndef COBALT_B200_H
#define COBALT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define COBALT_OK            0
#define COBALT_EINVAL       (-1)   /* bad argument (null pointer, shape, alignment, bits) */
#define COBALT_ESCRATCH     (-2)   /* scratch buffer missing or too small */
#define COBALT_ELAUNCH      (-3)   /* CUDA launch / runtime error (cudaGetLastError) */
#define COBALT_EARCH        (-4)   /* device is not compute capability 10.x */
#define COBALT_ETIMEOUT     (-5)   /* a bounded device-side wait gave up (see cobalt_device_status) */
#define COBALT_ETOOBIG      (-6)   /* size exceeds a stated maximum of the entry point */
#define COBALT_EUNSUPPORTED (-7)   /* this shape cannot take the fused path asked for; nothing was launched, use the separate entry points */

/* Descriptor of one packed matrix.  Replaces the reference's 9 x int64 MatDesc
 * {data,row_off,scale,zero,col_scale,K,N,G,layout}
 * (src/cobaltkernel/csrc/megakernel.cuh:21-28, built in src/cobaltkernel/runner.py:318-335). */
typedef struct CobaltMat {
    const void*     tiles;          /* first tile, 16-byte aligned */
    const uint32_t* tile_off;       /* n_row_blocks * n_col_tiles + 1 entries, 16-byte units */
    const void*     col_scale;      /* optional fp16[N] per-input-column scale (reference `scale2`), or NULL */
    int32_t K, N;                   /* out_features, in_features */
    int32_t bits;                   /* 2, 3 or 4 */
    int32_t group;                  /* 128 */
    int32_t n_row_blocks;           /* ceil(K / 16) */
    int32_t n_col_tiles;            /* ceil(N / 512) */
    uint32_t max_tile_bytes;        /* largest tile of this matrix */
    uint32_t max_tile_nnz;          /* most survivors in one tile */
    int64_t nnz;                    /* number of survivors */
} CobaltMat;

/* Library / ABI version (major << 16 | minor). */
int cobalt_version(void);

/* Human-readable text for a status code. */
const char* cobalt_strerror(int status);

/* Decode GEMV, M <= 16 tokens:  y[m, k] = bf16( sum_j bf16(W[k, j]) * x[m, j] (+ bias[k]) ), fp32 accumulate.
 * Replaces the reference's warp-per-row bitmap GEMV dispatcher cbk::gemv_rows<M>
 * (src/cobaltkernel/csrc/cobalt_gemv.cuh:1197-1213; gemv_sparse :216-301, gemv_sparse_expand :311-393)
 * and, above it, SparseQuantLinear.forward for small batches (benchmarks/benchmark_suite.py:1200-1217).
 * `scratch` holds split-K partial sums and per-row-block arrival counters; it must be at least
 * cobalt_gemv_scratch_bytes() bytes, 256-byte aligned and ZERO before its first use (the kernel
 * leaves the counters zero again).  Calls sharing one scratch buffer must not overlap on the GPU.
 * One zeroed buffer may serve cobalt_gemv() and cobalt_gemm() calls in any order as long as the matrix has at most
 * 16384 row blocks (K <= 262144): both kernels keep their arrival counters in the first 64 KB behind the status
 * word and return them to zero, and neither reads partial sums it has not written.  Taller matrices need a
 * buffer per kernel. */
int cobalt_gemv(const CobaltMat* w, const void* x, int64_t ldx, void* y, int64_t ldy,
                const void* bias, int M, void* scratch, size_t scratch_bytes, void* stream);
size_t cobalt_gemv_scratch_bytes(const CobaltMat* w, int M);

/* Up to 4 matrices that read the same activations (q|k|v, gate|up) in ONE launch: the tiles of all
 * matrices form one work list, so small projections no longer pay a launch each.  All matrices must
 * have the same in_features and bit width and no column scale.  Results are bit-identical to
 * separate cobalt_gemv() calls.  y[i], ldy[i], bias[i] belong to matrix i (bias may be NULL).
 * Replaces the row-concatenated qkv / gate-up matrices of the reference's packer
 * (docs/FORMAT.md:126-151, src/cobaltkernel/pack_cobalt.py:452-471, 647-660). */
int cobalt_gemv_fused(int n_mats, const CobaltMat* const* w, const void* x, int64_t ldx, void* const* y,
                      const int64_t* ldy, const void* const* bias, int M, void* scratch, size_t scratch_bytes,
                      void* stream);
size_t cobalt_gemv_fused_scratch_bytes(int n_mats, const CobaltMat* const* w, int M);

/* cobalt_gemv_fused() whose activation rows are COMPUTED while the kernel copies them into shared memory, so
 * that the element-wise step in front of a projection costs no launch and no round trip through memory:
 *   COBALT_IN_GLU      x = bf16( bf16(act(a)) * b ), act = SiLU (flavor 0) or tanh-GELU (flavor 1): what
 *                      cobalt_swiglu() computes.  The reference closes the gate in its gate|up epilogue
 *                      (docs/FORMAT.md:126-151, src/cobaltkernel/csrc/megakernel.cu:1805-1892).
 *   COBALT_IN_ADDNORM  h' = bf16(a + delta'), x = RMSNorm(h') * w: what cobalt_add_rmsnorm() computes, with
 *                      b = delta (or NULL), w_branch = Gemma's branch-norm weight (or NULL), flavor 0 Llama / 1 Gemma;
 *                      h' is written to h_out (may be NULL; must not alias a).  The reference normalises while it
 *                      writes its activation copy and adds the residual in the o/down epilogue
 *                      (src/cobaltkernel/csrc/megakernel.cu:270-288, 1904-1915).
 * a, b, h_out are [M, in_features] bf16 with row stride ld (elements), 16-byte aligned; results are bit-identical
 * to the separate entry points followed by cobalt_gemv_fused().  Only launches that stage their activations can
 * take this path (M <= 8 and M * in_features * 2 bytes beside the weight ring), and only while every CTA repeating the
 * step is cheaper than a kernel of its own: M * in_features <= 32768 for COBALT_IN_GLU, <= 8192 and in_features % 256 == 0
 * for COBALT_IN_ADDNORM.  Otherwise COBALT_EUNSUPPORTED is returned and nothing is launched.  COBALT_IN_PLAIN
 * (a = x) takes every shape.
 *
 * Tensor parallelism, the all-reduce of a row-parallel projection folded into the two kernels around it (the
 * reference runs on one GPU; its column/row split is docs/FORMAT.md:126-151 and it has no counterpart of this exchange):
 *   `push` (output side)   the raw fp32 sums of THIS rank are written to the staging area of its own peer buffer; the
 *                          last CTA of the launch to finish copies them into row `rank` of the current epoch's slot in
 *                          EVERY rank's peer buffer (plain NVLink stores; layout as for cobalt_allreduce_peer()) and
 *                          publishes the epoch in every rank's flag block.  One matrix, out_fp32 = 1, y is not
 *                          written (may be NULL).
 *   `in->b_slots` (input side, COBALT_IN_ADDNORM)  delta = bf16( sum over ranks, in rank order, of the rows pushed
 *                          into this rank's buffer ): the staging waits (bounded, about a second, then status
 *                          COBALT_ETIMEOUT through cobalt_device_status) for every rank's flag, then adds the rows
 *                          from local memory.  b must be NULL.
 *   cobalt_peer_sum()      the same sum as a kernel of its own, for consumers that cannot take the staged form.
 * Results equal cobalt_allreduce_peer() bit for bit.  All ranks must make the same sequence of calls on one buffer. */
#define COBALT_IN_PLAIN    0
#define COBALT_IN_GLU      1
#define COBALT_IN_ADDNORM  2
typedef struct CobaltPeerSlots {
    const uint64_t* peer_base;      /* [world] every rank's buffer as mapped into this process, 16-byte aligned */
    int rank, world;
    size_t slot_stride_bytes;       /* bytes of one row; flags_off_bytes >= (1 + 2 * world) * slot_stride_bytes */
    size_t flags_off_bytes;
} CobaltPeerSlots;
typedef struct CobaltStagedInput {
    int kind;                       /* COBALT_IN_PLAIN (a = x), COBALT_IN_GLU or COBALT_IN_ADDNORM */
    int flavor;
    const void* a;                  /* x, gate, or the residual stream h */
    const void* b;                  /* up, or delta (NULL: h' = h unless b_slots is given) */
    int64_t ld;
    const void* w;                  /* COBALT_IN_ADDNORM: norm weight [in_features] bf16 */
    const void* w_branch;           /* COBALT_IN_ADDNORM, flavor 1: weight of the norm applied to delta first, or NULL */
    void* h_out;                    /* COBALT_IN_ADDNORM: h' [M, in_features], or NULL */
    float eps;
    const CobaltPeerSlots* b_slots; /* COBALT_IN_ADDNORM: delta is the sum of the ranks' pushed partials, or NULL */
} CobaltStagedInput;
int cobalt_gemv_fused_staged(int n_mats, const CobaltMat* const* w, const CobaltStagedInput* in, void* const* y,
                             const int64_t* ldy, const void* const* bias, int M, int out_fp32,
                             const CobaltPeerSlots* push, void* scratch, size_t scratch_bytes, void* stream);
/* out[n] = bf16 (or fp32 when out_fp32) of the sum over ranks of the partials a pushing cobalt_gemv_fused_staged()
 * left in this rank's buffer: waits (bounded) for every rank's flag of the current epoch.  `status` as for
 * cobalt_allreduce_peer(). */
int cobalt_peer_sum(const CobaltPeerSlots* slots, size_t n, void* out, int out_fp32, void* status, void* stream);

/* cobalt_gemv() for callers that must not allocate device memory.
 *
 * Who needs it: code that runs where cudaMalloc is off limits -- a plug-in inside a serving
 * process whose memory pool is frozen after start-up, a real-time loop that cannot afford the
 * device-wide synchronisation an allocation implies, a host that hands this library raw pointers
 * from its own arena and forbids any other device allocation, or a process running so close to
 * the memory limit that an extra allocation may simply fail.  Such callers cannot size and own the scratch buffer that
 * cobalt_gemv() asks for, so this variant brings its own: a fixed
 * COBALT_STATIC_SCRATCH_BYTES array that is part of the library image on every GPU that
 * loads it, from load until the process exits.  Inputs and outputs are still the caller's.
 *
 *   - Same arguments (minus scratch), same kernel and bit-identical results as cobalt_gemv().
 *   - A matrix whose split-K bookkeeping does not fit the array is refused with
 *     COBALT_ETOOBIG; nothing is launched.  (The need grows with the number of row blocks;
 *     every 7B- and 27B-class projection, 262144-row heads included, fits.)
 *   - A bounded wait that gave up leaves its code in the array's status word; cobalt_device_status(NULL, ...)
 *     reads it.
 *   - It calls no cudaMalloc / cudaFree and no allocating library routine.  The first call on
 *     each device looks up the array's device address (cudaGetSymbolAddress, with that device
 *     current) -- make that first call outside any stream capture.
 *   - All calls on one GPU share the one array, and it keeps what the previous call left.  The
 *     entry point therefore zeroes the status word and the arrival counters on `stream` before
 *     every launch (cudaMemsetAsync, not an allocation).  Two calls that overlap on the GPU --
 *     different streams, or concurrent graph branches -- race on the array and produce wrong
 *     results; serialise them on one stream.
 * This entry point has no counterpart in the reference. */
#define COBALT_STATIC_SCRATCH_BYTES (8u << 20)
int cobalt_gemv_static(const CobaltMat* w, const void* x, int64_t ldx, void* y, int64_t ldy,
                       const void* bias, int M, void* stream);

/* Same contract and results as cobalt_gemv() through a plain one-thread-per-segment kernel
 * (no tensor cores, no bulk copies).  Bring-up and cross-check aid; needs no scratch. */
int cobalt_gemv_rowwalk(const CobaltMat* w, const void* x, int64_t ldx, void* y, int64_t ldy,
                        const void* bias, int M, void* stream);

/* Prefill GEMM, any M >= 1 (meant for M >= 17): same arithmetic contract as cobalt_gemv().
 * Weight tiles are dequantised to bf16 in shared memory and multiplied with tcgen05.mma,
 * accumulators in tensor memory; activations arrive through a TMA tensor map.  The tile image
 * must be followed by at least 64 readable bytes (the packer appends them).
 * Replaces cbk::gemm_tile + gemm_phase (src/cobaltkernel/csrc/cobalt_gemm.cuh:243-609,
 * src/cobaltkernel/csrc/prefill_kernel.cu:103-150).  `scratch` as for cobalt_gemv(). */
int cobalt_gemm(const CobaltMat* w, const void* x, int64_t ldx, void* y, int64_t ldy,
                const void* bias, int M, void* scratch, size_t scratch_bytes, void* stream);
size_t cobalt_gemm_scratch_bytes(const CobaltMat* w, int M);

/* Same product with the raw fp32 sums as output (no bias, no rounding): M <= 16 runs the GEMV,
 * larger M the GEMM.  For row-parallel tensor-parallel layers, whose partial outputs are added
 * across GPUs before the single rounding to bf16.  Scratch as for the kernel that runs.
 * No counterpart in the reference, which has no distributed code. */
int cobalt_linear_f32(const CobaltMat* w, const void* x, int64_t ldx, float* y, int64_t ldy, int M,
                      void* scratch, size_t scratch_bytes, void* stream);

/* Dense bf16 weight [K, N] (row-major, ld = N), bit-identical to the reference's
 * dequantize_sparse_sinq(...).to(bfloat16) (sinq/sparse_quant.py:1635-1681):
 * bf16_rne( fp32(q - z) * fp32(s) [* fp32(col_scale)] ) * keep.
 * Replaces cbk::dequant_row (src/cobaltkernel/csrc/cobalt_gemv.cuh:1218-1315). */
int cobalt_dequant(const CobaltMat* w, void* w_bf16, void* stream);

/* Recover the RAW schema (src/cobaltkernel/quantize_cobalt.py:326-329): codes u8[K, N]
 * (0 at pruned positions) and keep u8[K, N] in {0, 1}.  Either output may be NULL.
 * Replaces the host reader dequant_reference (src/cobaltkernel/pack_cobalt.py:277-334). */
int cobalt_unpack(const CobaltMat* w, uint8_t* codes, uint8_t* keep, void* stream);

/* End-to-end call with HOST activations and outputs: copies x host->device, runs the GEMV
 * (M <= 16) or GEMM, copies y device->host and synchronises `stream`.  The matrix itself
 * stays resident on the device.  `x_host` / `y_host` should be pinned for full speed.
 * `dev_x`, `dev_y`, `scratch` are caller-owned device staging buffers of at least
 * M*N*2, M*K*2 and max(cobalt_gemv_scratch_bytes, cobalt_gemm_scratch_bytes) bytes; `scratch` must be zeroed once
 * before its first use and then serves GEMV- and GEMM-sized calls in any order (every kernel leaves it clean).
 * Mirrors what a caller of SparseQuantLinear.forward pays when its tensors live on the host
 * (benchmarks/benchmark_suite.py:1200-1217). */
int cobalt_linear_host(const CobaltMat* w, const void* x_host, void* y_host, const void* bias, int M,
                       void* dev_x, void* dev_y, void* scratch, size_t scratch_bytes, void* stream);
/* The same without the final synchronisation: everything is stream-ordered; x_host and y_host must be pinned and
 * stay valid until the caller has synchronised the stream.  Lets a caller queue all projections of a block and
 * wait once. */
int cobalt_linear_host_async(const CobaltMat* w, const void* x_host, void* y_host, const void* bias, int M,
                             void* dev_x, void* dev_y, void* scratch, size_t scratch_bytes, void* stream);
/* cobalt_gemv_fused() for activations in host memory: ONE copy of x[M, in_features] host->device, one launch for up to
 * four matrices that read it (q|k|v, gate|up), one copy of every y[i] device->host; stream-ordered, no
 * synchronisation (buffers pinned and valid until the caller has synchronised).  dev_y[i] holds M * K_i bf16,
 * scratch at least cobalt_gemv_fused_scratch_bytes().  M <= 16.  Same results as cobalt_linear_host_async() per
 * matrix; it saves the repeated copy of x and the small launches (the reference packs q|k|v and gate|up as one
 * matrix for the same reason: docs/FORMAT.md:126-151). */
int cobalt_gemv_fused_host_async(int n_mats, const CobaltMat* const* w, const void* x_host, void* const* y_host, int M,
                                 void* dev_x, void* const* dev_y, void* scratch, size_t scratch_bytes, void* stream);

/* Fused element-wise steps of a decoder block around the linears, with the dtype policy of the
 * reference's executable specs (src/cobaltkernel/ref_llama.py:82-97, 139-143; src/cobaltkernel/ref_gemma3.py:138-143,
 * 173-174, 225-228; in the reference they are phases of its megakernel: src/cobaltkernel/csrc/megakernel.cu:270-288,
 * 667-774).  All tensors bf16.
 *   cobalt_add_rmsnorm : h_out = h + delta (delta, h_out may be NULL); rows [T, H] row-major;
 *                        flavor 0 (Llama): y = w * bf16(h_out * rsqrt(mean(h_out^2) + eps));
 *                        flavor 1 (Gemma): y = bf16(h_out * rsqrt(mean(h_out^2) + eps) * (1 + w)); with w_branch (may be
 *                        NULL) delta is first normalised the same way with (1 + w_branch) - the norm Gemma-3 applies to a
 *                        branch before it joins the residual.
 *   cobalt_rope_kv     : rotates q [T, n_heads*D] in place; rotates k and copies v [T, n_kv_heads*D] into the caches
 *                        [n_kv_heads][max_ctx][D] at positions[t] (a position outside [0, max_ctx) is read on the device
 *                        and simply not stored); inv_freq fp32 [D/2]; cos/sin rounded to bf16.  With
 *                        q_norm_w / k_norm_w (bf16 [D], both or neither) q and k first get Gemma-3's per-head norm
 *                        bf16(x * rsqrt(mean_D(x^2) + eps) * (1 + w)) (src/cobaltkernel/ref_gemma3.py:181-185).
 *                        cache_seq_stride (elements): token t writes at cache + t * cache_seq_stride - 0 when the T tokens
 *                        belong to one sequence, the size of one sequence's cache when T sequences decode one token each.
 *   cobalt_swiglu      : out = act(gate) * up over n elements; act 0 = SiLU, act 1 = GELU (tanh approximation).
 *   cobalt_attn_decode : grouped-query attention of one new token (q [n_heads*D], already rotated) over the caches
 *                        [n_kv_heads][max_ctx][D]; slots 0..positions[0] are attended (positions[0] is read on the device;
 *                        window > 0 keeps only the last `window` slots); out [n_heads*D].  Rounding points of
 *                        src/cobaltkernel/ref_llama.py:117-137: bf16 scores times `scale` rounded to bf16, fp32 softmax,
 *                        bf16 probabilities, bf16 context.  scratch: cobalt_attn_decode_scratch_bytes(), 256-byte aligned,
 *                        contents irrelevant.  n_heads/n_kv_heads <= 8, D in {64,128,192,256}, max_ctx <= 65536.
 *                        n_seq > 1 runs that many sequences at once (one new token each): q and out [n_seq][n_heads*D],
 *                        positions[n_seq], sequence b's caches at k_cache/v_cache + b * cache_seq_stride elements, scratch
 *                        n_seq times as large. */
int cobalt_add_rmsnorm(const void* h, const void* delta, const void* w, void* h_out, void* y, int T, int H, float eps,
                       int flavor, const void* w_branch, void* stream);
int cobalt_rope_kv(void* q, const void* k, const void* v, const int64_t* positions, const float* inv_freq, void* k_cache,
                   void* v_cache, int T, int n_heads, int n_kv_heads, int head_dim, int max_ctx, const void* q_norm_w,
                   const void* k_norm_w, float eps, int64_t cache_seq_stride, void* stream);
int cobalt_swiglu(const void* gate, const void* up, void* out, int64_t n, int act, void* stream);
size_t cobalt_attn_decode_scratch_bytes(int n_heads, int head_dim, int max_ctx);
int cobalt_attn_decode(const void* q, const void* k_cache, const void* v_cache, const int64_t* positions, void* scratch,
                       size_t scratch_bytes, void* out, int n_heads, int n_kv_heads, int head_dim, int max_ctx, int window,
                       float scale, int n_seq, int64_t cache_seq_stride, void* stream);
/* cobalt_attn_decode() as ONE kernel instead of three (cooperative launch: the CTAs of a head group wait for each other's
 * softmax statistics, with an iteration limit).  Same arguments and bit-identical results.  Differences: `scratch`
 * (cobalt_attn_decode_fused_scratch_bytes(), 256-byte aligned) must be ZERO before its first use - it starts with a
 * status word (cobalt_device_status(scratch, ...) reports COBALT_ETIMEOUT if a wait gave up) and arrival counters that
 * every launch returns to zero; and the whole grid (ceil(max_ctx / 128) * n_kv_heads * n_seq CTAs) must fit on the GPU
 * at once, else COBALT_EUNSUPPORTED is returned, nothing is launched and cobalt_attn_decode() is the way.  The reference
 * runs attention as a phase of its cooperative megakernel (src/cobaltkernel/csrc/megakernel.cu:842-1150). */
size_t cobalt_attn_decode_fused_scratch_bytes(int n_heads, int n_kv_heads, int head_dim, int max_ctx, int n_seq);
int cobalt_attn_decode_fused(const void* q, const void* k_cache, const void* v_cache, const int64_t* positions, void* scratch,
                             size_t scratch_bytes, void* out, int n_heads, int n_kv_heads, int head_dim, int max_ctx,
                             int window, float scale, int n_seq, int64_t cache_seq_stride, void* stream);

/* All-reduce (sum) of the fp32 partial outputs of a row-parallel layer over peer memory, for tensor-parallel decode
 * (the reference has no distributed code; this replaces the NCCL all-reduce that would follow cobalt_linear_f32).
 * Every rank owns one symmetric buffer mapped into all processes: [staging: slot_stride bytes][slot 0: world rows of
 * slot_stride bytes][slot 1: the same][flags at flags_off >= (1 + 2 * world) * slot_stride: 32 x u32], zero-initialised.
 * peer_base (host array, `world` entries) holds every rank's buffer address as seen by THIS process.  The caller has its
 * GEMV write the fp32 partial [n] into the staging area of its own buffer, then calls this on every rank with the same
 * n (all ranks make the same sequence of calls).  One CTA: pushes the partial into row `rank` of the slot of this call's
 * epoch (a counter kept on the device, so graph replays advance it) in EVERY rank's buffer (posted peer stores),
 * publishes the epoch in every peer's flags, waits (bounded, about a second; on expiry the status word is set and the
 * output is not written) until all peers have published theirs, adds the rows of its LOCAL slot in rank order
 * (deterministic) and writes bf16 (out_fp32 = 0) or fp32.  n % 4 == 0, n <= slot_stride/4, out 16-byte aligned,
 * world <= 8.  Plain peer stores only (no multicast, no load crosses NVLink). */
int cobalt_allreduce_peer(const uint64_t* peer_base, int rank, int world, size_t n, size_t slot_stride_bytes,
                          size_t flags_off_bytes, void* out, int out_fp32, void* status, void* stream);

/* Status word written by device code when a bounded wait gives up (0 = healthy).  Reads the
 * word at the start of `scratch` region reserved for it; synchronises `stream`.  scratch = NULL reads the word of
 * cobalt_gemv_static()'s private array on the current device (a copy from a cached address: nothing is allocated);
 * that word is cleared by every cobalt_gemv_static() call, so ask before the next one. */
int cobalt_device_status(const void* scratch, void* stream, uint32_t* status_out);

#ifdef __cplusplus
}
#endif
#endif /* COBALT_B200_H */
