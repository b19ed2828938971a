// Small fused kernels around the compressed linears of a decoder block: residual add + RMSNorm,
// RoPE + KV-cache append, SwiGLU / GeGLU, single-token attention over the KV cache.  They follow the dtype policy of the reference's
// executable specs (src/cobaltkernel/ref_llama.py:82-97, 139-143; src/cobaltkernel/ref_gemma3.py:138-143, 173-174,
// 225-228): every intermediate that the spec holds in a bf16 tensor is rounded to bf16 here as
// well, so that results agree with the spec up to the summation order of the mean.
#pragma once
#include "common.cuh"
#include "staged_input.cuh"

namespace cb {

// h_out = bf16(h + delta') (delta may be null);
// flavor 0 (Llama):  y = w * bf16( h_out * rsqrt(mean(h_out^2) + eps) ),  delta' = delta
// flavor 1 (Gemma):  y = bf16( h_out * rsqrt(mean(h_out^2) + eps) * (1 + w) ), all in fp32 before the one rounding;
//                    with w_branch the branch is normalised first: delta' = bf16( delta * rsqrt(mean(delta^2) + eps) * (1 + w_branch) )
//                    (the post-attention / post-feedforward norm of src/cobaltkernel/ref_gemma3.py:262-270)
// one block per row; any H (the fast kernel below takes rows of a multiple of 256 values)
__global__ void __launch_bounds__(256) add_rmsnorm_generic_kernel(const uint16_t* h, const uint16_t* delta, const uint16_t* w,
                                                          uint16_t* h_out, uint16_t* y, int H, float eps, int flavor,
                                                          const uint16_t* w_branch) {
    __shared__ float red[8];
    // the next kernel in the stream (usually a GEMV launched with programmatic serialisation) may run its prologue now;
    // it waits for this grid before it reads y
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const size_t base = (size_t)blockIdx.x * H;
    auto block_sum = [&](float v) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
        __syncthreads();                                               // `red` may still be read from the previous sum
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
        __syncthreads();
        float tot = 0.0f;
#pragma unroll
        for (int k = 0; k < 8; ++k) tot += red[k];
        return tot;
    };
    float rb = 0.0f;                                                   // branch norm factor
    const bool norm_branch = delta != nullptr && w_branch != nullptr;
    if (norm_branch) {
        float sb = 0.0f;
        for (int i = threadIdx.x; i < H; i += 256) { const float d = bf16_to_float(delta[base + i]); sb += d * d; }
        rb = rsqrtf(block_sum(sb) / (float)H + eps);
    }
    auto joined = [&](int i) {                                         // bf16(h + delta')
        float v = bf16_to_float(h[base + i]);
        if (delta) {
            float d = bf16_to_float(delta[base + i]);
            if (norm_branch) d = bf16_round(__fmul_rn(__fmul_rn(d, rb), __fadd_rn(1.0f, bf16_to_float(w_branch[i]))));
            v = bf16_round(v + d);
        }
        return v;
    };
    float ss = 0.0f;
    for (int i = threadIdx.x; i < H; i += 256) {
        const float v = joined(i);
        if (h_out) h_out[base + i] = float_to_bf16(v);
        ss += v * v;
    }
    const float r = rsqrtf(block_sum(ss) / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += 256) {
        const float v = h_out ? bf16_to_float(h_out[base + i]) : joined(i);
        if (flavor == 0) {
            const float n = bf16_round(v * r);
            y[base + i] = float_to_bf16(bf16_to_float(w[i]) * n);
        } else {
            y[base + i] = float_to_bf16(__fmul_rn(__fmul_rn(v, r), __fadd_rn(1.0f, bf16_to_float(w[i]))));
        }
    }
}

// The same for rows of H = 256 * k values, H <= 256 * ADDNORM_MAX_GROUPS: one block of 512 threads per row, every
// value read once with 16-byte loads and kept in registers between the two sums and the output.  Sums of squares in
// the order staged_input.cuh defines, which the decode GEMV reproduces when it applies this step while staging.
constexpr int ADDNORM_THREADS = 512;
constexpr int ADDNORM_MAX_ITERS = 4;                                   // chunks per thread: rows up to 16384 values
__global__ void __launch_bounds__(ADDNORM_THREADS) add_rmsnorm_kernel(const uint16_t* h, const uint16_t* delta, const uint16_t* w,
                                                                      uint16_t* h_out, uint16_t* y, int H, float eps, int flavor,
                                                                      const uint16_t* w_branch) {
    __shared__ float tot_branch[ADDNORM_MAX_ITERS * ADDNORM_THREADS / 32], tot_joined[ADDNORM_MAX_ITERS * ADDNORM_THREADS / 32];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const size_t base = (size_t)blockIdx.x * H;
    const int cpr = H / 8, groups = cpr / 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool norm_branch = delta != nullptr && w_branch != nullptr;
    float v[ADDNORM_MAX_ITERS][8], d[ADDNORM_MAX_ITERS][8];
#pragma unroll
    for (int q = 0; q < ADDNORM_MAX_ITERS; ++q) {
        const int c = threadIdx.x + q * ADDNORM_THREADS;
        if (c < cpr) {
            chunk_to_floats(__ldg(reinterpret_cast<const uint4*>(h + base) + c), v[q]);
            if (delta) chunk_to_floats(__ldg(reinterpret_cast<const uint4*>(delta + base) + c), d[q]);
        }
    }
    if (norm_branch) {
#pragma unroll
        for (int q = 0; q < ADDNORM_MAX_ITERS; ++q) {
            const int c = threadIdx.x + q * ADDNORM_THREADS;
            const float s = warp_butterfly_sum(c < cpr ? chunk_sumsq(d[q]) : 0.0f);
            if (lane == 0 && c < cpr) tot_branch[q * (ADDNORM_THREADS / 32) + warp] = s;
        }
        __syncthreads();
        const float rb = row_rsqrt(tot_branch, groups, H, eps);
#pragma unroll
        for (int q = 0; q < ADDNORM_MAX_ITERS; ++q) {
            const int c = threadIdx.x + q * ADDNORM_THREADS;
            if (c < cpr) {
                float wb[8];
                chunk_to_floats(__ldg(reinterpret_cast<const uint4*>(w_branch) + c), wb);
#pragma unroll
                for (int k = 0; k < 8; ++k) d[q][k] = branch_value(d[q][k], rb, wb[k]);
            }
        }
    }
#pragma unroll
    for (int q = 0; q < ADDNORM_MAX_ITERS; ++q) {
        const int c = threadIdx.x + q * ADDNORM_THREADS;
        if (c < cpr && delta) {
#pragma unroll
            for (int k = 0; k < 8; ++k) v[q][k] = joined_value(v[q][k], d[q][k]);
            if (h_out) reinterpret_cast<uint4*>(h_out + base)[c] = floats_to_chunk(v[q]);
        }
        const float s = warp_butterfly_sum(c < cpr ? chunk_sumsq(v[q]) : 0.0f);
        if (lane == 0 && c < cpr) tot_joined[q * (ADDNORM_THREADS / 32) + warp] = s;
    }
    __syncthreads();
    const float r = row_rsqrt(tot_joined, groups, H, eps);
#pragma unroll
    for (int q = 0; q < ADDNORM_MAX_ITERS; ++q) {
        const int c = threadIdx.x + q * ADDNORM_THREADS;
        if (c < cpr) {
            float wn[8], o[8];
            chunk_to_floats(__ldg(reinterpret_cast<const uint4*>(w) + c), wn);
#pragma unroll
            for (int k = 0; k < 8; ++k) o[k] = normed_value(v[q][k], r, wn[k], flavor);
            reinterpret_cast<uint4*>(y + base)[c] = floats_to_chunk(o);
        }
    }
}

// q [T, nh*D] rotated in place; k rotated and v copied into the caches [kvh][max_ctx][D] at positions[t]
// (token t writes at cache + t * seq_stride: 0 for the tokens of one sequence, the per-sequence cache size for a batch
// of sequences that decode one token each)
__global__ void rope_kv_kernel(uint16_t* q, const uint16_t* k, const uint16_t* v, const long long* positions,
                               const float* inv_freq, uint16_t* k_cache, uint16_t* v_cache, int T, int nh, int nkv,
                               int D, int max_ctx, long long seq_stride) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int half = D / 2;
    const int per_tok = (nh + 2 * nkv) * half;
    const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= (long long)T * per_tok) return;
    const int t = (int)(gid / per_tok);
    int rem = (int)(gid - (long long)t * per_tok);
    const int head = rem / half, d = rem - head * half;
    const long long pos = positions[t];
    const float ang = (float)pos * inv_freq[d];
    const float c = bf16_round(cosf(ang)), s = bf16_round(sinf(ang));
    if (head < nh + nkv) {
        const bool is_q = head < nh;
        const uint16_t* src = is_q ? q + ((size_t)t * nh + head) * D : k + ((size_t)t * nkv + (head - nh)) * D;
        const float x1 = bf16_to_float(src[d]), x2 = bf16_to_float(src[d + half]);
        const float o1 = bf16_round(bf16_round(x1 * c) + bf16_round(-x2 * s));
        const float o2 = bf16_round(bf16_round(x2 * c) + bf16_round(x1 * s));
        if (!is_q && (pos < 0 || pos >= max_ctx)) return;              // a position outside the cache is never stored
        uint16_t* dst = is_q ? q + ((size_t)t * nh + head) * D
                             : k_cache + (size_t)t * seq_stride + ((size_t)(head - nh) * max_ctx + (size_t)pos) * D;
        dst[d] = float_to_bf16(o1);
        dst[d + half] = float_to_bf16(o2);
    } else {
        if (pos < 0 || pos >= max_ctx) return;
        const int hv = head - nh - nkv;
        const uint16_t* src = v + ((size_t)t * nkv + hv) * D;
        uint16_t* dst = v_cache + (size_t)t * seq_stride + ((size_t)hv * max_ctx + (size_t)pos) * D;
        dst[d] = src[d];
        dst[d + half] = src[d + half];
    }
}

// The same with Gemma-3's per-head norm of q and k in front (src/cobaltkernel/ref_gemma3.py:181-185): one warp per (token, head);
// x' = bf16( x * rsqrt(mean_D(x^2) + eps) * (1 + w[d]) ), then the rotation on x'.  v is copied unchanged.
__global__ void __launch_bounds__(256) rope_kv_norm_kernel(uint16_t* q, const uint16_t* k, const uint16_t* v, const long long* positions,
                                                           const float* inv_freq, uint16_t* k_cache, uint16_t* v_cache, int T, int nh,
                                                           int nkv, int D, int max_ctx, const uint16_t* q_norm_w,
                                                           const uint16_t* k_norm_w, float eps, long long seq_stride) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int half = D / 2;
    const int heads = nh + 2 * nkv;
    const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= (long long)T * heads) return;
    const int t = (int)(wid / heads), head = (int)(wid - (long long)t * heads);
    const long long pos = positions[t];
    if (head >= nh && (pos < 0 || pos >= max_ctx)) return;             // a position outside the cache is never stored
    if (head >= nh + nkv) {                                            // v: plain copy into the cache
        const int hv = head - nh - nkv;
        const uint16_t* src = v + ((size_t)t * nkv + hv) * D;
        uint16_t* dst = v_cache + (size_t)t * seq_stride + ((size_t)hv * max_ctx + (size_t)pos) * D;
        for (int d = lane; d < D; d += 32) dst[d] = src[d];
        return;
    }
    const bool is_q = head < nh;
    const uint16_t* src = is_q ? q + ((size_t)t * nh + head) * D : k + ((size_t)t * nkv + (head - nh)) * D;
    const uint16_t* nw = is_q ? q_norm_w : k_norm_w;
    uint16_t* dst = is_q ? q + ((size_t)t * nh + head) * D : k_cache + (size_t)t * seq_stride + ((size_t)(head - nh) * max_ctx + (size_t)pos) * D;
    float ss = 0.0f;
    for (int d = lane; d < D; d += 32) { const float x = bf16_to_float(src[d]); ss += x * x; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
    const float r = rsqrtf(ss / (float)D + eps);
    for (int d = lane; d < half; d += 32) {
        const float x1 = bf16_round(__fmul_rn(__fmul_rn(bf16_to_float(src[d]), r), __fadd_rn(1.0f, bf16_to_float(nw[d]))));
        const float x2 = bf16_round(__fmul_rn(__fmul_rn(bf16_to_float(src[d + half]), r), __fadd_rn(1.0f, bf16_to_float(nw[d + half]))));
        const float ang = (float)pos * inv_freq[d];
        const float c = bf16_round(cosf(ang)), s = bf16_round(sinf(ang));
        const float o1 = bf16_round(bf16_round(x1 * c) + bf16_round(-x2 * s));
        const float o2 = bf16_round(bf16_round(x2 * c) + bf16_round(x1 * s));
        dst[d] = float_to_bf16(o1);
        dst[d + half] = float_to_bf16(o2);
    }
}

// out = bf16( bf16(act(g)) * u ); act 0 = SiLU, act 1 = GELU with the tanh approximation
__global__ void swiglu_kernel(const uint16_t* g, const uint16_t* u, uint16_t* out, long long n, int act) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    out[i] = float_to_bf16(glu_value(bf16_to_float(g[i]), bf16_to_float(u[i]), act));
}

// ----------------------------------------------------------------------------- single-token attention
// Grouped-query attention of ONE new token over the KV caches [n_kv][max_ctx][D], with the rounding points of the
// reference's executable spec (src/cobaltkernel/ref_llama.py:117-137): scores = bf16(q . k) (fp32 sum), times the scale
// rounded to bf16, softmax in fp32 over the allowed slots, probabilities rounded to bf16, context = bf16(sum p * v).
// The number of slots comes from positions[0] on the device, so a captured graph does the work of the current length.
// Three small kernels over (slot chunk, KV head) so that every SM takes part:
//   1. scores of a chunk of slots into att [n_heads][max_ctx] (fp32 holding bf16 values) + the chunk's max and
//      sum of exp per head;
//   2. global max / sum from the chunk statistics (a few dozen values), probabilities of the chunk, partial context
//      [chunk][n_heads][D] in fp32;
//   3. partial contexts added in chunk order, rounded to bf16.
// They are launched plainly: with programmatic serialisation their CTAs were scheduled early only to wait, and the
// three took 22.5 us instead of 19.2 us per layer.
constexpr int ATTN_MAX_REP = 8;            // query heads per KV head
constexpr int ATTN_CHUNK = 128;            // cache slots per CTA
constexpr int ATTN_WARPS = ATTN_CHUNK / 8; // every warp takes 8 slots of the chunk
constexpr int ATTN_THREADS = ATTN_WARPS * 32;
constexpr int ATTN_MAX_CHUNKS = 1024;      // max_ctx <= 65536

__device__ __forceinline__ bool attn_allowed(int s, long long pos, int window, int max_ctx) {
    return s < max_ctx && s <= pos && (window <= 0 || s > pos - window);
}

// grid (chunks, n_kv), block ATTN_THREADS: warp w takes slots s0 + w + ATTN_WARPS * i; lane holds D/32 contiguous dims (D % 64 == 0, D <= 256)
__global__ void __launch_bounds__(ATTN_THREADS) attn_scores_kernel(const uint16_t* q, const uint16_t* k_cache, const long long* positions,
                                                          float* att, float* chunk_stat, int rep, int D, int max_ctx, int window,
                                                          float scale, long long seq_stride) {
    __shared__ float sc[ATTN_MAX_REP][ATTN_CHUNK];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kvh = blockIdx.y, chunk = blockIdx.x, nchunks = gridDim.x;
    const int n_heads_all = (int)gridDim.y * rep;
    // blockIdx.z = sequence: its query, cache, position and scratch
    q += (size_t)blockIdx.z * n_heads_all * D;
    k_cache += (size_t)blockIdx.z * seq_stride;
    att += (size_t)blockIdx.z * n_heads_all * max_ctx;
    chunk_stat += (size_t)blockIdx.z * n_heads_all * nchunks * 2;
    const long long pos = positions[blockIdx.z];
    const int s0 = chunk * ATTN_CHUNK;
    float* stat = chunk_stat + ((size_t)(kvh * rep) * nchunks + chunk) * 2;     // [head][chunk][max, sum]
    if (s0 > pos || (window > 0 && s0 + ATTN_CHUNK - 1 <= pos - window)) {      // nothing allowed in this chunk
        if (threadIdx.x < rep) { stat[(size_t)threadIdx.x * nchunks * 2] = -INFINITY; stat[(size_t)threadIdx.x * nchunks * 2 + 1] = 0.0f; }
        return;
    }
    const int per = D / 32;
    uint32_t kraw[8][4], qraw[ATTN_MAX_REP][4];
    bool ok[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {                          // all loads first: their latencies overlap
        const int s = s0 + warp + ATTN_WARPS * i;
        ok[i] = attn_allowed(s, pos, window, max_ctx);
        const uint32_t* kp = reinterpret_cast<const uint32_t*>(k_cache + ((size_t)kvh * max_ctx + (ok[i] ? s : 0)) * D + lane * per);
#pragma unroll
        for (int e2 = 0; e2 < 4; ++e2) kraw[i][e2] = (ok[i] && e2 * 2 < per) ? __ldg(kp + e2) : 0u;
    }
#pragma unroll
    for (int h = 0; h < ATTN_MAX_REP; ++h) {
        const uint32_t* qp = reinterpret_cast<const uint32_t*>(q + ((size_t)kvh * rep + (h < rep ? h : 0)) * D + lane * per);
#pragma unroll
        for (int e2 = 0; e2 < 4; ++e2) qraw[h][e2] = (h < rep && e2 * 2 < per) ? __ldg(qp + e2) : 0u;
    }
#pragma unroll
    for (int h = 0; h < ATTN_MAX_REP; ++h) {
        if (h >= rep) break;
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            acc[i] = 0.0f;
#pragma unroll
            for (int e2 = 0; e2 < 4; ++e2) {
                acc[i] = fmaf(__uint_as_float(qraw[h][e2] << 16), __uint_as_float(kraw[i][e2] << 16), acc[i]);
                acc[i] = fmaf(__uint_as_float(qraw[h][e2] & 0xFFFF0000u), __uint_as_float(kraw[i][e2] & 0xFFFF0000u), acc[i]);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] += __shfl_xor_sync(0xFFFFFFFFu, acc[i], o);
        if (lane < 8) {                                    // lane i keeps slot i of this warp
            float mine = 0.0f;
            bool w_ok = false;
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (lane == i) { mine = acc[i]; w_ok = ok[i]; }
            const float v = w_ok ? bf16_round(bf16_round(mine) * scale) : -INFINITY;
            sc[h][warp + ATTN_WARPS * lane] = v;
            if (w_ok) att[((size_t)kvh * rep + h) * max_ctx + s0 + warp + ATTN_WARPS * lane] = v;
        }
    }
    __syncthreads();
    if (warp < rep) {                                                   // warp h: max and sum of exp of head h over the chunk
        float m = -INFINITY;
#pragma unroll
        for (int j = 0; j < ATTN_CHUNK; j += 32) m = fmaxf(m, sc[warp][lane + j]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
        float z = 0.0f;
#pragma unroll
        for (int j = 0; j < ATTN_CHUNK; j += 32) { const float a = sc[warp][lane + j]; z += a == -INFINITY ? 0.0f : expf(a - m); }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) z += __shfl_xor_sync(0xFFFFFFFFu, z, o);
        if (lane == 0) { stat[(size_t)warp * nchunks * 2] = m; stat[(size_t)warp * nchunks * 2 + 1] = z; }
    }
}

// grid (chunks, n_kv), block ATTN_THREADS = ATTN_WARPS warps x 32 dims: thread (w, l) adds the slots s0 + w + ATTN_WARPS * i of dims l, l+32, ... ;
// partial context of the chunk -> part [chunk][n_heads][D]
__global__ void __launch_bounds__(ATTN_THREADS) attn_context_kernel(const float* att, const float* chunk_stat, const uint16_t* v_cache,
                                                           const long long* positions, float* part, int rep, int D, int max_ctx,
                                                           int window, int n_heads, long long seq_stride) {
    __shared__ float gm[ATTN_MAX_REP], gz[ATTN_MAX_REP];
    __shared__ float pr[ATTN_MAX_REP][ATTN_CHUNK];
    __shared__ float red[ATTN_WARPS][ATTN_MAX_REP][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kvh = blockIdx.y, chunk = blockIdx.x, nchunks = gridDim.x;
    v_cache += (size_t)blockIdx.z * seq_stride;                         // blockIdx.z = sequence
    att += (size_t)blockIdx.z * n_heads * max_ctx;
    chunk_stat += (size_t)blockIdx.z * n_heads * nchunks * 2;
    part += (size_t)blockIdx.z * nchunks * n_heads * D;
    const long long pos = positions[blockIdx.z];
    const int s0 = chunk * ATTN_CHUNK;
    float* mine = part + ((size_t)chunk * n_heads + (size_t)kvh * rep) * D;
    if (s0 > pos || (window > 0 && s0 + ATTN_CHUNK - 1 <= pos - window)) return;   // the combine step skips chunks outside the range
    if (warp < rep) {                                                   // global max and sum of head `warp` from the chunk statistics
        const float* st = chunk_stat + (size_t)(kvh * rep + warp) * nchunks * 2;
        float m = -INFINITY;
        for (int c = lane; c < nchunks; c += 32) m = fmaxf(m, st[2 * c]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
        float z = 0.0f;
        for (int c = lane; c < nchunks; c += 32) { const float mc = st[2 * c]; if (mc != -INFINITY) z += st[2 * c + 1] * expf(mc - m); }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) z += __shfl_xor_sync(0xFFFFFFFFu, z, o);
        if (lane == 0) { gm[warp] = m; gz[warp] = z; }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < rep * ATTN_CHUNK; i += ATTN_THREADS) {        // probabilities of the chunk, rounded to bf16
        const int h = i / ATTN_CHUNK, j = i - h * ATTN_CHUNK, s = s0 + j;
        pr[h][j] = attn_allowed(s, pos, window, max_ctx) ? bf16_round(expf(att[((size_t)kvh * rep + h) * max_ctx + s] - gm[h]) / gz[h]) : 0.0f;
    }
    __syncthreads();
    for (int d0 = 0; d0 < D; d0 += 32) {
        float vv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int s = s0 + warp + ATTN_WARPS * i;
            vv[i] = attn_allowed(s, pos, window, max_ctx) ? bf16_to_float(v_cache[((size_t)kvh * max_ctx + s) * D + d0 + lane]) : 0.0f;
        }
#pragma unroll
        for (int h = 0; h < ATTN_MAX_REP; ++h) {
            if (h >= rep) break;
            float a = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) a = fmaf(pr[h][warp + ATTN_WARPS * i], vv[i], a);
            red[warp][h][lane] = a;
        }
        __syncthreads();
        if (warp < rep) {
            float a = 0.0f;
#pragma unroll
            for (int w = 0; w < ATTN_WARPS; ++w) a += red[w][warp][lane];
            mine[(size_t)warp * D + d0 + lane] = a;
        }
        __syncthreads();
    }
}

// grid ceil(n_heads * D / 256): out[h][d] = bf16( sum over chunks, in order, of part[chunk][h][d] ) for the chunks in range;
// the next kernel (the o projection's GEMV) may start its prologue at once
__global__ void __launch_bounds__(256) attn_combine_kernel(const float* part, const long long* positions, uint16_t* out, int n, int nchunks,
                                                           int window) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= n) return;
    part += (size_t)blockIdx.y * nchunks * n;                           // blockIdx.y = sequence
    out += (size_t)blockIdx.y * n;
    const long long pos = positions[blockIdx.y];
    int c1 = (int)(pos / ATTN_CHUNK) + 1;
    if (c1 > nchunks) c1 = nchunks;
    int c0 = 0;
    if (window > 0 && pos - window + 1 > 0) c0 = (int)((pos - window + 1) / ATTN_CHUNK);
    float a = 0.0f;
    for (int c = c0; c < c1; ++c) a += part[(size_t)c * n + i];
    out[i] = float_to_bf16(a);
}

// The three steps above as ONE kernel (cooperative launch: every CTA of the grid is resident, so CTAs may wait for each
// other).  grid (chunks, n_kv, n_seq).  A CTA computes the scores of its chunk and keeps them in shared memory, publishes
// the chunk's max / sum of exp, arrives on a counter of its (sequence, KV head) and waits - with an iteration limit -
// until all chunks in range have arrived; then it reads the statistics, forms the probabilities of its chunk and the
// partial context, and arrives on a second counter: the last CTA to do so adds the partial contexts in chunk order and
// rounds once.  Same arithmetic, in the same order, as the three kernels.  counters: [n_seq][n_kv][2] u32, zero before
// the first launch; the last CTA returns both to zero.  status: set to DEV_TIMEOUT_ATTN when the wait gives up (the
// outputs of that head group are then not written).
__device__ __forceinline__ void attn_chunk_range(long long pos, int window, int nchunks, int& c0, int& c1) {
    c1 = (int)(pos / ATTN_CHUNK) + 1;
    if (c1 > nchunks) c1 = nchunks;
    c0 = 0;
    if (window > 0 && pos - window + 1 > 0) c0 = (int)((pos - window + 1) / ATTN_CHUNK);
}

__global__ void __launch_bounds__(ATTN_THREADS) attn_decode_fused_kernel(const uint16_t* q, const uint16_t* k_cache, const uint16_t* v_cache,
                                                                         const long long* positions, float* chunk_stat, float* part,
                                                                         uint32_t* counters, uint32_t* status, uint16_t* out, int rep, int D,
                                                                         int max_ctx, int window, float scale, long long seq_stride) {
    __shared__ float sc[ATTN_MAX_REP][ATTN_CHUNK];
    __shared__ float gm[ATTN_MAX_REP], gz[ATTN_MAX_REP];
    __shared__ float red[ATTN_WARPS][ATTN_MAX_REP][32];
    __shared__ uint32_t flag_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kvh = blockIdx.y, chunk = blockIdx.x, nchunks = gridDim.x, n_kv = gridDim.y;
    const int n_heads = n_kv * rep;
    q += (size_t)blockIdx.z * n_heads * D;
    out += (size_t)blockIdx.z * n_heads * D;
    k_cache += (size_t)blockIdx.z * seq_stride;
    v_cache += (size_t)blockIdx.z * seq_stride;
    chunk_stat += (size_t)blockIdx.z * n_heads * nchunks * 2;
    part += (size_t)blockIdx.z * nchunks * n_heads * D;
    uint32_t* cnt = counters + ((size_t)blockIdx.z * n_kv + kvh) * 2;
    const long long pos = positions[blockIdx.z];
    int c0, c1;
    attn_chunk_range(pos, window, nchunks, c0, c1);
    if (chunk < c0 || chunk >= c1) return;                              // nothing allowed in this chunk: it takes no part
    const uint32_t expected = (uint32_t)(c1 - c0);
    const int s0 = chunk * ATTN_CHUNK;
    float* stat = chunk_stat + ((size_t)(kvh * rep) * nchunks + chunk) * 2;     // [head][chunk][max, sum]
    const int per = D / 32;
    {   // ---- scores of the chunk (as attn_scores_kernel), kept in shared memory
        uint32_t kraw[8][4], qraw[ATTN_MAX_REP][4];
        bool ok[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int s = s0 + warp + ATTN_WARPS * i;
            ok[i] = attn_allowed(s, pos, window, max_ctx);
            const uint32_t* kp = reinterpret_cast<const uint32_t*>(k_cache + ((size_t)kvh * max_ctx + (ok[i] ? s : 0)) * D + lane * per);
#pragma unroll
            for (int e2 = 0; e2 < 4; ++e2) kraw[i][e2] = (ok[i] && e2 * 2 < per) ? __ldg(kp + e2) : 0u;
        }
#pragma unroll
        for (int h = 0; h < ATTN_MAX_REP; ++h) {
            const uint32_t* qp = reinterpret_cast<const uint32_t*>(q + ((size_t)kvh * rep + (h < rep ? h : 0)) * D + lane * per);
#pragma unroll
            for (int e2 = 0; e2 < 4; ++e2) qraw[h][e2] = (h < rep && e2 * 2 < per) ? __ldg(qp + e2) : 0u;
        }
#pragma unroll
        for (int h = 0; h < ATTN_MAX_REP; ++h) {
            if (h >= rep) break;
            float acc[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                acc[i] = 0.0f;
#pragma unroll
                for (int e2 = 0; e2 < 4; ++e2) {
                    acc[i] = fmaf(__uint_as_float(qraw[h][e2] << 16), __uint_as_float(kraw[i][e2] << 16), acc[i]);
                    acc[i] = fmaf(__uint_as_float(qraw[h][e2] & 0xFFFF0000u), __uint_as_float(kraw[i][e2] & 0xFFFF0000u), acc[i]);
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] += __shfl_xor_sync(0xFFFFFFFFu, acc[i], o);
            if (lane < 8) {
                float mine = 0.0f;
                bool w_ok = false;
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (lane == i) { mine = acc[i]; w_ok = ok[i]; }
                sc[h][warp + ATTN_WARPS * lane] = w_ok ? bf16_round(bf16_round(mine) * scale) : -INFINITY;
            }
        }
    }
    __syncthreads();
    if (warp < rep) {                                                   // warp h: max and sum of exp of head h over the chunk
        float m = -INFINITY;
#pragma unroll
        for (int j = 0; j < ATTN_CHUNK; j += 32) m = fmaxf(m, sc[warp][lane + j]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
        float z = 0.0f;
#pragma unroll
        for (int j = 0; j < ATTN_CHUNK; j += 32) { const float a = sc[warp][lane + j]; z += a == -INFINITY ? 0.0f : expf(a - m); }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) z += __shfl_xor_sync(0xFFFFFFFFu, z, o);
        if (lane == 0) { stat[(size_t)warp * nchunks * 2] = m; stat[(size_t)warp * nchunks * 2 + 1] = z; }
    }
    // ---- every chunk of this (sequence, KV head) has published its statistics?  bounded wait
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(&cnt[0], 1u);
        uint32_t good = 0u;
        for (uint32_t it = 0; it < (1u << 20); ++it) {
            uint32_t v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(cnt) : "memory");
            if (v >= expected) { good = 1u; break; }
            if (it > 256) __nanosleep(64);
        }
        if (!good && status) atomicCAS(status, 0u, (uint32_t)DEV_TIMEOUT_ATTN);
        flag_s = good;
    }
    __syncthreads();
    if (flag_s == 0u) return;
    __threadfence();
    if (warp < rep) {                                                   // global max and sum of head `warp` from the chunk statistics
        const float* st = chunk_stat + (size_t)(kvh * rep + warp) * nchunks * 2;
        // same lanes, same order as attn_context_kernel (chunks outside the range count as empty there too)
        float m = -INFINITY;
        for (int c = lane; c < nchunks; c += 32)
            if (c >= c0 && c < c1) m = fmaxf(m, __ldcg(st + 2 * c));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
        float z = 0.0f;
        for (int c = lane; c < nchunks; c += 32)
            if (c >= c0 && c < c1) { const float mc = __ldcg(st + 2 * c); if (mc != -INFINITY) z += __ldcg(st + 2 * c + 1) * expf(mc - m); }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) z += __shfl_xor_sync(0xFFFFFFFFu, z, o);
        if (lane == 0) { gm[warp] = m; gz[warp] = z; }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < rep * ATTN_CHUNK; i += ATTN_THREADS) {        // probabilities of the chunk, rounded to bf16 (in place)
        const int h = i / ATTN_CHUNK, j = i - h * ATTN_CHUNK;
        const float a = sc[h][j];
        sc[h][j] = a == -INFINITY ? 0.0f : bf16_round(expf(a - gm[h]) / gz[h]);
    }
    __syncthreads();
    float* mine = part + ((size_t)chunk * n_heads + (size_t)kvh * rep) * D;
    for (int d0 = 0; d0 < D; d0 += 32) {
        float vv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int s = s0 + warp + ATTN_WARPS * i;
            vv[i] = attn_allowed(s, pos, window, max_ctx) ? bf16_to_float(v_cache[((size_t)kvh * max_ctx + s) * D + d0 + lane]) : 0.0f;
        }
#pragma unroll
        for (int h = 0; h < ATTN_MAX_REP; ++h) {
            if (h >= rep) break;
            float a = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) a = fmaf(sc[h][warp + ATTN_WARPS * i], vv[i], a);
            red[warp][h][lane] = a;
        }
        __syncthreads();
        if (warp < rep) {
            float a = 0.0f;
#pragma unroll
            for (int w = 0; w < ATTN_WARPS; ++w) a += red[w][warp][lane];
            mine[(size_t)warp * D + d0 + lane] = a;
        }
        __syncthreads();
    }
    // ---- the last chunk to finish adds the partial contexts in chunk order
    if (threadIdx.x == 0) {
        __threadfence();
        flag_s = atomicAdd(&cnt[1], 1u) == expected - 1u ? 1u : 0u;
    }
    __syncthreads();
    if (flag_s == 0u) return;
    __threadfence();
    for (int i = threadIdx.x; i < rep * D; i += ATTN_THREADS) {
        float a = 0.0f;
        for (int c = c0; c < c1; ++c) a += __ldcg(part + ((size_t)c * n_heads + (size_t)kvh * rep) * D + i);
        out[(size_t)kvh * rep * D + i] = float_to_bf16(a);
    }
    if (threadIdx.x == 0) { cnt[0] = 0u; cnt[1] = 0u; }
}

// ----------------------------------------------------------------------------- all-reduce over peer memory
// Sum of the fp32 partial outputs of a row-parallel layer, one [n]-vector per GPU, added in rank order and rounded
// to bf16 once.  Every rank runs this kernel (one CTA) on its own GPU.  It PUSHES: the partial goes from the local
// staging area (where the GEMV wrote it) into row `rank` of slot (epoch & 1) in EVERY rank's buffer (posted NVLink
// stores), then "my partial of epoch e is written" is published in each peer's flag array (release at system
// scope); the kernel waits (bounded) until all peers have published epoch e in its own flag array and adds the
// `world` rows of the slot from LOCAL memory - no load ever crosses NVLink.  The epoch counter lives on the device,
// so replaying a captured graph advances it like eager calls do.  Two slots alternate, so that a rank that is ahead
// never overwrites a row that a peer is still reading (a rank can only finish epoch e after every peer has started
// it, i.e. has finished reading epoch e-1).
struct PeerParams {
    unsigned long long base[PEER_MAX_RANKS];   // every rank's symmetric buffer, as mapped into this process
    int rank, world;
    unsigned int n;                            // floats to reduce
    unsigned long long slot_stride, flags_off; // bytes; staging at 0, slot s row r at (1 + s * world + r) * slot_stride
    uint16_t* out;                             // bf16 [n]
    float* out32;                              // or fp32 [n]
    uint32_t* status;
};

__global__ void __launch_bounds__(1024) peer_allreduce_kernel(const PeerParams P) {
    __shared__ uint32_t epoch_s;
    // Programmatic dependent launch: wait for the kernel that wrote the partial, and let the next kernel in the
    // stream begin its own prologue (it waits for this grid before it touches activations).
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    uint32_t* my_flags = reinterpret_cast<uint32_t*>(P.base[P.rank] + P.flags_off);
    if (threadIdx.x == 0) {
        const uint32_t e = my_flags[PEER_EPOCH_INDEX] + 1u;
        my_flags[PEER_EPOCH_INDEX] = e;
        epoch_s = e;
    }
    __syncthreads();
    const uint32_t epoch = epoch_s;
    const unsigned long long slot_off = (1ull + (unsigned long long)(epoch & 1u) * P.world) * P.slot_stride;   // row 0 of this epoch's slot
    const unsigned int n4 = P.n >> 2;                                  // n is a multiple of 4 (checked on the host)
    {   // staging -> row `rank` of this epoch's slot on every rank (the own copy included)
        const float4* stage = reinterpret_cast<const float4*>(P.base[P.rank]);
        const unsigned long long row_off = slot_off + (unsigned long long)P.rank * P.slot_stride;
        for (unsigned int i = threadIdx.x; i < n4; i += 1024) {
            const float4 v = stage[i];
#pragma unroll
            for (int q = 0; q < PEER_MAX_RANKS; ++q)
                if (q < P.world) reinterpret_cast<float4*>(P.base[q] + row_off)[i] = v;
        }
    }
    __syncthreads();                                                   // the release below covers every thread's stores
    bool good = true;
    if ((int)threadIdx.x < P.world) {
        uint32_t* theirs = reinterpret_cast<uint32_t*>(P.base[threadIdx.x] + P.flags_off) + P.rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
        const uint32_t* mine = my_flags + threadIdx.x;
        good = false;
        for (uint32_t it = 0; it < (1u << 20); ++it) {                 // about a second at the longest
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
            if ((int32_t)(v - epoch) >= 0) { good = true; break; }
            if (it > 1024) __nanosleep(128);
        }
    }
    if (!__syncthreads_and(good ? 1 : 0)) {
        if (threadIdx.x == 0 && P.status) atomicCAS(P.status, 0u, (uint32_t)DEV_TIMEOUT_PEER);
        return;
    }
    const unsigned long long mine_base = P.base[P.rank] + slot_off;
    for (unsigned int i = threadIdx.x; i < n4; i += 1024) {
        float4 v[PEER_MAX_RANKS];
#pragma unroll
        for (int q = 0; q < PEER_MAX_RANKS; ++q)                       // the rows the peers pushed, all loads in flight before the first add
            if (q < P.world) v[q] = ld_sys_f4(reinterpret_cast<const float*>(mine_base + (unsigned long long)q * P.slot_stride) + 4 * i);
        float4 s = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (int q = 0; q < PEER_MAX_RANKS; ++q)
            if (q < P.world) { s.x += v[q].x; s.y += v[q].y; s.z += v[q].z; s.w += v[q].w; }
        if (P.out32) {
            reinterpret_cast<float4*>(P.out32)[i] = s;
        } else {
            uint2 o;
            o.x = (uint32_t)float_to_bf16(s.x) | ((uint32_t)float_to_bf16(s.y) << 16);
            o.y = (uint32_t)float_to_bf16(s.z) | ((uint32_t)float_to_bf16(s.w) << 16);
            reinterpret_cast<uint2*>(P.out)[i] = o;
        }
    }
}

// The summing half alone, for partials that a pushing GEMV already placed in every rank's slot and published: waits
// (bounded) for all flags of the current epoch, adds the rows in rank order from local memory, rounds once.
__global__ void __launch_bounds__(1024) peer_sum_kernel(const PeerParams P) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t* my_flags = reinterpret_cast<const uint32_t*>(P.base[P.rank] + P.flags_off);
    const uint32_t epoch = *reinterpret_cast<const volatile uint32_t*>(my_flags + PEER_EPOCH_INDEX);
    if (!peer_wait_epoch(my_flags, P.world, epoch)) {
        if (threadIdx.x == 0 && P.status) atomicCAS(P.status, 0u, (uint32_t)DEV_TIMEOUT_PEER);
        return;
    }
    const uint8_t* row0 = reinterpret_cast<const uint8_t*>(P.base[P.rank] + (1ull + (unsigned long long)(epoch & 1u) * P.world) * P.slot_stride);
    for (unsigned int i = threadIdx.x; i < (P.n >> 3); i += 1024) {    // n is a multiple of 8 (checked on the host)
        if (P.out32) {
            float4 a = make_float4(0.0f, 0.0f, 0.0f, 0.0f), b = a;
            for (int q = 0; q < P.world; ++q) {
                const float* p = reinterpret_cast<const float*>(row0 + (unsigned long long)q * P.slot_stride) + 8 * (size_t)i;
                const float4 u = ld_sys_f4(p), v = ld_sys_f4(p + 4);
                a.x += u.x; a.y += u.y; a.z += u.z; a.w += u.w; b.x += v.x; b.y += v.y; b.z += v.z; b.w += v.w;
            }
            reinterpret_cast<float4*>(P.out32)[2 * i] = a;
            reinterpret_cast<float4*>(P.out32)[2 * i + 1] = b;
        } else {
            reinterpret_cast<uint4*>(P.out)[i] = peer_sum_chunk(row0, P.slot_stride, P.world, 8 * (size_t)i);
        }
    }
}

}  // namespace cb
