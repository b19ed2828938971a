// One-thread-per-segment kernels: RAW recovery, dense dequantisation and a plain GEMV.
// They read the tile image straight from global memory and walk the 128 positions of a
// segment bit by bit; they are the simple, obviously-correct side of the library.
#pragma once
#include "common.cuh"

namespace cb {

// 64 threads per block = the 16 x 4 segments of one tile; thread t <-> (row r = t/4, group gi = t%4).
// Returns the index of the thread's first survivor code within the tile and the tile pointers.
struct SegCtx {
    const uint32_t* mask;      // 4 words, valid when active
    const uint32_t* stream;    // code stream of the tile
    uint32_t sz;               // {scale, zero} bits
    uint32_t first;            // rank of the first survivor of this segment within the tile
    bool active;
    int w;
};

__device__ __forceinline__ SegCtx open_segment(const MatView& W, int rb, int ct, uint32_t* sh_cnt /*[64]*/) {
    SegCtx c;
    const int t = threadIdx.x, r = t >> 2, gi = t & 3;
    c.w = tile_width(W, ct);
    c.active = gi < c.w;
    const uint8_t* tile = W.tiles + (size_t)W.tile_off[rb * W.CT + ct] * 16;
    const int seg = r * c.w + gi;
    c.mask = (const uint32_t*)tile + seg * 4;
    c.stream = (const uint32_t*)(tile + TILE_ROWS * c.w * 20);
    uint32_t cnt = 0;
    c.sz = 0;
    if (c.active) {
        cnt = __popc(c.mask[0]) + __popc(c.mask[1]) + __popc(c.mask[2]) + __popc(c.mask[3]);
        c.sz = ((const uint32_t*)(tile + TILE_ROWS * c.w * 16))[seg];
    }
    __syncthreads();                 // protect sh_cnt against the previous tile's readers
    sh_cnt[t] = cnt;
    __syncthreads();
    uint32_t first = 0;
    for (int i = 0; i < t; ++i) first += sh_cnt[i];     // thread order == segment order among active threads
    c.first = first;
    return c;
}

// codes u8[K,N] (0 at pruned), keep u8[K,N], dense bf16[K,N]; any output may be null
__global__ void __launch_bounds__(64) unpack_kernel(MatView W, uint8_t* codes, uint8_t* keep, uint16_t* dense) {
    __shared__ uint32_t sh_cnt[64];
    const int ct = blockIdx.x, rb = blockIdx.y;
    SegCtx c = open_segment(W, rb, ct, sh_cnt);
    const int r = threadIdx.x >> 2, gi = threadIdx.x & 3;
    const int row = rb * TILE_ROWS + r;
    if (!c.active || row >= W.K) return;
    const int col0 = (ct * TILE_GROUPS + gi) * GROUP;
    const float s = half_bits_to_float(c.sz & 0xFFFFu), z = half_bits_to_float(c.sz >> 16);
    uint32_t bitpos = c.first * (uint32_t)W.bits;
    for (int j = 0; j < 4; ++j) {
        const uint32_t m = c.mask[j];
        for (int b = 0; b < 32; ++b) {
            const int col = col0 + 32 * j + b;
            const uint32_t kept = (m >> b) & 1u;
            uint32_t code = 0;
            if (kept) { code = extract_code(c.stream, bitpos, W.bits); bitpos += W.bits; }
            const size_t o = (size_t)row * W.N + col;
            if (codes) codes[o] = (uint8_t)code;
            if (keep) keep[o] = (uint8_t)kept;
            if (dense) {
                const float cs = W.col_scale ? half_bits_to_float(W.col_scale[col]) : 1.0f;
                // literal reference order: ((q - z) * s) * col_scale, then * keep, then one cast
                dense[o] = float_to_bf16(__fmul_rn(dequant_fp32((float)code, z, s, cs), (float)kept));
            }
        }
    }
}

// y[m,k] = bf16( sum_j bf16(W[k,j]) * x[m,j] + bias[k] ), one block of 64 threads per row block
template <int MM>
__global__ void __launch_bounds__(64) gemv_rowwalk_kernel(MatView W, const uint16_t* x, int64_t ldx, uint16_t* y,
                                                          int64_t ldy, const uint16_t* bias, int M) {
    __shared__ uint32_t sh_cnt[64];
    const int rb = blockIdx.x;
    const int r = threadIdx.x >> 2, gi = threadIdx.x & 3;
    const int row = rb * TILE_ROWS + r;
    float acc[MM];
#pragma unroll
    for (int m = 0; m < MM; ++m) acc[m] = 0.0f;
    for (int ct = 0; ct < W.CT; ++ct) {
        SegCtx c = open_segment(W, rb, ct, sh_cnt);
        if (!c.active) continue;
        const int col0 = (ct * TILE_GROUPS + gi) * GROUP;
        const float s = half_bits_to_float(c.sz & 0xFFFFu), z = half_bits_to_float(c.sz >> 16);
        uint32_t bitpos = c.first * (uint32_t)W.bits;
        for (int j = 0; j < 4; ++j) {
            uint32_t m = c.mask[j];
            while (m) {
                const int b = __ffs(m) - 1;
                m &= m - 1;
                const int col = col0 + 32 * j + b;
                const uint32_t code = extract_code(c.stream, bitpos, W.bits);
                bitpos += W.bits;
                const float cs = W.col_scale ? half_bits_to_float(W.col_scale[col]) : 1.0f;
                const float wv = bf16_to_float(float_to_bf16(dequant_fp32((float)code, z, s, cs)));
#pragma unroll
                for (int mm = 0; mm < MM; ++mm)
                    if (mm < M) acc[mm] = fmaf(wv, bf16_to_float(x[(size_t)mm * ldx + col]), acc[mm]);
            }
        }
    }
#pragma unroll
    for (int mm = 0; mm < MM; ++mm) {
        float v = acc[mm];
        v += __shfl_xor_sync(0xFFFFFFFFu, v, 1);
        v += __shfl_xor_sync(0xFFFFFFFFu, v, 2);
        if (gi == 0 && mm < M && row < W.K) {
            if (bias) v += bf16_to_float(bias[row]);
            y[(size_t)mm * ldy + row] = float_to_bf16(v);
        }
    }
}

}  // namespace cb
