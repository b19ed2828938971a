// Small fused kernels around the compressed linears of a decoder block: residual add + RMSNorm,
// RoPE + KV-cache append, SwiGLU / GeGLU.  They follow the dtype policy of the reference's
// executable specs (src/cobaltkernel/ref_llama.py:82-97, 139-143; src/cobaltkernel/ref_gemma3.py:138-143, 173-174,
// 225-228): every intermediate that the spec holds in a bf16 tensor is rounded to bf16 here as
// well, so that results agree with the spec up to the summation order of the mean.
#pragma once
#include "common.cuh"

namespace cb {

__device__ __forceinline__ float bf16_round(float f) { return bf16_to_float(float_to_bf16(f)); }

// h_out = bf16(h + delta) (delta may be null);
// flavor 0 (Llama):  y = w * bf16( h_out * rsqrt(mean(h_out^2) + eps) )
// flavor 1 (Gemma):  y = bf16( h_out * rsqrt(mean(h_out^2) + eps) * (1 + w) ), all in fp32 before the one rounding
// one block per row
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(const uint16_t* h, const uint16_t* delta, const uint16_t* w,
                                                          uint16_t* h_out, uint16_t* y, int H, float eps, int flavor) {
    __shared__ float red[8];
    const size_t base = (size_t)blockIdx.x * H;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < H; i += 256) {
        float v = bf16_to_float(h[base + i]);
        if (delta) v = bf16_round(v + bf16_to_float(delta[base + i]));
        if (h_out) h_out[base + i] = float_to_bf16(v);
        ss += v * v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) tot += red[k];
    const float r = rsqrtf(tot / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += 256) {
        float v = bf16_to_float(h[base + i]);
        if (delta) v = bf16_round(v + bf16_to_float(delta[base + i]));
        if (flavor == 0) {
            const float n = bf16_round(v * r);
            y[base + i] = float_to_bf16(bf16_to_float(w[i]) * n);
        } else {
            y[base + i] = float_to_bf16(__fmul_rn(__fmul_rn(v, r), __fadd_rn(1.0f, bf16_to_float(w[i]))));
        }
    }
}

// q [T, nh*D] rotated in place; k rotated and v copied into the caches [kvh][max_ctx][D] at positions[t]
__global__ void rope_kv_kernel(uint16_t* q, const uint16_t* k, const uint16_t* v, const long long* positions,
                               const float* inv_freq, uint16_t* k_cache, uint16_t* v_cache, int T, int nh, int nkv,
                               int D, int max_ctx) {
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
        uint16_t* dst = is_q ? q + ((size_t)t * nh + head) * D
                             : k_cache + ((size_t)(head - nh) * max_ctx + (size_t)pos) * D;
        dst[d] = float_to_bf16(o1);
        dst[d + half] = float_to_bf16(o2);
    } else {
        const int hv = head - nh - nkv;
        const uint16_t* src = v + ((size_t)t * nkv + hv) * D;
        uint16_t* dst = v_cache + ((size_t)hv * max_ctx + (size_t)pos) * D;
        dst[d] = src[d];
        dst[d + half] = src[d + half];
    }
}

// out = bf16( bf16(act(g)) * u ); act 0 = SiLU, act 1 = GELU with the tanh approximation
__global__ void swiglu_kernel(const uint16_t* g, const uint16_t* u, uint16_t* out, long long n, int act) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float x = bf16_to_float(g[i]);
    float a;
    if (act == 0) {
        a = x / (1.0f + expf(-x));
    } else {
        const float kBeta = 0.7978845608028654f, kKappa = 0.044715f;   // sqrt(2/pi)
        const float inner = kBeta * (x + kKappa * (x * x * x));
        a = 0.5f * x * (1.0f + tanhf(inner));
    }
    out[i] = float_to_bf16(bf16_round(a) * bf16_to_float(u[i]));
}

}  // namespace cb
