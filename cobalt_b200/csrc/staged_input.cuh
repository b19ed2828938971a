// Element-wise steps of a decoder block that sit between two compressed linears, written once so that the
// stand-alone kernels (glue_kernels.cuh) and the decode GEMV's activation staging (gemv_kernel.cuh) compute
// them with the same operations in the same order and therefore agree bit for bit:
//
//   * gated activation   out = bf16( bf16(act(g)) * u ), act = SiLU or tanh-GELU
//                        (src/cobaltkernel/ref_llama.py:139-143, src/cobaltkernel/ref_gemma3.py:272-279);
//   * residual + RMSNorm h' = bf16(h + delta'), y = norm(h') with the Llama rounding (w * bf16(h' * r)) or the Gemma
//                        one (bf16(h' * r * (1 + w))), delta' = delta or Gemma's normalised branch
//                        (src/cobaltkernel/ref_llama.py:82-86, src/cobaltkernel/ref_gemma3.py:138-143, 262-270).
//
// Sum of squares of a row, the one order-dependent quantity: the row is cut into 16-byte chunks of 8 values; a
// chunk's squares are added left to right with fused multiply-adds; 32 consecutive chunks are combined by an XOR
// butterfly over a warp; the warp totals are added in ascending order.  Rows must therefore hold a multiple of
// 256 values on this path.
#pragma once
#include "common.cuh"

namespace cb {

__device__ __forceinline__ float bf16_round(float f) { return bf16_to_float(float_to_bf16(f)); }

// ---- partial sums of a row-parallel layer exchanged over peer memory (layout shared by the GEMV's pushing epilogue,
// its summing activation staging and the stand-alone kernels in glue_kernels.cuh).  Every rank owns one buffer:
//   [0, stride)                              staging area of the copy-based all-reduce
//   (1 + s * world + r) * stride             row r (= the partial of rank r) of slot s, s = epoch & 1
//   flags_off + 4 * r                        epoch of the last complete partial received from rank r
//   flags_off + 4 * PEER_EPOCH_INDEX         epoch of the last all-reduce this rank started
constexpr int PEER_MAX_RANKS = 8;
constexpr int PEER_EPOCH_INDEX = 16;
__device__ __forceinline__ float4 ld_sys_f4(const float* p) {
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// waits (bounded, about a second) until flags[0 .. world) have all reached `epoch`; threads 0 .. world-1 poll, every
// thread of the CTA gets the verdict
__device__ __forceinline__ bool peer_wait_epoch(const uint32_t* flags, int world, uint32_t epoch) {
    bool good = true;
    if ((int)threadIdx.x < world) {
        good = false;
        for (uint32_t it = 0; it < (1u << 20); ++it) {
            if ((int32_t)(ld_acquire_sys_u32(flags + threadIdx.x) - epoch) >= 0) { good = true; break; }
            if (it > 1024) __nanosleep(128);
        }
    }
    return __syncthreads_and(good ? 1 : 0) != 0;
}
// 8 consecutive values of the sum over ranks (rank order, fp32), rounded to bf16 once
__device__ __forceinline__ uint4 peer_sum_chunk(const uint8_t* slot_row0, unsigned long long stride, int world, size_t first_float) {
    float s[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 1
    for (int q0 = 0; q0 < world; q0 += 4) {                            // four ranks' loads in flight at a time
        float4 v[4][2];
#pragma unroll
        for (int q = 0; q < 4; ++q)
            if (q0 + q < world) {
                const float* p = reinterpret_cast<const float*>(slot_row0 + (unsigned long long)(q0 + q) * stride) + first_float;
                v[q][0] = ld_sys_f4(p);
                v[q][1] = ld_sys_f4(p + 4);
            }
#pragma unroll
        for (int q = 0; q < 4; ++q)
            if (q0 + q < world) {
                s[0] += v[q][0].x; s[1] += v[q][0].y; s[2] += v[q][0].z; s[3] += v[q][0].w;
                s[4] += v[q][1].x; s[5] += v[q][1].y; s[6] += v[q][1].z; s[7] += v[q][1].w;
            }
    }
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) w[k] = (uint32_t)float_to_bf16(s[2 * k]) | ((uint32_t)float_to_bf16(s[2 * k + 1]) << 16);
    return make_uint4(w[0], w[1], w[2], w[3]);
}

__device__ __forceinline__ void chunk_to_floats(const uint4& c, float (&f)[8]) {
    const uint32_t w[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        f[2 * k] = __uint_as_float(w[k] << 16);
        f[2 * k + 1] = __uint_as_float(w[k] & 0xFFFF0000u);
    }
}
__device__ __forceinline__ uint4 floats_to_chunk(const float (&f)[8]) {      // rounds to bf16 (nearest even)
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) w[k] = (uint32_t)float_to_bf16(f[2 * k]) | ((uint32_t)float_to_bf16(f[2 * k + 1]) << 16);
    return make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ float chunk_sumsq(const float (&f)[8]) {
    float s = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) s = __fmaf_rn(f[k], f[k], s);
    return s;
}
__device__ __forceinline__ float warp_butterfly_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}
// total of `count` warp totals stored in ascending chunk order, then the norm factor
__device__ __forceinline__ float row_rsqrt(const float* warp_totals, int count, int H, float eps) {
    float tot = 0.0f;
    for (int k = 0; k < count; ++k) tot += warp_totals[k];
    return rsqrtf(tot / (float)H + eps);
}

// bf16( bf16(act(g)) * u ) as a float holding a bf16 value
__device__ __forceinline__ float glu_value(float g, float u, int act) {
    float a;
    if (act == 0) {
        a = g / (1.0f + expf(-g));
    } else {
        const float kBeta = 0.7978845608028654f, kKappa = 0.044715f;   // sqrt(2/pi)
        const float inner = kBeta * (g + kKappa * (g * g * g));
        a = 0.5f * g * (1.0f + tanhf(inner));
    }
    return bf16_round(bf16_round(a) * u);
}
__device__ __forceinline__ uint4 glu_chunk(const uint4& g, const uint4& u, int act) {
    float fg[8], fu[8], o[8];
    chunk_to_floats(g, fg);
    chunk_to_floats(u, fu);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = glu_value(fg[k], fu[k], act);
    return floats_to_chunk(o);
}

// Gemma's normalised branch: bf16( delta * r_branch * (1 + w_branch) )
__device__ __forceinline__ float branch_value(float d, float r_branch, float w_branch) {
    return bf16_round(__fmul_rn(__fmul_rn(d, r_branch), __fadd_rn(1.0f, w_branch)));
}
// bf16(h + delta')
__device__ __forceinline__ float joined_value(float h, float d) { return bf16_round(h + d); }
// the normalised output; flavor 0 = Llama, 1 = Gemma
__device__ __forceinline__ float normed_value(float v, float r, float w, int flavor) {
    if (flavor == 0) return bf16_round(w * bf16_round(v * r));
    return bf16_round(__fmul_rn(__fmul_rn(v, r), __fadd_rn(1.0f, w)));
}

}  // namespace cb
