// Shared device-side definitions: matrix view, PTX wrappers (mbarrier, bulk copy, fences),
// bounded waits.  sm_100a only.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include "../../include/cobalt_b200.h"
#include "decode_core.cuh"

namespace cb {

constexpr int GROUP = 128;
constexpr int TILE_ROWS = 16;
constexpr int TILE_GROUPS = 4;
constexpr int MAX_GEMV_M = 16;

// scratch layout shared by the GEMV and GEMM entry points
constexpr size_t SCRATCH_STATUS_BYTES = 256;     // [0]: status word written by bounded waits
constexpr size_t SCRATCH_COUNTER_BYTES = 65536;  // arrival counters of either kernel; partial sums start behind them

// device-side copy of CobaltMat with derived sizes
struct MatView {
    const uint8_t* tiles;
    const uint32_t* tile_off;
    const uint16_t* col_scale;   // fp16 bits or null
    int K, N, bits, G, RB, CT;
    uint32_t max_tile_bytes;
};

__host__ inline MatView make_view(const CobaltMat* m) {
    MatView v;
    v.tiles = (const uint8_t*)m->tiles;
    v.tile_off = m->tile_off;
    v.col_scale = (const uint16_t*)m->col_scale;
    v.K = m->K; v.N = m->N; v.bits = m->bits;
    v.G = m->N / GROUP;
    v.RB = m->n_row_blocks; v.CT = m->n_col_tiles;
    v.max_tile_bytes = m->max_tile_bytes;
    return v;
}

__device__ __forceinline__ int tile_width(const MatView& w, int ct) {
    int rem = w.G - TILE_GROUPS * ct;
    return rem < TILE_GROUPS ? rem : TILE_GROUPS;
}

// expansion table, constant-initialised at compile time
__device__ const LutTable g_lut = make_expand_lut();

// status codes a kernel may leave in the scratch status word
enum : uint32_t {
    DEV_OK = 0,
    DEV_TIMEOUT_TILE = 1,      // GEMV: a weight tile never arrived
    DEV_TIMEOUT_FULL = 2,      // GEMM: operand stage never filled
    DEV_TIMEOUT_EMPTY = 3,     // GEMM: operand stage never drained
    DEV_TIMEOUT_ACC = 4,       // GEMM: accumulator never completed
    DEV_TIMEOUT_STAGE = 5,     // GEMM: compressed tile group never arrived
    DEV_TIMEOUT_PEER = 6,      // peer all-reduce: a peer never published its partial
    DEV_TIMEOUT_ATTN = 7,      // one-kernel decode attention: a chunk of the head group never published its statistics
};

// ----------------------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void fence_acq_rel_gpu() {
    asm volatile("fence.acq_rel.gpu;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Wait with an iteration limit: returns false (and records `code`) instead of spinning forever.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint32_t* status, uint32_t code) {
    for (uint32_t it = 0; it < (1u << 18); ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if (it > 64) __nanosleep(128);
    }
    if (status) atomicCAS(status, 0u, code);
    return false;
}
// 1-D bulk async copy global -> shared, completion counted on an mbarrier (bytes % 16 == 0)
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void sts32(uint32_t addr, uint32_t a) {
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(a) : "memory");
}

__device__ __forceinline__ float bf16_to_float(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }
__device__ __forceinline__ uint16_t float_to_bf16(float f) { return (uint16_t)float_to_bf16_bits(f); }

}  // namespace cb
