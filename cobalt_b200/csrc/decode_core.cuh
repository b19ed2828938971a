// Lane-level decoder shared by the GEMV and GEMM kernels: occupancy bitmask + packed
// survivor codes -> dense bf16 weights, two per 32-bit register.
//
// The code compiles both as CUDA device code and as plain host C++ (define CB_HOST_ONLY);
// the host build exists so that the bit manipulation can be checked on a CPU.
//
// What it has to reproduce (reference: sinq/sparse_quant.py:1657-1681 followed by the cast in
// benchmarks/benchmark_suite.py:1211-1213):
//     W[k][j] = bf16_rne( fp32(q - z) * fp32(s) * fp32(col_scale[j]) ) * keep[k][j]
// with s, z the fp16 scale and zero point of the 128-wide group.
//
// Fast path (no column scale, zero point an integer in [0, 2^bits)):
//   * a 256-entry table indexed by one mask byte yields two byte-permute selectors that spread
//     the <= 8 survivor nibbles of those 8 positions to 8 dense byte slots; pruned slots pick a
//     byte that holds the zero point, so they decode to exactly 0;
//   * a dense code c becomes the bf16 pattern 0x4300|c (= 128 + c), two per register;
//   * d = (128+c) - (128+z) is exact; with s = s_hi + s_lo (top 8 / low 3 significand bits, both
//     exact in bf16), fma(d, s_hi, d*s_lo) rounds the exact product d*s once to bf16, which is
//     the reference value bit for bit (|d| < 16, so d*s_lo and d*s_hi are exact).
// Slow path (anything else): the fp32 sequence above, literally, one position at a time.
#pragma once
#include <stdint.h>

#if defined(CB_HOST_ONLY)
#define CB_HD inline
#define CB_DEVICE_CODE 0
#include <cmath>
#include <cstring>
#else
#define CB_HD __host__ __device__ __forceinline__
#if defined(__CUDA_ARCH__)
#define CB_DEVICE_CODE 1
#else
#define CB_DEVICE_CODE 0
#endif
#include <cmath>
#include <cstring>
#endif

namespace cb {

// ----------------------------------------------------------------------------- bit helpers
CB_HD uint32_t f2u(float f) {
#if CB_DEVICE_CODE
    return __float_as_uint(f);
#else
    uint32_t u; memcpy(&u, &f, 4); return u;
#endif
}
CB_HD float u2f(uint32_t u) {
#if CB_DEVICE_CODE
    return __uint_as_float(u);
#else
    float f; memcpy(&f, &u, 4); return f;
#endif
}

// byte permute with the semantics of PTX prmt.b32 (default mode), selector nibble bit 3 = replicate sign
CB_HD uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
#if CB_DEVICE_CODE
    uint32_t d;                                   // the intrinsic would mask the selector to 3 bits per nibble
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
#else
    uint64_t src = ((uint64_t)b << 32) | a;
    uint32_t out = 0;
    for (int i = 0; i < 4; ++i) {
        uint32_t s = (sel >> (4 * i)) & 0xF;
        uint32_t byte = (uint32_t)(src >> (8 * (s & 7))) & 0xFF;
        if (s & 8) byte = (byte & 0x80) ? 0xFF : 0x00;
        out |= byte << (8 * i);
    }
    return out;
#endif
}
CB_HD int popc(uint32_t x) {
#if CB_DEVICE_CODE
    return __popc(x);
#else
    int c = 0; while (x) { x &= x - 1; ++c; } return c;
#endif
}
// (a & b) | c in one instruction
CB_HD uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
#if CB_DEVICE_CODE
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
#else
    return (a & b) | c;
#endif
}
// low 32 bits of (hi:lo) >> (sh & 31)
CB_HD uint32_t funnel_r(uint32_t lo, uint32_t hi, uint32_t sh) {
#if CB_DEVICE_CODE
    return __funnelshift_r(lo, hi, sh);
#else
    sh &= 31; return sh ? (lo >> sh) | (hi << (32 - sh)) : lo;
#endif
}
// low 32 bits of (hi:lo) >> min(sh, 32)
CB_HD uint32_t funnel_rc(uint32_t lo, uint32_t hi, uint32_t sh) {
#if CB_DEVICE_CODE
    return __funnelshift_rc(lo, hi, sh);
#else
    if (sh >= 32) return hi; return sh ? (lo >> sh) | (hi << (32 - sh)) : lo;
#endif
}

// ----------------------------------------------------------------------------- fp16 / bf16 scalars
CB_HD float half_bits_to_float(uint32_t h) {
#if CB_DEVICE_CODE
    float f;
    asm("{\n\t.reg .b16 t;\n\tcvt.u16.u32 t, %1;\n\tcvt.f32.f16 %0, t;\n\t}" : "=f"(f) : "r"(h & 0xFFFFu));
    return f;
#endif
    h &= 0xFFFFu;
    uint32_t sign = (h & 0x8000u) << 16, e = (h >> 10) & 0x1Fu, m = h & 0x3FFu;
    if (e == 0) {
        float v = (float)m * 5.9604644775390625e-08f;        // m * 2^-24, exact
        return u2f(f2u(v) | sign);
    }
    if (e == 31) return u2f(sign | 0x7F800000u | (m << 13));
    return u2f(sign | ((e + 112u) << 23) | (m << 13));
}
// fp32 -> bf16 bits, round to nearest even (NaN kept quiet)
CB_HD uint32_t float_to_bf16_bits(float f) {
    uint32_t u = f2u(f);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (u >> 16) | 0x40u;
    return (u + 0x7FFFu + ((u >> 16) & 1u)) >> 16;
}
CB_HD float bf16_bits_to_float(uint32_t b) { return u2f((b & 0xFFFFu) << 16); }

// packed bf16x2 arithmetic on raw registers
#if CB_DEVICE_CODE
__device__ __forceinline__ uint32_t bf2_sub(uint32_t a, uint32_t b) {
    uint32_t d; asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d;
}
__device__ __forceinline__ uint32_t bf2_add(uint32_t a, uint32_t b) {
    uint32_t d; asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d;
}
__device__ __forceinline__ uint32_t bf2_mul(uint32_t a, uint32_t b) {
    uint32_t d; asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d;
}
__device__ __forceinline__ uint32_t bf2_fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d; asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d;
}
#else
inline uint32_t bf16_round_double(double v) {            // one RNE rounding of a double to bf16
    float f = (float)v;
    if ((double)f != v) {                                 // round-to-odd into fp32 first, then RNE to bf16
        if (std::fabs((double)f) > std::fabs(v)) f = std::nextafterf(f, 0.0f);
        f = u2f(f2u(f) | 1u);
    }
    return float_to_bf16_bits(f);
}
inline uint32_t bf2_sub(uint32_t a, uint32_t b) {
    uint32_t lo = bf16_round_double((double)bf16_bits_to_float(a) - (double)bf16_bits_to_float(b));
    uint32_t hi = bf16_round_double((double)bf16_bits_to_float(a >> 16) - (double)bf16_bits_to_float(b >> 16));
    return lo | (hi << 16);
}
inline uint32_t bf2_add(uint32_t a, uint32_t b) {
    uint32_t lo = bf16_round_double((double)bf16_bits_to_float(a) + (double)bf16_bits_to_float(b));
    uint32_t hi = bf16_round_double((double)bf16_bits_to_float(a >> 16) + (double)bf16_bits_to_float(b >> 16));
    return lo | (hi << 16);
}
inline uint32_t bf2_mul(uint32_t a, uint32_t b) {
    uint32_t lo = bf16_round_double((double)bf16_bits_to_float(a) * (double)bf16_bits_to_float(b));
    uint32_t hi = bf16_round_double((double)bf16_bits_to_float(a >> 16) * (double)bf16_bits_to_float(b >> 16));
    return lo | (hi << 16);
}
inline uint32_t bf2_fma(uint32_t a, uint32_t b, uint32_t c) {
    double l = (double)bf16_bits_to_float(a) * (double)bf16_bits_to_float(b) + (double)bf16_bits_to_float(c);
    double h = (double)bf16_bits_to_float(a >> 16) * (double)bf16_bits_to_float(b >> 16) +
               (double)bf16_bits_to_float(c >> 16);
    return bf16_round_double(l) | (bf16_round_double(h) << 16);
}
#endif

// exact fp32 reference sequence for one weight (keep applied by the caller)
CB_HD float dequant_fp32(float code, float z, float s, float cs) {
#if CB_DEVICE_CODE
    return __fmul_rn(__fmul_rn(__fsub_rn(code, z), s), cs);
#else
    volatile float d = code - z; volatile float p = d * s; volatile float r = p * cs; return r;
#endif
}

// ----------------------------------------------------------------------------- expansion table
// One entry per mask byte: .x spreads positions 0..3, .y positions 4..7, each into the byte
// order [p0, p2, p1, p3] so that bytes (0,2) and (1,3) form natural column pairs.
// Source bytes for prmt(lo, hi, sel): lo = window bits 0..31 (ranks 0,2,4,6 in the low nibble
// of bytes 0..3), hi = window >> 4 (ranks 1,3,5,7).  Pruned positions select source 7 (byte 3
// of hi), into which the caller injects the zero point unless all 8 positions are kept.
constexpr int LUT_ENTRIES = 256;
constexpr int LUT_COPIES = 16;          // shared-memory replicas, one bank pair per lane of a half warp

struct LutEntry { uint32_t x, y; };

constexpr void build_expand_lut(LutEntry* lut /*[256]*/) {
    for (int mb = 0; mb < 256; ++mb) {
        uint32_t s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        int rank = 0;
        for (int p = 0; p < 8; ++p) {
            if ((mb >> p) & 1) { s[p] = (rank & 1) ? 4u + (uint32_t)(rank >> 1) : (uint32_t)(rank >> 1); ++rank; }
            else s[p] = 7u;
        }
        // upper halves (ignored by prmt): .x = selector that builds the high view {hi.b0, hi.b1, hi.b2, z or hi.b3},
        // .y = window advance in bits (4 per survivor)
        const uint32_t self = (rank == 8) ? 0x3210u : 0x4210u;
        lut[mb].x = (s[0] | (s[2] << 4) | (s[1] << 8) | (s[3] << 12)) | (self << 16);
        lut[mb].y = (s[4] | (s[6] << 4) | (s[5] << 8) | (s[7] << 12)) | ((uint32_t)(4 * rank) << 16);
    }
}

struct LutTable { LutEntry e[LUT_ENTRIES]; };
constexpr LutTable make_expand_lut() {
    LutTable t{};
    build_expand_lut(t.e);
    return t;
}

// ----------------------------------------------------------------------------- per-segment constants
struct SegParams {
    float s, z;            // fp32 values of the stored fp16 scale / zero
    uint32_t zq;           // zero point as an integer (fast path)
    uint32_t zb24;         // zero point << 24 (fast path)
    uint32_t zb2;          // bf16x2 {-(128+z), -(128+z)}: added, so that no per-use negation is needed
    uint32_t shi2, slo2;   // bf16x2 {s_hi, s_hi}, {s_lo, s_lo}
    bool fast;
};

CB_HD SegParams make_seg_params(uint32_t sz_bits, int bits, bool has_col_scale) {
    SegParams p;
    p.s = half_bits_to_float(sz_bits & 0xFFFFu);
    p.z = half_bits_to_float(sz_bits >> 16);
    float top = (float)((1 << bits) - 1);
    int zi = (int)p.z;                                     // only used when the test below holds
    bool z_ok = (p.z >= 0.0f) && (p.z <= top) && ((float)zi == p.z);
    bool s_ok = (f2u(p.s) & 0x7F800000u) != 0x7F800000u;   // finite
    p.fast = z_ok && s_ok && !has_col_scale;
    uint32_t zq = p.fast ? (uint32_t)zi : 0u;
    p.zq = zq;
    p.zb24 = zq << 24;
    uint32_t zb = 0xC300u | zq;                            // sign bit set
    p.zb2 = zb | (zb << 16);
    uint32_t su = f2u(p.s);
    uint32_t hi = su & 0xFFFF0000u;
    float lo = p.s - u2f(hi);                              // exact: at most 3 significant bits
    uint32_t hb = hi >> 16, lb = f2u(lo) >> 16;
    p.shi2 = hb | (hb << 16);
    p.slo2 = lb | (lb << 16);
    return p;
}

// bf16x2 {128+c0, 128+c1} -> bf16x2 weights
CB_HD uint32_t dq_pair(uint32_t e, const SegParams& p) {
    uint32_t d = bf2_add(e, p.zb2);
    uint32_t t = bf2_mul(d, p.slo2);
    return bf2_fma(d, p.shi2, t);
}

// ----------------------------------------------------------------------------- 32 positions
// m        mask word (bit b = column b of this 32-column word)
// w0..w3   nibble stream of this word's survivors, already aligned so that the first survivor
//          is in bits 0..3 of w0 (up to 128 bits are consumed)
// lut      expansion table as seen by this lane; entry mb lives at lut[mb * LUT_STRIDE]
// cs       fp32 column scales of these 32 columns (slow path only; may be null = all ones)
// out[i]   bf16x2 weights of columns (2i, 2i+1)
template <int LUT_STRIDE>
CB_HD void decode32(uint32_t m, uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3, const SegParams& p,
                    const LutEntry* lut, const float* cs, uint32_t out[16]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t mb = (m >> (8 * i)) & 0xFFu;
        const LutEntry e = lut[mb * LUT_STRIDE];
        const uint32_t lo = w0;
        uint32_t hi = w0 >> 4;
        if (p.fast) {
            if (mb != 0xFFu) hi = (hi & 0x00FFFFFFu) | p.zb24;
            const uint32_t d0 = prmt(lo, hi, e.x), d1 = prmt(lo, hi, e.y);
            out[4 * i + 0] = dq_pair((d0 & 0x000F000Fu) | 0x43004300u, p);
            out[4 * i + 1] = dq_pair(((d0 >> 8) & 0x000F000Fu) | 0x43004300u, p);
            out[4 * i + 2] = dq_pair((d1 & 0x000F000Fu) | 0x43004300u, p);
            out[4 * i + 3] = dq_pair(((d1 >> 8) & 0x000F000Fu) | 0x43004300u, p);
        } else {
            const uint32_t d0 = prmt(lo, hi, e.x), d1 = prmt(lo, hi, e.y);
            // byte slot of position q within d0/d1: [p0, p2, p1, p3]
#pragma unroll
            for (int pr = 0; pr < 4; ++pr) {                 // pair pr = positions (2pr, 2pr+1) of this byte
                const uint32_t d = (pr < 2) ? d0 : d1;
                const int slot0 = (pr & 1) ? 1 : 0;          // bytes (0,2) for even pair, (1,3) for odd pair
                uint32_t packed = 0;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int pos = 8 * i + 2 * pr + h;
                    const float code = (float)((d >> (8 * (slot0 + 2 * h))) & 0xFu);
                    const float keepf = (float)((m >> pos) & 1u);
                    const float c = cs ? cs[pos] : 1.0f;
                    const float wv = dequant_fp32(code, p.z, p.s, c) * keepf;
                    packed |= float_to_bf16_bits(wv) << (16 * h);
                }
                out[4 * i + pr] = packed;
            }
        }
        const uint32_t amt = 4u * (uint32_t)popc(mb);
        if (i < 3) {
            w0 = funnel_rc(w0, w1, amt);
            if (i < 2) w1 = funnel_rc(w1, w2, amt);
            if (i < 1) w2 = funnel_rc(w2, w3, amt);
        }
        // words that later steps cannot reach are left stale on purpose
    }
}

// ----------------------------------------------------------------------------- 32 positions, fast segments only
// Same contract as decode32() for segments whose SegParams::fast is set, with the special cases
// folded into the table: the upper half of entry .x is the selector that builds the high view
// (byte 3 = zero point unless all eight positions are kept), the upper half of .y the window
// advance in bits.  `lut(idx)` returns the table entry of mask byte idx.
// (Right shifts stay on the integer pipe: a multiply-high costs four issue cycles on the pipe
// that also executes the bf16x2 arithmetic, a shift two on a pipe of its own.)

// Two mask bytes (16 positions): `m16` holds them in its low 16 bits.  The window words are
// advanced past the survivors consumed.  out[i] = bf16x2 weights of columns (2i, 2i+1), i < 8.
template <class LutFn>
CB_HD void decode16_fast(uint32_t m16, uint32_t& w0, uint32_t& w1, uint32_t& w2, uint32_t& w3, const SegParams& p,
                         LutFn lut, uint32_t out[8]) {
    const LutEntry e0 = lut(prmt(m16, 0u, 0x4440u));
    const LutEntry e1 = lut(prmt(m16, 0u, 0x4441u));
    const uint32_t zreg = p.zb24 >> 24;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const LutEntry e = i ? e1 : e0;
        // high view: (w0 >> 4) with byte 3 replaced by the zero point unless all eight positions are kept
        const uint32_t hi = prmt(w0 >> 4, zreg, e.x >> 16);
        const uint32_t d0 = prmt(w0, hi, e.x), d1 = prmt(w0, hi, e.y);
        out[4 * i + 0] = dq_pair(and_or(d0, 0x000F000Fu, 0x43004300u), p);
        out[4 * i + 1] = dq_pair(and_or(d0 >> 8, 0x000F000Fu, 0x43004300u), p);
        out[4 * i + 2] = dq_pair(and_or(d1, 0x000F000Fu, 0x43004300u), p);
        out[4 * i + 3] = dq_pair(and_or(d1 >> 8, 0x000F000Fu, 0x43004300u), p);
        const uint32_t amt = e.y >> 16;
        w0 = funnel_rc(w0, w1, amt);
        w1 = funnel_rc(w1, w2, amt);
        w2 = funnel_rc(w2, w3, amt);
    }
}

template <class LutFn>
CB_HD void decode32_fast(uint32_t m, uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3, const SegParams& p,
                         LutFn lut, uint32_t out[16]) {
    decode16_fast(m & 0xFFFFu, w0, w1, w2, w3, p, lut, out);
    decode16_fast(m >> 16, w0, w1, w2, w3, p, lut, out + 8);
}


// ----------------------------------------------------------------------------- 8 positions, any bit width
// One mask byte of a fast segment, decoded straight from the `BITS`-wide code stream (no re-pack to
// nibbles).  `w0` holds the codes of this byte's survivors from bit 0 upwards (8 * BITS bits are looked
// at).  code_view() turns them into a word whose byte k carries rank 2k in its low bits and whose copy
// shifted right by HI_SHIFT carries rank 2k+1 there; bits above the code width are junk and are masked
// off when the bf16 pattern is formed.
//   4 bit: the stream itself (nibbles);
//   3 bit: three shift-and-select steps spread the eight 3-bit fields to nibbles (bit 3 of each is junk);
//   2 bit: one byte permute puts ranks 0,2,4,6 into bits 0..1 of bytes 0..3 and ranks 1,3,5,7 into bits 2..3.
// selA / selB / self are the table fields of the mask byte (see Lut4), out[i] = bf16x2 weights of
// positions (2i, 2i+1).
struct Lut4 { uint32_t selA, selB, self, amt; };   // amt = BITS * number of survivors: window advance in bits

constexpr Lut4 make_lut4(const LutEntry& e, int bits) {
    return Lut4{e.x & 0xFFFFu, e.y & 0xFFFFu, e.x >> 16, ((e.y >> 16) / 4u) * (uint32_t)bits};
}

template <int BITS>
CB_HD uint32_t code_view(uint32_t w0) {
    if (BITS == 4) return w0;
    if (BITS == 2) return prmt(w0, w0 >> 4, 0x5140u);
    const uint32_t t = (w0 & 0x0000FFFFu) | ((w0 << 4) & 0xFFFF0000u);
    const uint32_t u = (t & 0x00FF00FFu) | ((t << 2) & 0xFF00FF00u);
    return (u & 0x0F0F0F0Fu) | ((u << 1) & 0xF0F0F0F0u);
}

template <int BITS>
CB_HD void decode8(uint32_t w0, uint32_t selA, uint32_t selB, uint32_t self, const SegParams& p, uint32_t out[4]) {
    constexpr uint32_t HI_SHIFT = BITS == 2 ? 2u : 4u;
    constexpr uint32_t CM = ((1u << BITS) - 1u) * 0x00010001u;
    const uint32_t v = code_view<BITS>(w0);
    const uint32_t hi = prmt(v >> HI_SHIFT, p.zq, self);      // byte 3 <- zero point unless all eight are kept
    const uint32_t d0 = prmt(v, hi, selA), d1 = prmt(v, hi, selB);
    out[0] = dq_pair(and_or(d0, CM, 0x43004300u), p);
    out[1] = dq_pair(and_or(d0 >> 8, CM, 0x43004300u), p);
    out[2] = dq_pair(and_or(d1, CM, 0x43004300u), p);
    out[3] = dq_pair(and_or(d1 >> 8, CM, 0x43004300u), p);
}

// Literal fp32 path for 32 positions of any segment (off-grid zero point, column scale): codes are read
// one at a time from the `BITS`-wide stream.  `stream` is a little-endian word stream, `bitpos` the bit
// offset of the first survivor of this word.  cs may be null.
template <class LoadWord>
CB_HD void decode32_slow(uint32_t m, LoadWord word_at, uint32_t bitpos, int bits, const SegParams& p, const float* cs,
                         uint32_t out[16]) {
    const uint32_t cmask = (1u << bits) - 1u;
    for (int i = 0; i < 16; ++i) {
        uint32_t packed = 0;
        for (int h = 0; h < 2; ++h) {
            const int pos = 2 * i + h;
            float wv = 0.0f;
            if ((m >> pos) & 1u) {
                const uint32_t wi = bitpos >> 5, sh = bitpos & 31u;
                uint32_t v = word_at(wi) >> sh;
                if (sh + (uint32_t)bits > 32u) v |= word_at(wi + 1) << (32u - sh);
                wv = dequant_fp32((float)(v & cmask), p.z, p.s, cs ? cs[pos] : 1.0f);
                bitpos += (uint32_t)bits;
            }
            packed |= float_to_bf16_bits(wv) << (16 * h);
        }
        out[i] = packed;
    }
}

// ----------------------------------------------------------------------------- 2/3-bit -> nibble
// 8 three-bit fields (bits 0..23) -> 8 nibbles
CB_HD uint32_t spread3(uint32_t x) {
    uint32_t t = (x & 0x00000FFFu) | ((x & 0x00FFF000u) << 4);
    uint32_t u = (t & 0x003F003Fu) | ((t & 0x0FC00FC0u) << 2);
    return (u & 0x07070707u) | ((u & 0x38383838u) << 1);
}
// 8 two-bit fields (bits 0..15) -> 8 nibbles
CB_HD uint32_t spread2(uint32_t x) {
    uint32_t t = x & 0xFFFFu;
    t = (t | (t << 8)) & 0x00FF00FFu;
    t = (t | (t << 4)) & 0x0F0F0F0Fu;
    return (t | (t << 2)) & 0x33333333u;
}

// generic b-bit field at bit position `bitpos` of a little-endian word stream
CB_HD uint32_t extract_code(const uint32_t* stream, uint32_t bitpos, int bits) {
    const uint32_t wi = bitpos >> 5, sh = bitpos & 31u;
    uint32_t v = stream[wi] >> sh;
    if (sh + (uint32_t)bits > 32u) v |= stream[wi + 1] << (32u - sh);
    return v & ((1u << bits) - 1u);
}

}  // namespace cb
