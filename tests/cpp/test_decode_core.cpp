// CPU check of the lane-level decoder (cobalt_b200/csrc/decode_core.cuh built as host C++).
// Prints "OK" and exits 0 when every case matches the literal fp32 reference sequence.
#define CB_HOST_ONLY 1
#include "../../cobalt_b200/csrc/decode_core.cuh"
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>

using namespace cb;

static uint32_t float_to_half_bits(float f) {          // RNE, enough for test inputs
    uint32_t u = f2u(f), sign = (u >> 16) & 0x8000u;
    int e = (int)((u >> 23) & 0xFF) - 127 + 15;
    uint32_t m = u & 0x7FFFFFu;
    if (e >= 31) return sign | 0x7C00u;
    if (e <= 0) {
        if (e < -10) return sign;
        m |= 0x800000u;
        int sh = 14 - e;
        uint32_t r = m >> sh, rem = m & ((1u << sh) - 1), half = 1u << (sh - 1);
        if (rem > half || (rem == half && (r & 1))) ++r;
        return sign | r;
    }
    uint32_t r = (uint32_t)(e << 10) | (m >> 13), rem = m & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1))) ++r;
    return sign | r;
}

int main() {
    int fails = 0;
    // 1. the split-scale product is exact for every finite fp16 scale and every |d| < 16
    for (uint32_t hb = 0; hb < 0x7C00u; ++hb) {
        for (int sgn = 0; sgn < 2; ++sgn) {
            uint32_t sb = hb | (sgn ? 0x8000u : 0u);
            for (int z = 0; z < 16; z += 5) {
                SegParams p = make_seg_params(sb | (float_to_half_bits((float)z) << 16), 4, false);
                if (!p.fast) { ++fails; continue; }
                for (int c = 0; c < 16; ++c) {
                    uint32_t e = (0x4300u | c) | ((0x4300u | (15 - c)) << 16);
                    uint32_t w = dq_pair(e, p);
                    uint32_t r0 = float_to_bf16_bits(dequant_fp32((float)c, p.z, p.s, 1.0f));
                    uint32_t r1 = float_to_bf16_bits(dequant_fp32((float)(15 - c), p.z, p.s, 1.0f));
                    // +0 / -0 are the same weight
                    auto same = [](uint32_t a, uint32_t b) { return a == b || (((a | b) & 0x7FFFu) == 0); };
                    if (!same(w & 0xFFFFu, r0) || !same(w >> 16, r1)) {
                        if (fails < 10) printf("split-scale mismatch s=%04x z=%d c=%d got %08x want %04x %04x\n", sb, z, c, w, r0, r1);
                        ++fails;
                    }
                }
            }
        }
    }
    // 2. decode32 against a direct walk, fast and slow segments, bits 2/3/4, all densities
    std::vector<LutEntry> lut1(256);
    build_expand_lut(lut1.data());
    std::vector<LutEntry> lut(256 * LUT_COPIES);
    for (int i = 0; i < 256; ++i) for (int c = 0; c < LUT_COPIES; ++c) lut[i * LUT_COPIES + c] = lut1[i];
    std::mt19937 rng(1234);
    for (int iter = 0; iter < 20000; ++iter) {
        int bits = 2 + (iter % 3);
        int top = (1 << bits) - 1;
        double dens = (iter % 11) / 10.0;
        uint32_t m = 0;
        for (int b = 0; b < 32; ++b) if ((rng() % 1000) < dens * 1000) m |= 1u << b;
        if (iter % 97 == 0) m = 0xFFFFFFFFu;
        if (iter % 89 == 0) m = 0xFF00FF00u;
        int codes[32];
        uint32_t w[5] = {0, 0, 0, 0, 0};
        int r = 0;
        for (int b = 0; b < 32; ++b) {
            codes[b] = 0;
            if ((m >> b) & 1) { codes[b] = rng() % (top + 1); w[r / 8] |= (uint32_t)codes[b] << (4 * (r % 8)); ++r; }
        }
        for (int k = r; k < 32; ++k) w[k / 8] |= (rng() & 0xFu) << (4 * (k % 8));      // garbage after the survivors
        float s = ((rng() % 10000) / 10000.0f) * 0.01f + 0.0007f;
        float z;
        bool use_cs = false;
        switch (iter % 5) {
            case 0: z = (float)(rng() % (top + 1)); break;
            case 1: z = -(float)(rng() % 40); break;                      // negative: slow path
            case 2: z = (float)(top + 1 + rng() % 300); break;            // above the grid: slow path
            case 3: z = (float)(rng() % (top + 1)); use_cs = true; break; // column scale: slow path
            default: z = (float)(rng() % (top + 1)); s = -s; break;
        }
        uint32_t szb = float_to_half_bits(s) | (float_to_half_bits(z) << 16);
        SegParams p = make_seg_params(szb, bits, use_cs);
        float cs[32];
        for (int b = 0; b < 32; ++b) cs[b] = half_bits_to_float(float_to_half_bits(0.5f + (rng() % 1500) / 1000.0f));
        uint32_t out[16];
        decode32<LUT_COPIES>(m, w[0], w[1], w[2], w[3], p, lut.data() + (iter % LUT_COPIES), use_cs ? cs : nullptr, out);
        if (p.fast) {                                   // the fast variant must agree with the generic one
            uint32_t out2[16];
            const LutEntry* lp = lut.data() + (iter % LUT_COPIES);
            decode32_fast(m, w[0], w[1], w[2], w[3], p, [lp](uint32_t i) { return lp[i * LUT_COPIES]; }, out2);
            for (int k = 0; k < 16; ++k) if (out2[k] != out[k]) {
                if (fails < 10) printf("decode32_fast mismatch iter=%d k=%d m=%08x got %08x want %08x\n", iter, k, m, out2[k], out[k]);
                ++fails;
            }
        }
        for (int b = 0; b < 32; ++b) {
            uint32_t got = (out[b / 2] >> (16 * (b & 1))) & 0xFFFFu;
            float keepf = (float)((m >> b) & 1);
            uint32_t want = float_to_bf16_bits(dequant_fp32((float)codes[b], p.z, p.s, use_cs ? cs[b] : 1.0f) * keepf);
            bool same = got == want || (((got | want) & 0x7FFFu) == 0);
            if (!same) {
                if (fails < 10) printf("decode32 mismatch iter=%d bits=%d b=%d m=%08x fast=%d got %04x want %04x\n", iter, bits, b, m, (int)p.fast, got, want);
                ++fails;
            }
        }
    }
    // 3. field spreading
    for (int iter = 0; iter < 100000; ++iter) {
        uint32_t x = rng();
        uint32_t a = spread3(x & 0xFFFFFFu), b = spread2(x & 0xFFFFu);
        for (int i = 0; i < 8; ++i) {
            if (((a >> (4 * i)) & 0xF) != ((x >> (3 * i)) & 7)) ++fails;
            if (((b >> (4 * i)) & 0xF) != ((x >> (2 * i)) & 3)) ++fails;
        }
    }
    // 4. generic field extraction
    {
        std::vector<uint32_t> st(64);
        for (auto& v : st) v = rng();
        for (int bits = 2; bits <= 4; ++bits)
            for (uint32_t pos = 0; pos + bits <= 63 * 32; pos += bits) {
                uint32_t want = 0;
                for (int i = 0; i < bits; ++i) want |= ((st[(pos + i) >> 5] >> ((pos + i) & 31)) & 1u) << i;
                if (extract_code(st.data(), pos, bits) != want) ++fails;
            }
    }
    // 5. decode8 on the raw `bits`-wide stream (no nibble re-pack), every mask byte, and the literal slow path
    for (int bits = 2; bits <= 4; ++bits) {
        const int top = (1 << bits) - 1;
        for (int iter = 0; iter < 40000; ++iter) {
            const uint32_t mb = (iter < 256) ? (uint32_t)iter : (rng() & 0xFFu);
            int codes[8];
            uint64_t stream = 0;
            int r = 0;
            for (int b = 0; b < 8; ++b) {
                codes[b] = 0;
                if ((mb >> b) & 1) { codes[b] = rng() % (top + 1); stream |= (uint64_t)codes[b] << (bits * r); ++r; }
            }
            stream |= ((uint64_t)rng() << 32 | rng()) << (bits * r);                 // garbage after the survivors
            const float s = ((rng() % 10000) / 10000.0f) * 0.01f + 0.0007f;
            const float z = (float)(rng() % (top + 1));
            SegParams p = make_seg_params(float_to_half_bits((iter & 1) ? -s : s) | (float_to_half_bits(z) << 16), bits, false);
            if (!p.fast) { ++fails; continue; }
            const Lut4 e = make_lut4(lut1[mb], bits);
            if (e.amt != (uint32_t)(bits * r)) ++fails;
            uint32_t out[4];
            const uint32_t w0 = (uint32_t)stream;
            if (bits == 2) decode8<2>(w0, e.selA, e.selB, e.self, p, out);
            else if (bits == 3) decode8<3>(w0, e.selA, e.selB, e.self, p, out);
            else decode8<4>(w0, e.selA, e.selB, e.self, p, out);
            for (int b = 0; b < 8; ++b) {
                const uint32_t got = (out[b / 2] >> (16 * (b & 1))) & 0xFFFFu;
                const float keepf = (float)((mb >> b) & 1);
                const uint32_t want = float_to_bf16_bits(dequant_fp32((float)codes[b], p.z, p.s, 1.0f) * keepf);
                const bool same = got == want || (((got | want) & 0x7FFFu) == 0);
                if (!same) {
                    if (fails < 10) printf("decode8 mismatch bits=%d mb=%02x b=%d got %04x want %04x\n", bits, mb, b, got, want);
                    ++fails;
                }
            }
        }
        for (int iter = 0; iter < 4000; ++iter) {                                    // decode32_slow
            uint32_t m = rng() & rng();
            if (iter % 7 == 0) m = 0xFFFFFFFFu;
            std::vector<uint32_t> st(8, 0);
            const uint32_t start = rng() % 64;
            int codes[32];
            uint32_t bp = start;
            for (int b = 0; b < 32; ++b) {
                codes[b] = 0;
                if ((m >> b) & 1) {
                    codes[b] = rng() % (top + 1);
                    for (int i = 0; i < bits; ++i) if ((codes[b] >> i) & 1) st[(bp + i) >> 5] |= 1u << ((bp + i) & 31);
                    bp += bits;
                }
            }
            const float s = 0.003f, z = (iter & 1) ? -3.0f : 2.5f;
            SegParams p = make_seg_params(float_to_half_bits(s) | (float_to_half_bits(z) << 16), bits, false);
            uint32_t out[16];
            decode32_slow(m, [&](uint32_t i) { return st[i]; }, start, bits, p, nullptr, out);
            for (int b = 0; b < 32; ++b) {
                const uint32_t got = (out[b / 2] >> (16 * (b & 1))) & 0xFFFFu;
                const float keepf = (float)((m >> b) & 1);
                const uint32_t want = float_to_bf16_bits(dequant_fp32((float)codes[b], p.z, p.s, 1.0f) * keepf);
                if (!(got == want || (((got | want) & 0x7FFFu) == 0))) ++fails;
            }
        }
    }
    if (fails) { printf("FAILED: %d mismatches\n", fails); return 1; }
    printf("OK\n");
    return 0;
}
