// CPU unit test of csrc/khq_kdecode.cuh: the register-level K decode against a plain per-dim
// decode of the same code words (symbols, residual nibbles, sign bits), including rows with more
// than 50 outlier symbols, which the format cannot hold and the reference decodes as -c.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>

#include "khq_kdecode.cuh"

static float half_bits_to_float(uint16_t h) {
    const int s = h >> 15, e = (h >> 10) & 31, m = h & 1023;
    float v = e == 0 ? std::ldexp((float)m, -24) : std::ldexp((float)(m + 1024), e - 25);
    return s ? -v : v;
}

int main() {
    using namespace khq;
    KdLutEntry lut[KD_LUT_ENTRIES];
    for (uint32_t f = 0; f < KD_LUT_ENTRIES; ++f) lut[f] = kd_make_lut_entry(f);
    std::mt19937 rng(1234);
    long checked = 0;
    for (int iter = 0; iter < 20000; ++iter) {
        const double p_out = (iter % 7 == 0) ? 0.35 : 0.11;  // some rows overflow 50 outliers
        uint32_t mask[16] = {0}, kp[10] = {0};
        int sym[256];
        for (int i = 0; i < 256; ++i) {
            const double u = (rng() & 0xFFFFFF) / double(0x1000000);
            sym[i] = u < p_out ? 3 : (u < p_out + 0.3 ? 0 : (u < p_out + 0.6 ? 1 : 2));
            mask[i / 16] |= (uint32_t)sym[i] << (2 * (i % 16));
        }
        uint8_t* pb = reinterpret_cast<uint8_t*>(kp);
        for (int b = 0; b < 40; ++b) pb[b] = (uint8_t)rng();
        pb[36] = 2; pb[37] = pb[38] = pb[39] = 0;
        // expected per dim
        int t_exp[256], r_exp[256], j = 0;
        for (int i = 0; i < 256; ++i) {
            t_exp[i] = sym[i] == 2 ? 1 : (sym[i] == 1 ? -1 : 0);
            r_exp[i] = 0;
            if (sym[i] == 3) {
                const bool ok = j < 50;
                const int sgn = (ok && ((pb[29 + j / 8] >> (j % 8)) & 1)) ? 1 : -1;
                const int code = ok ? ((pb[4 + j / 2] >> ((j % 2) * 4)) & 15) : 0;
                t_exp[i] = sgn;
                r_exp[i] = sgn * code;
                ++j;
            }
        }
        // register-level decode, one "thread" per 64-dim quarter
        uint32_t base = 0;
        for (int t = 0; t < 4; ++t) {
            const KdSigns sg = kd_signs(kp);
            uint32_t wbase = base;
            for (int wi = 0; wi < 4; ++wi) {
                const KdWord w = kd_word(mask[4 * t + wi]);
                for (int q = 0; q < 4; ++q) {
                    const KdStep r = kd_step(w, q, wbase + kd_prefix(w, q), kp, sg, lut);
                    const int d0 = 64 * t + 16 * wi + 4 * q;
                    const int dims[4] = {d0, d0 + 2, d0 + 1, d0 + 3};
                    const uint16_t th[4] = {(uint16_t)r.t0, (uint16_t)(r.t0 >> 16), (uint16_t)r.t1, (uint16_t)(r.t1 >> 16)};
                    const uint16_t hh[4] = {(uint16_t)r.h0, (uint16_t)(r.h0 >> 16), (uint16_t)r.h1, (uint16_t)(r.h1 >> 16)};
                    for (int k = 0; k < 4; ++k) {
                        const float tv = half_bits_to_float(th[k]);
                        const float res = tv * -1024.0f + half_bits_to_float(hh[k]);
                        if ((int)tv != t_exp[dims[k]] || (int)res != r_exp[dims[k]]) {
                            std::printf("MISMATCH iter %d dim %d: t %g (want %d) res %g (want %d)\n", iter, dims[k], tv,
                                        t_exp[dims[k]], res, r_exp[dims[k]]);
                            return 1;
                        }
                        ++checked;
                    }
                }
                wbase += kd_count(w);
            }
            for (int i = 64 * t; i < 64 * t + 64; ++i) base += sym[i] == 3;
            if (wbase != base) { std::printf("stream position drifted\n"); return 1; }
        }
    }
    std::printf("ok %ld dims\n", checked);
    return 0;
}
