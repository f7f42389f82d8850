// CPU unit test of csrc/khq_kdecode3.cuh: the register-level decode of one mask word (ternary
// fp16 pairs and sign-matched 1024 + code pairs, in operand order) and of the V payload's 12-bit
// fields against plain per-dim / per-patch decodes, including words with more than eight
// outliers and rows with more than 50 outlier symbols.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>

#include "khq_kdecode3.cuh"

int main() {
    using namespace khq3;
    std::mt19937 rng(4321);
    long checked = 0, slow_words = 0;
    for (int iter = 0; iter < 30000; ++iter) {
        const double p_out = (iter % 7 == 0) ? 0.35 : ((iter % 11 == 0) ? 0.7 : 0.11);
        uint32_t mask[16] = {0}, kp[10] = {0};
        int sym[256];
        for (int i = 0; i < 256; ++i) {
            const double u = (rng() & 0xFFFFFF) / double(0x1000000);
            sym[i] = u < p_out ? 3 : (u < p_out + 0.3 * (1 - p_out) ? 0 : (u < p_out + 0.65 * (1 - p_out) ? 1 : 2));
            mask[i / 16] |= (uint32_t)sym[i] << (2 * (i % 16));
        }
        unsigned char* pb = reinterpret_cast<unsigned char*>(kp);
        for (int b = 0; b < 40; ++b) pb[b] = (unsigned char)rng();
        int t_exp[256], c_exp[256], j = 0;
        for (int i = 0; i < 256; ++i) {
            t_exp[i] = sym[i] == 2 ? 1 : (sym[i] == 1 ? -1 : 0);
            c_exp[i] = 0;
            if (sym[i] == 3) {
                const bool ok = j < 50;
                const int sgn = (ok && ((pb[29 + j / 8] >> (j % 8)) & 1)) ? 1 : -1;
                const int code = ok ? ((pb[4 + j / 2] >> ((j % 2) * 4)) & 15) : 0;
                t_exp[i] = sgn;
                c_exp[i] = code;
                ++j;
            }
        }
        uint32_t ob = 0;
        for (int wi = 0; wi < 16; ++wi) {
            uint32_t t2[8], h2[8];
            const uint32_t cnt = k3_word(mask[wi], ob, kp, t2, h2);
            if (cnt != k3_count(mask[wi])) { printf("count mismatch\n"); return 1; }
            if (cnt > 8 || ob + cnt > 50) ++slow_words;
            for (int i = 0; i < 16; ++i) {
                const int d = 16 * wi + k3_dim_of(i);
                if (k3_index_of(k3_dim_of(i)) != i) { printf("index map broken\n"); return 1; }
                const uint32_t tb = (t2[i >> 1] >> (16 * (i & 1))) & 0xFFFFu;
                const uint32_t hb = (h2[i >> 1] >> (16 * (i & 1))) & 0xFFFFu;
                const uint32_t t_want = t_exp[d] > 0 ? 0x3C00u : (t_exp[d] < 0 ? 0xBC00u : 0u);
                const uint32_t h_want = t_exp[d] == 0 ? 0u : ((t_exp[d] > 0 ? 0x6400u : 0xE400u) | (uint32_t)c_exp[d]);
                if (tb != t_want || hb != h_want) {
                    printf("iter %d word %d index %d (dim %d): t %04x want %04x, h %04x want %04x (ob %u cnt %u)\n", iter, wi, i, d,
                           tb, t_want, hb, h_want, ob, cnt);
                    return 1;
                }
                ++checked;
            }
            ob += cnt;
        }
    }
    // V fields
    for (int iter = 0; iter < 20000; ++iter) {
        uint32_t f_exp[8], w[3] = {0, 0, 0}, f[8];
        unsigned long long lo = 0, hi = 0;  // 96 bits
        for (int p = 0; p < 8; ++p) {
            f_exp[p] = rng() & 0xFFFu;
            const int bit = 12 * p;
            for (int b = 0; b < 12; ++b)
                if ((f_exp[p] >> b) & 1u) {
                    const int pos = bit + b;
                    if (pos < 64) lo |= 1ull << pos; else hi |= 1ull << (pos - 64);
                }
        }
        w[0] = (uint32_t)lo; w[1] = (uint32_t)(lo >> 32); w[2] = (uint32_t)hi;
        v3_fields(w[0], w[1], w[2], f);
        for (int p = 0; p < 8; ++p)
            if (f[p] != f_exp[p]) { printf("field %d: %03x want %03x\n", p, f[p], f_exp[p]); return 1; }
    }
    printf("ok: %ld operand entries checked (%ld words on the per-dim path)\n", checked, slow_words);
    return 0;
}
