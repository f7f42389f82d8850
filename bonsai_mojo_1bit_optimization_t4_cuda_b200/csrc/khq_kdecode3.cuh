// khq_kdecode3.cuh -- thread-per-row decode of KHQ code words into tensor-core operand words
// (third-generation decode kernel).  Host-callable so that a CPU unit test can check every bit
// trick against a plain per-dim decode.
//
// K.  A row is 256 two-bit symbols (0: zero, 1: -c, 2: +c, 3: outlier) in 16 mask words plus, for
// the outliers in dim order, a 4-bit residual code stream (payload bytes 4..28) and a sign-bit
// stream (bytes 29..35, 1 = positive).  k3_word turns one mask word (16 dims) into eight fp16x2
// words of the ternary part t in {-1, 0, +1} (outliers carry their sign) and eight fp16x2 words h
// with h = t * (1024 + code): the signed residual code is then t * -1024 + h, one exact fused
// multiply-add.  Order of the 16 dims inside the eight words ("operand order"):
//     word j < 4 : dims (4j, 4j + 2)              even dims first,
//     word j >= 4: dims (4(j-4) + 1, 4(j-4) + 3)  then the odd ones,
// i.e. operand index 2j + e of a word holds dim K3_DIM_OF[2j + e].
// Everything is done on whole registers: the symbols of a word, one per nibble, are byte-permute
// selectors into the table {0, -1, +1, +1}; an outlier's ordinal inside the word comes from a
// nibble-wise prefix sum (one multiply) and is the permute selector that fetches its code and
// sign from the next eight stream entries; selector bit 3 (sign-replicate mode on a byte whose
// top bit is clear) yields zero for the dims that are not outliers.
// Words with more than eight outliers, and rows that run past the 50 entries the format holds
// (the reference decodes those symbols as -c, code 0), take a per-dim path.
//
// V.  A row is 64 twelve-bit fields (7 low bits of the VQ code, 1 bit choosing the dim-3
// centroid, 4-bit dim-3 residual) packed eight to three words, plus the codes' high bits in
// words 24 and 25.  v3_fields unpacks the eight fields of one three-word group.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define KHQ3_HD __host__ __device__ __forceinline__
#else
#define KHQ3_HD inline
#endif

namespace khq3 {

KHQ3_HD uint32_t k3_prmt(uint32_t x, uint32_t y, uint32_t s) {
#if defined(__CUDA_ARCH__)
    // the instruction itself, not __byte_perm: selector bit 3 (replicate the selected byte's top
    // bit) is part of the decode
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(x), "r"(y), "r"(s));
    return r;
#else
    // bytes 0..3 of x are sources 0..3, bytes of y are 4..7; selector bit 3 replicates the
    // selected byte's top bit over the whole output byte
    const uint64_t v = ((uint64_t)y << 32) | x;
    uint32_t r = 0;
    for (int i = 0; i < 4; ++i) {
        const uint32_t sel = (s >> (4 * i)) & 0xFu;
        uint32_t b = (uint32_t)((v >> (8 * (sel & 7u))) & 0xFFu);
        if (sel & 8u) b = (b & 0x80u) ? 0xFFu : 0x00u;
        r |= b << (8 * i);
    }
    return r;
#endif
}
KHQ3_HD uint32_t k3_funnel_r(uint32_t lo, uint32_t hi, uint32_t sh) {
#if defined(__CUDA_ARCH__)
    return __funnelshift_r(lo, hi, sh);
#else
    sh &= 31;
    return sh ? ((lo >> sh) | (hi << (32 - sh))) : lo;
#endif
}
KHQ3_HD uint32_t k3_popc(uint32_t x) {
#if defined(__CUDA_ARCH__)
    return (uint32_t)__popc(x);
#else
    return (uint32_t)__builtin_popcount(x);
#endif
}

// dim (inside its mask word) held at operand index i of the word
KHQ3_HD int k3_dim_of(int i) { return i < 8 ? 2 * i : 2 * (i - 8) + 1; }
// operand index (inside its word) of dim d
KHQ3_HD int k3_index_of(int d) { return (d & 1) ? 8 + (d >> 1) : (d >> 1); }

// Number of outlier symbols in a mask word.
KHQ3_HD uint32_t k3_count(uint32_t w) { return k3_popc(w & (w >> 1) & 0x55555555u); }

// Per-dim path of k3_word: any count, any ordinal.  Rare: kept out of line on the device.
#if defined(__CUDACC__)
__host__ __device__ __noinline__
#else
inline
#endif
void k3_word_slow(uint32_t w, uint32_t ob, const uint32_t* kp, uint32_t (&t2)[8], uint32_t (&h2)[8]) {
    const unsigned char* pb = reinterpret_cast<const unsigned char*>(kp);
#pragma unroll
    for (int j = 0; j < 8; ++j) t2[j] = h2[j] = 0u;
    uint32_t ord = ob;
#pragma unroll 1
    for (int d = 0; d < 16; ++d) {
        const uint32_t sym = (w >> (2 * d)) & 3u;
        uint32_t t = 0u, h = 0u;  // fp16 bit patterns
        if (sym == 1u) {
            t = 0xBC00u;
            h = 0xE400u;
        } else if (sym == 2u) {
            t = 0x3C00u;
            h = 0x6400u;
        } else if (sym == 3u) {
            uint32_t code = 0u, pos = 0u;
            if (ord < 50u) {
                code = (pb[4 + (ord >> 1)] >> (4 * (ord & 1u))) & 15u;
                pos = (pb[29 + (ord >> 3)] >> (ord & 7u)) & 1u;
            }
            t = pos ? 0x3C00u : 0xBC00u;
            h = (pos ? 0x6400u : 0xE400u) | code;
            ++ord;
        }
        const int i = k3_index_of(d);
        const int sh = 16 * (i & 1);
        // static word index for the register arrays: select with a switch-free loop
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (j == (i >> 1)) {
                t2[j] |= t << sh;
                h2[j] |= h << sh;
            }
    }
}

// Decode mask word `w`, whose first outlier (if any) has ordinal `ob` in its row; `kp` = the
// row's ten payload words.  Returns the number of outliers of the word.
KHQ3_HD uint32_t k3_word(uint32_t w, uint32_t ob, const uint32_t* kp, uint32_t (&t2)[8], uint32_t (&h2)[8]) {
    const uint32_t E = w & 0x33333333u, O = (w >> 2) & 0x33333333u;  // even / odd symbols, one per nibble
    const uint32_t e3 = E & (E >> 1) & 0x11111111u, o3 = O & (O >> 1) & 0x11111111u;
    const uint32_t cnt = k3_popc(e3 | (o3 << 1));
    if (cnt > 8u || ob + cnt > 50u) {
        uint32_t ts[8], hs[8];  // only these have their address taken: t2 / h2 stay in registers
        k3_word_slow(w, ob, kp, ts, hs);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            t2[j] = ts[j];
            h2[j] = hs[j];
        }
        return cnt;
    }
    uint32_t g[4] = {0u, 0u, 0u, 0u};  // per dim: code | negative << 4, zero off the outliers
    if (cnt != 0u) {
        // ordinal of every dim inside the word: nibble-wise prefix sums (at most 8, no carries)
        const uint32_t incE = e3 * 0x11111111u, incO = o3 * 0x11111111u;
        const uint32_t exO = incO - o3;
        const uint32_t ordE = (incE - e3) + exO, ordO = incE + exO;
        const uint32_t selE = ordE | ((e3 ^ 0x11111111u) << 3), selO = ordO | ((o3 ^ 0x11111111u) << 3);
        // the next eight stream entries, one per byte: code | negative << 4
        const uint32_t cbit = 32u + 4u * ob;
        const uint32_t cw = k3_funnel_r(kp[cbit >> 5], kp[(cbit >> 5) + 1u], cbit & 31u);
        const uint32_t sbit = 232u + ob;
        const uint32_t ng = ~k3_funnel_r(kp[sbit >> 5], kp[(sbit >> 5) + 1u], sbit & 31u);
        const uint32_t lo4 = cw & 0x0F0F0F0Fu, hi4 = (cw >> 4) & 0x0F0F0F0Fu;
        const uint32_t a = k3_prmt(lo4, hi4, 0x5140u) | (((ng & 0xFu) * 0x02040810u) & 0x10101010u);
        const uint32_t b = k3_prmt(lo4, hi4, 0x7362u) | ((((ng >> 4) & 0xFu) * 0x02040810u) & 0x10101010u);
        g[0] = k3_prmt(a, b, selE);
        g[1] = k3_prmt(a, b, selE >> 16);
        g[2] = k3_prmt(a, b, selO);
        g[3] = k3_prmt(a, b, selO >> 16);
    }
    const uint32_t lut = 0x3C3CBC00u;  // fp16 high bytes of 0, -1, +1, +1
    const uint32_t t[4] = {k3_prmt(lut, 0u, E), k3_prmt(lut, 0u, E >> 16), k3_prmt(lut, 0u, O), k3_prmt(lut, 0u, O >> 16)};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const uint32_t tq = t[q] ^ ((g[q] & 0x10101010u) << 3);   // negative outliers: 0x3C -> 0xBC
        const uint32_t hq = tq + (tq & 0x04040404u) * 10u;         // +-1 -> +-1024: 0x3C -> 0x64, 0xBC -> 0xE4
        const uint32_t gc = g[q] & 0x0F0F0F0Fu;
        t2[2 * q] = k3_prmt(tq, 0u, 0x1404u);
        t2[2 * q + 1] = k3_prmt(tq, 0u, 0x3424u);
        h2[2 * q] = k3_prmt(hq, gc, 0x1504u);
        h2[2 * q + 1] = k3_prmt(hq, gc, 0x3726u);
    }
    return cnt;
}

// The eight 12-bit fields of one three-word group of a V payload row.
KHQ3_HD void v3_fields(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t (&f)[8]) {
    f[0] = w0 & 0xFFFu;
    f[1] = (w0 >> 12) & 0xFFFu;
    f[2] = k3_funnel_r(w0, w1, 24) & 0xFFFu;
    f[3] = (w1 >> 4) & 0xFFFu;
    f[4] = (w1 >> 16) & 0xFFFu;
    f[5] = k3_funnel_r(w1, w2, 28) & 0xFFFu;
    f[6] = (w2 >> 8) & 0xFFFu;
    f[7] = w2 >> 20;
}

}  // namespace khq3
