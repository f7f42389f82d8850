// khq_kdecode.cuh -- SIMD-within-a-register decode of KHQ K code words into fp16 operand pairs.
//
// A K row is 256 two-bit symbols (0: zero, 1: -c, 2: +c, 3: outlier) plus, for the outliers in
// dim order, a 4-bit residual code stream and a sign-bit stream.  The tensor-core decode kernel
// needs, for four consecutive dims at a time, two fp16 pairs of the ternary part
// t in {-1, 0, +1} (outliers carry their sign) and two fp16 pairs of the signed residual code
// sign*code in [-15, 15].  Everything here works on whole 32-bit registers with byte permutes:
//
//   E, O    the mask word's even / odd symbols, one per nibble          (per 16 dims)
//   X3      outlier flags of the word, byte q = flags of dims 4q..4q+3  (per 16 dims)
//   step q  byte q of E and O is a 4-nibble permute selector into the table {0, -1, +1, +1}
//           (as fp16 high bytes 0x00, 0xBC, 0x3C, 0x3C); the next <= 4 stream entries
//           (code | sign << 7, one per byte) are scattered to their dims by a permute whose
//           selector comes from a 52-entry table indexed by the four outlier flags; the sign bit
//           flips the high byte of negative outliers; 1024 + code is assembled next to the
//           ternary value so that one fused multiply-add (t * -1024 + h) yields sign*code exactly.
//
// Output dim order inside a step is [4q, 4q+2 | 4q+1, 4q+3]: pair 0 = dims (4q, 4q+2), pair 1 =
// dims (4q+1, 4q+3).  The helpers are host-callable so that a CPU unit test can check them.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define KHQ_HD __host__ __device__ __forceinline__
#else
#define KHQ_HD inline
#endif

namespace khq {

KHQ_HD uint32_t kd_prmt(uint32_t x, uint32_t y, uint32_t s) {
#if defined(__CUDA_ARCH__)
    return __byte_perm(x, y, s);
#else
    const uint64_t v = ((uint64_t)y << 32) | x;
    uint32_t r = 0;
    for (int i = 0; i < 4; ++i) r |= (uint32_t)((v >> (8 * ((s >> (4 * i)) & 7))) & 0xFF) << (8 * i);
    return r;
#endif
}
KHQ_HD uint32_t kd_funnel_r(uint32_t lo, uint32_t hi, uint32_t sh) {
#if defined(__CUDA_ARCH__)
    return __funnelshift_r(lo, hi, sh);
#else
    sh &= 31;
    return sh ? ((lo >> sh) | (hi << (32 - sh))) : lo;
#endif
}

// Scatter table entry for outlier-flag byte f (bit0: dim 4q, bit1: 4q+1, bit4: 4q+2, bit5: 4q+3).
//   x: bits 0..15 permute selector, bits 16..23 = 4*count, bits 24..31 = count
//   y: 0x80 in every output byte that belongs to an outlier dim
// Output byte order: [dim 4q, dim 4q+2, dim 4q+1, dim 4q+3].
struct KdLutEntry {
    uint32_t x, y;
};
constexpr int KD_LUT_ENTRIES = 0x34;

KHQ_HD KdLutEntry kd_make_lut_entry(uint32_t f) {
    const uint32_t flag[4] = {f & 1u, (f >> 1) & 1u, (f >> 4) & 1u, (f >> 5) & 1u};  // dims 0..3
    const int out_dim[4] = {0, 2, 1, 3};                                                // byte -> dim
    uint32_t sel = 0, ob = 0, n = 0;
    uint32_t ord[4];
    for (int d = 0; d < 4; ++d) {
        ord[d] = n;
        n += flag[d];
    }
    for (int b = 0; b < 4; ++b) {
        const int d = out_dim[b];
        sel |= (flag[d] ? ord[d] : 4u) << (4 * b);
        ob |= (flag[d] ? 0x80u : 0u) << (8 * b);
    }
    KdLutEntry e;
    e.x = sel | ((4u * n) << 16) | (n << 24);
    e.y = ob;
    return e;
}

// Per mask word (16 dims).
struct KdWord {
    uint32_t E, O, X3;
};
KHQ_HD KdWord kd_word(uint32_t w) {
    KdWord r;
    r.E = w & 0x33333333u;
    r.O = (w >> 2) & 0x33333333u;
    const uint32_t e3 = r.E & (r.E >> 1) & 0x11111111u;
    const uint32_t o3 = r.O & (r.O >> 1) & 0x11111111u;
    r.X3 = e3 | (o3 << 1);
    return r;
}

// The sign-bit stream of a row: bits 0..49 = payload bytes 29..35.
struct KdSigns {
    uint32_t lo, hi;
};
KHQ_HD KdSigns kd_signs(const uint32_t* kp) {
    KdSigns r;
    r.lo = kd_funnel_r(kp[7], kp[8], 8);
    r.hi = kd_funnel_r(kp[8], kp[9], 8) & 0x00FFFFFFu;
    return r;
}

// Number of outliers of a word before its step q (q = 0..3).
KHQ_HD uint32_t kd_prefix(const KdWord& w, int q) {
#if defined(__CUDA_ARCH__)
    return (uint32_t)__popc(w.X3 & ((1u << (8 * q)) - 1u));
#else
    return (uint32_t)__builtin_popcount(w.X3 & ((1u << (8 * q)) - 1u));
#endif
}
KHQ_HD uint32_t kd_count(const KdWord& w) {
#if defined(__CUDA_ARCH__)
    return (uint32_t)__popc(w.X3);
#else
    return (uint32_t)__builtin_popcount(w.X3);
#endif
}

struct KdStep {
    uint32_t t0, t1;  // fp16x2 ternary values: dims (4q, 4q+2), (4q+1, 4q+3)
    uint32_t h0, h1;  // fp16x2 of sign-matched (1024 + code); residual = t * -1024 + h
};

// Decode step q (0..3) of a mask word.  `pos` = ordinal (in the row) of the step's first outlier,
// `kp` = the row's 10 payload words, `sg` = its sign stream, `lut` = the scatter table.  Nothing
// is carried from one step to the next, so the steps of a row are independent instruction streams.
KHQ_HD KdStep kd_step(const KdWord& w, int q, uint32_t pos, const uint32_t* kp, const KdSigns& sg,
                      const KdLutEntry* lut) {
    const uint32_t f = (w.X3 >> (8 * q)) & 0xFFu;
    const KdLutEntry e = lut[f];
    // next four residual nibbles -> bytes [n0, n1, n2, n3]
    const uint32_t p = pos < 50u ? pos : 50u;  // never read past the 50-entry stream
    const uint32_t bit = 32u + 4u * p;
    const uint32_t cw = kd_funnel_r(kp[bit >> 5], kp[(bit >> 5) + 1], bit & 31u);
    const uint32_t cb = kd_prmt(cw & 0x0F0Fu, (cw >> 4) & 0x0F0Fu, 0x5140u);
    // next four sign bits -> 0x80 in bytes 0..3
    const uint32_t s4 = kd_funnel_r(p < 32u ? sg.lo : sg.hi, p < 32u ? sg.hi : 0u, p & 31u);
    uint32_t sb = (((s4 & 0xFu) * 0x10204080u) & 0x80808080u) | cb;
    if (pos > 46u) {  // entries with ordinal >= 50 do not exist: code 0, negative sign
        const uint32_t nv = pos >= 50u ? 0u : (50u - pos);
        if (nv < 4u) sb &= (1u << (8u * nv)) - 1u;
    }
    const uint32_t pd = kd_prmt(sb, 0u, e.x);  // per dim: code | positive << 7, zero off the outliers
    // ternary high bytes from the symbols; negative outliers get their sign bit flipped
    const uint32_t selq = kd_prmt(w.E, w.O, (uint32_t)q | ((uint32_t)(4 + q) << 4));
    uint32_t H = kd_prmt(0x3C3CBC00u, 0u, selq);
    H ^= e.y ^ (pd & 0x80808080u);
    const uint32_t H2 = H + (H & 0x04040404u) * 10u;  // 0x3C -> 0x64, 0xBC -> 0xE4: +-1 -> +-1024
    const uint32_t pdc = pd & 0x0F0F0F0Fu;
    KdStep r;
    r.t0 = kd_prmt(H, 0u, 0x1404u);
    r.t1 = kd_prmt(H, 0u, 0x3424u);
    r.h0 = kd_prmt(H2, pdc, 0x1504u);
    r.h1 = kd_prmt(H2, pdc, 0x3726u);
    return r;
}

}  // namespace khq
