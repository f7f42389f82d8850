/*
 * khq_oracle.c -- CPU restatement of the KHQ attention path (TEST INFRASTRUCTURE ONLY).
 *
 * This file is the checker for the CUDA library: the tests, the smoke entry and the
 * benchmark's CPU-baseline leg are the only callers.  Nothing in the shipped package
 * imports, links or executes it, and the shipped package has no CPU fallback.
 *
 * Every function restates one piece of the reference project's algorithm (paths are
 * relative to the reference project's root):
 *
 *   khq_oracle_compress        src/csrc/qmv_sm75_kernel.cu:1256-1467  (khq_compress_kernel)
 *   khq_oracle_decode_k/_v     src/csrc/qmv_sm75_kernel.cu:1608-1699, 1739-1761, 1776-1826
 *   khq_oracle_attn_partial    src/csrc/qmv_sm75_kernel.cu:1471-1831  (khq_attn_kernel)
 *   khq_oracle_attn_reduce     src/csrc/qmv_sm75_kernel.cu:1836-1877  (khq_attn_reduce_kernel)
 *   khq_oracle_attn_launch     src/csrc/qmv_sm75_kernel.cu:4314-4375  (launch_khq_attn_fp16)
 *   khq_oracle_window_attn     src/csrc/qmv_sm75_kernel.cu:1882-1965  (khq_window_attn_kernel)
 *   khq_oracle_merge_gate      src/csrc/qmv_sm75_kernel.cu:1983-2010  (khq_merge_gate_kernel)
 *   khq_oracle_gqa_attention   src/kernels/elementwise_sm75.mojo:1091-1231 and its FP64 twin
 *                              tests/test_gqa_attention_gpu.mojo:36-83
 *   khq_oracle_partial_rope    src/kernels/elementwise_sm75.mojo:1023-1061,
 *                              tests/test_rope_gpu.mojo:20-47
 *
 * Parity pinning: the reference holds no golden vector for any KHQ kernel; the code words
 * this file produces are pinned against outputs of the reference's own CUDA source compiled
 * unmodified for sm_100a (tests/golden/, produced by tests/golden/make_golden_gpu.py).  The
 * fp16-KV attention and RoPE functions are pinned against the reference's own test fixtures.
 *
 * Numerics.  The compress path is integer/bit-exact work and therefore follows the
 * reference's fp32 evaluation order step by step, with fmaf() written out wherever the
 * device compiler fuses a multiply into the following add (the device build of the
 * reference uses the default -fmad=true).  Build with -ffp-contract=off so the host
 * compiler adds no fusion of its own.  The attention path is tolerance-checked, so after the
 * fp32 decode of each code word it accumulates in double: it is an "at least fp32" reference.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define KHQ_D 256
#define KHQ_NP 64
#define KHQ_K_PAYLOAD 40
#define KHQ_V_PAYLOAD 104
#define KHQ_MAX_OUTLIERS 50

/* ---------------------------------------------------------------- fp16 <-> fp32 */
static float h2f(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1Fu;
    uint32_t m = h & 0x3FFu;
    uint32_t bits;
    if (e == 0) {
        if (m == 0) {
            bits = sign;
        } else { /* subnormal: normalise */
            int shift = 0;
            while (!(m & 0x400u)) { m <<= 1; ++shift; }
            m &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - shift + 1) << 23) | (m << 13);
        }
    } else if (e == 31) {
        bits = sign | 0x7F800000u | (m << 13);
    } else {
        bits = sign | ((e + 112u) << 23) | (m << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* round-to-nearest-even, the conversion __float2half performs */
static uint16_t f2h(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | ((ax > 0x7F800000u) ? 0x200u : 0u));
    }
    if (ax >= 0x477FF000u) { /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7C00u);
    }
    if (ax < 0x33000001u) { /* below half of the smallest subnormal -> 0 */
        return (uint16_t)sign;
    }
    int32_t e = (int32_t)(ax >> 23) - 127;
    uint32_t m = (ax & 0x7FFFFFu) | 0x800000u;
    if (e < -14) { /* subnormal result */
        int shift = (-14 - e) + 13;
        uint32_t rem_mask = (1u << shift) - 1u;
        uint32_t rem = m & rem_mask;
        uint32_t half = 1u << (shift - 1);
        uint32_t r = m >> shift;
        if (rem > half || (rem == half && (r & 1u))) ++r;
        return (uint16_t)(sign | r);
    }
    uint32_t r = ((uint32_t)(e + 15) << 10) | ((m >> 13) & 0x3FFu);
    uint32_t rem = m & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1u))) ++r;
    return (uint16_t)(sign | r);
}

uint16_t khq_oracle_f2h(float f) { return f2h(f); }
float khq_oracle_h2f(uint16_t h) { return h2f(h); }

/* roundf of the device library: half away from zero, same as C99 roundf */

/* unnormalised FWHT-256, natural order, stages 1,2,..,128 (qmv_sm75_kernel.cu:1285-1292) */
static void fwht256_f(float* r) {
    for (int step = 1; step < KHQ_D; step <<= 1)
        for (int i = 0; i < KHQ_D; i += 2 * step)
            for (int j = 0; j < step; ++j) {
                float a = r[i + j], b = r[i + j + step];
                r[i + j] = a + b;
                r[i + j + step] = a - b;
            }
}
static void fwht256_d(double* r) {
    for (int step = 1; step < KHQ_D; step <<= 1)
        for (int i = 0; i < KHQ_D; i += 2 * step)
            for (int j = 0; j < step; ++j) {
                double a = r[i + j], b = r[i + j + step];
                r[i + j] = a + b;
                r[i + j + step] = a - b;
            }
}

/* ============================================================== compress ====== */
/* Common front end: norm, x*d/norm, FWHT, 4x4 rotor per patch.
 * qmv_sm75_kernel.cu:1273-1303.  Returns the fp16 bits of the stored norm. */
static uint16_t compress_front(const uint16_t* x, const uint16_t* d_vec, const uint16_t* rotor,
                               float* rot /*256*/) {
    float sum_sq = 0.0f;
    for (int i = 0; i < KHQ_D; ++i) {
        float v = h2f(x[i]);
        sum_sq = fmaf(v, v, sum_sq); /* v*v is exact in fp32, so fused == unfused */
    }
    float norm = sqrtf(sum_sq + 1e-8f);
    float r[KHQ_D];
    float den = norm + 1e-8f;
    for (int i = 0; i < KHQ_D; ++i) r[i] = (h2f(x[i]) * h2f(d_vec[i])) / den;
    fwht256_f(r);
    for (int p = 0; p < KHQ_NP; ++p)
        for (int c = 0; c < 4; ++c) {
            float acc = 0.0f;
            for (int k = 0; k < 4; ++k) acc = fmaf(r[p * 4 + k], h2f(rotor[p * 16 + k * 4 + c]), acc);
            rot[p * 4 + c] = acc;
        }
    return f2h(norm);
}

/* One row of the K branch (qmv_sm75_kernel.cu:1314-1351, 1430-1465). */
static void compress_row_k(const float* rot, const uint16_t* cents, float ts, uint32_t* mask16,
                           uint16_t* r_norm, uint8_t* pay /*40*/, uint8_t* shared_meta /*4*/) {
    const float f_s = 0.0625f; /* rsqrtf(256.f) */
    uint32_t plan[16];
    memset(plan, 0, sizeof plan);
    float out_abs[KHQ_MAX_OUTLIERS];
    uint32_t out_dim[KHQ_MAX_OUTLIERS], out_sign[KHQ_MAX_OUTLIERS];
    uint32_t n_out = 0;
    float sum_normals = 0.0f, sum_cbase = 0.0f;
    const float th_out = 1.60f * f_s, th_lo = 0.47f * f_s;
    for (int i = 0; i < KHQ_D; ++i) {
        float proj = rot[i] * f_s;
        float proj_scaled = proj * ts;
        float ap = fabsf(proj);
        uint32_t sym;
        if (ap > th_out) {
            if (n_out < KHQ_MAX_OUTLIERS) {
                sym = 3;
                out_abs[n_out] = fabsf(proj_scaled);
                out_dim[n_out] = (uint32_t)i;
                out_sign[n_out] = (proj > 0.0f) ? 1u : 0u;
                ++n_out;
            } else {
                sym = (proj > 0.0f) ? 2u : 1u; /* overflow outliers stay out of the sums */
            }
        } else {
            if (proj > th_lo) sym = 2;
            else if (proj < -th_lo) sym = 1;
            else sym = 0;
            if (sym == 1 || sym == 2) {
                sum_normals += ap;
                sum_cbase += h2f(cents[2 * KHQ_D + i]);
            }
        }
        plan[i / 16] |= sym << ((i % 16) * 2);
    }
    memcpy(mask16, plan, sizeof plan);

    float mult = (sum_cbase > 1e-5f) ? (sum_normals / sum_cbase) : 1.0f;
    if (mult < 0.1f || mult > 10.0f || isnan(mult)) mult = 1.0f;
    float max_res = 0.0f;
    float res[KHQ_MAX_OUTLIERS];
    for (uint32_t j = 0; j < n_out; ++j) {
        float c = h2f(cents[2 * KHQ_D + out_dim[j]]);
        /* abs - c*mult: device compiler fuses the multiply into the subtract */
        float rj = fmaxf(0.0f, fmaf(-c, mult, out_abs[j]));
        res[j] = rj;
        if (rj > max_res) max_res = rj;
    }
    float rscale = (n_out > 0) ? (fmaxf(max_res, 1e-4f) / 15.0f) : 0.0f;
    *r_norm = f2h(rscale);
    uint32_t mult_u = (uint32_t)(mult * 1000.0f);
    memcpy(pay, &mult_u, 4);
    memset(pay + 4, 0, 36);
    for (uint32_t j = 0; j < n_out; ++j) {
        if (rscale > 0.0f) {
            float r4 = roundf(res[j] / rscale);
            uint8_t v = (uint8_t)fmaxf(0.0f, fminf(15.0f, r4));
            pay[4 + (j / 2)] |= (uint8_t)(v << ((j % 2) * 4));
        }
        if (out_sign[j]) pay[29 + (j / 8)] |= (uint8_t)(1u << (j % 8));
    }
    pay[36] = 0x02;
    memset(shared_meta, 0, 4);
}

/* One row of the V branch (qmv_sm75_kernel.cu:1353-1428). */
static void compress_row_v(const float* rot, const uint16_t* cents, const uint16_t* vq, float alpha,
                           uint16_t* r_norm, uint8_t* pay /*104*/, uint8_t* shared_meta /*4*/,
                           uint32_t* near_ties) {
    const float f_s = 0.0625f;
    uint32_t code[KHQ_NP], sel[KHQ_NP], dump[KHQ_NP];
    float pres[KHQ_NP], e_true[KHQ_NP], e_vq[KHQ_NP];
    float max_res = 0.0f;
    for (int p = 0; p < KHQ_NP; ++p) {
        float v0 = rot[p * 4 + 0] * f_s, v1 = rot[p * 4 + 1] * f_s, v2 = rot[p * 4 + 2] * f_s;
        const uint16_t* cb = vq + (size_t)p * 256 * 3;
        float best_d = 1e20f, second_d = 1e20f;
        uint32_t best = 0;
        for (uint32_t i = 0; i < 256; ++i) {
            float c0 = h2f(cb[i * 3 + 0]), c1 = h2f(cb[i * 3 + 1]), c2 = h2f(cb[i * 3 + 2]);
            float d0 = fmaf(-c0, alpha, v0), d1 = fmaf(-c1, alpha, v1), d2 = fmaf(-c2, alpha, v2);
            /* d0*d0 + d1*d1 + d2*d2 as the device compiler contracts it */
            float dist = fmaf(d2, d2, fmaf(d0, d0, d1 * d1));
            if (dist < best_d) { second_d = best_d; best_d = dist; best = i; }
            else if (dist < second_d) second_d = dist;
        }
        if (near_ties && second_d == best_d) ++*near_ties;
        code[p] = best;
        float b0 = h2f(cb[best * 3 + 0]) * alpha, b1 = h2f(cb[best * 3 + 1]) * alpha,
              b2 = h2f(cb[best * 3 + 2]) * alpha;
        e_true[p] = fmaf(v2, v2, fmaf(v0, v0, v1 * v1));
        e_vq[p] = fmaf(b2, b2, fmaf(b0, b0, b1 * b1));

        float v3 = rot[p * 4 + 3] * f_s;
        float best_s = 1e20f;
        uint32_t s = 0;
        for (uint32_t i = 0; i < 2; ++i) {
            float c = h2f(cents[i * KHQ_D + p * 4 + 3]);
            float dist = fabsf(fmaf(-c, alpha, v3));
            if (dist < best_s) { best_s = dist; s = i; }
        }
        sel[p] = s;
        float cbest = h2f(cents[s * KHQ_D + p * 4 + 3]);
        float residual = fmaf(-cbest, alpha, v3);
        pres[p] = residual;
        if (fabsf(residual) > max_res) max_res = fabsf(residual);
    }
    memcpy(shared_meta, &max_res, 4);
    float rs = fmaxf(max_res, 1e-4f);
    for (int p = 0; p < KHQ_NP; ++p) {
        float scaled = fmaf(pres[p] / rs, 7.0f, 8.0f);
        dump[p] = (uint32_t)fmaxf(0.0f, fminf(15.0f, roundf(scaled)));
    }
    uint32_t w[26];
    for (int g = 0; g < 8; ++g) {
        uint32_t f[8];
        for (int i = 0; i < 8; ++i) {
            int p = g * 8 + i;
            f[i] = (code[p] & 0x7Fu) | ((sel[p] & 1u) << 7) | ((dump[p] & 0xFu) << 8);
        }
        w[g * 3 + 0] = f[0] | (f[1] << 12) | ((f[2] & 0xFFu) << 24);
        w[g * 3 + 1] = (f[2] >> 8) | (f[3] << 4) | (f[4] << 16) | ((f[5] & 0xFu) << 28);
        w[g * 3 + 2] = (f[5] >> 4) | (f[6] << 8) | (f[7] << 20);
    }
    uint32_t lo = 0, hi = 0;
    for (int i = 0; i < 32; ++i) {
        lo |= ((code[i] >> 7) & 1u) << i;
        hi |= ((code[32 + i] >> 7) & 1u) << i;
    }
    w[24] = lo;
    w[25] = hi;
    memcpy(pay, w, sizeof w);
    float st = 0.0f, sv = 0.0f;
    for (int p = 0; p < KHQ_NP; ++p) { st += e_true[p]; sv += e_vq[p]; }
    *r_norm = f2h(sqrtf(st / (sv + 1e-8f)));
}

/* launch_khq_compress_fp16 semantics (qmv_sm75_kernel.cu:4279-4310): returns 0, or -100 on
 * n<=0 / d!=256.  out_mask is written for K rows only; out_shared_meta gets 0 (K) or the fp32
 * max residual (V).  near_ties (optional) counts V patches whose two best codes are at exactly
 * the same distance. */
int khq_oracle_compress(const uint16_t* x, const uint16_t* d_vec, const uint16_t* rotor,
                        const uint16_t* cents, const uint16_t* vq, uint32_t* out_mask,
                        uint16_t* out_norms, uint16_t* out_r_norms, uint8_t* out_payload,
                        uint8_t* out_shared_meta, int n, int d, float threshold_scale, float alpha,
                        int is_v, uint32_t* near_ties) {
    if (n <= 0 || d != KHQ_D) return -100;
    uint32_t ties_total = 0;
#pragma omp parallel for schedule(static) reduction(+ : ties_total)
    for (int row = 0; row < n; ++row) {
        float rot[KHQ_D];
        out_norms[row] = compress_front(x + (size_t)row * KHQ_D, d_vec, rotor, rot);
        if (is_v) {
            uint32_t t = 0;
            compress_row_v(rot, cents, vq, alpha, out_r_norms + row,
                           out_payload + (size_t)row * KHQ_V_PAYLOAD,
                           out_shared_meta + (size_t)row * 4, &t);
            ties_total += t;
        } else {
            compress_row_k(rot, cents, threshold_scale, out_mask + (size_t)row * 16,
                           out_r_norms + row, out_payload + (size_t)row * KHQ_K_PAYLOAD,
                           out_shared_meta + (size_t)row * 4);
        }
    }
    if (near_ties) *near_ties = ties_total;
    return 0;
}

/* ============================================================ decompress ====== */
/* K code words of one row -> the rotated-domain vector y = k_val * alpha_k * k_norm in fp32,
 * exactly the per-dimension decode of qmv_sm75_kernel.cu:1608-1644. */
static void decode_k_codes(const uint8_t* pay, const uint32_t* mask16, uint16_t norm_h,
                           uint16_t rnorm_h, const uint16_t* cents, float alpha_k, float* y) {
    float k_norm = h2f(norm_h), rscale = h2f(rnorm_h);
    uint32_t mult_u;
    memcpy(&mult_u, pay, 4);
    float mult = (float)mult_u / 1000.0f;
    if (mult < 0.1f || mult > 10.0f || isnan(mult)) mult = 1.0f;
    const uint8_t* res = pay + 4;
    const uint8_t* sgn = pay + 29;
    uint32_t j = 0;
    for (int i = 0; i < KHQ_D; ++i) {
        uint32_t sym = (mask16[i / 16] >> ((i % 16) * 2)) & 3u;
        float cb = h2f(cents[2 * KHQ_D + i]) * mult;
        float kv = 0.0f;
        if (sym == 3) {
            float sign = (j < KHQ_MAX_OUTLIERS && ((sgn[j / 8] >> (j % 8)) & 1u)) ? 1.0f : -1.0f;
            float r4 = (j < KHQ_MAX_OUTLIERS) ? (float)((res[j / 2] >> ((j % 2) * 4)) & 0xFu) : 0.0f;
            kv = sign * (cb + r4 * rscale);
            ++j;
        } else if (sym == 2) kv = cb;
        else if (sym == 1) kv = -cb;
        y[i] = kv * alpha_k * k_norm;
    }
}

/* Full K reconstruction before RoPE: inverse rotor (transpose), FWHT, /256/(d+1e-8)
 * (qmv_sm75_kernel.cu:1646-1687).  out in double. */
void khq_oracle_decode_k(const uint8_t* pay, const uint32_t* mask16, uint16_t norm_h,
                         uint16_t rnorm_h, const uint16_t* cents, const uint16_t* rotor,
                         const uint16_t* d_vec, float alpha_k, double* out /*256*/) {
    float y[KHQ_D];
    decode_k_codes(pay, mask16, norm_h, rnorm_h, cents, alpha_k, y);
    double z[KHQ_D];
    for (int p = 0; p < KHQ_NP; ++p)
        for (int c = 0; c < 4; ++c) {
            double a = 0.0;
            for (int k = 0; k < 4; ++k) a += (double)y[p * 4 + k] * (double)h2f(rotor[p * 16 + c * 4 + k]);
            z[p * 4 + c] = a;
        }
    fwht256_d(z);
    for (int i = 0; i < KHQ_D; ++i) {
        float dinv = (1.0f / 256.0f) / (h2f(d_vec[i]) + 1e-8f);
        out[i] = z[i] * (double)dinv;
    }
}

/* V code words of one row -> rotated-domain vector (before the final inverse rotor / FWHT),
 * qmv_sm75_kernel.cu:1739-1761. */
static void decode_v_codes(const uint8_t* pay, uint16_t norm_h, uint16_t energy_h, float sm_scale,
                           const uint16_t* cents_v, const uint16_t* vq, float alpha_v, float* v) {
    float vn = h2f(norm_h), energy = h2f(energy_h);
    float pre_v = alpha_v * vn * energy;
    float pre_res = sm_scale * vn;
    uint32_t w[26];
    memcpy(w, pay, sizeof w);
    for (int p = 0; p < KHQ_NP; ++p) {
        int g = p / 8, sub = p % 8;
        uint64_t lo64 = ((uint64_t)w[3 * g + 1] << 32) | w[3 * g + 0];
        uint64_t hi64 = ((uint64_t)w[3 * g + 2] << 32) | w[3 * g + 1];
        uint32_t f = (sub < 4) ? (uint32_t)((lo64 >> (sub * 12)) & 0xFFFu)
                               : (uint32_t)((hi64 >> ((sub - 4) * 12 + 16)) & 0xFFFu);
        uint32_t hb = (p < 32) ? ((w[24] >> p) & 1u) : ((w[25] >> (p - 32)) & 1u);
        uint32_t code = (f & 0x7Fu) | (hb << 7);
        uint32_t s3 = (f >> 7) & 1u, dump = (f >> 8) & 0xFu;
        for (int k = 0; k < 3; ++k) v[p * 4 + k] = h2f(vq[((size_t)p * 256 + code) * 3 + k]) * pre_v;
        float c = h2f(cents_v[s3 * KHQ_D + p * 4 + 3]) * alpha_v;
        v[p * 4 + 3] = (c * vn) + (((float)dump - 8.0f) / 7.0f * pre_res);
    }
}

/* Inverse rotor + FWHT + /16/(d+1e-8) of an accumulated rotated-domain vector
 * (qmv_sm75_kernel.cu:1776-1826). */
static void v_epilogue(const double* acc, const uint16_t* rotor_v, const uint16_t* d_vec_v,
                       double* out) {
    double z[KHQ_D];
    for (int p = 0; p < KHQ_NP; ++p)
        for (int c = 0; c < 4; ++c) {
            double a = 0.0;
            for (int k = 0; k < 4; ++k) a += acc[p * 4 + k] * (double)h2f(rotor_v[p * 16 + c * 4 + k]);
            z[p * 4 + c] = a;
        }
    fwht256_d(z);
    for (int i = 0; i < KHQ_D; ++i)
        out[i] = (z[i] * (double)(1.0f / 16.0f)) / (double)(h2f(d_vec_v[i]) + 1e-8f);
}

void khq_oracle_decode_v(const uint8_t* pay, uint16_t norm_h, uint16_t energy_h, float sm_scale,
                         const uint16_t* cents_v, const uint16_t* vq, const uint16_t* rotor_v,
                         const uint16_t* d_vec_v, float alpha_v, double* out /*256*/) {
    float v[KHQ_D];
    double a[KHQ_D];
    decode_v_codes(pay, norm_h, energy_h, sm_scale, cents_v, vq, alpha_v, v);
    for (int i = 0; i < KHQ_D; ++i) a[i] = v[i];
    v_epilogue(a, rotor_v, d_vec_v, out);
}

/* ============================================== compressed-region attention === */
/* Partial over tokens [s_lo, s_hi) for every query head: out (num_heads, 258) =
 * unnormalised acc[256], max_s, sum_exp, with max_s = -1e20 and zeros for an empty range.
 * RoPE pairs (m, m+32), m<32, freq = powf(base, -2m/64), angle (start_pos+s)*freq
 * (qmv_sm75_kernel.cu:1514-1521, 1572-1579, 1689-1699).  The angle is evaluated in double here;
 * the reference evaluates it in fp32 at every re-synchronisation point and advances it by a
 * rotation recurrence in between. */
void khq_oracle_attn_partial(const uint16_t* q, const uint8_t* k_payload, const uint8_t* v_payload,
                             const uint8_t* v_shared_meta, const uint32_t* k_mask,
                             const uint16_t* k_norms, const uint16_t* k_r_norms,
                             const uint16_t* v_norms, const uint16_t* v_r_norms,
                             const uint16_t* cents_k, const uint16_t* cents_v, const uint16_t* vq,
                             const uint16_t* k_rotor, const uint16_t* v_rotor,
                             const uint16_t* d_vec_k, const uint16_t* d_vec_v, float* out,
                             int num_heads, int n_rep, float scale, float alpha_k, float alpha_v,
                             float rope_base, int start_pos, int s_lo, int s_hi) {
    int h_kv = (n_rep > 0) ? num_heads / n_rep : 1;
    double freq[32];
    for (int m = 0; m < 32; ++m) freq[m] = (double)powf(rope_base, -2.0f * (float)m / 64.0f);

#pragma omp parallel for schedule(dynamic, 1)
    for (int g = 0; g < h_kv; ++g) {
        int nh = n_rep;
        double* acc = (double*)calloc((size_t)nh * KHQ_D, sizeof(double));
        double* mx = (double*)malloc((size_t)nh * sizeof(double));
        double* se = (double*)calloc((size_t)nh, sizeof(double));
        double* qd = (double*)malloc((size_t)nh * KHQ_D * sizeof(double));
        for (int r = 0; r < nh; ++r) {
            mx[r] = -1e20;
            const uint16_t* qp = q + (size_t)(g * n_rep + r) * 2 * KHQ_D;
            for (int i = 0; i < KHQ_D; ++i) qd[r * KHQ_D + i] = h2f(qp[i]);
        }
        for (int s = s_lo; s < s_hi; ++s) {
            size_t row = (size_t)s * h_kv + g;
            double kh[KHQ_D];
            khq_oracle_decode_k(k_payload + row * KHQ_K_PAYLOAD, k_mask + row * 16, k_norms[row],
                                k_r_norms[row], cents_k, k_rotor, d_vec_k, alpha_k, kh);
            for (int m = 0; m < 32; ++m) {
                double th = (double)(start_pos + s) * freq[m];
                double c = cos(th), sn = sin(th);
                double a = kh[m], b = kh[m + 32];
                kh[m] = a * c - b * sn;
                kh[m + 32] = a * sn + b * c;
            }
            float vv[KHQ_D];
            float sm;
            memcpy(&sm, v_shared_meta + row * 4, 4);
            decode_v_codes(v_payload + row * KHQ_V_PAYLOAD, v_norms[row], v_r_norms[row], sm,
                           cents_v, vq, alpha_v, vv);
            for (int r = 0; r < nh; ++r) {
                double dot = 0.0;
                for (int i = 0; i < KHQ_D; ++i) dot += qd[r * KHQ_D + i] * kh[i];
                double sv = dot * (double)scale;
                double p;
                if (sv > mx[r]) {
                    double fac = exp(mx[r] - sv);
                    se[r] = se[r] * fac + 1.0;
                    for (int i = 0; i < KHQ_D; ++i) acc[r * KHQ_D + i] *= fac;
                    mx[r] = sv;
                    p = 1.0;
                } else {
                    p = exp(sv - mx[r]);
                    se[r] += p;
                }
                for (int i = 0; i < KHQ_D; ++i) acc[r * KHQ_D + i] += p * (double)vv[i];
            }
        }
        for (int r = 0; r < nh; ++r) {
            double o[KHQ_D];
            v_epilogue(acc + (size_t)r * KHQ_D, v_rotor, d_vec_v, o);
            float* ob = out + (size_t)(g * n_rep + r) * (KHQ_D + 2);
            for (int i = 0; i < KHQ_D; ++i) ob[i] = (float)o[i];
            ob[KHQ_D] = (float)mx[r];
            ob[KHQ_D + 1] = (float)se[r];
        }
        free(acc); free(mx); free(se); free(qd);
    }
}

/* LSE merge of split partials (qmv_sm75_kernel.cu:1836-1877):
 * partial (nq, splits, 258) -> out (nq, 258), still unnormalised. */
void khq_oracle_attn_reduce(const float* partial, float* out, int nq, int splits) {
    const int st = KHQ_D + 2;
    for (int qi = 0; qi < nq; ++qi) {
        const float* base = partial + (size_t)qi * splits * st;
        double M = -1e20;
        for (int sp = 0; sp < splits; ++sp)
            if ((double)base[(size_t)sp * st + KHQ_D] > M) M = base[(size_t)sp * st + KHQ_D];
        double den = 0.0;
        for (int sp = 0; sp < splits; ++sp)
            den += (double)base[(size_t)sp * st + KHQ_D + 1] * exp((double)base[(size_t)sp * st + KHQ_D] - M);
        float* o = out + (size_t)qi * st;
        for (int d = 0; d < KHQ_D; ++d) {
            double num = 0.0;
            for (int sp = 0; sp < splits; ++sp)
                num += (double)base[(size_t)sp * st + d] * exp((double)base[(size_t)sp * st + KHQ_D] - M);
            o[d] = (float)num;
        }
        o[KHQ_D] = (float)M;
        o[KHQ_D + 1] = (float)den;
    }
}

/* launch_khq_attn_fp16 semantics for L_q == 1 (qmv_sm75_kernel.cu:4314-4375, split ranges
 * 1546-1553): returns 0, -100 (num_queries<=0 or c_len<=0) or -101 (splits>1 without a partial
 * buffer). */
int khq_oracle_attn_launch(const uint16_t* q, const uint8_t* k_payload, const uint8_t* v_payload,
                           const uint8_t* v_shared_meta, const uint32_t* k_mask,
                           const uint16_t* k_norms, const uint16_t* k_r_norms,
                           const uint16_t* v_norms, const uint16_t* v_r_norms,
                           const uint16_t* cents_k, const uint16_t* cents_v, const uint16_t* vq,
                           const uint16_t* k_rotor, const uint16_t* v_rotor,
                           const uint16_t* d_vec_k, const uint16_t* d_vec_v, float* out_attn,
                           float* out_partial, int num_queries, int num_heads, int c_len, int n_rep,
                           float scale, float alpha_k, float alpha_v, float rope_base, int start_pos,
                           int num_splits) {
    if (num_queries <= 0 || c_len <= 0) return -100;
    if (num_splits < 1) num_splits = 1;
    if (num_splits > 1 && !out_partial) return -101;
    if (num_splits == 1) {
        khq_oracle_attn_partial(q, k_payload, v_payload, v_shared_meta, k_mask, k_norms, k_r_norms,
                                v_norms, v_r_norms, cents_k, cents_v, vq, k_rotor, v_rotor, d_vec_k,
                                d_vec_v, out_attn, num_heads, n_rep, scale, alpha_k, alpha_v,
                                rope_base, start_pos, 0, c_len);
        return 0;
    }
    const int st = KHQ_D + 2;
    int per = (c_len + num_splits - 1) / num_splits;
    float* tmp = (float*)malloc((size_t)num_heads * st * sizeof(float));
    for (int sp = 0; sp < num_splits; ++sp) {
        int lo = sp * per; if (lo > c_len) lo = c_len;
        int hi = lo + per; if (hi > c_len) hi = c_len;
        khq_oracle_attn_partial(q, k_payload, v_payload, v_shared_meta, k_mask, k_norms, k_r_norms,
                                v_norms, v_r_norms, cents_k, cents_v, vq, k_rotor, v_rotor, d_vec_k,
                                d_vec_v, tmp, num_heads, n_rep, scale, alpha_k, alpha_v, rope_base,
                                start_pos, lo, hi);
        for (int h = 0; h < num_heads && h < num_queries; ++h)
            memcpy(out_partial + ((size_t)h * num_splits + sp) * st, tmp + (size_t)h * st,
                   st * sizeof(float));
    }
    free(tmp);
    khq_oracle_attn_reduce(out_partial, out_attn, num_queries, num_splits);
    return 0;
}

/* ====================================================== raw-ring window ======= */
/* qmv_sm75_kernel.cu:1882-1965: ring rows are token-major, row = slot*H_kv + kv_head. */
int khq_oracle_window_attn(const uint16_t* q, const uint16_t* ring_k, const uint16_t* ring_v,
                           float* out, int win_start, int win_len, int ring_cap, int H_q, int H_kv,
                           int d, float scale) {
    if (H_q <= 0 || win_len <= 0) return -100;
    int n_rep = H_q / H_kv;
#pragma omp parallel for schedule(static)
    for (int h = 0; h < H_q; ++h) {
        int g = h / n_rep;
        double acc[KHQ_D];
        for (int i = 0; i < d; ++i) acc[i] = 0.0;
        double mx = -1e20, se = 0.0;
        for (int s = 0; s < win_len; ++s) {
            int slot = (win_start + s) % ring_cap;
            const uint16_t* kr = ring_k + ((size_t)slot * H_kv + g) * d;
            const uint16_t* vr = ring_v + ((size_t)slot * H_kv + g) * d;
            double dot = 0.0;
            for (int i = 0; i < d; ++i) dot += (double)h2f(q[(size_t)h * 2 * d + i]) * (double)h2f(kr[i]);
            double sv = dot * (double)scale, p;
            if (sv > mx) {
                double fac = exp(mx - sv);
                se = se * fac + 1.0;
                for (int i = 0; i < d; ++i) acc[i] *= fac;
                mx = sv;
                p = 1.0;
            } else {
                p = exp(sv - mx);
                se += p;
            }
            for (int i = 0; i < d; ++i) acc[i] += p * (double)h2f(vr[i]);
        }
        float* o = out + (size_t)h * (d + 2);
        for (int i = 0; i < d; ++i) o[i] = (float)acc[i];
        o[d] = (float)mx;
        o[d + 1] = (float)se;
    }
    return 0;
}

/* ========================================================== merge + gate ====== */
/* qmv_sm75_kernel.cu:1983-2010.  out is fp16 (H_q, d). */
int khq_oracle_merge_gate(const float* attn_c, const float* attn_w, const uint16_t* q_gate,
                          uint16_t* out, int H_q, int d, int has_w) {
    if (H_q <= 0 || d <= 0) return -100;
    for (int h = 0; h < H_q; ++h) {
        const float* cc = attn_c + (size_t)h * (d + 2);
        for (int i = 0; i < d; ++i) {
            double num = cc[i], den = cc[d + 1];
            if (has_w) {
                const float* cw = attn_w + (size_t)h * (d + 2);
                double mc = cc[d], mw = cw[d];
                double M = mc > mw ? mc : mw;
                double wc = exp(mc - M), ww = exp(mw - M);
                num = num * wc + (double)cw[i] * ww;
                den = den * wc + (double)cw[d + 1] * ww;
            }
            double val = num / (den + (double)1e-8f);
            double g = h2f(q_gate[(size_t)h * 2 * d + d + i]);
            val = val * (1.0 / (1.0 + exp(-g)));
            out[(size_t)h * d + i] = f2h((float)val);
        }
    }
    return 0;
}

/* ===================================================== fp16-KV attention ====== */
/* One query row over cache rows [0, seq_len): softmax(q.K^T*scale) V * sigmoid(gate) with the
 * kernel's 1/(Z + 1e-9) denominator (elementwise_sm75.mojo:1140-1231;
 * tests/test_gqa_attention_gpu.mojo:36-83).  q_gate/k/v are fp32 arrays here so that the
 * reference's fp32 test fixtures can be fed unchanged; out is fp64. */
void khq_oracle_gqa_attention_f32(const float* q_gate, const float* k_cache, const float* v_cache,
                                  double* out, int seq_len, int H_q, int H_kv, int d, double scale) {
    int group = H_q / H_kv, kv_dim = H_kv * d;
    double* sc = (double*)malloc((size_t)(seq_len > 0 ? seq_len : 1) * sizeof(double));
    for (int h = 0; h < H_q; ++h) {
        int g = h / group;
        double m = -3.0e38;
        for (int t = 0; t < seq_len; ++t) {
            double dot = 0.0;
            for (int i = 0; i < d; ++i)
                dot += (double)q_gate[(size_t)h * 2 * d + i] * (double)k_cache[(size_t)t * kv_dim + g * d + i];
            sc[t] = dot * scale;
            if (sc[t] > m) m = sc[t];
        }
        double z = 0.0;
        for (int t = 0; t < seq_len; ++t) { sc[t] = exp(sc[t] - m); z += sc[t]; }
        double inv = 1.0 / (z + 1e-9);
        for (int i = 0; i < d; ++i) {
            double ctx = 0.0;
            for (int t = 0; t < seq_len; ++t) ctx += sc[t] * inv * (double)v_cache[(size_t)t * kv_dim + g * d + i];
            double gate = q_gate[(size_t)h * 2 * d + d + i];
            out[(size_t)h * d + i] = ctx * (1.0 / (1.0 + exp(-gate)));
        }
    }
    free(sc);
}

/* Causal prefill of T rows: row t attends cache rows 0..t (the per-token loop of
 * src/models/qwen3_5/layer.mojo:630-641 over the kernel above).  q_gate (T, H_q, 2d) fp16,
 * k/v (T, H_kv, d) fp16 with K already RoPE'd, out (T, H_q, d) fp32. */
void khq_oracle_gqa_prefill(const uint16_t* q_gate, const uint16_t* k, const uint16_t* v, float* out,
                            int T, int H_q, int H_kv, int d, float scale) {
    int group = H_q / H_kv, kv_dim = H_kv * d;
#pragma omp parallel for schedule(dynamic, 4)
    for (int t = T - 1; t >= 0; --t) {
        double* sc = (double*)malloc((size_t)(t + 1) * sizeof(double));
        for (int h = 0; h < H_q; ++h) {
            int g = h / group;
            const uint16_t* qp = q_gate + ((size_t)t * H_q + h) * 2 * d;
            double qd[KHQ_D];
            for (int i = 0; i < d; ++i) qd[i] = h2f(qp[i]);
            double m = -3.0e38;
            for (int u = 0; u <= t; ++u) {
                const uint16_t* kp = k + (size_t)u * kv_dim + g * d;
                double dot = 0.0;
                for (int i = 0; i < d; ++i) dot += qd[i] * (double)h2f(kp[i]);
                sc[u] = dot * (double)scale;
                if (sc[u] > m) m = sc[u];
            }
            double z = 0.0;
            for (int u = 0; u <= t; ++u) { sc[u] = exp(sc[u] - m); z += sc[u]; }
            double inv = 1.0 / (z + 1e-9);
            double ctx[KHQ_D];
            for (int i = 0; i < d; ++i) ctx[i] = 0.0;
            for (int u = 0; u <= t; ++u) {
                const uint16_t* vp = v + (size_t)u * kv_dim + g * d;
                double p = sc[u] * inv;
                for (int i = 0; i < d; ++i) ctx[i] += p * (double)h2f(vp[i]);
            }
            for (int i = 0; i < d; ++i) {
                double gate = h2f(qp[d + i]);
                out[((size_t)t * H_q + h) * d + i] = (float)(ctx[i] * (1.0 / (1.0 + exp(-gate))));
            }
        }
        free(sc);
    }
}

/* ================================================================== RoPE ====== */
/* Half-split partial RoPE in place on fp16 (elementwise_sm75.mojo:1023-1061):
 * pairs (i, i+rotary/2), freq = expf(logf(theta) * (-2i/rotary)), fp32 angle pos*freq. */
void khq_oracle_partial_rope(uint16_t* vec, int num_heads, int head_dim, int rotary_dim, int pos,
                             float theta, int stride) {
    int half = rotary_dim / 2;
    int st = stride > 0 ? stride : head_dim;
    for (int h = 0; h < num_heads; ++h)
        for (int i = 0; i < half; ++i) {
            float ex = -(float)(2 * i) / (float)rotary_dim;
            float freq = expf(logf(theta) * ex);
            float ang = (float)pos * freq;
            float c = cosf(ang), s = sinf(ang);
            float x0 = h2f(vec[(size_t)h * st + i]), x1 = h2f(vec[(size_t)h * st + i + half]);
            vec[(size_t)h * st + i] = f2h(x0 * c - x1 * s);
            vec[(size_t)h * st + i + half] = f2h(x0 * s + x1 * c);
        }
}

/* ============================================================ head RMSNorm ==== */
/* Per-head RMSNorm in place on fp16 (src/kernels/elementwise_sm75.mojo:362-423): one warp per
 * head; lane t sums the squares of dims t, t+32, ... in fp32, the 32 partial sums go through a
 * shuffle-down tree (offsets 16, 8, 4, 2, 1; lane 0 holds the total), scale =
 * 1/sqrt(sum/dim + eps), out = fp16(x*scale [* weight]).  The tree is reproduced so that the
 * result is bit-identical. */
void khq_oracle_head_rmsnorm(uint16_t* x, int num_heads, int head_dim, int stride, const float* weight,
                             float eps) {
    int st = stride > 0 ? stride : head_dim;
    for (int h = 0; h < num_heads; ++h) {
        uint16_t* p = x + (size_t)h * st;
        float part[64];
        for (int t = 0; t < 64; ++t) part[t] = 0.0f;
        for (int t = 0; t < 32; ++t)
            for (int d = t; d < head_dim; d += 32) {
                float v = h2f(p[d]);
                part[t] += v * v;
            }
        for (int off = 16; off > 0; off >>= 1) {
            float nxt[32];
            for (int t = 0; t < 32; ++t) nxt[t] = part[t] + ((t + off < 32) ? part[t + off] : part[t]);
            for (int t = 0; t < 32; ++t) part[t] = nxt[t];
        }
        float scale = 1.0f / sqrtf(part[0] / (float)head_dim + eps);
        for (int d = 0; d < head_dim; ++d) {
            float n = h2f(p[d]) * scale;
            if (weight) n *= weight[d];
            p[d] = f2h(n);
        }
    }
}

/* K-static calibration fit (src/csrc/qmv_sm75_kernel.cu:2645-2680, cal_kstatic_p_kernel +
 * cal_kstatic_f_kernel): per-dim sigma of the projected sample rot (rows, 256) fp32 by a serial
 * mean and a serial sum of squared deviations, ts = 16 / sqrt(sum_i 0.528756 (0.935 sigma_i)^2 +
 * 0.464545 sigma_i^2) summed serially, centroid rows {0, -cb, cb, cb} with cb = 0.935 sigma ts.
 * The device build of the reference fuses dv*dv into the running sum (-fmad=true), restated here
 * with fmaf; which product of the two-term psum expression it fuses is the compiler's choice, so
 * callers compare ts and the centroids within a few ulp. */
void khq_oracle_cal_kstatic(const float* rot, int rows, float* cents, float* out_ts, float* sigma) {
    float psum[256], sg_[256];
    for (int i = 0; i < 256; ++i) {
        float m = 0.0f;
        for (int r = 0; r < rows; ++r) m += rot[(size_t)r * 256 + i];
        m /= (float)rows;
        float v = 0.0f;
        for (int r = 0; r < rows; ++r) {
            float dv = rot[(size_t)r * 256 + i] - m;
            v = fmaf(dv, dv, v);
        }
        float sg = sqrtf(v / (float)rows);
        sg_[i] = sg;
        if (sigma) sigma[i] = sg;
        float cb = 0.9350f * sg;
        psum[i] = fmaf(0.464545f * sg, sg, 0.528756f * cb * cb);
    }
    float se = 0.0f;
    for (int i = 0; i < 256; ++i) se += psum[i];
    float ts = 16.0f / sqrtf(se);
    for (int i = 0; i < 256; ++i) {
        float cb = 0.9350f * sg_[i] * ts;
        cents[0 * 256 + i] = 0.0f;
        cents[1 * 256 + i] = -cb;
        cents[2 * 256 + i] = cb;
        cents[3 * 256 + i] = cb;
    }
    out_ts[0] = ts;
}
