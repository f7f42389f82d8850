// khq_compress.cu -- KHQ compress for sm_100a: one warp per (token, kv-head) row, or per group of
// two (K) or four (V) rows in large launches.
//
// Code words must be bit-identical to the reference kernel's, which evaluates every row in one
// thread in a fixed fp32 order.  The work is therefore split in two kinds:
//   * order-insensitive steps run lane-parallel: the FWHT butterflies (each output of a stage is
//     the same a+b / a-b whatever thread computes it), the per-patch 4x4 rotor (the k-chain of a
//     patch stays inside one lane), the 64x256 VQ search (lexicographic (distance, index)
//     minimum == first strict minimum of an ascending scan), max reductions, bit packing;
//   * the few order-sensitive scalar sums (sum of squares over 256 dims, the two conditional
//     sums behind the K base multiplier, the two 64-term energy sums of V) are staged in shared
//     memory and accumulated strictly in index order; with a group of R rows lane l follows the
//     chain of row l % R, so one pass serves R rows.
// Arithmetic that feeds a threshold or a rounding is written with explicit __fmaf_rn where the
// reference's build (default -fmad=true) fuses a multiply into the following add/subtract.
#include "khq_common.cuh"

namespace khq {

constexpr int CMP_WARPS = 4;  // warps per block, each on its own row or group of rows
constexpr int CMP_KROWS = 2;  // rows of a K group (large launches); four would halve the blocks per SM
constexpr int CMP_VROWS = 4;  // rows a warp carries through the V code search together (large launches)
// Below this a launch keeps one row per warp: groups of rows would leave SMs without work
// (148 SMs x 8 blocks x 4 warps x 4 rows = 18 944 rows fill the GPU once).
constexpr long long CMP_VROWS_MIN_N = 24576;

// One run of rows of a batched launch: source rows (fp16, D per row, contiguous) and the first
// output row in the launch's output arrays (mirrored in include/khq_b200.h).
struct KhqCompressSeg {
    const __half* x;
    long long row0;
};
static_assert(sizeof(KhqCompressSeg) == 16, "ABI");

// Row strides of D + 4 (and NP + 4) floats: the in-order sums read R rows at once (lane l
// follows row l % R), and the odd multiple of 16 bytes keeps those 16-byte reads on different banks.
template <int R>
struct CompressScratchK {
    float a[R][D + 4];      // x as float, then per-dim |proj| contributions
    float b[R][D + 4];      // per-dim centroid contributions
    float q[R][D];          // the rotated projection
    int incl[R][32];        // per lane: outlier candidates up to and including the lane's dims
    unsigned char oc[64];   // outlier 4-bit codes, by outlier ordinal
    unsigned char os[64];   // outlier sign flags, by outlier ordinal
};

template <int R>
struct CompressScratchV {
    float p[R][D + 4];           // x as float, then the rotated projection, per row of the group
    float a[R][NP + 4];          // per-patch true energies
    float b[R][NP + 4];          // per-patch codebook energies
    unsigned short code[R][NP];  // chosen code per (row, patch)
};

// One launch over one contiguous run of rows (segs == nullptr: input row = output row), or over
// many runs of rows_per_seg rows, each with its own source and first output row.
__device__ __forceinline__ const __half* compress_map_row(const __half* x, const KhqCompressSeg* segs,
                                                          int rows_per_seg, long long x_byte_offset,
                                                          long long lrow, long long& row) {
    row = lrow;
    if (segs == nullptr) return x + lrow * D;
    const KhqCompressSeg sg = segs[lrow / rows_per_seg];
    const long long rr = lrow % rows_per_seg;
    row = sg.row0 + rr;
    return reinterpret_cast<const __half*>(reinterpret_cast<const char*>(sg.x) + x_byte_offset) + rr * D;
}

// Normalisation, FWHT-256 and the 4x4 rotor of one row whose norm is known; lane owns dims
// 8*lane .. 8*lane+7 (xv).
__device__ __forceinline__ void compress_rotate(const float (&xv)[8], float norm,
                                                const __half* __restrict__ d_vec,
                                                const __half* __restrict__ rotor, float f_s, int lane,
                                                float (&proj)[8]) {
    const float den = norm + 1e-8f;

    const uint4 draw = *reinterpret_cast<const uint4*>(d_vec + lane * 8);
    const __half* hd = reinterpret_cast<const __half*>(&draw);
    float r[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = __fdiv_rn(xv[j] * __half2float(hd[j]), den);
    fwht256_lane8(r, lane);

    // 4x4 rotor of the lane's two patches: rot[c] = sum_k r[k] * R[k][c], k ascending
#pragma unroll
    for (int p = 0; p < 2; ++p) {
        const uint4* rp = reinterpret_cast<const uint4*>(rotor + (lane * 2 + p) * 16);
        const uint4 r0 = rp[0], r1 = rp[1];
        __half hr[16];
        *reinterpret_cast<uint4*>(&hr[0]) = r0;
        *reinterpret_cast<uint4*>(&hr[8]) = r1;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            float acc = 0.0f;
#pragma unroll
            for (int k = 0; k < 4; ++k)
                acc = __fmaf_rn(r[p * 4 + k], __half2float(hr[k * 4 + c]), acc);
            proj[p * 4 + c] = acc * f_s;
        }
    }
}

// ============ K rows: a warp takes a group of R rows; their in-order sums run side by side ============
// The three order-sensitive sums of a K row (256 squares, then the two conditional 256-term sums
// behind the base multiplier) are dependent chains that every lane of the warp would compute
// alike; with R rows per warp lane l follows row l % R, so one pass over shared memory serves R
// rows.  Between the passes a row's projection and outlier ordinals wait in shared memory.
template <int R>
__global__ void __launch_bounds__(CMP_WARPS * 32, 8)
khq_compress_k_kernel(const __half* __restrict__ x, const __half* __restrict__ d_vec,
                      const __half* __restrict__ rotor, const __half* __restrict__ cents,
                      unsigned int* __restrict__ out_mask, __half* __restrict__ out_norms,
                      __half* __restrict__ out_r_norms, unsigned char* __restrict__ out_payload,
                      unsigned char* __restrict__ out_shared_meta, int d_val, int n, float ts,
                      const KhqCompressSeg* __restrict__ segs, int rows_per_seg,
                      long long x_byte_offset) {
    __shared__ __align__(16) CompressScratchK<R> scratch[CMP_WARPS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    CompressScratchK<R>& S = scratch[warp];
    // The reference computes this factor at run time from the dimension argument.
    const float f_s = rsqrtf((float)d_val);
    const float th_out = 1.60f * f_s, th_lo = 0.47f * f_s;
    const long long n_groups = ((long long)n + R - 1) / R;
    const int cr = lane & (R - 1);
    float cb[8];  // the lane's 8 dims of the centroid row the base multiplier is fitted to
    {
        const uint4 craw = *reinterpret_cast<const uint4*>(cents + 2 * D + lane * 8);
        const __half* hc = reinterpret_cast<const __half*>(&craw);
#pragma unroll
        for (int j = 0; j < 8; ++j) cb[j] = __half2float(hc[j]);
    }

    for (long long grp = (long long)blockIdx.x * CMP_WARPS + warp; grp < n_groups;
         grp += (long long)gridDim.x * CMP_WARPS) {
        const long long l0 = grp * R;
        const int nr = (n - l0 < R) ? (int)(n - l0) : R;
        // ---- the rows as fp32 in shared memory, then their sums of squares in dim order ----------
#pragma unroll 1
        for (int r = 0; r < nr; ++r) {
            long long row;
            const __half* xrow = compress_map_row(x, segs, rows_per_seg, x_byte_offset, l0 + r, row);
            const uint4 raw = *reinterpret_cast<const uint4*>(xrow + lane * 8);
            const __half2* hx = reinterpret_cast<const __half2*>(&raw);
            const float2 x0 = __half22float2(hx[0]), x1 = __half22float2(hx[1]), x2 = __half22float2(hx[2]),
                         x3 = __half22float2(hx[3]);
            *reinterpret_cast<float4*>(&S.a[r][lane * 8]) = make_float4(x0.x, x0.y, x1.x, x1.y);
            *reinterpret_cast<float4*>(&S.a[r][lane * 8 + 4]) = make_float4(x2.x, x2.y, x3.x, x3.y);
        }
        __syncwarp();
        float sum_sq = 0.0f;
#pragma unroll 8
        for (int i = 0; i < D; i += 4) {
            const float4 t = *reinterpret_cast<const float4*>(&S.a[cr][i]);
            sum_sq = __fmaf_rn(t.x, t.x, sum_sq);
            sum_sq = __fmaf_rn(t.y, t.y, sum_sq);
            sum_sq = __fmaf_rn(t.z, t.z, sum_sq);
            sum_sq = __fmaf_rn(t.w, t.w, sum_sq);
        }
        __syncwarp();
        // ---- per row: projection, symbols, mask words, the terms of the two conditional sums ------
#pragma unroll 1
        for (int r = 0; r < nr; ++r) {
            long long row;
            (void)compress_map_row(x, segs, rows_per_seg, x_byte_offset, l0 + r, row);
            const float norm = sqrtf(__shfl_sync(0xFFFFFFFFu, sum_sq, r) + 1e-8f);
            if (lane == 0) out_norms[row] = __float2half(norm);
            float xv[8], proj[8];
            *reinterpret_cast<float4*>(&xv[0]) = *reinterpret_cast<const float4*>(&S.a[r][lane * 8]);
            *reinterpret_cast<float4*>(&xv[4]) = *reinterpret_cast<const float4*>(&S.a[r][lane * 8 + 4]);
            compress_rotate(xv, norm, d_vec, rotor, f_s, lane, proj);
            *reinterpret_cast<float4*>(&S.q[r][lane * 8]) = make_float4(proj[0], proj[1], proj[2], proj[3]);
            *reinterpret_cast<float4*>(&S.q[r][lane * 8 + 4]) = make_float4(proj[4], proj[5], proj[6], proj[7]);

            unsigned cand = 0;  // dims whose |proj| is above the outlier threshold
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (fabsf(proj[j]) > th_out) cand |= 1u << j;
            // ordinal of the lane's first candidate among all candidates, in dim order
            const int cnt = __popc(cand);
            int incl = cnt;
#pragma unroll
            for (int dlt = 1; dlt < 32; dlt <<= 1) {
                const int t = __shfl_up_sync(0xFFFFFFFFu, incl, dlt);
                if (lane >= dlt) incl += t;
            }
            S.incl[r][lane] = incl;
            int ord = incl - cnt;

            unsigned sym16 = 0;
            float cn[8], cc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float pj = proj[j];
                unsigned sym;
                cn[j] = 0.0f;
                cc[j] = 0.0f;
                if (cand & (1u << j)) {
                    // kept outlier, or overflow outlier (not part of the sums)
                    sym = (ord < MAX_OUT) ? 3u : ((pj > 0.0f) ? 2u : 1u);
                    ++ord;
                } else {
                    if (pj > th_lo) sym = 2;
                    else if (pj < -th_lo) sym = 1;
                    else sym = 0;
                    if (sym != 0) { cn[j] = fabsf(pj); cc[j] = cb[j]; }
                }
                sym16 |= sym << (2 * j);
            }
            // adding +0.0f leaves a non-negative fp32 sum unchanged
            *reinterpret_cast<float4*>(&S.a[r][lane * 8]) = make_float4(cn[0], cn[1], cn[2], cn[3]);
            *reinterpret_cast<float4*>(&S.a[r][lane * 8 + 4]) = make_float4(cn[4], cn[5], cn[6], cn[7]);
            *reinterpret_cast<float4*>(&S.b[r][lane * 8]) = make_float4(cc[0], cc[1], cc[2], cc[3]);
            *reinterpret_cast<float4*>(&S.b[r][lane * 8 + 4]) = make_float4(cc[4], cc[5], cc[6], cc[7]);
            // mask word w = dims 16w..16w+15 = lanes 2w (low half) and 2w+1 (high half)
            const unsigned hi16 = __shfl_down_sync(0xFFFFFFFFu, sym16, 1);
            if ((lane & 1) == 0) out_mask[row * 16 + (lane >> 1)] = sym16 | (hi16 << 16);
        }
        __syncwarp();
        // ---- the two conditional sums in dim order, R rows side by side ------------------------
        float sum_n = 0.0f, sum_c = 0.0f;
#pragma unroll 8
        for (int i = 0; i < D; i += 4) {
            const float4 ta = *reinterpret_cast<const float4*>(&S.a[cr][i]);
            const float4 tb = *reinterpret_cast<const float4*>(&S.b[cr][i]);
            sum_n += ta.x; sum_c += tb.x;
            sum_n += ta.y; sum_c += tb.y;
            sum_n += ta.z; sum_c += tb.z;
            sum_n += ta.w; sum_c += tb.w;
        }
        float mult_own = (sum_c > 1e-5f) ? __fdiv_rn(sum_n, sum_c) : 1.0f;
        if (mult_own < 0.1f || mult_own > 10.0f || isnan(mult_own)) mult_own = 1.0f;
        // ---- per row: residuals of the kept outliers, their scale, the 40 payload bytes ----------
#pragma unroll 1
        for (int r = 0; r < nr; ++r) {
            long long row;
            (void)compress_map_row(x, segs, rows_per_seg, x_byte_offset, l0 + r, row);
            const float mult = __shfl_sync(0xFFFFFFFFu, mult_own, r);
            float proj[8];
            *reinterpret_cast<float4*>(&proj[0]) = *reinterpret_cast<const float4*>(&S.q[r][lane * 8]);
            *reinterpret_cast<float4*>(&proj[4]) = *reinterpret_cast<const float4*>(&S.q[r][lane * 8 + 4]);
            unsigned cand = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (fabsf(proj[j]) > th_out) cand |= 1u << j;
            int ord = S.incl[r][lane] - __popc(cand);
            const int total_cand = S.incl[r][31];
            const int n_out = total_cand < MAX_OUT ? total_cand : MAX_OUT;

            float res[8];
            int o_ord[8];
            float max_res = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                res[j] = 0.0f;
                o_ord[j] = -1;
                if (cand & (1u << j)) {
                    if (ord < MAX_OUT) {
                        o_ord[j] = ord;
                        res[j] = fmaxf(0.0f, __fmaf_rn(-cb[j], mult, fabsf(proj[j] * ts)));
                        max_res = fmaxf(max_res, res[j]);
                    }
                    ++ord;
                }
            }
#pragma unroll
            for (int m = 16; m > 0; m >>= 1)
                max_res = fmaxf(max_res, __shfl_xor_sync(0xFFFFFFFFu, max_res, m));
            const float rscale = (n_out > 0) ? __fdiv_rn(fmaxf(max_res, 1e-4f), 15.0f) : 0.0f;
            if (lane == 0) {
                out_r_norms[row] = __float2half(rscale);
                *reinterpret_cast<unsigned int*>(out_shared_meta + row * 4) = 0u;
            }
            // stage codes and signs by ordinal, then assemble the 40 payload bytes
            if (lane < 16) reinterpret_cast<unsigned int*>(S.oc)[lane] = 0u;
            else reinterpret_cast<unsigned int*>(S.os)[lane - 16] = 0u;
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (o_ord[j] >= 0) {
                    unsigned char code = 0;
                    if (rscale > 0.0f) {
                        const float r4 = roundf(__fdiv_rn(res[j], rscale));
                        code = (unsigned char)fmaxf(0.0f, fminf(15.0f, r4));
                    }
                    S.oc[o_ord[j]] = code;
                    S.os[o_ord[j]] = (proj[j] > 0.0f) ? 1 : 0;
                }
            }
            __syncwarp();
            if (lane < 10) {
                unsigned int word = 0;
#pragma unroll
                for (int bb = 0; bb < 4; ++bb) {
                    const int byte = lane * 4 + bb;
                    unsigned int v = 0;
                    if (byte < 4) {
                        const unsigned int mu = (unsigned int)(mult * 1000.0f);
                        v = (mu >> (8 * byte)) & 0xFFu;
                    } else if (byte < 29) {
                        const int j0 = (byte - 4) * 2;
                        v = (unsigned)S.oc[j0] | ((unsigned)S.oc[j0 + 1] << 4);
                    } else if (byte < 36) {
                        const int j0 = (byte - 29) * 8;
#pragma unroll
                        for (int t = 0; t < 8; ++t)
                            if (j0 + t < MAX_OUT) v |= (unsigned)S.os[j0 + t] << t;
                    } else if (byte == 36) {
                        v = 0x02u;
                    }
                    word |= v << (8 * bb);
                }
                reinterpret_cast<unsigned int*>(out_payload + row * K_PAY)[lane] = word;
            }
            __syncwarp();
        }
    }
}

// packed pairs of fp32: one instruction, each half rounded like the scalar operation
__device__ __forceinline__ unsigned long long f2_pack(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void f2_unpack(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long f2_fma(unsigned long long a, unsigned long long b,
                                                     unsigned long long c) {
    unsigned long long r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ unsigned long long f2_mul(unsigned long long a, unsigned long long b) {
    unsigned long long r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

__device__ __forceinline__ float f_min3(float a, float b, float c) {
    float d;
    asm("min.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// Code search of one (row, patch): every lane scans its 8 consecutive codes in ascending order, then
// the warp takes the lexicographic (distance, index) minimum.  cc[k][i] = (code 2i, code 2i+1) of
// dim k of the lane's 8 codes, as packed fp32 pairs.
__device__ __forceinline__ void v_search_row(const float* __restrict__ proj_row, unsigned short* __restrict__ code_row,
                                             int p, const unsigned long long (&cc)[3][4],
                                             unsigned long long nalpha2, int lane) {
    const float4 v = *reinterpret_cast<const float4*>(&proj_row[p * 4]);
    const unsigned long long v0 = f2_pack(v.x, v.x), v1 = f2_pack(v.y, v.y), v2 = f2_pack(v.z, v.z);
    float dist[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        // d = v - c * alpha with one rounding (c * -alpha is the exact negative of c * alpha),
        // dist = d2*d2 + (d0*d0 + d1*d1) in the reference's order
        const unsigned long long d0 = f2_fma(cc[0][i], nalpha2, v0);
        const unsigned long long d1 = f2_fma(cc[1][i], nalpha2, v1);
        const unsigned long long d2 = f2_fma(cc[2][i], nalpha2, v2);
        f2_unpack(f2_fma(d2, d2, f2_fma(d0, d0, f2_mul(d1, d1))), dist[2 * i], dist[2 * i + 1]);
    }
    // The reference's ascending scan from 1e20 with a strict '<' ends on the smallest distance
    // below 1e20 and on the first index that has it: the minimum first (three-input minima, which
    // pass over a NaN), then the first index equal to it.
    const float best = f_min3(f_min3(dist[0], dist[1], dist[2]), f_min3(dist[3], dist[4], dist[5]),
                              f_min3(dist[6], dist[7], 1e20f));
    unsigned bl = 7;  // index among the lane's 8 codes
#pragma unroll
    for (int i = 6; i >= 0; --i)
        if (dist[i] == best) bl = i;
    // warp minimum of (distance, index): a lane's best is a non-negative, non-NaN float (at most
    // 1e20), so its bit pattern orders like the value and two hardware warp reductions do the
    // work of five shuffle-and-compare steps
    const unsigned best_bits = __reduce_min_sync(0xFFFFFFFFu, __float_as_uint(best));
    unsigned bi = __reduce_min_sync(0xFFFFFFFFu, (__float_as_uint(best) == best_bits) ? (unsigned)(lane * 8) + bl : 0xFFFFFFFFu);
    // The reference starts from min=1e20 with a strict '<': if no distance is below 1e20
    // (NaN/inf input) it keeps code 0.
    if (!(__uint_as_float(best_bits) < 1e20f)) bi = 0;
    if (lane == 0) code_row[p] = (unsigned short)bi;
}

// ============ V rows: a warp takes R rows through the code search on one codebook load ============
// The search dominates a V row (64 patches x 256 codes); the codebook slice a lane scans (8 codes
// of the patch) is loaded and converted once per patch and used for the R rows of the group.
template <int R>
__global__ void __launch_bounds__(CMP_WARPS * 32, 8)
khq_compress_v_kernel(const __half* __restrict__ x, const __half* __restrict__ d_vec,
                      const __half* __restrict__ rotor, const __half* __restrict__ cents,
                      const __half* __restrict__ vq, __half* __restrict__ out_norms,
                      __half* __restrict__ out_r_norms, unsigned char* __restrict__ out_payload,
                      unsigned char* __restrict__ out_shared_meta, int d_val, int n, float alpha,
                      const KhqCompressSeg* __restrict__ segs, int rows_per_seg,
                      long long x_byte_offset) {
    __shared__ __align__(16) CompressScratchV<R> scratch[CMP_WARPS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    CompressScratchV<R>& S = scratch[warp];
    const float f_s = rsqrtf((float)d_val);
    const long long n_groups = ((long long)n + R - 1) / R;

    for (long long grp = (long long)blockIdx.x * CMP_WARPS + warp; grp < n_groups;
         grp += (long long)gridDim.x * CMP_WARPS) {
        const long long l0 = grp * R;
        const int nr = (n - l0 < R) ? (int)(n - l0) : R;
        // ---- front of every row of the group; the projection stays in shared memory ------------
#pragma unroll 1
        for (int r = 0; r < nr; ++r) {
            long long row;
            const __half* xrow = compress_map_row(x, segs, rows_per_seg, x_byte_offset, l0 + r, row);
            const uint4 raw = *reinterpret_cast<const uint4*>(xrow + lane * 8);
            const __half2* hx = reinterpret_cast<const __half2*>(&raw);
            const float2 x0 = __half22float2(hx[0]), x1 = __half22float2(hx[1]), x2 = __half22float2(hx[2]),
                         x3 = __half22float2(hx[3]);
            *reinterpret_cast<float4*>(&S.p[r][lane * 8]) = make_float4(x0.x, x0.y, x1.x, x1.y);
            *reinterpret_cast<float4*>(&S.p[r][lane * 8 + 4]) = make_float4(x2.x, x2.y, x3.x, x3.y);
        }
        __syncwarp();
        // sums of squares strictly in dim order, the R rows at once: lane l follows row l % R
        const int cr = lane & (R - 1);
        float sum_sq = 0.0f;
#pragma unroll 8
        for (int i = 0; i < D; i += 4) {
            const float4 t = *reinterpret_cast<const float4*>(&S.p[cr][i]);
            sum_sq = __fmaf_rn(t.x, t.x, sum_sq);
            sum_sq = __fmaf_rn(t.y, t.y, sum_sq);
            sum_sq = __fmaf_rn(t.z, t.z, sum_sq);
            sum_sq = __fmaf_rn(t.w, t.w, sum_sq);
        }
        __syncwarp();
#pragma unroll 1
        for (int r = 0; r < nr; ++r) {
            long long row;
            (void)compress_map_row(x, segs, rows_per_seg, x_byte_offset, l0 + r, row);
            const float norm = sqrtf(__shfl_sync(0xFFFFFFFFu, sum_sq, r) + 1e-8f);
            if (lane == 0) out_norms[row] = __float2half(norm);
            float xv[8], proj[8];
            *reinterpret_cast<float4*>(&xv[0]) = *reinterpret_cast<const float4*>(&S.p[r][lane * 8]);
            *reinterpret_cast<float4*>(&xv[4]) = *reinterpret_cast<const float4*>(&S.p[r][lane * 8 + 4]);
            compress_rotate(xv, norm, d_vec, rotor, f_s, lane, proj);
            *reinterpret_cast<float4*>(&S.p[r][lane * 8]) = make_float4(proj[0], proj[1], proj[2], proj[3]);
            *reinterpret_cast<float4*>(&S.p[r][lane * 8 + 4]) = make_float4(proj[4], proj[5], proj[6], proj[7]);
        }
        __syncwarp();
        // ---- code search: for each patch every lane scans 8 consecutive codes in ascending
        // order, then the warp takes the lexicographic (distance, index) minimum -----------------
        const unsigned long long nalpha2 = f2_pack(-alpha, -alpha);
#pragma unroll 1
        for (int p = 0; p < NP; ++p) {
            const uint4* cbp = reinterpret_cast<const uint4*>(vq + ((size_t)p * 256 + lane * 8) * 3);
            __half hcb[24];
            *reinterpret_cast<uint4*>(&hcb[0]) = __ldg(cbp);
            *reinterpret_cast<uint4*>(&hcb[8]) = __ldg(cbp + 1);
            *reinterpret_cast<uint4*>(&hcb[16]) = __ldg(cbp + 2);
            // the lane's 8 codes x 3 dims as fp32 (exact), paired by neighbouring codes:
            // cc[k][i] = (code 2i, code 2i+1) of dim k
            unsigned long long cc[3][4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int k = 0; k < 3; ++k)
                    cc[k][i] = f2_pack(__half2float(hcb[6 * i + k]), __half2float(hcb[6 * i + 3 + k]));
            if (nr == R) {
#pragma unroll
                for (int r = 0; r < R; ++r)
                    v_search_row(S.p[r], S.code[r], p, cc, nalpha2, lane);
            } else {
                for (int r = 0; r < nr; ++r) v_search_row(S.p[r], S.code[r], p, cc, nalpha2, lane);
            }
        }
        __syncwarp();
        // ---- per row: energies, dim-3 centroid choice, residual, packing ------------------------
#pragma unroll 1
        for (int r = 0; r < nr; ++r) {
            long long row;
            (void)compress_map_row(x, segs, rows_per_seg, x_byte_offset, l0 + r, row);
            float proj[8];
            *reinterpret_cast<float4*>(&proj[0]) = *reinterpret_cast<const float4*>(&S.p[r][lane * 8]);
            *reinterpret_cast<float4*>(&proj[4]) = *reinterpret_cast<const float4*>(&S.p[r][lane * 8 + 4]);
            unsigned code[2];
            {
                const unsigned pr = *reinterpret_cast<const unsigned*>(&S.code[r][lane * 2]);
                code[0] = pr & 0xFFFFu;
                code[1] = pr >> 16;
            }
            // per-patch energies, dim-3 centroid choice and residual (in the owning lane)
            float e_true[2], e_vq[2], pres[2];
            unsigned sel[2];
            float max_res = 0.0f;
#pragma unroll
            for (int p = 0; p < 2; ++p) {
                const int pid = lane * 2 + p;
                const float v0 = proj[p * 4 + 0], v1 = proj[p * 4 + 1], v2 = proj[p * 4 + 2];
                const __half* cbp = vq + ((size_t)pid * 256 + code[p]) * 3;
                const float b0 = __half2float(cbp[0]) * alpha;
                const float b1 = __half2float(cbp[1]) * alpha;
                const float b2 = __half2float(cbp[2]) * alpha;
                e_true[p] = __fmaf_rn(v2, v2, __fmaf_rn(v0, v0, v1 * v1));
                e_vq[p] = __fmaf_rn(b2, b2, __fmaf_rn(b0, b0, b1 * b1));
                const float v3 = proj[p * 4 + 3];
                const float c0 = __half2float(cents[0 * D + pid * 4 + 3]);
                const float c1 = __half2float(cents[1 * D + pid * 4 + 3]);
                const float dist0 = fabsf(__fmaf_rn(-c0, alpha, v3));
                const float dist1 = fabsf(__fmaf_rn(-c1, alpha, v3));
                // ascending scan from min=1e20 with strict '<': index 1 only when strictly closer
                unsigned s = 0;
                float bd = 1e20f;
                if (dist0 < bd) { bd = dist0; s = 0; }
                if (dist1 < bd) { bd = dist1; s = 1; }
                sel[p] = s;
                const float cbest = s ? c1 : c0;
                pres[p] = __fmaf_rn(-cbest, alpha, v3);
                max_res = fmaxf(max_res, fabsf(pres[p]));
                S.a[r][pid] = e_true[p];
                S.b[r][pid] = e_vq[p];
            }
#pragma unroll
            for (int m = 16; m > 0; m >>= 1)
                max_res = fmaxf(max_res, __shfl_xor_sync(0xFFFFFFFFu, max_res, m));
            if (lane == 0) *reinterpret_cast<float*>(out_shared_meta + row * 4) = max_res;
            const float rs = fmaxf(max_res, 1e-4f);
            unsigned f24 = 0, hb = 0;
#pragma unroll
            for (int p = 0; p < 2; ++p) {
                const float scaled = __fmaf_rn(__fdiv_rn(pres[p], rs), 7.0f, 8.0f);
                const unsigned dump = (unsigned)fmaxf(0.0f, fminf(15.0f, roundf(scaled)));
                const unsigned f = (code[p] & 0x7Fu) | ((sel[p] & 1u) << 7) | ((dump & 0xFu) << 8);
                f24 |= f << (12 * p);
                hb |= ((code[p] >> 7) & 1u) << p;
            }
            // 8 patches = 4 lanes = 96 bits = 3 words; lane k of the quad holds bits [24k, 24k+24)
            const unsigned nxt = __shfl_down_sync(0xFFFFFFFFu, f24, 1);
            unsigned int* prow = reinterpret_cast<unsigned int*>(out_payload + row * V_PAY);
            const int k4 = lane & 3, g = lane >> 2;
            if (k4 == 0) prow[g * 3 + 0] = f24 | (nxt << 24);
            else if (k4 == 1) prow[g * 3 + 1] = (f24 >> 8) | (nxt << 16);
            else if (k4 == 2) prow[g * 3 + 2] = (f24 >> 16) | (nxt << 8);
            const unsigned hv = hb << (2 * (lane & 15));
            const unsigned lo = __reduce_or_sync(0xFFFFFFFFu, lane < 16 ? hv : 0u);
            const unsigned hi = __reduce_or_sync(0xFFFFFFFFu, lane >= 16 ? hv : 0u);
            if (lane == 0) { prow[24] = lo; prow[25] = hi; }
        }
        __syncwarp();
        // the two energy sums strictly in patch order, the R rows at once
        float st = 0.0f, sv = 0.0f;
#pragma unroll 4
        for (int i = 0; i < NP; i += 4) {
            const float4 ta = *reinterpret_cast<const float4*>(&S.a[cr][i]);
            const float4 tb = *reinterpret_cast<const float4*>(&S.b[cr][i]);
            st += ta.x; sv += tb.x;
            st += ta.y; sv += tb.y;
            st += ta.z; sv += tb.z;
            st += ta.w; sv += tb.w;
        }
        if (lane < nr) {
            long long row;
            (void)compress_map_row(x, segs, rows_per_seg, x_byte_offset, l0 + lane, row);
            out_r_norms[row] = __float2half(sqrtf(__fdiv_rn(st, sv + 1e-8f)));
        }
        __syncwarp();
    }
}

}  // namespace khq

namespace {
int compress_launch(const __half* x, const void* d_vec, const void* rotor, const void* centroids,
                    const void* vq_centroids, void* out_mask, void* out_norms, void* out_r_norms,
                    void* out_payload, void* out_shared_meta, int d, int n, float threshold_scale, float alpha,
                    int is_v, const khq::KhqCompressSeg* segs, int rows_per_seg, long long x_byte_offset,
                    cudaStream_t stream) {
    using namespace khq;
    const long long cap = 148LL * 64;  // grid-stride beyond this
    const auto grid = [&](long long units) {
        long long blocks = (units + CMP_WARPS - 1) / CMP_WARPS;
        return (unsigned)(blocks > cap ? cap : blocks);
    };
    const __half* dv = static_cast<const __half*>(d_vec);
    const __half* ro = static_cast<const __half*>(rotor);
    const __half* ce = static_cast<const __half*>(centroids);
    __half* on = static_cast<__half*>(out_norms);
    __half* orn = static_cast<__half*>(out_r_norms);
    unsigned char* op = static_cast<unsigned char*>(out_payload);
    unsigned char* om = static_cast<unsigned char*>(out_shared_meta);
    if (!is_v && n >= CMP_VROWS_MIN_N) {
        khq_compress_k_kernel<CMP_KROWS><<<grid(((long long)n + CMP_KROWS - 1) / CMP_KROWS), CMP_WARPS * 32, 0,
                                           stream>>>(x, dv, ro, ce, static_cast<unsigned int*>(out_mask), on, orn, op,
                                                     om, d, n, threshold_scale, segs, rows_per_seg, x_byte_offset);
    } else if (!is_v) {
        khq_compress_k_kernel<1><<<grid(n), CMP_WARPS * 32, 0, stream>>>(
            x, dv, ro, ce, static_cast<unsigned int*>(out_mask), on, orn, op, om, d, n, threshold_scale, segs,
            rows_per_seg, x_byte_offset);
    } else if (n >= CMP_VROWS_MIN_N) {
        khq_compress_v_kernel<CMP_VROWS><<<grid(((long long)n + CMP_VROWS - 1) / CMP_VROWS), CMP_WARPS * 32, 0,
                                           stream>>>(x, dv, ro, ce, static_cast<const __half*>(vq_centroids), on, orn,
                                                     op, om, d, n, alpha, segs, rows_per_seg, x_byte_offset);
    } else {
        khq_compress_v_kernel<1><<<grid(n), CMP_WARPS * 32, 0, stream>>>(
            x, dv, ro, ce, static_cast<const __half*>(vq_centroids), on, orn, op, om, d, n, alpha, segs,
            rows_per_seg, x_byte_offset);
    }
    const cudaError_t err = cudaGetLastError();
    return (err == cudaSuccess) ? 0 : static_cast<int>(err);
}
}  // namespace

extern "C" int launch_khq_compress_fp16(const void* x, const void* d_vec, const void* rotor,
                                        const void* centroids, const void* vq_centroids,
                                        void* out_mask, void* out_norms, void* out_r_norms,
                                        void* out_payload, void* out_shared_meta, int n, int d,
                                        float threshold_scale, float alpha, int is_v,
                                        cudaStream_t stream) {
    using namespace khq;
    if (n <= 0 || d != D) return -100;
    return compress_launch(static_cast<const __half*>(x), d_vec, rotor, centroids, vq_centroids, out_mask,
                           out_norms, out_r_norms, out_payload, out_shared_meta, d, n, threshold_scale,
                           alpha, is_v, nullptr, 1, 0, stream);
}

// Many compression events in one launch: `n_seg` runs of `rows_per_seg` rows (512 = the 128 oldest
// tokens of one sequence's ring), run i read from segs[i].x and written to rows segs[i].row0 .. of
// the output arrays.  `segs` is a device array; x_byte_offset is added to every run's source address
// (a host that keeps K and V rings at a fixed distance uses one table for both launches).  Same
// arithmetic, row by row, as the single launch.
extern "C" int launch_khq_compress_batched_fp16(const void* segs, int n_seg, int rows_per_seg, const void* d_vec,
                                                const void* rotor, const void* centroids, const void* vq_centroids,
                                                void* out_mask, void* out_norms, void* out_r_norms, void* out_payload,
                                                void* out_shared_meta, int d, float threshold_scale, float alpha,
                                                int is_v, long long x_byte_offset, cudaStream_t stream) {
    using namespace khq;
    if (n_seg <= 0 || rows_per_seg <= 0 || d != D || !segs) return -100;
    if ((x_byte_offset & 15) != 0) return -104;
    const long long n = (long long)n_seg * rows_per_seg;
    if (n > 0x7FFFFFFFLL) return -100;
    return compress_launch(nullptr, d_vec, rotor, centroids, vq_centroids, out_mask, out_norms, out_r_norms,
                           out_payload, out_shared_meta, d, (int)n, threshold_scale, alpha, is_v,
                           static_cast<const khq::KhqCompressSeg*>(segs), rows_per_seg, x_byte_offset, stream);
}
