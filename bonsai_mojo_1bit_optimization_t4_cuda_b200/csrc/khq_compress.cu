// khq_compress.cu -- KHQ compress for sm_100a: one warp per (token, kv-head) row.
//
// Code words must be bit-identical to the reference kernel's, which evaluates every row in one
// thread in a fixed fp32 order.  The work is therefore split in two kinds:
//   * order-insensitive steps run lane-parallel: the FWHT butterflies (each output of a stage is
//     the same a+b / a-b whatever thread computes it), the per-patch 4x4 rotor (the k-chain of a
//     patch stays inside one lane), the 64x256 VQ search (lexicographic (distance, index)
//     minimum == first strict minimum of an ascending scan), max reductions, bit packing;
//   * the few order-sensitive scalar sums (sum of squares over 256 dims, the two conditional
//     sums behind the K base multiplier, the two 64-term energy sums of V) are staged in shared
//     memory and accumulated strictly in index order.
// Arithmetic that feeds a threshold or a rounding is written with explicit __fmaf_rn where the
// reference's build (default -fmad=true) fuses a multiply into the following add/subtract.
#include "khq_common.cuh"

namespace khq {

constexpr int CMP_WARPS = 4;  // rows per block

// One run of rows of a batched launch: source rows (fp16, D per row, contiguous) and the first
// output row in the launch's output arrays (mirrored in include/khq_b200.h).
struct KhqCompressSeg {
    const __half* x;
    long long row0;
};
static_assert(sizeof(KhqCompressSeg) == 16, "ABI");

struct CompressScratch {
    float a[D];             // x as float, then per-dim |proj| contributions
    float b[D];             // per-dim centroid contributions
    unsigned char oc[64];   // outlier 4-bit codes, by outlier ordinal
    unsigned char os[64];   // outlier sign flags, by outlier ordinal
};

__global__ void __launch_bounds__(CMP_WARPS * 32, 8)
khq_compress_kernel(const __half* __restrict__ x, const __half* __restrict__ d_vec,
                    const __half* __restrict__ rotor, const __half* __restrict__ cents,
                    const __half* __restrict__ vq, unsigned int* __restrict__ out_mask,
                    __half* __restrict__ out_norms, __half* __restrict__ out_r_norms,
                    unsigned char* __restrict__ out_payload,
                    unsigned char* __restrict__ out_shared_meta, int d_val, int n, float ts,
                    float alpha, int is_v, const KhqCompressSeg* __restrict__ segs, int rows_per_seg,
                    long long x_byte_offset) {
    __shared__ CompressScratch scratch[CMP_WARPS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    CompressScratch& S = scratch[warp];
    // The reference computes this factor at run time from the dimension argument.
    const float f_s = rsqrtf((float)d_val);

    for (long long lrow = (long long)blockIdx.x * CMP_WARPS + warp; lrow < n;
         lrow += (long long)gridDim.x * CMP_WARPS) {
        // One launch over one contiguous run of rows (segs == nullptr: input row = output row), or
        // over many runs of rows_per_seg rows, each with its own source and first output row.
        long long row = lrow;
        const __half* xrow = x + lrow * D;
        if (segs != nullptr) {
            const KhqCompressSeg sg = segs[lrow / rows_per_seg];
            const long long rr = lrow % rows_per_seg;
            row = sg.row0 + rr;
            xrow = reinterpret_cast<const __half*>(reinterpret_cast<const char*>(sg.x) + x_byte_offset) + rr * D;
        }
        // ---- load: lane owns dims 8*lane .. 8*lane+7 ---------------------------------------
        const uint4 raw = *reinterpret_cast<const uint4*>(xrow + lane * 8);
        const __half* hx = reinterpret_cast<const __half*>(&raw);
        float xv[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            xv[j] = __half2float(hx[j]);
            S.a[lane * 8 + j] = xv[j];
        }
        __syncwarp();
        // sum of squares strictly in dim order (every lane computes the same chain)
        float sum_sq = 0.0f;
#pragma unroll 8
        for (int i = 0; i < D; i += 4) {
            const float4 t = *reinterpret_cast<const float4*>(&S.a[i]);
            sum_sq = __fmaf_rn(t.x, t.x, sum_sq);
            sum_sq = __fmaf_rn(t.y, t.y, sum_sq);
            sum_sq = __fmaf_rn(t.z, t.z, sum_sq);
            sum_sq = __fmaf_rn(t.w, t.w, sum_sq);
        }
        __syncwarp();
        const float norm = sqrtf(sum_sq + 1e-8f);
        if (lane == 0) out_norms[row] = __float2half(norm);
        const float den = norm + 1e-8f;

        const uint4 draw = *reinterpret_cast<const uint4*>(d_vec + lane * 8);
        const __half* hd = reinterpret_cast<const __half*>(&draw);
        float r[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) r[j] = __fdiv_rn(xv[j] * __half2float(hd[j]), den);
        fwht256_lane8(r, lane);

        // ---- 4x4 rotor of the lane's two patches: rot[c] = sum_k r[k] * R[k][c], k ascending
        float proj[8];
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

        if (!is_v) {
            // =============================== K branch ======================================
            const float th_out = 1.60f * f_s, th_lo = 0.47f * f_s;
            const uint4 craw = *reinterpret_cast<const uint4*>(cents + 2 * D + lane * 8);
            const __half* hc = reinterpret_cast<const __half*>(&craw);
            float cb[8];
            unsigned cand = 0;  // dims whose |proj| is above the outlier threshold
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                cb[j] = __half2float(hc[j]);
                if (fabsf(proj[j]) > th_out) cand |= 1u << j;
            }
            // ordinal of the lane's first candidate among all candidates, in dim order
            const int cnt = __popc(cand);
            int incl = cnt;
#pragma unroll
            for (int dlt = 1; dlt < 32; dlt <<= 1) {
                const int t = __shfl_up_sync(0xFFFFFFFFu, incl, dlt);
                if (lane >= dlt) incl += t;
            }
            int ord = incl - cnt;
            const int total_cand = __shfl_sync(0xFFFFFFFFu, incl, 31);
            const int n_out = total_cand < MAX_OUT ? total_cand : MAX_OUT;

            unsigned sym16 = 0;
            float o_abs[8];
            int o_ord[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float pj = proj[j];
                const float ap = fabsf(pj);
                unsigned sym;
                float cn = 0.0f, cc = 0.0f;
                o_ord[j] = -1;
                o_abs[j] = 0.0f;
                if (cand & (1u << j)) {
                    if (ord < MAX_OUT) {
                        sym = 3;
                        o_ord[j] = ord;
                        o_abs[j] = fabsf(pj * ts);
                    } else {
                        sym = (pj > 0.0f) ? 2u : 1u;  // overflow outlier: not part of the sums
                    }
                    ++ord;
                } else {
                    if (pj > th_lo) sym = 2;
                    else if (pj < -th_lo) sym = 1;
                    else sym = 0;
                    if (sym != 0) { cn = ap; cc = cb[j]; }
                }
                sym16 |= sym << (2 * j);
                S.a[lane * 8 + j] = cn;  // adding +0.0f leaves a non-negative fp32 sum unchanged
                S.b[lane * 8 + j] = cc;
            }
            // mask word w = dims 16w..16w+15 = lanes 2w (low half) and 2w+1 (high half)
            const unsigned hi16 = __shfl_down_sync(0xFFFFFFFFu, sym16, 1);
            if ((lane & 1) == 0) out_mask[row * 16 + (lane >> 1)] = sym16 | (hi16 << 16);
            __syncwarp();
            float sum_n = 0.0f, sum_c = 0.0f;
#pragma unroll 8
            for (int i = 0; i < D; i += 4) {
                const float4 ta = *reinterpret_cast<const float4*>(&S.a[i]);
                const float4 tb = *reinterpret_cast<const float4*>(&S.b[i]);
                sum_n += ta.x; sum_c += tb.x;
                sum_n += ta.y; sum_c += tb.y;
                sum_n += ta.z; sum_c += tb.z;
                sum_n += ta.w; sum_c += tb.w;
            }
            __syncwarp();
            float mult = (sum_c > 1e-5f) ? __fdiv_rn(sum_n, sum_c) : 1.0f;
            if (mult < 0.1f || mult > 10.0f || isnan(mult)) mult = 1.0f;

            float res[8];
            float max_res = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                res[j] = 0.0f;
                if (o_ord[j] >= 0) {
                    res[j] = fmaxf(0.0f, __fmaf_rn(-cb[j], mult, o_abs[j]));
                    max_res = fmaxf(max_res, res[j]);
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
        } else {
            // =============================== V branch ======================================
            // VQ search: for each patch every lane scans 8 consecutive codes in ascending order,
            // then the warp takes the lexicographic (distance, index) minimum.
            unsigned code[2] = {0, 0};
#pragma unroll 1
            for (int p = 0; p < NP; ++p) {
                const int src = p >> 1, off = (p & 1) * 4;
                // v0..v2 of patch p live in lane p/2
                const float s0 = (p & 1) ? proj[4] : proj[0];
                const float s1 = (p & 1) ? proj[5] : proj[1];
                const float s2 = (p & 1) ? proj[6] : proj[2];
                (void)off;
                const float v0 = __shfl_sync(0xFFFFFFFFu, s0, src);
                const float v1 = __shfl_sync(0xFFFFFFFFu, s1, src);
                const float v2 = __shfl_sync(0xFFFFFFFFu, s2, src);
                const uint4* cbp =
                    reinterpret_cast<const uint4*>(vq + ((size_t)p * 256 + lane * 8) * 3);
                __half hcb[24];
                *reinterpret_cast<uint4*>(&hcb[0]) = __ldg(cbp);
                *reinterpret_cast<uint4*>(&hcb[8]) = __ldg(cbp + 1);
                *reinterpret_cast<uint4*>(&hcb[16]) = __ldg(cbp + 2);
                float cf[24];  // the lane's 8 codes x 3 dims as fp32 (exact), converted two at a time
#pragma unroll
                for (int e = 0; e < 24; e += 2) {
                    const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&hcb[e]));
                    cf[e] = f2.x;
                    cf[e + 1] = f2.y;
                }
                float best = 1e20f;
                unsigned bi = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float d0 = __fmaf_rn(-cf[i * 3 + 0], alpha, v0);
                    const float d1 = __fmaf_rn(-cf[i * 3 + 1], alpha, v1);
                    const float d2 = __fmaf_rn(-cf[i * 3 + 2], alpha, v2);
                    const float dist = __fmaf_rn(d2, d2, __fmaf_rn(d0, d0, d1 * d1));
                    if (dist < best) { best = dist; bi = (unsigned)(lane * 8 + i); }
                }
                // warp minimum of (distance, index): a lane's best is a non-negative, non-NaN float
                // (it starts at 1e20 and only a strictly smaller distance replaces it), so its bit
                // pattern orders like the value and two hardware warp reductions do the work of
                // five shuffle-and-compare steps
                const unsigned best_bits = __reduce_min_sync(0xFFFFFFFFu, __float_as_uint(best));
                bi = __reduce_min_sync(0xFFFFFFFFu, (__float_as_uint(best) == best_bits) ? bi : 0xFFFFFFFFu);
                best = __uint_as_float(best_bits);
                // The reference starts from min=1e20 with a strict '<': if no distance is below
                // 1e20 (NaN/inf input) it keeps code 0.
                if (!(best < 1e20f)) bi = 0;
                if (src == lane) code[p & 1] = bi;
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
                S.a[pid] = e_true[p];
                S.b[pid] = e_vq[p];
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
            __syncwarp();
            float st = 0.0f, sv = 0.0f;
#pragma unroll 4
            for (int i = 0; i < NP; i += 4) {
                const float4 ta = *reinterpret_cast<const float4*>(&S.a[i]);
                const float4 tb = *reinterpret_cast<const float4*>(&S.b[i]);
                st += ta.x; sv += tb.x;
                st += ta.y; sv += tb.y;
                st += ta.z; sv += tb.z;
                st += ta.w; sv += tb.w;
            }
            if (lane == 0)
                out_r_norms[row] = __float2half(sqrtf(__fdiv_rn(st, sv + 1e-8f)));
            __syncwarp();
        }
    }
}

}  // namespace khq

extern "C" int launch_khq_compress_fp16(const void* x, const void* d_vec, const void* rotor,
                                        const void* centroids, const void* vq_centroids,
                                        void* out_mask, void* out_norms, void* out_r_norms,
                                        void* out_payload, void* out_shared_meta, int n, int d,
                                        float threshold_scale, float alpha, int is_v,
                                        cudaStream_t stream) {
    using namespace khq;
    if (n <= 0 || d != D) return -100;
    long long blocks = ((long long)n + CMP_WARPS - 1) / CMP_WARPS;
    const long long cap = 148LL * 64;  // grid-stride beyond this
    if (blocks > cap) blocks = cap;
    khq_compress_kernel<<<(unsigned)blocks, CMP_WARPS * 32, 0, stream>>>(
        static_cast<const __half*>(x), static_cast<const __half*>(d_vec),
        static_cast<const __half*>(rotor), static_cast<const __half*>(centroids),
        static_cast<const __half*>(vq_centroids), static_cast<unsigned int*>(out_mask),
        static_cast<__half*>(out_norms), static_cast<__half*>(out_r_norms),
        static_cast<unsigned char*>(out_payload), static_cast<unsigned char*>(out_shared_meta), d,
        n, threshold_scale, alpha, is_v, nullptr, 1, 0);
    const cudaError_t err = cudaGetLastError();
    return (err == cudaSuccess) ? 0 : static_cast<int>(err);
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
    long long blocks = (n + CMP_WARPS - 1) / CMP_WARPS;
    const long long cap = 148LL * 64;
    if (blocks > cap) blocks = cap;
    khq_compress_kernel<<<(unsigned)blocks, CMP_WARPS * 32, 0, stream>>>(
        nullptr, static_cast<const __half*>(d_vec), static_cast<const __half*>(rotor),
        static_cast<const __half*>(centroids), static_cast<const __half*>(vq_centroids),
        static_cast<unsigned int*>(out_mask), static_cast<__half*>(out_norms), static_cast<__half*>(out_r_norms),
        static_cast<unsigned char*>(out_payload), static_cast<unsigned char*>(out_shared_meta), d, (int)n,
        threshold_scale, alpha, is_v, static_cast<const KhqCompressSeg*>(segs), rows_per_seg, x_byte_offset);
    const cudaError_t err = cudaGetLastError();
    return (err == cudaSuccess) ? 0 : static_cast<int>(err);
}
