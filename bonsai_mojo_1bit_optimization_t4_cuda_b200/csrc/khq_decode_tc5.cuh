// khq_decode_tc5.cuh -- third-generation compressed-region decode: both contractions of the
// attention on the fifth-generation tensor cores (tcgen05.mma, accumulators in tensor memory),
// code words decoded one payload row per thread.  Included by khq_decode.cu.
//
// Tile = 128 payload rows = 32 tokens x 4 kv-heads, exactly as they lie in memory (row =
// token * 4 + kv_head), so the tile is eight contiguous byte ranges staged by bulk copies and
// tensor-memory lane r / MMA row r is payload row r of the tile.  Rows of different kv-heads share
// one MMA because the query side is the N dimension:
//
//   K side   D[128 rows, 96] = A[128, 256] B[256, 96]
//     A  (tensor memory, fp16): a_i = alpha_i * t_i + rho * beta_i * sign_i * code_i with t the
//        ternary symbol (outliers carry their sign), rho = residual_scale / mult of the row,
//        beta_i = 1 / c_i the inverse base centroid (alpha_i = 1; a dim whose centroid is ~0
//        uses beta_i = 1, alpha_i = 0).  y_i = alpha_k * k_norm * mult * c_i * a_i is the
//        reference's de-quantised value before the inverse rotor.
//     B  (shared memory, K-major, fp16): columns 0..23 = per query head the folded query
//        c_i * [R^T H256 (q * dinv * [dim >= 64])]_i (the pass-through dims of the reference's
//        RoPE), columns 32..95 = c_i * W[m][i], W = the linear map from y to the 64 rotary dims of
//        K^ (inverse rotor, the first 64 outputs of H256, /256/(d+eps)); 24..31 unused (their
//        shared memory carries the exchange of partial rotary sums between a row's two threads).
//     Score of head h for row r: sp_r * (D[r, h] + sum_m q_h[m] * RoPE_pos(D[r, 32..95])[m]).
//   V side   O[48, 256] += P[48, 128 rows] V[128 rows, 256]
//     V  (shared memory, dims contiguous): raw fp16 codebook entries for dims 0..2 of a patch,
//        fp16(c3[s] * alpha_v + (dump - 8) * max_res / 7) for dim 3.
//     P  (shared memory, K-major): rows 0..23 = p * alpha_v * v_norm * energy (used for dims 0..2),
//        rows 24..47 = p * v_norm (used for dim 3); a row's p is nonzero only in the columns of
//        its own kv-head's six heads.  MMA rows 48..127 read whatever follows in shared memory and
//        produce tensor-memory lanes nobody reads.
// p = 2^(s - M[h]) against a per-head reference M that is raised (by the new maximum + 8) only
// when a score exceeds it; O and the running sums are rescaled then.
//
// Warps: 0-7 decode (thread pair (r, r + 128) owns row r: K dims [128 half, +128), three of the
// row's six query heads each), 8 = bulk-copy producer, 9 = MMA issuer.  Every wait is bounded; a
// wait that runs out sets the device status word and a CTA-wide abort flag, after which every
// other wait returns at once and the CTA leaves (tensor memory is always released).
#pragma once
#include "khq_kdecode3.cuh"

namespace khq {
namespace m3 {

constexpr int DEC_T = 256;       // decode threads
constexpr int THREADS = 320;
constexpr int TILE_TOK = 32;
constexpr int ROWS = 128;
constexpr int NK = 96;           // columns of the K-side GEMM
constexpr int ROT0 = 32;         // first rotary column

constexpr int BK_GROUP = NK * 128;                   // bytes per 64-deep K group of B
constexpr int SM_BK = 0;
constexpr int V_CHUNK = 16384, V_GROUP = 4096;       // 32 rows x 256 dims; one 64-dim group
constexpr int SM_V = SM_BK + 4 * BK_GROUP;           // two chunk buffers
constexpr int P_ROWS = 48, P_GROUP = P_ROWS * 128;
constexpr int SM_P = SM_V + 2 * V_CHUNK;
constexpr int SM_STAGE = SM_P + 2 * P_GROUP;
// stage: "K part" (needed by the K decode) then "V part"
constexpr int ST_MASK = 0;
constexpr int ST_KPAY = ST_MASK + ROWS * 64;
constexpr int ST_KN = ST_KPAY + ROWS * K_PAY;
constexpr int ST_KRN = ST_KN + ROWS * 2;
constexpr int ST_VN = ST_KRN + ROWS * 2;
constexpr int ST_VRN = ST_VN + ROWS * 2;
constexpr int ST_VPAY = ST_VRN + ROWS * 2;
constexpr int ST_VSM = ST_VPAY + ROWS * V_PAY;
constexpr int STAGE_BYTES = ST_VSM + ROWS * 4;       // 28160
constexpr int VQA_STRIDE = 65;                       // words per code row of the (d0, d1) table
constexpr int VQB_STRIDE = 130;                      // bytes per code row of the d2 table
constexpr int SM_VQA = SM_STAGE + STAGE_BYTES;
constexpr int SM_VQB = SM_VQA + 256 * VQA_STRIDE * 4;
constexpr int QROT_KVH = NREP * 64 + 4;              // floats per kv-head group (+4: the four groups sit on different banks)
constexpr int SM_QROT = SM_VQB + 256 * VQB_STRIDE;
constexpr int SM_BETA = SM_QROT + HKV * QROT_KVH * 4;  // 128 x {beta2, amask}
constexpr int SM_C3 = SM_BETA + 128 * 8;               // 64 x float2
constexpr int SM_RSTEP = SM_C3 + 64 * 8;               // 32 x float2: rotation by 32 positions
constexpr int SM_FREQ = SM_RSTEP + 32 * 8;             // 32 floats
constexpr int SM_SOFT = SM_FREQ + 128;                 // M[24], fac[24], tmax[24], lsum[24], grow[2], abort, all_alpha
constexpr int SM_BARS = SM_SOFT + 4 * 24 * 4 + 32;
constexpr int SM_TOTAL = SM_BARS + 16 * 8;
static_assert(SM_TOTAL <= 227 * 1024, "shared memory budget");
static_assert(SM_V % 1024 == 0 && SM_P % 1024 == 0 && BK_GROUP % 1024 == 0 && P_GROUP % 1024 == 0 && SM_STAGE % 16 == 0 &&
                  ST_KPAY % 16 == 0 && ST_KN % 16 == 0 && ST_KRN % 16 == 0 && ST_VN % 16 == 0 && ST_VRN % 16 == 0 &&
                  ST_VPAY % 16 == 0 && ST_VSM % 16 == 0 && SM_VQA % 16 == 0 && SM_VQB % 4 == 0 && SM_QROT % 16 == 0 &&
                  SM_BETA % 16 == 0 && SM_BARS % 8 == 0,
              "alignment");
static_assert(HQ * 257 * 4 <= 2 * V_CHUNK && HKV * MERGE_FLOATS * 4 <= 2 * V_CHUNK, "item scratch aliases the V buffers");

constexpr uint32_t TM_COLS = 512, TM_A = 0, TM_D = 128, TM_O = 256;
constexpr float M_HEADROOM = 8.0f;   // log2 units added to a new maximum
constexpr float M_NONE = -1.0e30f;
constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;

enum Bar { B_KFULL = 0, B_VFULL, B_KFREE, B_VFREE, B_AREADY, B_DREADY, B_DFREE, B_VREADY0, B_VREADY1, B_VDONE0, B_VDONE1,
           B_PREADY, B_PVDONE, B_COUNT };
static_assert(B_COUNT <= 15, "barrier area (the last slot holds the tensor-memory address)");

struct Soft {  // SM_SOFT
    float M[24], fac[24];
    int tmax[24];
    float lsum[24];
    int grow[2];
    int abort_flag, all_alpha, next_item, pad;
};

// ---- small wrappers --------------------------------------------------------------------------
__device__ __forceinline__ uint32_t idesc_f16(int n, bool b_mn_major) {
    // fp32 accumulate, fp16 A and B, A K-major, M = 128
    return (1u << 4) | (b_mn_major ? (1u << 16) : 0u) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ uint32_t sdesc_lo(uint32_t addr, uint32_t lbo) {
    return ((addr & 0x3FFFFu) >> 4) | (((lbo >> 4) & 0x3FFFu) << 16);
}
constexpr uint32_t SDESC_HI = ((1024u >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);  // 8-row groups 1024 B apart, 128-byte swizzle
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .b64 da, db;\n\t.reg .pred p;\n\t"
        "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %2};\n\t"
        "setp.ne.u32 p, %5, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}" ::"r"(d_tmem),
        "r"(a_lo), "r"(SDESC_HI), "r"(b_lo), "r"(idesc), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .b64 db;\n\t.reg .pred p;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "setp.ne.u32 p, %5, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "r"(b_lo), "r"(SDESC_HI), "r"(idesc), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tm_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tm_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// Tensor-memory stores carry no "memory" clobber: they do not touch ordinary memory, and the clobber would stop
// the compiler from overlapping the shared-memory loads of one mask word with the stores of the previous one.
// They stay ordered among themselves and with the waits and fences (all asm volatile).
__device__ __forceinline__ void tm_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%8], {%0,%1,%2,%3,%4,%5,%6,%7};" ::"r"(r[0]), "r"(r[1]), "r"(r[2]),
                 "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(taddr));
}
__device__ __forceinline__ void tm_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tm_ld32(uint32_t taddr, uint32_t* r) {
    tm_ld16(taddr, r);
    tm_ld16(taddr + 16, r + 16);
}
__device__ __forceinline__ void tm_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15};" ::"r"(r[0]),
        "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(taddr));
}
__device__ __forceinline__ float ex2f(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void dec_barrier() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
__device__ __forceinline__ uint32_t hfma2_u(uint32_t a, uint32_t b, uint32_t c) {
    const __half2 r = __hfma2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b),
                              *reinterpret_cast<const __half2*>(&c));
    return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t hmul2_u(uint32_t a, uint32_t b) {
    const __half2 r = __hmul2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
}
// order-preserving int key of a float (for atomicMax)
__device__ __forceinline__ int fkey(float f) {
    const int i = __float_as_int(f);
    return i >= 0 ? i : (i ^ 0x7FFFFFFF);
}
__device__ __forceinline__ float funkey(int k) { return __int_as_float(k >= 0 ? k : (k ^ 0x7FFFFFFF)); }

// Bounded wait that gives up at once when the CTA has already aborted.
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    if (*abort_flag) return false;
    for (uint32_t it = 0; it < (1u << 21); ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if (it > 32) {
            __nanosleep(64);
            if ((it & 255u) == 0u && *abort_flag) return false;
        }
    }
    *abort_flag = 1;
    atomicExch(&g_status, 1);
    return false;
}

// Byte offsets inside the shared-memory operands (128-byte-swizzle canonical layouts).
__device__ __forceinline__ uint32_t bk_off(int n, int kap) {  // B of the K side: column n, operand index kap
    return (uint32_t)((kap >> 6) * BK_GROUP + n * 128 + ((((kap >> 3) & 7) ^ (n & 7)) << 4) + (kap & 7) * 2);
}
__device__ __forceinline__ uint32_t p_off(int m, int k) {  // A of the V side: row m (head / 24 + head), tile row k
    return (uint32_t)((k >> 6) * P_GROUP + m * 128 + ((((k >> 3) & 7) ^ (m & 7)) << 4) + (k & 7) * 2);
}
// operand index (0..255) of K dim d: mask word d / 16, then the word's even dims, then its odd ones
__device__ __forceinline__ int kap_of_dim(int d) { return (d & ~15) + khq3::k3_index_of(d & 15); }

// ---- per-layer tables -------------------------------------------------------------------------
// V codebook, rotary columns of B, beta / alpha tables, dim-3 centroids, RoPE constants.  All
// NT threads of the CTA; must be followed by a CTA barrier (and a proxy fence before the next MMA).
template <int NT = THREADS>
__device__ __forceinline__ void setup_layer(unsigned char* smem, const CompressedKV& P, int tid) {
    Soft* soft = reinterpret_cast<Soft*>(smem + SM_SOFT);
    unsigned short* vqa = reinterpret_cast<unsigned short*>(smem + SM_VQA);
    unsigned short* vqb = reinterpret_cast<unsigned short*>(smem + SM_VQB);
    stage_vq_codebook<NT, VQA_STRIDE, VQB_STRIDE>(P.vq, reinterpret_cast<unsigned int*>(vqa), vqb, tid);
    // rotary columns: B[kap(i)][32 + m] = ceff_i * dinv_m * sum_c' R[p][c'][k] * (-1)^popc(m & ((4p + c') & 63))
    for (int e = tid; e < 64 * D; e += NT) {
        const int m = e & 63, i = e >> 6;
        const int p = i >> 2, k = i & 3;
        float acc = 0.0f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const float sgn = (__popc(m & ((4 * p + c) & 63)) & 1) ? -1.0f : 1.0f;
            acc += sgn * __half2float(P.k_rotor[p * 16 + c * 4 + k]);
        }
        const float cb = __half2float(P.cents_k[2 * D + i]);
        const float ceff = fabsf(cb) >= 6.2e-5f ? cb : 1.0f;
        const float dinv = (1.0f / 256.0f) / (__half2float(P.d_k[m]) + 1e-8f);
        *reinterpret_cast<__half*>(smem + SM_BK + bk_off(ROT0 + m, kap_of_dim(i))) = __float2half(acc * dinv * ceff);
    }
    if (tid < 128) {
        uint32_t beta2 = 0u, amask = 0u;
        bool all_one = true;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int kap = 2 * tid + e;
            const int d = (kap & ~15) + khq3::k3_dim_of(kap & 15);
            const float cb = __half2float(P.cents_k[2 * D + d]);
            const bool live = fabsf(cb) >= 6.2e-5f;
            const float beta = live ? 1.0f / cb : 1.0f;
            beta2 |= (uint32_t)__half_as_ushort(__float2half(beta)) << (16 * e);
            amask |= (live ? 0xFFFFu : 0u) << (16 * e);
            all_one = all_one && live;
        }
        reinterpret_cast<uint2*>(smem + SM_BETA)[tid] = make_uint2(beta2, amask);
        if (!all_one) soft->all_alpha = 0;
    }
    if (tid >= 128 && tid < 192) {
        const int p = tid - 128;
        reinterpret_cast<float2*>(smem + SM_C3)[p] = make_float2(__half2float(P.cents_v[0 * D + 4 * p + 3]) * P.alpha_v,
                                                                 __half2float(P.cents_v[1 * D + 4 * p + 3]) * P.alpha_v);
    }
    if (tid >= 192 && tid < 224) {
        const int m = tid - 192;
        const float f = powf(P.rope_base, -2.0f * (float)m / 64.0f);
        reinterpret_cast<float*>(smem + SM_FREQ)[m] = f;
        double th = 32.0 * (double)f;
        th -= rint(th * 0.15915494309189535) * 6.283185307179586;
        reinterpret_cast<float2*>(smem + SM_RSTEP)[m] = make_float2((float)cos(th), (float)sin(th));
    }
}

// ---- per-item query-side set-up (decode threads) ------------------------------------------------
// Folded query columns of B, the raw rotary query dims, the softmax state.  scratch: 8 warps x
// 256 floats (the V buffers).  Followed by a decoder barrier by the caller.
__device__ __forceinline__ void setup_item(unsigned char* smem, const __half* __restrict__ q, size_t q_head_stride,
                                           const CompressedKV& P, int tid) {
    const int warp = tid >> 5, lane = tid & 31;
    Soft* soft = reinterpret_cast<Soft*>(smem + SM_SOFT);
    float dv[8], cf[8], rr[2][16];
    {
        const uint4 dr = *reinterpret_cast<const uint4*>(P.d_k + lane * 8);
        const uint4 cr = *reinterpret_cast<const uint4*>(P.cents_k + 2 * D + lane * 8);
        const __half* hd = reinterpret_cast<const __half*>(&dr);
        const __half* hc = reinterpret_cast<const __half*>(&cr);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            dv[j] = (lane >= 8) ? (1.0f / 256.0f) / (__half2float(hd[j]) + 1e-8f) : 0.0f;
            const float cb = __half2float(hc[j]);
            cf[j] = fabsf(cb) >= 6.2e-5f ? cb : 1.0f;
        }
#pragma unroll
        for (int p = 0; p < 2; ++p)
#pragma unroll
            for (int i = 0; i < 16; ++i) rr[p][i] = __half2float(P.k_rotor[(lane * 2 + p) * 16 + i]);
    }
#pragma unroll 1
    for (int hh = 0; hh < 3; ++hh) {
        const int h = warp * 3 + hh;
        const uint4 qraw = *reinterpret_cast<const uint4*>(q + (size_t)h * q_head_stride + lane * 8);
        const __half* hq = reinterpret_cast<const __half*>(&qraw);
        float x[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = __half2float(hq[j]) * dv[j];
        fwht256_lane8(x, lane);
#pragma unroll
        for (int p = 0; p < 2; ++p)
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float a = 0.0f;
#pragma unroll
                for (int c = 0; c < 4; ++c) a = fmaf(rr[p][c * 4 + k], x[p * 4 + c], a);
                const int d = lane * 8 + p * 4 + k;
                *reinterpret_cast<__half*>(smem + SM_BK + bk_off(h, kap_of_dim(d))) = __float2half(a * cf[p * 4 + k]);
            }
    }
    float* qrot = reinterpret_cast<float*>(smem + SM_QROT);
    for (int e = tid; e < HQ * 64; e += DEC_T) {
        const int h = e >> 6, m = e & 63;
        qrot[(h / NREP) * QROT_KVH + (h % NREP) * 64 + m] = __half2float(q[(size_t)h * q_head_stride + m]);
    }
    if (tid < 24) {
        soft->M[tid] = M_NONE;
        soft->fac[tid] = 1.0f;
        soft->tmax[tid] = fkey(M_NONE);
        soft->lsum[tid] = 0.0f;
    }
    if (tid < 2) soft->grow[tid] = 0;
}

// ---- bulk-copy producer ------------------------------------------------------------------------
// Stages `ntok` tokens from token `tok0`: part 0 = what the K decode reads (mask, K payload, the four
// norm arrays), part 1 = V payload and V meta.  Whole warp; lane 0 issues the bulk copies of the
// even-token part, the lanes copy an odd last token with plain loads, lane 0 arrives.
__device__ __forceinline__ void stage_part(const CompressedKV& P, unsigned char* stage, uint64_t* bar, int part, int tok0,
                                           int ntok, int lane) {
    const size_t r0 = (size_t)tok0 * HKV;
    const unsigned char* src[6];
    int dst[6], bpr[6], n;
    if (part == 0) {
        src[0] = reinterpret_cast<const unsigned char*>(P.k_mask) + r0 * 64; dst[0] = ST_MASK; bpr[0] = 64;
        src[1] = P.k_payload + r0 * K_PAY; dst[1] = ST_KPAY; bpr[1] = K_PAY;
        src[2] = reinterpret_cast<const unsigned char*>(P.k_norms) + r0 * 2; dst[2] = ST_KN; bpr[2] = 2;
        src[3] = reinterpret_cast<const unsigned char*>(P.k_r_norms) + r0 * 2; dst[3] = ST_KRN; bpr[3] = 2;
        src[4] = reinterpret_cast<const unsigned char*>(P.v_norms) + r0 * 2; dst[4] = ST_VN; bpr[4] = 2;
        src[5] = reinterpret_cast<const unsigned char*>(P.v_r_norms) + r0 * 2; dst[5] = ST_VRN; bpr[5] = 2;
        n = 6;
    } else {
        src[0] = P.v_payload + r0 * V_PAY; dst[0] = ST_VPAY; bpr[0] = V_PAY;
        src[1] = P.v_shared_meta + r0 * 4; dst[1] = ST_VSM; bpr[1] = 4;
        n = 2;
    }
    const int rows_b = (ntok & ~1) * HKV;
    if (ntok & 1) {
        for (int a = 0; a < n; ++a) {
            const int words = HKV * bpr[a] / 4;  // one token = 4 rows: always whole words
            const unsigned int* s = reinterpret_cast<const unsigned int*>(src[a] + (size_t)rows_b * bpr[a]);
            unsigned int* d = reinterpret_cast<unsigned int*>(stage + dst[a] + rows_b * bpr[a]);
            for (int i = lane; i < words; i += 32) d[i] = s[i];
        }
    }
    __syncwarp();
    if (lane == 0) {
        int per_row = 0;
        for (int a = 0; a < n; ++a) per_row += bpr[a];
        if (rows_b > 0) {
            mbar_arrive_expect_tx(bar, (uint32_t)(rows_b * per_row));
            for (int a = 0; a < n; ++a) bulk_g2s(stage + dst[a], src[a], (uint32_t)(rows_b * bpr[a]), bar);
        } else {
            mbar_arrive(bar);
        }
    }
}

// ---- the compressed range of one work item ------------------------------------------------------
// Running counts of how often each barrier has completed in this CTA's life.
struct Counters {
    unsigned tiles;   // tiles whose K decode / score step / V staging have been started
    unsigned vph;     // V decode phases (two per tile)
};

// All THREADS threads call it.  On return the decode warps 0..3 hold the item's merged state in `ws`
// (first generation's layout: warp = kv-head, lane = 8 dims, rotated V domain).
__device__ __forceinline__ void compressed_range(unsigned char* smem, uint32_t tmem, const __half* __restrict__ q,
                                                 size_t q_head_stride, const CompressedKV& P, int my_lo, int my_hi,
                                                 float scale, Counters& cn, WarpState& ws) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    Soft* soft = reinterpret_cast<Soft*>(smem + SM_SOFT);
    volatile int* abortf = &soft->abort_flag;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM_BARS);
    unsigned char* stage = smem + SM_STAGE;
    const int base = my_lo & ~1;
    const int ntiles = (my_hi > my_lo) ? (my_hi - base + TILE_TOK - 1) / TILE_TOK : 0;
    const unsigned g0 = cn.tiles, v0 = cn.vph;
    ws.init();

    if (warp == 8) {
        // ================================ producer =================================================
#pragma unroll 1
        for (int t = 0; t < ntiles; ++t) {
            const unsigned g = g0 + t;
            const int tok0 = base + t * TILE_TOK;
            const int ntok = min(TILE_TOK, P.c_len - tok0);
            bool ok = true;
            if (lane == 0 && g >= 1) ok = wait_bar(&bars[B_KFREE], (g - 1) & 1u, abortf);
            ok = __shfl_sync(0xFFFFFFFFu, ok ? 1 : 0, 0) != 0;
            if (ok) stage_part(P, stage, &bars[B_KFULL], 0, tok0, ntok, lane);
            if (lane == 0 && g >= 1) ok = wait_bar(&bars[B_VFREE], (g - 1) & 1u, abortf);
            ok = __shfl_sync(0xFFFFFFFFu, ok ? 1 : 0, 0) != 0;
            if (ok) stage_part(P, stage, &bars[B_VFULL], 1, tok0, ntok, lane);
        }
    } else if (warp == 9) {
        // ================================ MMA issuer ===============================================
        if (lane == 0) {
            const uint32_t sbase = smem_u32(smem);
            const uint32_t idesc_k = idesc_f16(NK, false), idesc_v = idesc_f16(D, true);
            const uint32_t bk_lo = sdesc_lo(sbase + SM_BK, 16), p_lo = sdesc_lo(sbase + SM_P, 16);
            const uint32_t v_lo = sdesc_lo(sbase + SM_V, V_GROUP);
            bool ok = true;
            auto issue_pv = [&](int tile_first, int phase) {  // chunks 2*phase, 2*phase+1 from buffers 0, 1
#pragma unroll
                for (int b = 0; b < 2; ++b) {
#pragma unroll
                    for (int kk = 0; kk < 2; ++kk) {
                        const int ks = (2 * phase + b) * 2 + kk;  // K step of the tile (16 rows each)
                        const uint32_t oa = (uint32_t)((ks >> 2) * P_GROUP + (ks & 3) * 32) >> 4;
                        const uint32_t ob = (uint32_t)(b * V_CHUNK + kk * 2048) >> 4;
                        mma_ss(tmem + TM_O, p_lo + oa, v_lo + ob, idesc_v, (tile_first && ks == 0) ? 0u : 1u);
                    }
                    mma_commit(&bars[B_VDONE0 + b]);
                }
            };
#pragma unroll 1
            for (int i = -1; i < ntiles && ok; ++i) {
                if (i + 1 < ntiles) {
                    const unsigned g = g0 + i + 1;
                    ok = wait_bar(&bars[B_AREADY], g & 1u, abortf);
                    if (ok && g >= 1) ok = wait_bar(&bars[B_DFREE], (g - 1) & 1u, abortf);
                    if (!ok) break;
                    tc_after();
#pragma unroll
                    for (int s = 0; s < 16; ++s) {
                        const uint32_t ob = (uint32_t)((s >> 2) * BK_GROUP + (s & 3) * 32) >> 4;
                        mma_ts(tmem + TM_D, tmem + TM_A + 8 * s, bk_lo + ob, idesc_k, s > 0 ? 1u : 0u);
                    }
                    mma_commit(&bars[B_DREADY]);
                }
                if (i >= 0) {
                    const unsigned vp = v0 + 2 * i + 1;
                    ok = wait_bar(&bars[B_VREADY0], vp & 1u, abortf) && wait_bar(&bars[B_VREADY1], vp & 1u, abortf);
                    if (!ok) break;
                    tc_after();
                    issue_pv(0, 1);
                    mma_commit(&bars[B_PVDONE]);
                }
                if (i + 1 < ntiles) {
                    const unsigned g = g0 + i + 1, vp = v0 + 2 * (i + 1);
                    ok = wait_bar(&bars[B_PREADY], g & 1u, abortf) && wait_bar(&bars[B_VREADY0], vp & 1u, abortf) &&
                         wait_bar(&bars[B_VREADY1], vp & 1u, abortf);
                    if (!ok) break;
                    tc_after();
                    issue_pv(i + 1 == 0, 0);
                }
            }
        }
    } else {
        // ================================ decode warps ==============================================
        const int r = tid & 127, half = tid >> 7, kvh = r & 3;
        const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const float* qrot = reinterpret_cast<const float*>(smem + SM_QROT) + kvh * QROT_KVH + half * 16;
        const uint4* betat = reinterpret_cast<const uint4*>(smem + SM_BETA);
        const float2* c3t = reinterpret_cast<const float2*>(smem + SM_C3);
        const float2* rstep = reinterpret_cast<const float2*>(smem + SM_RSTEP) + 16 * half;
        const unsigned char* vqa = smem + SM_VQA;
        const unsigned char* vqb = smem + SM_VQB;
        const int h0 = kvh * NREP + half * 3;   // the three query heads this thread finishes
        const bool all_alpha = soft->all_alpha != 0;
        // partial rotary dot products are swapped with the row's other thread through the unused columns
        // 24..31 of B (1 KB per 64-deep group; whatever lies there only reaches D columns nobody reads)
        float* xmine = reinterpret_cast<float*>(smem + SM_BK + (2 * half + (r >> 6)) * BK_GROUP + 24 * 128) + (r & 63) * 3;
        const float* xother =
            reinterpret_cast<const float*>(smem + SM_BK + (2 * (half ^ 1) + (r >> 6)) * BK_GROUP + 24 * 128) + (r & 63) * 3;

        // RoPE cos/sin of this row's token for this thread's 16 pairs m = 16 half + j, advanced by 32
        // positions per tile
        float rc[16], rs[16];
        if (ntiles > 0) {
            const float* freq = reinterpret_cast<const float*>(smem + SM_FREQ) + 16 * half;
            const int pos = P.start_pos + base + (r >> 2);
#pragma unroll
            for (int m = 0; m < 16; ++m) {
                double th = (double)pos * (double)freq[m];
                th -= rint(th * 0.15915494309189535) * 6.283185307179586;
                __sincosf((float)th, &rs[m], &rc[m]);
            }
        }
        float lrun[3] = {0.0f, 0.0f, 0.0f};
        float sp2 = 0.0f, s1 = 0.0f, s2 = 0.0f;  // row scalars kept from the K decode to the score step

        // Order of the phases: K(0) S(0) | V(0,0) K(1) V(0,1) S(1) | V(1,0) K(2) V(1,1) S(2) | ...  (K = code
        // words -> A operand, S = scores + softmax + P, V(t, ph) = chunks 2 ph, 2 ph + 1 of tile t): the K-side
        // MMAs of a tile run under the V decode of the tile before, its P V MMAs under the next K decode.
#pragma unroll 1
        for (int step = 0; step < 2 * ntiles + 2; ++step) {
            const int t = (step >> 1) - 1, ph = step & 1;  // V decode of tile t, then K (ph 0) or S (ph 1) of tile t + 1
            // ---------------- V decode of chunks 2 ph, 2 ph + 1 of tile t -----------------------------
            if (t >= 0) {
                const unsigned vp = v0 + 2 * t + ph;
                const int b = warp >> 2, grp = warp & 3;
                const int rr = 32 * (2 * ph + b) + lane;
                if (ph == 0) wait_bar(&bars[B_VFULL], (g0 + t) & 1u, abortf);
                if (vp >= 1) wait_bar(&bars[B_VDONE0 + b], (vp - 1) & 1u, abortf);
                const unsigned char* vrow = stage + ST_VPAY + rr * V_PAY;
                const int tok = base + t * TILE_TOK + (rr >> 2);
                const bool valid = tok >= my_lo && tok < my_hi;
                const float smv7 = valid ? reinterpret_cast<const float*>(stage + ST_VSM)[rr] * (1.0f / 7.0f) : 0.0f;
                const uint32_t hb = (reinterpret_cast<const uint32_t*>(vrow)[24 + (grp >> 1)] >> (16 * (grp & 1))) & 0xFFFFu;
                unsigned char* dst = smem + SM_V + b * V_CHUNK + grp * V_GROUP + lane * 128;
#pragma unroll 1
                for (int g8 = 0; g8 < 2; ++g8) {
                    const uint32_t* wp = reinterpret_cast<const uint32_t*>(vrow) + 6 * grp + 3 * g8;
                    uint32_t f[8];
                    khq3::v3_fields(wp[0], wp[1], wp[2], f);
#pragma unroll
                    for (int u = 0; u < 8; u += 2) {
                        uint32_t ow[4];
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const int p = 16 * grp + 8 * g8 + u + e;
                            const uint32_t fld = f[u + e];
                            const uint32_t hbit = ((hb >> (8 * g8)) << (7 - (u + e))) & 0x80u;
                            const uint32_t code = (fld & 0x7Fu) | hbit;
                            const uint32_t e01 = *reinterpret_cast<const uint32_t*>(vqa + code * (VQA_STRIDE * 4) + p * 4);
                            const uint32_t e2 = *reinterpret_cast<const unsigned short*>(vqb + code * VQB_STRIDE + p * 2);
                            const float2 cc = c3t[p];
                            const float c3 = (fld & 0x80u) ? cc.y : cc.x;
                            const float v3 = fmaf(__uint_as_float(0x4B000000u | (fld >> 8)) - 8388616.0f, smv7, c3);  // (dump - 8)
                            ow[2 * e] = e01;
                            ow[2 * e + 1] = e2 | ((uint32_t)__half_as_ushort(__float2half_rn(v3)) << 16);
                        }
                        const int cc16 = (8 * g8 + u) >> 1;  // 16-byte chunk of the row's 128 bytes
                        *reinterpret_cast<uint4*>(dst + ((cc16 ^ (lane & 7)) << 4)) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
                    }
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&bars[B_VREADY0 + b]);
                    if (ph == 1) mbar_arrive(&bars[B_VFREE]);
                }
            }
            if (t + 1 >= ntiles) continue;
            const unsigned g = g0 + t + 1;
            if (ph == 0) {
                // ---------------- K decode of tile t + 1: code words -> A operand in tensor memory -------
                wait_bar(&bars[B_KFULL], g & 1u, abortf);
                const uint32_t* kp = reinterpret_cast<const uint32_t*>(stage + ST_KPAY + r * K_PAY);
                const uint32_t* mrow = reinterpret_cast<const uint32_t*>(stage + ST_MASK + r * 64);
                uint32_t ob = 0;
                if (half) {  // outliers of the row's first 128 dims come before this thread's
                    const uint4 a = reinterpret_cast<const uint4*>(mrow)[0], b4 = reinterpret_cast<const uint4*>(mrow)[1];
                    ob = khq3::k3_count(a.x) + khq3::k3_count(a.y) + khq3::k3_count(a.z) + khq3::k3_count(a.w) +
                         khq3::k3_count(b4.x) + khq3::k3_count(b4.y) + khq3::k3_count(b4.z) + khq3::k3_count(b4.w);
                }
                float mult = (float)kp[0] / 1000.0f;
                if (mult < 0.1f || mult > 10.0f || isnan(mult)) mult = 1.0f;
                const float rsc = hbits2f(reinterpret_cast<const uint16_t*>(stage + ST_KRN)[r]);
                const float kn = hbits2f(reinterpret_cast<const uint16_t*>(stage + ST_KN)[r]);
                const float vn = hbits2f(reinterpret_cast<const uint16_t*>(stage + ST_VN)[r]);
                const float en = hbits2f(reinterpret_cast<const uint16_t*>(stage + ST_VRN)[r]);
                sp2 = P.alpha_k * kn * mult * scale * LOG2E;
                s1 = P.alpha_v * vn * en;
                s2 = vn;
                const __half2 rh = __float2half2_rn(rsc / mult);
                const uint32_t ratio2 = *reinterpret_cast<const uint32_t*>(&rh);
                const uint32_t neg1024 = 0xE400E400u;
#ifndef M3_WORD_UNROLL
#define M3_WORD_UNROLL 2
#endif
#define M3_STR2(x) #x
#define M3_STR(x) M3_STR2(x)
_Pragma(M3_STR(unroll M3_WORD_UNROLL))
                for (int w = 0; w < 8; ++w) {  // not fully unrolled: the loop body is large and the instruction cache is not
                    uint32_t t2[8], h2[8], a2[8];
                    ob += khq3::k3_word(mrow[8 * half + w], ob, kp, t2, h2);
                    const int col0 = 8 * (8 * half + w);
#pragma unroll
                    for (int j = 0; j < 8; j += 2) {
                        const uint4 bt = betat[(col0 + j) >> 1];  // {beta2, mask} of two operand words
                        const uint32_t c0 = hfma2_u(t2[j], neg1024, h2[j]), c1 = hfma2_u(t2[j + 1], neg1024, h2[j + 1]);  // sign * code
                        a2[j] = hfma2_u(c0, hmul2_u(ratio2, bt.x), all_alpha ? t2[j] : (t2[j] & bt.y));
                        a2[j + 1] = hfma2_u(c1, hmul2_u(ratio2, bt.z), all_alpha ? t2[j + 1] : (t2[j + 1] & bt.w));
                    }
                    tm_st8(lane_base + TM_A + col0, a2);
                }
                tm_st_wait();
                tc_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&bars[B_AREADY]);
                    mbar_arrive(&bars[B_KFREE]);
                }
            } else {
                // ---------------- scores, softmax and P of tile t + 1 ---------------------------------
                const int tt = t + 1;
                wait_bar(&bars[B_DREADY], g & 1u, abortf);
                tc_after();
                float acc[3], part[6];
                {
                    uint32_t pc[32], lo[16], hi[16];
                    tm_ld32(lane_base + TM_D, pc);
                    tm_ld16(lane_base + TM_D + ROT0 + 16 * half, lo);
                    tm_ld16(lane_base + TM_D + ROT0 + 32 + 16 * half, hi);
                    tm_ld_wait();
                    // every column of D this thread needs has been read: the next tile's K-side MMAs may overwrite it
                    tc_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars[B_DFREE]);
#pragma unroll
                    for (int j = 0; j < 3; ++j) {
                        const uint32_t v0_ = half ? pc[3 + j] : pc[j], v1_ = half ? pc[9 + j] : pc[6 + j];
                        const uint32_t v2_ = half ? pc[15 + j] : pc[12 + j], v3_ = half ? pc[21 + j] : pc[18 + j];
                        acc[j] = __uint_as_float(kvh == 0 ? v0_ : (kvh == 1 ? v1_ : (kvh == 2 ? v2_ : v3_)));
                    }
                    // rotate this thread's 16 pairs (m, m + 32), m = 16 half + mm, and advance their table by one tile
                    float ka[16], kb[16];
#pragma unroll
                    for (int mm = 0; mm < 16; ++mm) {
                        const float k0 = __uint_as_float(lo[mm]), k1 = __uint_as_float(hi[mm]);
                        ka[mm] = k0 * rc[mm] - k1 * rs[mm];
                        kb[mm] = k0 * rs[mm] + k1 * rc[mm];
                        const float2 st = rstep[mm];
                        const float c = rc[mm] * st.x - rs[mm] * st.y, s = rs[mm] * st.x + rc[mm] * st.y;
                        rc[mm] = c;
                        rs[mm] = s;
                    }
                    // partial dot products with the raw rotary query dims of the six heads of this row's group
#pragma unroll
                    for (int j = 0; j < 6; ++j) {
                        float a = 0.0f;
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4) {
                            const float4 qa = *reinterpret_cast<const float4*>(qrot + j * 64 + 4 * q4);
                            const float4 qb = *reinterpret_cast<const float4*>(qrot + j * 64 + 32 + 4 * q4);
                            a = fmaf(ka[4 * q4], qa.x, fmaf(ka[4 * q4 + 1], qa.y, fmaf(ka[4 * q4 + 2], qa.z, fmaf(ka[4 * q4 + 3], qa.w, a))));
                            a = fmaf(kb[4 * q4], qb.x, fmaf(kb[4 * q4 + 1], qb.y, fmaf(kb[4 * q4 + 2], qb.z, fmaf(kb[4 * q4 + 3], qb.w, a))));
                        }
                        part[j] = a;
                    }
                }
                // hand the other thread of the row the three heads it finishes, take mine from it
#pragma unroll
                for (int j = 0; j < 3; ++j) xmine[j] = half ? part[j] : part[3 + j];
                asm volatile("bar.sync %0, 64;" ::"r"(2 + (warp & 3)) : "memory");
                const int tok = base + tt * TILE_TOK + (r >> 2);
                const bool valid = tok >= my_lo && tok < my_hi;
                float sc[3];
                bool need = false;
#pragma unroll
                for (int j = 0; j < 3; ++j) {
                    const float tot = acc[j] + (half ? part[3 + j] : part[j]) + xother[j];
                    sc[j] = valid ? sp2 * tot : M_NONE;
                    need = need || (valid && sc[j] > soft->M[h0 + j]);
                }
                const int par = tt & 1;
                if (__any_sync(0xFFFFFFFFu, need)) {
                    if (need) {
#pragma unroll
                        for (int j = 0; j < 3; ++j)
                            if (sc[j] > soft->M[h0 + j]) atomicMax(&soft->tmax[h0 + j], fkey(sc[j]));
                        soft->grow[par] = 1;
                    }
                }
                dec_barrier();
                if (soft->grow[par]) {
                    if (tid < 24) {
                        const float mo = soft->M[tid], tm = funkey(soft->tmax[tid]);
                        float f = 1.0f;
                        if (tm > mo) {
                            const float mn = tm + M_HEADROOM;
                            f = (mo <= -1.0e29f) ? 0.0f : ex2f(mo - mn);
                            soft->M[tid] = mn;
                        }
                        soft->fac[tid] = f;
                        soft->tmax[tid] = fkey(M_NONE);
                    }
                    dec_barrier();
                    if (tid == 0) soft->grow[par] = 0;
#pragma unroll
                    for (int j = 0; j < 3; ++j) lrun[j] *= soft->fac[h0 + j];
                    if (tt > 0 && warp < 2) {
                        // O holds earlier tiles of this item.  Rows: lane m < 24 = head m (dims 0..2 of the
                        // patches), 24..47 = head m - 24 (dim 3)
                        wait_bar(&bars[B_PVDONE], (g - 1) & 1u, abortf);
                        tc_after();
                        const int m = warp * 32 + lane;
                        const float f = m < 48 ? soft->fac[m < 24 ? m : m - 24] : 1.0f;
#pragma unroll 1
                        for (int cb = 0; cb < 16; ++cb) {
                            uint32_t o[16];
                            tm_ld16(lane_base + TM_O + 16 * cb, o);
                            tm_ld_wait();
#pragma unroll
                            for (int e = 0; e < 16; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * f);
                            tm_st16(lane_base + TM_O + 16 * cb, o);
                        }
                        tm_st_wait();
                        tc_before();
                    }
                }
                float pw[3];
#pragma unroll
                for (int j = 0; j < 3; ++j) {
                    pw[j] = valid ? ex2f(sc[j] - soft->M[h0 + j]) : 0.0f;
                    lrun[j] += pw[j];
                }
                // P of the previous tile must have been consumed before it is overwritten
                if (g >= 1) wait_bar(&bars[B_PVDONE], (g - 1) & 1u, abortf);
#pragma unroll
                for (int j = 0; j < 3; ++j) {
                    // rows outside the item write an exact zero: their row scalars are whatever the staging area held
                    *reinterpret_cast<__half*>(smem + SM_P + p_off(h0 + j, r)) = __float2half(valid ? pw[j] * s1 : 0.0f);
                    *reinterpret_cast<__half*>(smem + SM_P + p_off(24 + h0 + j, r)) = __float2half(valid ? pw[j] * s2 : 0.0f);
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars[B_PREADY]);
            }
        }
        // ---------------- item epilogue: O and the running sums -> the first generation's state ------
        if (ntiles > 0) {
            const unsigned glast = g0 + ntiles - 1;
            wait_bar(&bars[B_PVDONE], glast & 1u, abortf);
            tc_after();
#pragma unroll
            for (int j = 0; j < 3; ++j) {
                float v = lrun[j];
                v += __shfl_xor_sync(0xFFFFFFFFu, v, 4);
                v += __shfl_xor_sync(0xFFFFFFFFu, v, 8);
                v += __shfl_xor_sync(0xFFFFFFFFu, v, 16);
                if (lane < 4) atomicAdd(&soft->lsum[h0 + j], v);  // lane = kv-head of this thread
            }
            float* scr = reinterpret_cast<float*>(smem + SM_V);  // [24 heads][257]
            if (warp < 2) {
                const int m = warp * 32 + lane;
#pragma unroll 1
                for (int cb = 0; cb < 16; ++cb) {
                    uint32_t o[16];
                    tm_ld16(lane_base + TM_O + 16 * cb, o);
                    tm_ld_wait();
                    if (m < 24) {
#pragma unroll
                        for (int e = 0; e < 16; ++e)
                            if ((e & 3) != 3) scr[m * 257 + 16 * cb + e] = __uint_as_float(o[e]);
                    } else if (m < 48) {
#pragma unroll
                        for (int e = 3; e < 16; e += 4) scr[(m - 24) * 257 + 16 * cb + e] = __uint_as_float(o[e]);
                    }
                }
                tc_before();
            }
            dec_barrier();
            if (warp < 4) {  // kv-head = warp
#pragma unroll
                for (int h = 0; h < NREP; ++h) {
                    const int hd = warp * NREP + h;
#pragma unroll
                    for (int j = 0; j < 8; ++j) ws.acc[h][j] = scr[hd * 257 + lane * 8 + j];
                    const float M = soft->M[hd];
                    ws.m[h] = (M <= -1.0e29f) ? NEG_BIG : M * LN2;
                    ws.l[h] = soft->lsum[hd];
                }
            }
        }
    }
    cn.tiles = g0 + (unsigned)ntiles;
    cn.vph = v0 + 2u * (unsigned)ntiles;
}

// Persistent batched kernel, third generation (same contract as khq_decode_batched_kernel).
__global__ void __launch_bounds__(THREADS, 1)
khq_decode_batched_tc5_kernel(const KhqSeqDesc* __restrict__ descs, const KhqTablesDesc* __restrict__ tables,
                              const KhqWorkItem* __restrict__ items, int n_items, int* __restrict__ counter,
                              float* __restrict__ partials, float scale, float rope_base, int ring_cap) {
    extern __shared__ __align__(1024) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM_BARS);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM_BARS + 15 * 8);
    Soft* soft = reinterpret_cast<Soft*>(smem + SM_SOFT);
    if ((smem_u32(smem) & 1023u) != 0) {  // the swizzled operand layouts need a 1024-byte aligned base
        if (tid == 0) atomicExch(&g_status, 2);
        return;
    }
    if (tid == 0) {
        mbar_init(&bars[B_KFULL], 1);
        mbar_init(&bars[B_VFULL], 1);
        mbar_init(&bars[B_KFREE], 8);
        mbar_init(&bars[B_VFREE], 8);
        mbar_init(&bars[B_AREADY], 8);
        mbar_init(&bars[B_DREADY], 1);
        mbar_init(&bars[B_DFREE], 8);
        mbar_init(&bars[B_VREADY0], 4);
        mbar_init(&bars[B_VREADY1], 4);
        mbar_init(&bars[B_VDONE0], 1);
        mbar_init(&bars[B_VDONE1], 1);
        mbar_init(&bars[B_PREADY], 8);
        mbar_init(&bars[B_PVDONE], 1);
        fence_barrier_init();
        soft->abort_flag = 0;
        soft->all_alpha = 1;
    }
    // P starts as zeros: a row only ever writes the columns of its own kv-head's heads
    for (int e = tid; e < 2 * P_GROUP / 16; e += THREADS) reinterpret_cast<uint4*>(smem + SM_P)[e] = make_uint4(0u, 0u, 0u, 0u);
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "n"(TM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_before();
    __syncthreads();
    tc_after();
    const uint32_t tmem = *tmem_slot;

    int cur_table = -1;
    Counters cn = {0u, 0u};
#pragma unroll 1
    while (true) {
        __syncthreads();  // previous item fully retired
        if (tid == 0) soft->next_item = soft->abort_flag ? n_items : atomicAdd(counter, 1);
        __syncthreads();
        const int it = soft->next_item;
        if (it >= n_items) break;
        const KhqWorkItem w = items[it];
        const KhqSeqDesc d = descs[w.desc];
        const int kvh = warp & 3, sub = warp >> 2;
        float* ob[NREP];
#pragma unroll
        for (int h = 0; h < NREP; ++h) ob[h] = partials + ((size_t)w.slot * HQ + kvh * NREP + h) * PART;
        if (w.kind == 0) {
            const KhqTablesDesc tb = tables[d.table_id];
            CompressedKV P;
            P.k_payload = d.k_payload; P.v_payload = d.v_payload; P.v_shared_meta = d.v_shared_meta;
            P.k_mask = d.k_mask; P.k_norms = d.k_norms; P.k_r_norms = d.k_r_norms;
            P.v_norms = d.v_norms; P.v_r_norms = d.v_r_norms;
            P.cents_k = tb.cents_k; P.cents_v = tb.cents_v; P.vq = tb.vq; P.k_rotor = tb.k_rotor;
            P.v_rotor = tb.v_rotor; P.d_k = tb.d_k; P.d_v = tb.d_v;
            P.alpha_k = tb.alpha_k; P.alpha_v = tb.alpha_v; P.rope_base = rope_base;
            P.start_pos = d.start_pos; P.c_len = d.c_len; P.bulk_ok = 1; P.pos_chunk = 0; P.pos_stride = 0;
            // this generation advances RoPE by whole tiles: chunk-cyclic positions are not supported (status 4)
            if (d.pos_pack != 0 && tid == 0) atomicExch(&g_status, 4);
            if (d.table_id != cur_table) {
                if (tid == 0) soft->all_alpha = 1;
                __syncthreads();
                setup_layer(smem, P, tid);
                cur_table = d.table_id;
            }
            if (warp < 8) setup_item(smem, d.q_gate, (size_t)2 * D, P, tid);
            fence_proxy_async();  // B columns were written with ordinary stores, the tensor core reads them
            __syncthreads();
            WarpState ws;
            compressed_range(smem, tmem, d.q_gate, (size_t)2 * D, P, w.lo, w.hi, scale, cn, ws);
            if (warp < 4) v_epilogue_store(ws, P, lane, ob);
        } else if (warp < 8) {
            WarpState ws;
            ws.init();
            window_range(d.q_gate, d.ring_k, d.ring_v, d.win_start, w.lo + sub, 2, w.hi, ring_cap, scale, kvh, lane, ws);
            float* rec = reinterpret_cast<float*>(smem + SM_V) + kvh * MERGE_FLOATS;
            if (sub == 1) store_record(ws, rec, lane);
            dec_barrier();
            if (sub == 0) {
                merge_from(ws, rec, lane);
                raw_store(ws, lane, ob);
            }
        }
    }
    tc_before();
    __syncthreads();
    if (warp == 9) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(TM_COLS) : "memory");
    }
}

}  // namespace m3
}  // namespace khq
