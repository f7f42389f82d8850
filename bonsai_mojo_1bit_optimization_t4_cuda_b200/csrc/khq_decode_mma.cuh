// khq_decode_mma.cuh -- second-generation compressed-region decode: the two contractions of
// attention (q.K^T and p.V), the inverse K rotor + block sum, and the 64-dim rotary dot product
// run on the tensor cores with the 16 tokens of a block as the M dimension and the GQA group's
// six query heads (padded to 8) as N.  Included by khq_decode.cu (shares its helpers).
//
// Algebra.  K^ = RoPE_s( dinv * H256 * R * y ), y = alpha_k*k_norm*(mult*c*t + rs*sign*code).
// Everything left of y is linear, so it moves to the query side once per (sequence, layer):
//   * non-rotary output dims (>= 64):  q.K^ = y . q~,  q~ = R^T H256 (q * dinv * [dim >= 64])
//     -> one GEMM  S_pass[token, head] = T[token, dim] Q1[dim, head] + C[token, dim] Q2[dim, head]
//        with T = ternary symbols (exact in fp16), C = sign*code*(rs/mult), Q1 = q~*c, Q2 = q~;
//   * rotary output dims (< 64): the first 64 outputs of H256 are H64 of the sum of the four
//     64-dim blocks, so u[token, 64] = T * (R c)-blocks + C * R-blocks is a second GEMM with the
//     same A operands; H64, /d, the rotation by the token's angle, and a 64-deep GEMM with the raw
//     query finish it.
// V is accumulated in the rotated domain exactly as the first-generation kernel does:
//   O^T[dim, head] += V^T[dim, token] P^T[token, head], V^T = raw fp16 codebook entries (exact),
//   the per-token scales (alpha_v*v_norm*energy etc.) folded into three variants of P.
//
// Thread mapping (mma.sync.m16n8k16 fragments): lane = 4*g + t.  K side: token rows g and g+8,
// thread t owns the 64-dim quarter [64t, 64t+64) of both rows (mask words 4t..4t+3), k-step s
// covers dims 64t'+4s..+3 of all four quarters, i.e. the four patches that the rotor block sum
// adds up.  V side: thread (g, t) owns patch group g (patches 8g..8g+7) of tokens 2t, 2t+1,
// 2t+8, 2t+9.
//
// Registers and warps.  Twelve warps (three per scheduler) of at most 168 registers: what a warp keeps for a
// whole work item or layer -- the query-side and rotor-side B fragments and the 64 O^T accumulators -- lives in
// tensor memory, used here as a per-lane scratch file (tcgen05.st / tcgen05.ld; no tcgen05.mma), see M2_TM_COLS.
#pragma once
#include "khq_kdecode3.cuh"

namespace khq {

constexpr int M2_WPK = 3;           // warps per kv-head (12 warps: three per scheduler, at most 168 registers each)
constexpr int M2_TT = 16 * M2_WPK;  // tokens per tile: every warp of a kv-head takes 16
constexpr int M2_THREADS = 32 * HKV * M2_WPK;
constexpr int M2_NSTAGE = 2;
constexpr int M2_ROWS = M2_TT * HKV;
constexpr int M2_OFF_MASK = 0;
constexpr int M2_OFF_KPAY = M2_OFF_MASK + M2_ROWS * 64;
constexpr int M2_OFF_VPAY = M2_OFF_KPAY + M2_ROWS * K_PAY;
constexpr int M2_OFF_KN = M2_OFF_VPAY + M2_ROWS * V_PAY;
constexpr int M2_OFF_KRN = M2_OFF_KN + M2_ROWS * 2;
constexpr int M2_OFF_VN = M2_OFF_KRN + M2_ROWS * 2;
constexpr int M2_OFF_VRN = M2_OFF_VN + M2_ROWS * 2;
constexpr int M2_OFF_VSM = M2_OFF_VRN + M2_ROWS * 2;
constexpr int M2_STAGE_BYTES = M2_OFF_VSM + M2_ROWS * 4;  // 28160

constexpr int M2_SM_STAGES = 0;
// V codebook, split so that it fits beside everything else: (d0, d1) as one 32-bit word per
// (code, patch) and d2 as one half.  Rows of 65 words / 65 halfs instead of 64: the bank of a
// look-up then depends on the code as well as on the patch, which spreads the warp's 32
// look-ups (8 patches x 4 tokens per instruction) over the banks.
constexpr int M2_VQA_STRIDE = 65;                                    // words per code row
constexpr int M2_VQB_STRIDE = 130;                                   // bytes per code row
constexpr int M2_SM_VQ = M2_SM_STAGES + M2_NSTAGE * M2_STAGE_BYTES;  // (d0, d1): 256 x 65 x 4 B
constexpr int M2_SM_VQB = M2_SM_VQ + 256 * M2_VQA_STRIDE * 4;        // d2: 256 x 130 B
constexpr int M2_SM_ROPE = M2_SM_VQB + 256 * M2_VQB_STRIDE;          // 2 x M2_TT tokens x 32 float2
constexpr int M2_SM_BROT = M2_SM_ROPE + 2 * M2_TT * 32 * 8;          // 4 kinds x 16 steps x 32 lanes x 8 B
constexpr int M2_SM_FREQ = M2_SM_BROT + 4 * 16 * 32 * 8;
constexpr int M2_SM_DINV = M2_SM_FREQ + 128;                         // 64 floats
constexpr int M2_SM_BARS = M2_SM_DINV + 256;
constexpr int M2_SM_C3 = M2_SM_BARS + 64;              // 64 patches x float2: dim-3 centroids x alpha_v
constexpr int M2_SM_RSTEP = M2_SM_C3 + NP * 8;                          // 32 x float2: cos / sin of one tile's worth (32 positions) of each rotary pair
constexpr int M2_SM_QR = M2_SM_RSTEP + 32 * 8;                             // raw rotary query fragments: 4 kv-heads x 4 k-steps x 32 lanes x 8 B
constexpr int M2_SM_TOTAL = M2_SM_QR + HKV * 4 * 32 * 8;
// Tensor memory as a second register file.  The B fragments of the K side are per-lane constants: the query
// side (ternary part q1 and residual part q2, fp16 hi and lo, eight registers per k-step) for a whole work
// item, the rotor side (rotor x centroid and rotor, hi and lo, eight registers per k-step) for a whole layer.
// Held in registers the hi query fragments alone took 64 of the 255 across the tile loop, and the rest came
// from shared memory with six loads per k-step.  They are written to tensor memory (tcgen05.st: the query side
// once per item, the rotor side once per layer) and fetched one k-step ahead of use with two tcgen05.ld.
// Warp w owns lanes 32 (w & 3) .. +31, which it shares with the other warps of its kv-head.  Columns: 0 .. 127 =
// the kv-head's query fragments (eight per k-step: q1.x, q1.y, q2.x, q2.y and their low-order halves; written by
// the kv-head's first warp), 128 .. 255 = the rotor fragments of the lane quadrant (eight per k-step: b1.x, b1.y,
// b2.x, b2.y and their low-order halves; the same values in all four quadrants), 256 + 64 (w >> 2) .. +63 = the
// warp's O^T accumulators, which are in registers only while the V side of a block runs.
constexpr uint32_t M2_TM_COLS = 512, M2_TM_ROT = 128, M2_TM_ACC = 256;
static_assert(M2_TM_ACC + 64 * M2_WPK <= M2_TM_COLS, "tensor-memory columns");
static_assert(M2_SM_TOTAL <= 227 * 1024 && M2_SM_C3 % 16 == 0 && M2_SM_ROPE % 16 == 0 && M2_SM_VQB % 16 == 0,
              "shared memory budget");
static_assert(HKV * MERGE_FLOATS * 4 <= 256 * M2_VQA_STRIDE * 4, "cluster export records alias the codebook");
static_assert(HKV * M2_WPK * MERGE_FLOATS * 4 <= M2_NSTAGE * M2_STAGE_BYTES, "records alias the stages");
static_assert(HKV * NREP * D * 4 <= M2_NSTAGE * M2_STAGE_BYTES, "prologue scratch aliases the stages");
static_assert(M2_STAGE_BYTES % 16 == 0 && M2_OFF_KPAY % 16 == 0 && M2_OFF_VPAY % 16 == 0 && M2_OFF_KN % 16 == 0 &&
                  M2_OFF_VSM % 16 == 0, "bulk copy alignment");

__device__ __forceinline__ void m2_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t m2_movmatrix_t(uint32_t x) {
    uint32_t r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(x));
    return r;
}
// low-order ("what fp16 lost") products go through the same instruction
#define m2_mma_lo(c, a, b0, b1) m2_mma(c, a, b0, b1)
__device__ __forceinline__ uint32_t m2_pack(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}
// fp16x2 of (a, b) and fp16x2 of what that rounding lost: hi + lo carries ~22 mantissa bits.
__device__ __forceinline__ void m2_pack_hilo(float a, float b, uint32_t& hi, uint32_t& lo) {
    const __half2 h = __floats2half2_rn(a, b);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = m2_pack(a - __low2float(h), b - __high2float(h));
}
__device__ __forceinline__ uint32_t m2_hfma2(uint32_t a, uint32_t b, uint32_t c) {
    const __half2 r = __hfma2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b),
                              *reinterpret_cast<const __half2*>(&c));
    return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t m2_hmul2(uint32_t a, uint32_t b) {
    const __half2 r = __hmul2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
}

// Stage `ntok` tokens starting at `tok0` (same contract as stage_tile of the first generation).
__device__ __forceinline__ void m2_stage_tile(const CompressedKV& P, unsigned char* stage, uint64_t* bar, int tok0,
                                              int ntok, int tid) {
    const size_t r0 = (size_t)tok0 * HKV;
    const int rows = ntok * HKV;
    const unsigned char* src[8] = {reinterpret_cast<const unsigned char*>(P.k_mask) + r0 * 64,
                                   P.k_payload + r0 * K_PAY,
                                   P.v_payload + r0 * V_PAY,
                                   reinterpret_cast<const unsigned char*>(P.k_norms) + r0 * 2,
                                   reinterpret_cast<const unsigned char*>(P.k_r_norms) + r0 * 2,
                                   reinterpret_cast<const unsigned char*>(P.v_norms) + r0 * 2,
                                   reinterpret_cast<const unsigned char*>(P.v_r_norms) + r0 * 2,
                                   P.v_shared_meta + r0 * 4};
    const int dst[8] = {M2_OFF_MASK, M2_OFF_KPAY, M2_OFF_VPAY, M2_OFF_KN, M2_OFF_KRN, M2_OFF_VN, M2_OFF_VRN, M2_OFF_VSM};
    const int bpr[8] = {64, K_PAY, V_PAY, 2, 2, 2, 2, 4};
    const bool bulk = P.bulk_ok && ((tok0 & 1) == 0) && ((ntok & 1) == 0);
    if (bulk) {
        if (tid == 0) {
            mbar_arrive_expect_tx(bar, (uint32_t)(rows * 220));
#pragma unroll
            for (int a = 0; a < 8; ++a) bulk_g2s(stage + dst[a], src[a], (uint32_t)(rows * bpr[a]), bar);
        }
    } else {
#pragma unroll
        for (int a = 0; a < 8; ++a) {
            const int words = rows * bpr[a] / 4;
            const unsigned int* s = reinterpret_cast<const unsigned int*>(src[a]);
            unsigned int* d = reinterpret_cast<unsigned int*>(stage + dst[a]);
            for (int i = tid; i < words; i += M2_THREADS) d[i] = s[i];
        }
        fence_proxy_async();
        __syncthreads();
        if (tid == 0) mbar_arrive(bar);
    }
}

__device__ __forceinline__ void m2_fill_rope(float2* tab, const float* freq, const CompressedKV& P, int tok0, int tid) {
    for (int e = tid; e < M2_TT * 32; e += M2_THREADS) {
        const int t = e >> 5, m = e & 31;
        double th = (double)token_pos(P, tok0 + t) * (double)freq[m];
        th -= rint(th * 0.15915494309189535) * 6.283185307179586;
        float s, c;
        __sincosf((float)th, &s, &c);
        tab[e] = make_float2(c, s);
    }
}

// The next tile's RoPE table from this tile's: every entry turns by 32 positions of its pair (four FMAs
// instead of a range reduction and a sincos).  The caller re-seeds with m2_fill_rope every M2_ROPE_RESEED
// tiles, so that rounding never accumulates over more than that many turns (< 4e-6), and whenever the
// positions are not contiguous.
constexpr int M2_ROPE_RESEED = 64;
__device__ __forceinline__ void m2_step_rope(float2* dst, const float2* src, const float2* step, int tid) {
#pragma unroll
    for (int e = tid; e < M2_TT * 32; e += M2_THREADS) {
        const float2 a = src[e], d = step[e & 31];
        dst[e] = make_float2(a.x * d.x - a.y * d.y, a.y * d.x + a.x * d.y);
    }
}

// Per-layer constants in shared memory: RoPE frequencies, dinv of the 64 rotary dims, the rotor B fragments (with and without the centroid factor) and the V
// codebook.  Must be followed by __syncthreads().
__device__ __forceinline__ void m2_setup_tables(unsigned char* smem, const CompressedKV& P, int tid) {
    float* freq_s = reinterpret_cast<float*>(smem + M2_SM_FREQ);
    float* dinv_s = reinterpret_cast<float*>(smem + M2_SM_DINV);
    uint2* brot = reinterpret_cast<uint2*>(smem + M2_SM_BROT);
    unsigned short* vqa = reinterpret_cast<unsigned short*>(smem + M2_SM_VQ);
    unsigned short* vqb = reinterpret_cast<unsigned short*>(smem + M2_SM_VQB);
    if (tid < 32) freq_s[tid] = powf(P.rope_base, -2.0f * (float)tid / 64.0f);
    if (tid >= 128 && tid < 128 + NP)
        reinterpret_cast<float2*>(smem + M2_SM_C3)[tid - 128] = make_float2(__half2float(P.cents_v[0 * D + 4 * (tid - 128) + 3]) * P.alpha_v,
                                                                             __half2float(P.cents_v[1 * D + 4 * (tid - 128) + 3]) * P.alpha_v);
    if (tid < 64) dinv_s[tid] = (1.0f / 256.0f) / (__half2float(P.d_k[tid]) + 1e-8f);
    if (tid >= 192 && tid < 224) {
        const int m = tid - 192;
        double th = (double)M2_TT * (double)powf(P.rope_base, -2.0f * (float)m / 64.0f);
        th -= rint(th * 0.15915494309189535) * 6.283185307179586;
        reinterpret_cast<float2*>(smem + M2_SM_RSTEP)[m] = make_float2((float)cos(th), (float)sin(th));
    }
    // Rotor B fragments with the three low index bits of the 64-point Hadamard transform folded
    // in: u[8j + n] is produced by step s = 2j + (n >> 2) as rotor output c = n & 3, and
    // H64 = H8 (bits 0..2, inside a tile) x H8 (bits 3..5, across tiles), so column n' of the
    // folded operand is sum_n H8[n][n'] * (column n of the plain one).
    for (int e = tid; e < 16 * 32; e += M2_THREADS) {
        const int s = e >> 5, lane = e & 31;
        const int g = lane >> 2, t = lane & 3;
        const int patch = 16 * t + s;
        const int kk[4] = {0, 2, 1, 3};  // dims 64t+4s + {0, 2, 1, 3}
        float rc[4], r1[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float acc = 0.0f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int n = 4 * (s & 1) + c;
                const float sgn = (__popc(n & g) & 1) ? -1.0f : 1.0f;
                acc += sgn * __half2float(P.k_rotor[patch * 16 + c * 4 + kk[i]]);
            }
            r1[i] = acc;
            rc[i] = acc * __half2float(P.cents_k[2 * D + 64 * t + 4 * s + kk[i]]);
        }
        uint2 hi, lo;
        m2_pack_hilo(rc[0], rc[1], hi.x, lo.x);
        m2_pack_hilo(rc[2], rc[3], hi.y, lo.y);
        brot[e] = hi;          // rotor * centroid (ternary operand), fp16 hi
        brot[1024 + e] = lo;   //   and what fp16 lost
        m2_pack_hilo(r1[0], r1[1], hi.x, lo.x);
        m2_pack_hilo(r1[2], r1[3], hi.y, lo.y);
        brot[512 + e] = hi;    // rotor (residual operand), fp16 hi
        brot[1536 + e] = lo;   //   and what fp16 lost
    }
    stage_vq_codebook<M2_THREADS, M2_VQA_STRIDE, M2_VQB_STRIDE>(P.vq, reinterpret_cast<unsigned int*>(vqa), vqb, tid);
}

// Query-side operands of one (sequence, layer, kv-head): this warp's B fragments.
struct M2Query {
    uint32_t tm;   // tensor-memory address of this warp's query fragments
    uint32_t rot;  // ... and of its lane quadrant's rotor fragments
};

__device__ __forceinline__ void m2_tm_st4(uint32_t taddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%4], {%0,%1,%2,%3};" ::"r"(a), "r"(b), "r"(c), "r"(d), "r"(taddr) : "memory");
}
__device__ __forceinline__ void m2_tm_ld4(uint32_t taddr, uint32_t (&r)[4]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void m2_tm_st8(uint32_t taddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t e, uint32_t f,
                                          uint32_t g, uint32_t h) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%8], {%0,%1,%2,%3,%4,%5,%6,%7};" ::"r"(a), "r"(b), "r"(c), "r"(d), "r"(e),
                 "r"(f), "r"(g), "r"(h), "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void m2_tm_ld8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void m2_tm_st16f(uint32_t taddr, const float* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15};" ::"f"(r[0]),
        "f"(r[1]), "f"(r[2]), "f"(r[3]), "f"(r[4]), "f"(r[5]), "f"(r[6]), "f"(r[7]), "f"(r[8]), "f"(r[9]), "f"(r[10]), "f"(r[11]),
        "f"(r[12]), "f"(r[13]), "f"(r[14]), "f"(r[15]), "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void m2_tm_ld16f(uint32_t taddr, float* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7]), "=f"(r[8]), "=f"(r[9]),
          "=f"(r[10]), "=f"(r[11]), "=f"(r[12]), "=f"(r[13]), "=f"(r[14]), "=f"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void m2_tm_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void m2_tm_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// Allocation by warp 0 of a CTA (one CTA per SM by shared memory, so the columns are always free); the address goes
// through `slot` in shared memory.  Followed by a CTA barrier by the caller.
__device__ __forceinline__ void m2_tm_alloc(uint32_t* slot, int warp) {
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "n"(M2_TM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
// After a CTA barrier behind the last use.
__device__ __forceinline__ void m2_tm_free(uint32_t tmem, int warp) {
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(M2_TM_COLS) : "memory");
    }
}

// The layer's rotor fragments from their shared-memory staging table into the tensor memory of every lane
// quadrant (warps 0..3, one quadrant each).  After the CTA barrier that follows m2_setup_tables; the readers
// pass another CTA barrier and a tcgen05 fence before their first load.
__device__ __forceinline__ void m2_rotor_to_tmem(const unsigned char* smem, uint32_t tmem, int warp, int lane) {
    if (warp < 4) {
        const uint2* brot = reinterpret_cast<const uint2*>(smem + M2_SM_BROT);
        const uint32_t dst = tmem + ((uint32_t)(32 * warp) << 16) + M2_TM_ROT;
#pragma unroll 4
        for (int s = 0; s < 16; ++s) {
            const uint2 b1 = brot[s * 32 + lane], b2 = brot[512 + s * 32 + lane], b1l = brot[1024 + s * 32 + lane],
                        b2l = brot[1536 + s * 32 + lane];
            m2_tm_st8(dst + 8 * s, b1.x, b1.y, b2.x, b2.y, b1l.x, b1l.y, b2l.x, b2l.y);
        }
        m2_tm_st_wait();
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

// q: (H_q, ..) with `q_head_stride` halfs between heads.  scratch: this warp's NREP*D floats.
__device__ __forceinline__ void m2_build_query(M2Query& Q, const __half* __restrict__ q, size_t q_head_stride,
                                               const CompressedKV& P, int kvh, int sub, int lane, float* scratch,
                                               uint2* qr_s /* this kv-head's [4][32] raw rotary query fragments */) {
    // The M2_WPK warps of a kv-head share the work (it runs once per work item, on the critical path): warp `sub`
    // transforms query heads sub, sub + M2_WPK, ... into the kv-head's scratch, the warps meet at a named barrier,
    // then warp `sub` builds the B fragments of k-steps sub, sub + M2_WPK, ... .  Every global load is issued before
    // the first one is needed.
    const int g = lane >> 2, t = lane & 3;
    constexpr int HPW = NREP / M2_WPK;  // heads per warp
    static_assert(NREP % M2_WPK == 0, "query heads split evenly over the warps of a kv-head");
    float dv[8], rr[2][16];
    uint4 qraw[HPW];
#pragma unroll
    for (int i = 0; i < HPW; ++i)
        qraw[i] = *reinterpret_cast<const uint4*>(q + (size_t)(kvh * NREP + sub + M2_WPK * i) * q_head_stride + lane * 8);
    // for the fragments built after the transforms: the centroids of dims 64 t + 4 s + {0..3} and the raw rotary query dims
    constexpr int SPW = (16 + M2_WPK - 1) / M2_WPK;  // k-steps per warp (the last warps may have one less)
    uint2 cck[SPW];
    uint32_t qrw[4][2];
#pragma unroll
    for (int i = 0; i < SPW; ++i) {
        const int s = sub + M2_WPK * i;
        cck[i] = (g < NREP && s < 16) ? *reinterpret_cast<const uint2*>(P.cents_k + 2 * D + 64 * t + 4 * s) : make_uint2(0u, 0u);
    }
    if (sub == 0) {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            const __half* qh = q + (size_t)(kvh * NREP + (g < NREP ? g : 0)) * q_head_stride + 16 * kk + 2 * t;
            qrw[kk][0] = (g < NREP) ? *reinterpret_cast<const uint32_t*>(qh) : 0u;
            qrw[kk][1] = (g < NREP) ? *reinterpret_cast<const uint32_t*>(qh + 8) : 0u;
        }
    }
    {
        const uint4 dr = *reinterpret_cast<const uint4*>(P.d_k + lane * 8);
        const uint4* rp = reinterpret_cast<const uint4*>(P.k_rotor + lane * 32);
        const uint4 r0 = rp[0], r1 = rp[1], r2 = rp[2], r3 = rp[3];
        const __half* hd = reinterpret_cast<const __half*>(&dr);
#pragma unroll
        for (int j = 0; j < 8; ++j) dv[j] = (lane >= 8) ? (1.0f / 256.0f) / (__half2float(hd[j]) + 1e-8f) : 0.0f;
        __half hr[32];
        *reinterpret_cast<uint4*>(&hr[0]) = r0;
        *reinterpret_cast<uint4*>(&hr[8]) = r1;
        *reinterpret_cast<uint4*>(&hr[16]) = r2;
        *reinterpret_cast<uint4*>(&hr[24]) = r3;
#pragma unroll
        for (int p = 0; p < 2; ++p)
#pragma unroll
            for (int i = 0; i < 16; ++i) rr[p][i] = __half2float(hr[p * 16 + i]);
    }
    // q~ in the lane-owns-8-dims layout: q~ = R^T H256 (q * dinv * [dim >= 64])
#pragma unroll
    for (int i = 0; i < HPW; ++i) {
        const int h = sub + M2_WPK * i;
        const __half* hq = reinterpret_cast<const __half*>(&qraw[i]);
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
                scratch[h * D + lane * 8 + p * 4 + k] = a;
            }
    }
    asm volatile("bar.sync %0, %1;" ::"r"(2 + kvh), "n"(32 * M2_WPK) : "memory");  // the kv-head's warps: all six heads are in the scratch
#pragma unroll
    for (int i = 0; i < SPW; ++i) {
        const int s = sub + M2_WPK * i;
        if (s < 16) {
            const int d0 = 64 * t + 4 * s;
            float v[4] = {0.0f, 0.0f, 0.0f, 0.0f}, c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            if (g < NREP) {
                const float4 qq = *reinterpret_cast<const float4*>(scratch + g * D + d0);
                const __half* hc = reinterpret_cast<const __half*>(&cck[i]);
                v[0] = qq.x; v[1] = qq.z; v[2] = qq.y; v[3] = qq.w;  // dims d0 + {0, 2, 1, 3}
                c[0] = __half2float(hc[0]); c[1] = __half2float(hc[2]); c[2] = __half2float(hc[1]); c[3] = __half2float(hc[3]);
            }
            uint2 lo, hi;
            m2_pack_hilo(v[0] * c[0], v[1] * c[1], hi.x, lo.x);
            m2_pack_hilo(v[2] * c[2], v[3] * c[3], hi.y, lo.y);
            uint2 lo2, hi2;
            m2_pack_hilo(v[0], v[1], hi2.x, lo2.x);
            m2_pack_hilo(v[2], v[3], hi2.y, lo2.y);
            m2_tm_st8(Q.tm + 8 * s, hi.x, hi.y, hi2.x, hi2.y, lo.x, lo.y, lo2.x, lo2.y);
        }
    }
    m2_tm_st_wait();
    if (sub == 0) {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) qr_s[kk * 32 + lane] = make_uint2(qrw[kk][0], qrw[kk][1]);
    }
    __syncwarp();
}

// Running attention state of a warp in fragment layout: thread (g, t) holds heads 2t, 2t+1.
struct M2State {
    uint32_t tm_o;  // tensor-memory address of the warp's 64 accumulator columns: O^T tiles [0..11] dims 0..2 of the
                    // patches, [12..15] dim 3 of the patches, four registers each; in registers only during the V side
    float m[2], l[2];
    __device__ __forceinline__ void init() {  // whole warp
        float z[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) z[i] = 0.0f;
#pragma unroll
        for (int c = 0; c < 4; ++c) m2_tm_st16f(tm_o + 16 * c, z);
        m2_tm_st_wait();
        m[0] = m[1] = NEG_BIG;
        l[0] = l[1] = 0.0f;
    }
};

// Packed pairs of fp32 (one instruction for two neighbouring accumulator registers; each half is
// rounded like the scalar operation).
__device__ __forceinline__ void m2_add2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
    asm("{.reg .b64 a, b, d; mov.b64 a, {%2, %3}; mov.b64 b, {%4, %5}; add.rn.f32x2 d, a, b; mov.b64 {%0, %1}, d;}"
        : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
__device__ __forceinline__ void m2_sub2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
    asm("{.reg .b64 a, b, d; mov.b64 a, {%2, %3}; mov.b64 b, {%4, %5}; sub.rn.f32x2 d, a, b; mov.b64 {%0, %1}, d;}"
        : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
__device__ __forceinline__ void m2_fma2(float& d0, float& d1, float a0, float a1, float b0, float b1, float c0,
                                        float c1) {
    asm("{.reg .b64 a, b, c, d; mov.b64 a, {%2, %3}; mov.b64 b, {%4, %5}; mov.b64 c, {%6, %7};"
        " fma.rn.f32x2 d, a, b, c; mov.b64 {%0, %1}, d;}"
        : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1), "f"(c0), "f"(c1));
}

// One block of 16 tokens (rows r0..r0+15 of the staged tile) of kv-head `kvh`.
// valid_lo/valid_hi: block-relative range of tokens that belong to the caller's range.
__device__ __forceinline__ void m2_block(const unsigned char* __restrict__ S, const unsigned char* __restrict__ smem,
                                         const float2* __restrict__ rope, int r0, int kvh, int lane, int valid_lo,
                                         int valid_hi, const M2Query& Q, const CompressedKV& P, float scale,
                                         M2State& st) {
    const int g = lane >> 2, t = lane & 3;
    const float* dinv_s = reinterpret_cast<const float*>(smem + M2_SM_DINV);
    const unsigned char* vqa = smem + M2_SM_VQ;
    const unsigned char* vqb = smem + M2_SM_VQB;
    const float2* c3s = reinterpret_cast<const float2*>(smem + M2_SM_C3) + 8 * g;
    const uint2* qr_s = reinterpret_cast<const uint2*>(smem + M2_SM_QR) + kvh * 4 * 32;

    // ================================ K side: scores ==========================================
    const uint32_t* kp[2];
    uint4 mw[2];
    uint32_t wbase[2];
    float sp[2], sp2[2];
    float ratio[2];  // rs / mult of rows g, g + 8: scales the residual part of the rotor sums after their GEMM
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        const int row = (r0 + g + 8 * x) * HKV + kvh;
        kp[x] = reinterpret_cast<const uint32_t*>(S + M2_OFF_KPAY + row * K_PAY);
        mw[x] = *reinterpret_cast<const uint4*>(S + M2_OFF_MASK + row * 64 + 16 * t);
        // outliers of this thread's quarter, then the ordinal of its first one (scan over the quad)
        int cnt = (int)(khq3::k3_count(mw[x].x) + khq3::k3_count(mw[x].y) + khq3::k3_count(mw[x].z) + khq3::k3_count(mw[x].w));
        int incl = cnt;
        int up = __shfl_up_sync(0xFFFFFFFFu, incl, 1);
        if (t >= 1) incl += up;
        up = __shfl_up_sync(0xFFFFFFFFu, incl, 2);
        if (t >= 2) incl += up;
        wbase[x] = (uint32_t)(incl - cnt);
        float mult = (float)kp[x][0] / 1000.0f;
        if (mult < 0.1f || mult > 10.0f || isnan(mult)) mult = 1.0f;
        const float rs = hbits2f(reinterpret_cast<const uint16_t*>(S + M2_OFF_KRN)[row]);
        const float kn = hbits2f(reinterpret_cast<const uint16_t*>(S + M2_OFF_KN)[row]);
        sp[x] = P.alpha_k * kn * mult * scale;
        sp2[x] = P.alpha_k * kn * rs * scale;
        ratio[x] = rs / mult;
    }
    const uint32_t neg1024 = 0xE400E400u;  // fp16x2 (-1024, -1024)
    float cs[4] = {0.0f, 0.0f, 0.0f, 0.0f};   // pass-part scores, ternary part: rows g (0,1), g+8 (2,3); heads 2t, 2t+1
    float cs2[4] = {0.0f, 0.0f, 0.0f, 0.0f};  // pass-part scores, residual part (exact integer operand)
    float cu[8][4];                          // rotor block sums u[token, 8j + n]
    float cur[4];                            // their residual part, before the row scale
#pragma unroll
    for (int j = 0; j < 8; ++j) cu[j][0] = cu[j][1] = cu[j][2] = cu[j][3] = 0.0f;
    uint32_t qf[2][8], rf[2][8];  // this and the next k-step's query and rotor fragments
    m2_tm_ld8(Q.tm, qf[0]);
    m2_tm_ld8(Q.rot, rf[0]);
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
        const uint32_t wa = wi == 0 ? mw[0].x : wi == 1 ? mw[0].y : wi == 2 ? mw[0].z : mw[0].w;
        const uint32_t wb = wi == 0 ? mw[1].x : wi == 1 ? mw[1].y : wi == 2 ? mw[1].z : mw[1].w;
        // a whole mask word (16 dims = this thread's share of four k-steps) of each of the two rows at once
        uint32_t ta[8], ha[8], tb[8], hb[8];
        wbase[0] += khq3::k3_word(wa, wbase[0], kp[0], ta, ha);
        wbase[1] += khq3::k3_word(wb, wbase[1], kp[1], tb, hb);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int s = wi * 4 + q;
            const uint32_t a1[4] = {ta[q], tb[q], ta[4 + q], tb[4 + q]};  // dims (4q, 4q + 2) and (4q + 1, 4q + 3) of rows g, g + 8
            const uint32_t ax[4] = {m2_hfma2(ta[q], neg1024, ha[q]), m2_hfma2(tb[q], neg1024, hb[q]),
                                    m2_hfma2(ta[4 + q], neg1024, ha[4 + q]), m2_hfma2(tb[4 + q], neg1024, hb[4 + q])};  // sign*code, exact
            m2_tm_ld_wait();
            if (s + 1 < 16) {
                m2_tm_ld8(Q.tm + 8 * (s + 1), qf[(s + 1) & 1]);
                m2_tm_ld8(Q.rot + 8 * (s + 1), rf[(s + 1) & 1]);
            }
            const uint32_t(&qq)[8] = qf[s & 1];  // q1.x, q1.y, q2.x, q2.y, then their low-order halves
            const uint32_t(&rr)[8] = rf[s & 1];  // b1.x, b1.y, b2.x, b2.y, then their low-order halves
            m2_mma(cs, a1, qq[0], qq[1]);
            m2_mma_lo(cs, a1, qq[4], qq[5]);  // low-order halves of the query operands: the code operands are exact
            m2_mma(cs2, ax, qq[2], qq[3]);
            m2_mma_lo(cs2, ax, qq[6], qq[7]);
            m2_mma(cu[s >> 1], a1, rr[0], rr[1]);
            m2_mma_lo(cu[s >> 1], a1, rr[4], rr[5]);
            // residual part of the same rotor sums: exact integer operand first, the row's rs / mult in fp32 after the
            // two k-steps that feed this tile
            if ((s & 1) == 0) cur[0] = cur[1] = cur[2] = cur[3] = 0.0f;
            m2_mma(cur, ax, rr[2], rr[3]);
            m2_mma_lo(cur, ax, rr[6], rr[7]);
            if (s & 1) {
                float* c = cu[s >> 1];
                m2_fma2(c[0], c[1], ratio[0], ratio[0], cur[0], cur[1], c[0], c[1]);
                m2_fma2(c[2], c[3], ratio[1], ratio[1], cur[2], cur[3], c[2], c[3]);
            }
        }
    }
    // ---- rotary part: rest of H64 over idx = 8j + 2t + e, /d, rotation, dot with the raw query ----
    float cr[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    {
        // index bits 0..2 were transformed inside the GEMM (folded into the rotor operand)
        // bits 3, 4, 5 (j)
#pragma unroll
        for (int m = 1; m <= 4; m <<= 1)
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if ((j & m) == 0)
#pragma unroll
                    for (int e = 0; e < 4; e += 2) {
                        const float a0 = cu[j][e], a1 = cu[j][e + 1], b0 = cu[j | m][e], b1 = cu[j | m][e + 1];
                        m2_add2(cu[j][e], cu[j][e + 1], a0, a1, b0, b1);
                        m2_sub2(cu[j | m][e], cu[j | m][e + 1], a0, a1, b0, b1);
                    }
        // scale by dinv, rotate pairs (idx, idx + 32) = tiles (j, j + 4)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 dlo = *reinterpret_cast<const float2*>(dinv_s + 8 * j + 2 * t);
            const float2 dhi = *reinterpret_cast<const float2*>(dinv_s + 32 + 8 * j + 2 * t);
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                const float4 rc = *reinterpret_cast<const float4*>(rope + (r0 + g + 8 * x) * 32 + 8 * j + 2 * t);
                const float z0 = cu[j][2 * x] * dlo.x, z1 = cu[j][2 * x + 1] * dlo.y;
                const float w0 = cu[j + 4][2 * x] * dhi.x, w1 = cu[j + 4][2 * x + 1] * dhi.y;
                cu[j][2 * x] = z0 * rc.x - w0 * rc.y;
                cu[j + 4][2 * x] = z0 * rc.y + w0 * rc.x;
                cu[j][2 * x + 1] = z1 * rc.z - w1 * rc.w;
                cu[j + 4][2 * x + 1] = z1 * rc.w + w1 * rc.z;
            }
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            uint32_t a[4], al[4];  // rotated K^ dims as fp16 hi + lo: the raw query operand is exact
            m2_pack_hilo(cu[2 * kk][0], cu[2 * kk][1], a[0], al[0]);
            m2_pack_hilo(cu[2 * kk][2], cu[2 * kk][3], a[1], al[1]);
            m2_pack_hilo(cu[2 * kk + 1][0], cu[2 * kk + 1][1], a[2], al[2]);
            m2_pack_hilo(cu[2 * kk + 1][2], cu[2 * kk + 1][3], a[3], al[3]);
            const uint2 qrk = qr_s[kk * 32 + lane];
            m2_mma(cr, a, qrk.x, qrk.y);
            m2_mma_lo(cr, al, qrk.x, qrk.y);
        }
    }
    // ================================ softmax over the block ====================================
    float sc[2][2], pw[2][2];  // [row x: g, g+8][head e: 2t, 2t+1]
    bool valid[2];
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        valid[x] = (g + 8 * x) >= valid_lo && (g + 8 * x) < valid_hi;
#pragma unroll
        for (int e = 0; e < 2; ++e)
            sc[x][e] = valid[x] ? fmaf(sp[x], cs[2 * x + e] + cr[2 * x + e], sp2[x] * cs2[2 * x + e]) : -1e30f;
    }
    float corr[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        float bm = fmaxf(sc[0][e], sc[1][e]);
        bm = fmaxf(bm, __shfl_xor_sync(0xFFFFFFFFu, bm, 4));
        bm = fmaxf(bm, __shfl_xor_sync(0xFFFFFFFFu, bm, 8));
        bm = fmaxf(bm, __shfl_xor_sync(0xFFFFFFFFu, bm, 16));
        const float mn = fmaxf(st.m[e], bm);
        corr[e] = __expf(st.m[e] - mn);
        st.m[e] = mn;
        pw[0][e] = valid[0] ? __expf(sc[0][e] - mn) : 0.0f;
        pw[1][e] = valid[1] ? __expf(sc[1][e] - mn) : 0.0f;
        st.l[e] = st.l[e] * corr[e] + pw[0][e] + pw[1][e];
    }
    const bool rescale = __any_sync(0xFFFFFFFFu, corr[0] != 1.0f || corr[1] != 1.0f);
    // three scaled variants of P, transposed into B fragments (tokens = k, heads = n)
    uint32_t pb[3][2], pl_[3][2];  // fp16 hi and the fp16 of what hi lost
    {
        float s1[2], s2[2], s3[2];
#pragma unroll
        for (int x = 0; x < 2; ++x) {
            const int row = (r0 + g + 8 * x) * HKV + kvh;
            const float vn = hbits2f(reinterpret_cast<const uint16_t*>(S + M2_OFF_VN)[row]);
            const float en = hbits2f(reinterpret_cast<const uint16_t*>(S + M2_OFF_VRN)[row]);
            const float sm = reinterpret_cast<const float*>(S + M2_OFF_VSM)[row];
            s1[x] = valid[x] ? P.alpha_v * vn * en : 0.0f;     // dims 0..2: codebook entry
            s2[x] = valid[x] ? vn : 0.0f;                      // dim 3: centroid * alpha_v (folded in c3)
            s3[x] = valid[x] ? sm * vn * (1.0f / 7.0f) : 0.0f;  // dim 3: (dump - 8)
        }
#pragma unroll
        for (int x = 0; x < 2; ++x) {
            uint32_t hi, lo;
            m2_pack_hilo(pw[x][0] * s1[x], pw[x][1] * s1[x], hi, lo);
            pb[0][x] = m2_movmatrix_t(hi);
            pl_[0][x] = m2_movmatrix_t(lo);
            m2_pack_hilo(pw[x][0] * s2[x], pw[x][1] * s2[x], hi, lo);
            pb[1][x] = m2_movmatrix_t(hi);
            pl_[1][x] = m2_movmatrix_t(lo);
            m2_pack_hilo(pw[x][0] * s3[x], pw[x][1] * s3[x], hi, lo);
            pb[2][x] = m2_movmatrix_t(hi);
            pl_[2][x] = m2_movmatrix_t(lo);
        }
    }
    // ================================ V side: O^T += V^T P^T ====================================
    // the accumulators come out of tensor memory for this part only
    float o[16][4];
#pragma unroll
    for (int c = 0; c < 4; ++c) m2_tm_ld16f(st.tm_o + 16 * c, &o[4 * c][0]);
    m2_tm_ld_wait();
    if (rescale) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            o[i][0] *= corr[0];
            o[i][1] *= corr[1];
            o[i][2] *= corr[0];
            o[i][3] *= corr[1];
        }
    }
    // thread (g, t): patch group g of tokens 2t, 2t+1, 2t+8, 2t+9
    uint32_t vw[4][3], hb[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int tok = 2 * t + (i & 1) + 8 * (i >> 1);
        const uint32_t* vp = reinterpret_cast<const uint32_t*>(S + M2_OFF_VPAY + ((r0 + tok) * HKV + kvh) * V_PAY);
        vw[i][0] = vp[3 * g];
        vw[i][1] = vp[3 * g + 1];
        vw[i][2] = vp[3 * g + 2];
        hb[i] = ((vp[24 + (g >> 2)] >> (8 * (g & 3))) & 0xFFu) << 7;  // bit 7 + pl = high code bit of patch pl
    }
#pragma unroll
    for (int pp = 0; pp < 4; ++pp) {  // patch pairs (2pp, 2pp+1) -> tiles 3pp .. 3pp+2
        uint32_t ex[2][4], ey[2][4];  // [patch of the pair][token i]: (d0,d1), (d2,-)
        uint32_t f3[2][4];            // 12-bit fields
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int pl = 2 * pp + u;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint32_t f;
                switch (pl) {
                    case 0: f = vw[i][0]; break;
                    case 1: f = vw[i][0] >> 12; break;
                    case 2: f = (vw[i][0] >> 24) | (vw[i][1] << 8); break;
                    case 3: f = vw[i][1] >> 4; break;
                    case 4: f = vw[i][1] >> 16; break;
                    case 5: f = (vw[i][1] >> 28) | (vw[i][2] << 4); break;
                    case 6: f = vw[i][2] >> 8; break;
                    default: f = vw[i][2] >> 20; break;
                }
                f &= 0xFFFu;
                f3[u][i] = f;
                const uint32_t code = (f & 0x7Fu) | ((hb[i] >> pl) & 0x80u);
                ex[u][i] = *reinterpret_cast<const uint32_t*>(vqa + (code * M2_VQA_STRIDE + 8 * g + pl) * 4);
                ey[u][i] = *reinterpret_cast<const unsigned short*>(vqb + code * M2_VQB_STRIDE + (8 * g + pl) * 2);
            }
        }
        // rows: idx = 2j + r -> (patch idx/3, dim idx%3); the pair's six (patch, dim) rows in order
        uint32_t lo[6], hi[6];  // token pairs (2t, 2t+1) and (2t+8, 2t+9)
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            lo[3 * u + 0] = __byte_perm(ex[u][0], ex[u][1], 0x5410);
            lo[3 * u + 1] = __byte_perm(ex[u][0], ex[u][1], 0x7632);
            lo[3 * u + 2] = __byte_perm(ey[u][0], ey[u][1], 0x5410);
            hi[3 * u + 0] = __byte_perm(ex[u][2], ex[u][3], 0x5410);
            hi[3 * u + 1] = __byte_perm(ex[u][2], ex[u][3], 0x7632);
            hi[3 * u + 2] = __byte_perm(ey[u][2], ey[u][3], 0x5410);
        }
#pragma unroll
        for (int jj = 0; jj < 3; ++jj) {
            const uint32_t a[4] = {lo[2 * jj], lo[2 * jj + 1], hi[2 * jj], hi[2 * jj + 1]};
            m2_mma(o[3 * pp + jj], a, pb[0][0], pb[0][1]);
            m2_mma_lo(o[3 * pp + jj], a, pl_[0][0], pl_[0][1]);
        }
        // dim 3 of the two patches (rows 0, 1 of tile 12 + pp): centroid choice and (dump - 8)
        uint32_t ca[4], da[4];  // a0..a3 of the two extra MMAs
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int pl = 2 * pp + u;
            float cv[4];
            uint32_t dv[4];
            const float2 c3p = c3s[pl];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                cv[i] = ((f3[u][i] >> 7) & 1u) ? c3p.y : c3p.x;
                dv[i] = 0x6400u | (f3[u][i] >> 8);  // fp16 bits of 1024 + dump
            }
            ca[u] = m2_pack(cv[0], cv[1]);
            ca[2 + u] = m2_pack(cv[2], cv[3]);
            const uint32_t bias = 0x64086408u;  // fp16x2 (1032, 1032): (1024 + dump) - 1032 = dump - 8
            const uint32_t plo = dv[0] | (dv[1] << 16), phi = dv[2] | (dv[3] << 16);
            const __half2 d_lo = __hsub2(*reinterpret_cast<const __half2*>(&plo), *reinterpret_cast<const __half2*>(&bias));
            const __half2 d_hi = __hsub2(*reinterpret_cast<const __half2*>(&phi), *reinterpret_cast<const __half2*>(&bias));
            da[u] = *reinterpret_cast<const uint32_t*>(&d_lo);
            da[2 + u] = *reinterpret_cast<const uint32_t*>(&d_hi);
        }
        m2_mma(o[12 + pp], ca, pb[1][0], pb[1][1]);
        m2_mma_lo(o[12 + pp], ca, pl_[1][0], pl_[1][1]);
        m2_mma(o[12 + pp], da, pb[2][0], pb[2][1]);
        m2_mma_lo(o[12 + pp], da, pl_[2][0], pl_[2][1]);
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) m2_tm_st16f(st.tm_o + 16 * c, &o[4 * c][0]);
    m2_tm_st_wait();
}

// Attention of all 24 query heads over compressed tokens [my_lo, my_hi) of P; the CTA's 12 warps
// are (kv-head = warp & 3) x (16-token third of each 48-token tile = warp >> 2).  On return,
// warps 0..3 hold in `ws` the merged state of their kv-head's six heads in the first generation's
// layout (lane = 8 dims, rotated V domain), ready for merge_from / v_epilogue_store.  Tables must
// be set up; all M2_THREADS threads call it.
template <bool ALL_WARPS_MERGE = false>  // true: every warp of a kv-head returns the kv-head's merged state
__device__ __forceinline__ void m2_compressed_range(unsigned char* smem, const __half* __restrict__ q,
                                                    size_t q_head_stride, const CompressedKV& P, int my_lo, int my_hi,
                                                    float scale, unsigned& tiles_done, WarpState& ws, uint32_t tmem) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kvh = warp & 3, sub = warp >> 2, g = lane >> 2, t = lane & 3;
    float2* rope_tab = reinterpret_cast<float2*>(smem + M2_SM_ROPE);
    const float* freq_s = reinterpret_cast<const float*>(smem + M2_SM_FREQ);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + M2_SM_BARS);

    M2Query Q;
    Q.tm = tmem + ((uint32_t)(32 * kvh) << 16);
    Q.rot = tmem + ((uint32_t)(32 * kvh) << 16) + M2_TM_ROT;
    m2_build_query(Q, q, q_head_stride, P, kvh, sub, lane, reinterpret_cast<float*>(smem + M2_SM_STAGES) + kvh * NREP * D,
                   reinterpret_cast<uint2*>(smem + M2_SM_QR) + kvh * 4 * 32);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();  // the query scratch aliases the stages
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");  // the query and rotor fragments other warps stored

    const int base = my_lo & ~1;
    const int ntiles = (my_hi > my_lo) ? (my_hi - base + M2_TT - 1) / M2_TT : 0;
    const unsigned t0 = tiles_done;
    if (ntiles > 0) {
        m2_fill_rope(rope_tab, freq_s, P, base, tid);
        m2_stage_tile(P, smem + M2_SM_STAGES + (t0 % M2_NSTAGE) * M2_STAGE_BYTES, &bars[t0 % M2_NSTAGE], base,
                      min(M2_TT, P.c_len - base), tid);
    }
    __syncthreads();
    M2State st;
    st.tm_o = tmem + ((uint32_t)(32 * kvh) << 16) + M2_TM_ACC + 64u * (uint32_t)sub;
    st.init();
#pragma unroll 1
    for (int i = 0; i < ntiles; ++i) {
        const unsigned gi = t0 + i;
        const int stg = gi % M2_NSTAGE;
        if (i + 1 < ntiles) {
            const int tok0 = base + (i + 1) * M2_TT;
            m2_stage_tile(P, smem + M2_SM_STAGES + ((gi + 1) % M2_NSTAGE) * M2_STAGE_BYTES, &bars[(gi + 1) % M2_NSTAGE],
                          tok0, min(M2_TT, P.c_len - tok0), tid);
            if (P.pos_chunk == 0 && ((i + 1) % M2_ROPE_RESEED) != 0)
                m2_step_rope(rope_tab + ((i + 1) & 1) * M2_TT * 32, rope_tab + (i & 1) * M2_TT * 32,
                             reinterpret_cast<const float2*>(smem + M2_SM_RSTEP), tid);
            else
                m2_fill_rope(rope_tab + ((i + 1) & 1) * M2_TT * 32, freq_s, P, tok0, tid);
        }
        mbar_wait_bounded(&bars[stg], (uint32_t)((gi / M2_NSTAGE) & 1), &g_status);
        const int blk0 = base + i * M2_TT + 16 * sub;
        const int vlo = max(my_lo - blk0, 0), vhi = min(my_hi - blk0, 16);
        if (vhi > vlo)
            m2_block(smem + M2_SM_STAGES + stg * M2_STAGE_BYTES, smem, rope_tab + (i & 1) * M2_TT * 32, 16 * sub, kvh,
                     lane, vlo, vhi, Q, P, scale, st);
        __syncthreads();  // stage and rope buffer free for the tile after next
    }
    tiles_done = t0 + (unsigned)ntiles;

    // ---- per-warp record in the first generation's layout, then merge + inverse V transform --------
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        st.l[e] += __shfl_xor_sync(0xFFFFFFFFu, st.l[e], 4);
        st.l[e] += __shfl_xor_sync(0xFFFFFFFFu, st.l[e], 8);
        st.l[e] += __shfl_xor_sync(0xFFFFFFFFu, st.l[e], 16);
    }
    float* rec = reinterpret_cast<float*>(smem + M2_SM_STAGES) + warp * MERGE_FLOATS;
    float o[16][4];
#pragma unroll
    for (int c = 0; c < 4; ++c) m2_tm_ld16f(st.tm_o + 16 * c, &o[4 * c][0]);
    m2_tm_ld_wait();
    if (t < 3) {
#pragma unroll
        for (int j = 0; j < 16; ++j)
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int idx = 2 * j + r;
                const int dim = j < 12 ? 4 * (8 * g + idx / 3) + idx % 3 : 4 * (8 * g + 2 * (j - 12) + r) + 3;
                rec[(2 * t) * D + dim] = o[j][2 * r];
                rec[(2 * t + 1) * D + dim] = o[j][2 * r + 1];
            }
        if (g == 0) {
            rec[NREP * D + 2 * t] = st.m[0];
            rec[NREP * D + 2 * t + 1] = st.m[1];
            rec[NREP * D + NREP + 2 * t] = st.l[0];
            rec[NREP * D + NREP + 2 * t + 1] = st.l[1];
        }
    }
    __syncthreads();
    ws.init();
    if (ALL_WARPS_MERGE || warp < 4) {
#pragma unroll
        for (int r = 0; r < M2_WPK; ++r)
            merge_from(ws, reinterpret_cast<const float*>(smem + M2_SM_STAGES) + (kvh + 4 * r) * MERGE_FLOATS, lane);
    }
}

// Persistent batched kernel, second generation (same contract as khq_decode_batched_kernel).
__global__ void __launch_bounds__(M2_THREADS, 1)
khq_decode_batched_mma_kernel(const KhqSeqDesc* __restrict__ descs, const KhqTablesDesc* __restrict__ tables,
                              const KhqWorkItem* __restrict__ items, int n_items, int* __restrict__ counter,
                              float* __restrict__ partials, float scale, float rope_base, int ring_cap) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_next;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kvh = warp & 3, sub = warp >> 2;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + M2_SM_BARS);
    uint32_t* tm_slot = reinterpret_cast<uint32_t*>(smem + M2_SM_BARS + 32);
    if (tid == 0) {
        for (int s = 0; s < M2_NSTAGE; ++s) mbar_init(&bars[s], 1);
        fence_barrier_init();
    }
    m2_tm_alloc(tm_slot, warp);
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tm_slot;
    int cur_table = -1;
    unsigned tiles_done = 0;
#pragma unroll 1
    while (true) {
        __syncthreads();
        if (tid == 0) s_next = atomicAdd(counter, 1);
        __syncthreads();
        const int it = s_next;
        if (it >= n_items) break;
        const KhqWorkItem w = items[it];
        const KhqSeqDesc d = descs[w.desc];
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
            P.start_pos = d.start_pos; P.c_len = d.c_len; P.bulk_ok = 1;
            unpack_pos(d.pos_pack, P);
            if (d.table_id != cur_table) {
                m2_setup_tables(smem, P, tid);
                cur_table = d.table_id;
                __syncthreads();
                m2_rotor_to_tmem(smem, tmem, warp, lane);
            }
            WarpState ws;
            m2_compressed_range<true>(smem, d.q_gate, (size_t)2 * D, P, w.lo, w.hi, scale, tiles_done, ws, tmem);
            // the three warps of a kv-head transform and store two heads each
            static_assert(M2_WPK == 3 && NREP == 6, "head split of the item epilogue");
            if (sub == 0) v_epilogue_store<0, 2>(ws, P, lane, ob);
            else if (sub == 1) v_epilogue_store<2, 4>(ws, P, lane, ob);
            else v_epilogue_store<4, 6>(ws, P, lane, ob);
        } else {
            WarpState ws;
            ws.init();
            window_range(d.q_gate, d.ring_k, d.ring_v, d.win_start, w.lo + sub, M2_WPK, w.hi, ring_cap, scale, kvh, lane, ws);
            float* rec = reinterpret_cast<float*>(smem + M2_SM_STAGES);
            if (sub > 0) store_record(ws, rec + (kvh + 4 * (sub - 1)) * MERGE_FLOATS, lane);
            __syncthreads();
            if (sub == 0) {
#pragma unroll
                for (int r = 0; r < M2_WPK - 1; ++r) merge_from(ws, rec + (kvh + 4 * r) * MERGE_FLOATS, lane);
                raw_store(ws, lane, ob);
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    m2_tm_free(tmem, warp);
}

// Drop-in (single sequence-layer) variant: grid = num_splits * cluster_size CTAs; the CTAs of a
// cluster share one of the caller's splits and merge through distributed shared memory.
__global__ void __launch_bounds__(M2_THREADS, 1)
khq_attn_compressed_mma_kernel(const __half* __restrict__ q, CompressedKV P, float* __restrict__ out_attn,
                               float* __restrict__ out_partial, int num_splits, int L_q, int l_idx, int s_limit,
                               float scale) {
    extern __shared__ __align__(128) unsigned char smem[];
    cg::cluster_group cluster = cg::this_cluster();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int csize = (int)cluster.num_blocks(), crank = (int)cluster.block_rank();
    const int split_id = blockIdx.x / csize;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + M2_SM_BARS);
    int s_lo = 0, s_hi = s_limit;
    if (num_splits > 1) {
        const int per = (s_limit + num_splits - 1) / num_splits;
        s_lo = min(split_id * per, s_limit);
        s_hi = min(s_lo + per, s_limit);
    }
    const int len = s_hi - s_lo;
    const int chunk = (((len + csize - 1) / csize) + 1) & ~1;
    const int my_lo = min(s_lo + crank * chunk, s_hi);
    const int my_hi = min(my_lo + chunk, s_hi);
    uint32_t* tm_slot = reinterpret_cast<uint32_t*>(smem + M2_SM_BARS + 32);
    if (tid == 0) {
        for (int s = 0; s < M2_NSTAGE; ++s) mbar_init(&bars[s], 1);
        fence_barrier_init();
    }
    m2_tm_alloc(tm_slot, warp);
    m2_setup_tables(smem, P, tid);
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tm_slot;
    m2_rotor_to_tmem(smem, tmem, warp, lane);
    unsigned tiles_done = 0;
    WarpState ws;
    m2_compressed_range(smem, q + (size_t)l_idx * 2 * D, (size_t)L_q * 2 * D, P, my_lo, my_hi, scale, tiles_done, ws, tmem);
    // the query fragments are not needed any more; everything below is ordinary memory
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    m2_tm_free(tmem, warp);
    // cluster merge: records exported over the (no longer needed) codebook area
    float* exp_rec = reinterpret_cast<float*>(smem + M2_SM_VQ) + (warp & 3) * MERGE_FLOATS;
    if (csize > 1) {
        __syncthreads();  // every warp is done with the codebook
        if (warp < 4) store_record(ws, exp_rec, lane);
        cluster.sync();
        if (crank == 0 && warp < 4) {
#pragma unroll 1
            for (int r = 1; r < csize; ++r) merge_from(ws, cluster.map_shared_rank(exp_rec, r), lane);
        }
        cluster.sync();
    }
    if (crank == 0 && warp < 4) {
        float* ob[NREP];
#pragma unroll
        for (int h = 0; h < NREP; ++h) {
            const int total_id = (warp * NREP + h) * L_q + l_idx;
            ob[h] = (num_splits > 1) ? out_partial + ((size_t)total_id * num_splits + split_id) * PART
                                     : out_attn + (size_t)total_id * PART;
        }
        v_epilogue_store(ws, P, lane, ob);
    }
}

}  // namespace khq
