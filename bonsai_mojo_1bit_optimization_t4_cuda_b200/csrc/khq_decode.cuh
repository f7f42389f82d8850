// khq_decode.cuh -- device building blocks of the two-region KHQ decode attention (sm_100a).
//
// Work shape.  A CTA owns a range of tokens for ALL four kv-heads, because the payload arrays
// are token-major with the kv-heads interleaved: a token tile is then eight fully contiguous
// byte ranges (mask, K payload, V payload, four fp16 norm arrays, V meta) that 1-D bulk
// asynchronous copies (cp.async.bulk + mbarrier, no multicast) stage into shared memory.
// Inside the CTA a warp owns one kv-head and serves its six query heads from ONE decode of each
// compressed row (the reference decodes every row once per query head).  A lane owns the eight
// consecutive dims 8*lane..8*lane+7 of the 256-dim row.
#pragma once
#include <cooperative_groups.h>

#include "khq_common.cuh"

namespace khq {
namespace cg = cooperative_groups;

constexpr int DEC_WPK = 3;                    // warps per kv-head
constexpr int DEC_WARPS = HKV * DEC_WPK;      // 12
constexpr int DEC_THREADS = DEC_WARPS * 32;   // 384
constexpr int TT = 24;                        // tokens per staged tile (even)
constexpr int NSTAGE = 3;
constexpr int TROWS = TT * HKV;               // 96 rows per tile

// byte offsets inside one stage (all multiples of 16)
constexpr int OFF_MASK = 0;
constexpr int OFF_KPAY = OFF_MASK + TROWS * 64;
constexpr int OFF_VPAY = OFF_KPAY + TROWS * K_PAY;
constexpr int OFF_KN = OFF_VPAY + TROWS * V_PAY;
constexpr int OFF_KRN = OFF_KN + TROWS * 2;
constexpr int OFF_VN = OFF_KRN + TROWS * 2;
constexpr int OFF_VRN = OFF_VN + TROWS * 2;
constexpr int OFF_VSM = OFF_VRN + TROWS * 2;
constexpr int STAGE_BYTES = OFF_VSM + TROWS * 4;  // 21120
static_assert(STAGE_BYTES % 16 == 0 && OFF_KPAY % 16 == 0 && OFF_VPAY % 16 == 0 &&
                  OFF_KN % 16 == 0 && OFF_KRN % 16 == 0 && OFF_VN % 16 == 0 &&
                  OFF_VRN % 16 == 0 && OFF_VSM % 16 == 0,
              "stage sub-buffers must be 16-byte aligned for bulk copies");

constexpr int SM_STAGES = 0;
constexpr int SM_ROPE = SM_STAGES + NSTAGE * STAGE_BYTES;   // 2 x TT x 32 float2
constexpr int SM_ROTOR = SM_ROPE + 2 * TT * 32 * 8;         // 32 lanes x 36 floats
constexpr int SM_FREQ = SM_ROTOR + 32 * 36 * 4;             // 32 floats
constexpr int SM_BARS = SM_FREQ + 32 * 4;                   // NSTAGE mbarriers
constexpr int SM_TOTAL = SM_BARS + 64;                      // without the V codebook
constexpr int SM_VQ = SM_TOTAL;                             // 256 codes x 64 patches x 4 halfs
constexpr int SM_TOTAL_VQ = SM_VQ + 256 * NP * 8;
static_assert(SM_VQ % 16 == 0 && SM_TOTAL_VQ <= 227 * 1024, "shared memory budget");
// Per-kv-head merge record: acc[NREP][D], m[NREP], l[NREP]  (+pad to 16 B)
constexpr int MERGE_FLOATS = NREP * D + 2 * NREP + 4;       // 1552
constexpr int SM_MERGE_A = 0;                               // aliases the stages after the loop
constexpr int SM_MERGE_E = SM_MERGE_A + HKV * MERGE_FLOATS * 4;
static_assert(SM_MERGE_E + HKV * MERGE_FLOATS * 4 <= NSTAGE * STAGE_BYTES, "merge areas alias the stages");

// ---- batched decode: device-resident descriptor tables (mirrored in include/khq_b200.h) -------
struct KhqSeqDesc {  // one (sequence, layer) decode problem
    const __half* q_gate;
    const unsigned char* k_payload;
    const unsigned char* v_payload;
    const unsigned char* v_shared_meta;
    const unsigned int* k_mask;
    const __half* k_norms;
    const __half* k_r_norms;
    const __half* v_norms;
    const __half* v_r_norms;
    const __half* ring_k;
    const __half* ring_v;
    __half* out;
    int table_id, c_len, start_pos, win_start, win_len, first_slot, n_slots;
    int pos_pack;  // 0: token s of the arrays sits at position start_pos + s; else (pos_chunk << 16) | (pos_stride / pos_chunk)
};
struct KhqTablesDesc {  // one layer's calibration tables
    const __half* cents_k;
    const __half* cents_v;
    const __half* vq;
    const __half* k_rotor;
    const __half* v_rotor;
    const __half* d_k;
    const __half* d_v;
    float alpha_k, alpha_v;
};
struct KhqWorkItem {  // one CTA-sized piece of a problem
    int desc, kind, lo, hi, slot, r0, r1, r2;  // kind 0: compressed tokens [lo,hi); 1: window tokens [lo,hi)
};
static_assert(sizeof(KhqSeqDesc) == 128 && sizeof(KhqTablesDesc) == 64 && sizeof(KhqWorkItem) == 32, "ABI");

struct CompressedKV {  // device pointers of one sequence-layer's compressed region + tables
    const unsigned char* k_payload;
    const unsigned char* v_payload;
    const unsigned char* v_shared_meta;
    const unsigned int* k_mask;
    const __half* k_norms;
    const __half* k_r_norms;
    const __half* v_norms;
    const __half* v_r_norms;
    const __half* cents_k;
    const __half* cents_v;
    const __half* vq;
    const __half* k_rotor;
    const __half* v_rotor;
    const __half* d_k;
    const __half* d_v;
    float alpha_k, alpha_v, rope_base;
    int start_pos;  // absolute position of compressed token 0
    int c_len;      // valid tokens in the arrays
    int bulk_ok;    // all eight arrays 16-byte aligned
    // Positions of a slice that holds every G-th chunk of a longer context (chunk-cyclic context
    // partition): token s of the arrays sits at start_pos + (s / pos_chunk) * pos_stride + s % pos_chunk.
    // pos_chunk == 0: consecutive positions.
    int pos_chunk, pos_stride;
};

// Stages a layer's V codebook (NP patches x 256 codes x 3 halfs; entry e = patch * 256 + code starts at
// half 3e) into the two shared-memory tables of the tensor-core generations: the (d0, d1) word at
// vqa[code * STRIDE_A_WORDS + patch], the d2 half at vqb[code * (STRIDE_B_BYTES / 2) + patch].  Two
// entries (three words) per thread and iteration, eight iterations' loads in flight: the staging runs
// once per CTA and layer and is bound by load latency, not by bytes.
template <int NT, int STRIDE_A_WORDS, int STRIDE_B_BYTES>
__device__ __forceinline__ void stage_vq_codebook(const __half* __restrict__ vq, unsigned int* __restrict__ vqa,
                                                  unsigned short* __restrict__ vqb, int tid) {
    const unsigned int* src = reinterpret_cast<const unsigned int*>(vq);
#pragma unroll 8
    for (int u = tid; u < NP * 256 / 2; u += NT) {
        const unsigned int w0 = __ldg(src + 3 * u), w1 = __ldg(src + 3 * u + 1), w2 = __ldg(src + 3 * u + 2);
        const int e = 2 * u, patch = e >> 8, code = e & 255;  // the pair never straddles a patch (256 codes)
        vqa[code * STRIDE_A_WORDS + patch] = w0;
        vqb[code * (STRIDE_B_BYTES / 2) + patch] = (unsigned short)(w1 & 0xFFFFu);
        vqa[(code + 1) * STRIDE_A_WORDS + patch] = (w1 >> 16) | (w2 << 16);
        vqb[(code + 1) * (STRIDE_B_BYTES / 2) + patch] = (unsigned short)(w2 >> 16);
    }
}

// Chunk-cyclic positions of a descriptor (KhqSeqDesc::pos_pack) into P.
__host__ __device__ __forceinline__ void unpack_pos(int pos_pack, CompressedKV& P) {
    P.pos_chunk = (int)((unsigned)pos_pack >> 16);
    P.pos_stride = P.pos_chunk * (pos_pack & 0xFFFF);
}

// Absolute position of token `tok` of the arrays.
__device__ __forceinline__ int token_pos(const CompressedKV& P, int tok) {
    return P.start_pos + (P.pos_chunk > 0 ? (tok / P.pos_chunk) * P.pos_stride + tok % P.pos_chunk : tok);
}

// Per-warp running state: 6 query heads x the lane's 8 dims.
struct WarpState {
    float acc[NREP][8];
    float m[NREP];
    float l[NREP];
    __device__ __forceinline__ void init() {
#pragma unroll
        for (int h = 0; h < NREP; ++h) {
            m[h] = NEG_BIG;
            l[h] = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[h][j] = 0.0f;
        }
    }
};

// Sum six per-lane partial dot products over the warp; every lane ends with all six totals.
__device__ __forceinline__ void reduce6(float (&s)[NREP], int lane) {
    const bool upper = (lane & 16) != 0;
    float keep[3];
#pragma unroll
    for (int i = 0; i < 3; ++i) {
        const float send = upper ? s[i] : s[i + 3];
        const float recv = __shfl_xor_sync(0xFFFFFFFFu, send, 16);
        keep[i] = (upper ? s[i + 3] : s[i]) + recv;
    }
#pragma unroll
    for (int m = 8; m > 0; m >>= 1)
#pragma unroll
        for (int i = 0; i < 3; ++i) keep[i] += __shfl_xor_sync(0xFFFFFFFFu, keep[i], m);
#pragma unroll
    for (int i = 0; i < 3; ++i) {
        const float other = __shfl_xor_sync(0xFFFFFFFFu, keep[i], 16);
        s[i] = upper ? other : keep[i];
        s[i + 3] = upper ? keep[i] : other;
    }
}

// Online-softmax step for the six heads of a warp given the six scaled scores; p[h] is the
// weight to apply to this token's V row.
__device__ __forceinline__ void softmax_step(WarpState& st, const float (&s)[NREP], float (&p)[NREP]) {
#pragma unroll
    for (int h = 0; h < NREP; ++h) {
        if (s[h] > st.m[h]) {  // warp-uniform: every lane holds the same score and max
            const float fac = __expf(st.m[h] - s[h]);
            st.l[h] = st.l[h] * fac + 1.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) st.acc[h][j] *= fac;
            st.m[h] = s[h];
            p[h] = 1.0f;
        } else {
            p[h] = __expf(s[h] - st.m[h]);
            st.l[h] += p[h];
        }
    }
}

__device__ __forceinline__ void accumulate_v(WarpState& st, const float (&p)[NREP], const float (&v)[8]) {
#pragma unroll
    for (int h = 0; h < NREP; ++h)
#pragma unroll
        for (int j = 0; j < 8; ++j) st.acc[h][j] = fmaf(p[h], v[j], st.acc[h][j]);
}

// st <- LSE-merge(st, record in memory).  rec may point to this CTA's or a peer CTA's shared
// memory (distributed shared memory of the cluster).
__device__ __forceinline__ void merge_from(WarpState& st, const float* rec, int lane) {
#pragma unroll
    for (int h = 0; h < NREP; ++h) {
        const float mo = rec[NREP * D + h], lo = rec[NREP * D + NREP + h];
        const float M = fmaxf(st.m[h], mo);
        const float fa = __expf(st.m[h] - M), fb = __expf(mo - M);
        st.l[h] = st.l[h] * fa + lo * fb;
        const float4 a0 = *reinterpret_cast<const float4*>(rec + h * D + lane * 8);
        const float4 a1 = *reinterpret_cast<const float4*>(rec + h * D + lane * 8 + 4);
        const float o[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) st.acc[h][j] = st.acc[h][j] * fa + o[j] * fb;
        st.m[h] = M;
    }
}

__device__ __forceinline__ void store_record(const WarpState& st, float* rec, int lane) {
#pragma unroll
    for (int h = 0; h < NREP; ++h) {
        *reinterpret_cast<float4*>(rec + h * D + lane * 8) =
            make_float4(st.acc[h][0], st.acc[h][1], st.acc[h][2], st.acc[h][3]);
        *reinterpret_cast<float4*>(rec + h * D + lane * 8 + 4) =
            make_float4(st.acc[h][4], st.acc[h][5], st.acc[h][6], st.acc[h][7]);
    }
#pragma unroll
    for (int h = 0; h < NREP; ++h)
        if (lane == h) {  // static indices keep the state in registers
            rec[NREP * D + h] = st.m[h];
            rec[NREP * D + NREP + h] = st.l[h];
        }
}

// Merge the DEC_WPK warps of each kv-head inside the CTA, then the CTAs of the cluster.  On
// return the sub==0 warps of cluster rank 0 hold the merged state.  `area` is shared memory no
// longer used for anything else (>= 2*HKV*MERGE_FLOATS floats).  Must be called by all threads
// of all CTAs of the cluster.
__device__ __forceinline__ void merge_cta_and_cluster(WarpState& st, float* area, int kvh, int sub,
                                                      int lane) {
    cg::cluster_group cluster = cg::this_cluster();
    float* recA = area + kvh * MERGE_FLOATS;
    float* recE = area + (HKV + kvh) * MERGE_FLOATS;
    __syncthreads();
#pragma unroll
    for (int src = 1; src < DEC_WPK; ++src) {
        if (sub == src) store_record(st, recA, lane);
        __syncthreads();
        if (sub == 0) merge_from(st, recA, lane);
        __syncthreads();
    }
    const unsigned nblk = cluster.num_blocks();
    if (nblk > 1) {
        if (sub == 0) store_record(st, recE, lane);
        cluster.sync();
        if (cluster.block_rank() == 0 && sub == 0) {
#pragma unroll 1
            for (unsigned r = 1; r < nblk; ++r) {
                const float* remote = cluster.map_shared_rank(recE, r);
                merge_from(st, remote, lane);
            }
        }
        cluster.sync();  // peers must stay resident until rank 0 has read their records
    }
}

}  // namespace khq
