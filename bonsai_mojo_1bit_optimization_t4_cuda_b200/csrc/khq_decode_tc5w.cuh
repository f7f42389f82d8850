// khq_decode_tc5w.cuh -- fourth-generation compressed-region decode: the third generation's
// formulation (same operands, same tensor-memory and shared-memory layouts, see khq_decode_tc5.cuh)
// run by 32 warps of at most 64 registers instead of 8 decode warps of 168.  The third generation
// was bound by the latency of its 2 decode warps per scheduler; here every scheduler has 8 warps,
// and the work is cut into small per-thread pieces:
//
//   K step   thread (row r, part s = 0..7) decodes mask words 2s, 2s + 1 of its row into operand
//            columns 16 s .. 16 s + 15 of A (tensor-memory lane r);
//   V step   thread (row of a 32-row chunk, warp w) decodes patches 2w, 2w + 1 (one 16-byte store);
//   S1 step  thread (r, s) rotates rotary pairs 4s .. 4s + 3 of D in place in tensor memory;
//   S2 step  thread (r, head slot j = 0..5; 24 of the 32 warps) finishes the score of head
//            6 * kv_head(r) + j, its softmax weight and the two P entries.
//
// All 32 warps walk the same sequence of steps and meet at CTA-wide barriers; after a barrier warp
// 0 issues what the step made ready (the K-side MMAs, the P V MMAs of a chunk pair, the next bulk
// copies) and goes on with its share of the next step.  Per tile i of an item:
//
//   K(i) |A| V(i-1) chunks 0,1 |B| S1(i) |C| V(i-1) chunks 2,3 |D| S2(i) scores |E| S2(i) weights, P
//
// so the K-side MMAs of tile i run under the V decode of tile i - 1, and the P V MMAs of tile i - 1
// under S1 and S2 of tile i.  Every wait on an mbarrier is bounded (m3::wait_bar).
#pragma once
#include "khq_decode_tc5.cuh"

namespace khq {
namespace m3 {  // shares the third generation's layouts, descriptors, wrappers and set-up

constexpr int W_THREADS = 1024;
enum WBar { W_KFULL = 0, W_VFULL, W_DREADY, W_VDONE, W_PVDONE, W_COUNT };

#ifndef M4_WORD_UNROLL
#define M4_WORD_UNROLL 1
#endif

__device__ __forceinline__ void tm_ld4(uint32_t taddr, uint32_t (&r)[4]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tm_st4(uint32_t taddr, const uint32_t (&r)[4]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%4], {%0,%1,%2,%3};" ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]),
                 "r"(taddr));
}
__device__ __forceinline__ uint32_t tm_ld1(uint32_t taddr) {
    uint32_t r;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r) : "r"(taddr) : "memory");
    return r;
}

// Row scalars kept from the K step to the S2 step: three float arrays of 128 in the unused B columns
// 24..31 (1 KB per 64-deep group; whatever lies there only reaches D columns nobody reads).
__device__ __forceinline__ float* row_scalar(unsigned char* smem, int which) {
    return reinterpret_cast<float*>(smem + SM_BK + which * BK_GROUP + 24 * 128);
}

// The parts of an item that need many registers (the first generation's per-warp state is 60 floats)
// are kept out of line, so that their spills stay out of the tile loop, which has 64 registers.
__device__ __noinline__ void w_setup_item(unsigned char* smem, const __half* q, size_t q_head_stride, const CompressedKV& P,
                                          int tid) {
    setup_item(smem, q, q_head_stride, P, tid);
}
// Raw-window item: warps 0..7 (kv-head = warp & 3, two warps per kv-head take alternate tokens).
__device__ __noinline__ void w_window_item(const KhqSeqDesc& d, const KhqWorkItem& w, unsigned char* smem, int ring_cap,
                                           float scale, float* const (&ob)[NREP]) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kvh = warp & 3, sub = warp >> 2;
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
// End of a compressed item, warps 0..3 (kv-head = warp): the O rows and running sums that the tile
// loop left in shared memory -> the first generation's state -> inverse rotor and partial record.
__device__ __noinline__ void w_item_store(unsigned char* smem, const CompressedKV& P, bool empty, float* const (&ob)[NREP]) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const Soft* soft = reinterpret_cast<const Soft*>(smem + SM_SOFT);
    const float* scr = reinterpret_cast<const float*>(smem + SM_V);  // [24 heads][257]
    WarpState ws;
    ws.init();
    if (!empty) {
#pragma unroll
        for (int h = 0; h < NREP; ++h) {
            const int hh = warp * NREP + h;
#pragma unroll
            for (int j = 0; j < 8; ++j) ws.acc[h][j] = scr[hh * 257 + lane * 8 + j];
            const float M = soft->M[hh];
            ws.m[h] = (M <= -1.0e29f) ? NEG_BIG : M * LN2;
            ws.l[h] = soft->lsum[hh];
        }
    }
    v_epilogue_store(ws, P, lane, ob);
}

struct WCounters {
    unsigned tiles;   // tiles started in this CTA's life (K / V staging, D, P V completion)
    unsigned vdone;   // P V chunk pairs committed
};

// The compressed range [my_lo, my_hi) of one work item.  All W_THREADS threads call it.  Returns false
// for an empty range; otherwise leaves the 24 O rows ([24][257] floats at SM_V), M and the running sums
// in shared memory for w_item_store, after a CTA barrier.
__device__ __forceinline__ bool compressed_range_w(unsigned char* smem, uint32_t tmem, const CompressedKV& P, int my_lo,
                                                   int my_hi, float scale, WCounters& cn) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quad = warp & 3, sub = warp >> 2;
    const int r = 32 * quad + lane, kvh = lane & 3;
    Soft* soft = reinterpret_cast<Soft*>(smem + SM_SOFT);
    volatile int* abortf = &soft->abort_flag;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM_BARS);
    unsigned char* stage = smem + SM_STAGE;
    const int base = my_lo & ~1;
    const int ntiles = (my_hi > my_lo) ? (my_hi - base + TILE_TOK - 1) / TILE_TOK : 0;
    const unsigned g0 = cn.tiles, vd0 = cn.vdone;
    const uint32_t lane_base = tmem + ((uint32_t)(quad * 32) << 16);
    const bool all_alpha = soft->all_alpha != 0;
    const int hd = kvh * NREP + sub;  // S2: this thread's query head (warps 0..23)
    if (ntiles == 0) return false;

    const uint32_t sbase = smem_u32(smem);
    const uint32_t idesc_k = idesc_f16(NK, false), idesc_v = idesc_f16(D, true);
    const uint32_t bk_lo = sdesc_lo(sbase + SM_BK, 16), p_lo = sdesc_lo(sbase + SM_P, 16);
    const uint32_t v_lo = sdesc_lo(sbase + SM_V, V_GROUP);

    auto stage_tile = [&](int part, int t) {  // warp 0
        const int tok0 = base + t * TILE_TOK;
        stage_part(P, stage, &bars[part == 0 ? W_KFULL : W_VFULL], part, tok0, min(TILE_TOK, P.c_len - tok0), lane);
    };
    auto issue_pv = [&](int tile, int pair) {  // one thread: chunks 2 pair, 2 pair + 1 from buffers 0, 1
#pragma unroll
        for (int b = 0; b < 2; ++b)
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
                const int ks = (2 * pair + b) * 2 + kk;  // K step of the tile (16 rows each)
                const uint32_t oa = (uint32_t)((ks >> 2) * P_GROUP + (ks & 3) * 32) >> 4;
                const uint32_t ob = (uint32_t)(b * V_CHUNK + kk * 2048) >> 4;
                mma_ss(tmem + TM_O, p_lo + oa, v_lo + ob, idesc_v, (tile == 0 && ks == 0) ? 0u : 1u);
            }
        mma_commit(&bars[W_VDONE]);
    };
    // chunks 2 pair, 2 pair + 1 of tile t -> the two V buffers
    auto v_pair = [&](int t, int pair) {
        const unsigned char* vqa = smem + SM_VQA;
        const unsigned char* vqb = smem + SM_VQB;
        const float2* c3t = reinterpret_cast<const float2*>(smem + SM_C3);
        const int p0 = 2 * warp;                       // patches p0, p0 + 1
        const int q8 = warp & 3;                       // their 24 bits start at bit 24 q8 of the three-word group
        const int wi = (24 * q8) >> 5, sh = (24 * q8) & 31;
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            const int rr = 32 * (2 * pair + b) + lane;
            const uint32_t* vrow = reinterpret_cast<const uint32_t*>(stage + ST_VPAY + rr * V_PAY);
            const int tok = base + t * TILE_TOK + (rr >> 2);
            const bool valid = tok >= my_lo && tok < my_hi;
            const float smv7 = valid ? reinterpret_cast<const float*>(stage + ST_VSM)[rr] * (1.0f / 7.0f) : 0.0f;
            const uint32_t* wp = vrow + 3 * (warp >> 2);
            const uint32_t two = khq3::k3_funnel_r(wp[wi], wp[min(wi + 1, 2)], (uint32_t)sh) & 0xFFFFFFu;
            const uint32_t hb2 = vrow[24 + (warp >> 4)] >> ((2 * warp) & 31);
            uint32_t ow[4];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const uint32_t fld = (two >> (12 * e)) & 0xFFFu;
                const uint32_t code = (fld & 0x7Fu) | (((hb2 >> e) & 1u) << 7);
                const uint32_t e01 = *reinterpret_cast<const uint32_t*>(vqa + code * (VQA_STRIDE * 4) + (p0 + e) * 4);
                const uint32_t e2 = *reinterpret_cast<const unsigned short*>(vqb + code * VQB_STRIDE + (p0 + e) * 2);
                const float2 cc = c3t[p0 + e];
                const float c3 = (fld & 0x80u) ? cc.y : cc.x;
                const float v3 = fmaf(__uint_as_float(0x4B000000u | (fld >> 8)) - 8388616.0f, smv7, c3);  // (dump - 8)
                ow[2 * e] = e01;
                ow[2 * e + 1] = e2 | ((uint32_t)__half_as_ushort(__float2half_rn(v3)) << 16);
            }
            unsigned char* dst = smem + SM_V + b * V_CHUNK + (warp >> 3) * V_GROUP + lane * 128;
            *reinterpret_cast<uint4*>(dst + (((warp & 7) ^ (lane & 7)) << 4)) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
        }
        fence_proxy_async();
    };

    if (warp == 0) {
        stage_tile(0, 0);
        stage_tile(1, 0);
    }
    // RoPE cos/sin of this row's token for rotary pairs 4 sub + j, advanced by 32 positions per tile
    float rc[4], rs[4];
    {
        const float* freq = reinterpret_cast<const float*>(smem + SM_FREQ) + 4 * sub;
        const int pos = P.start_pos + base + (r >> 2);
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            double th = (double)pos * (double)freq[m];
            th -= rint(th * 0.15915494309189535) * 6.283185307179586;
            __sincosf((float)th, &rs[m], &rc[m]);
        }
    }
    float lrun = 0.0f;

#pragma unroll 1
    for (int i = 0; i <= ntiles; ++i) {
        const bool has_k = i < ntiles, has_v = i >= 1;
        const unsigned g = g0 + (unsigned)i;
        // ---------------- K step: code words of tile i -> A operand ---------------------------------
        if (has_k) {
            wait_bar(&bars[W_KFULL], g & 1u, abortf);
            const uint32_t* kp = reinterpret_cast<const uint32_t*>(stage + ST_KPAY + r * K_PAY);
            const uint32_t* mrow = reinterpret_cast<const uint32_t*>(stage + ST_MASK + r * 64);
            uint32_t ob = 0;  // outliers of the row before mask word 2 sub
#pragma unroll 1
            for (int jq = 0; jq < (sub >> 1); ++jq) {
                const uint4 a = reinterpret_cast<const uint4*>(mrow)[jq];
                ob += khq3::k3_count(a.x) + khq3::k3_count(a.y) + khq3::k3_count(a.z) + khq3::k3_count(a.w);
            }
            if (sub & 1) {
                const uint2 a = reinterpret_cast<const uint2*>(mrow)[sub - 1];
                ob += khq3::k3_count(a.x) + khq3::k3_count(a.y);
            }
            float mult = (float)kp[0] / 1000.0f;
            if (mult < 0.1f || mult > 10.0f || isnan(mult)) mult = 1.0f;
            const float rsc = hbits2f(reinterpret_cast<const uint16_t*>(stage + ST_KRN)[r]);
            if (sub == 0) {
                const float kn = hbits2f(reinterpret_cast<const uint16_t*>(stage + ST_KN)[r]);
                const float vn = hbits2f(reinterpret_cast<const uint16_t*>(stage + ST_VN)[r]);
                const float en = hbits2f(reinterpret_cast<const uint16_t*>(stage + ST_VRN)[r]);
                row_scalar(smem, 0)[r] = P.alpha_k * kn * mult * scale * LOG2E;
                row_scalar(smem, 1)[r] = P.alpha_v * vn * en;
                row_scalar(smem, 2)[r] = vn;
            }
            const __half2 rh = __float2half2_rn(rsc / mult);
            const uint32_t ratio2 = *reinterpret_cast<const uint32_t*>(&rh);
            const uint32_t neg1024 = 0xE400E400u;
            const uint4* betat = reinterpret_cast<const uint4*>(smem + SM_BETA);
_Pragma(M3_STR(unroll M4_WORD_UNROLL))
            for (int ww = 0; ww < 2; ++ww) {
                uint32_t t2[8], h2[8], a2[8];
                const int wj = 2 * sub + ww;
                ob += khq3::k3_word(mrow[wj], ob, kp, t2, h2);
                const int col0 = 8 * wj;
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
        }
        __syncthreads();  // A: the A operand and the row scalars of tile i are complete, the K part of the stage is free
        if (warp == 0) {
            if (has_k && lane == 0) {
                tc_after();
#pragma unroll
                for (int s = 0; s < 16; ++s) {
                    const uint32_t ob = (uint32_t)((s >> 2) * BK_GROUP + (s & 3) * 32) >> 4;
                    mma_ts(tmem + TM_D, tmem + TM_A + 8 * s, bk_lo + ob, idesc_k, s > 0 ? 1u : 0u);
                }
                mma_commit(&bars[W_DREADY]);
            }
            __syncwarp();
            if (i + 1 < ntiles) stage_tile(0, i + 1);
        }
        // ---------------- V step, chunks 0 and 1 of tile i - 1 ---------------------------------------
        if (has_v) {
            wait_bar(&bars[W_VFULL], (g - 1) & 1u, abortf);
            const unsigned vc = vd0 + 2u * (unsigned)(i - 1);  // pairs committed before this one
            if (vc >= 1) wait_bar(&bars[W_VDONE], (vc - 1) & 1u, abortf);
            v_pair(i - 1, 0);
        }
        __syncthreads();  // B
        if (warp == 0 && lane == 0 && has_v) {
            tc_after();
            issue_pv(i - 1, 0);
        }
        // ---------------- S1 step: RoPE on the rotary columns of D, in place -------------------------
        if (has_k) {
            wait_bar(&bars[W_DREADY], g & 1u, abortf);
            tc_after();
            uint32_t lo[4], hi[4];
            tm_ld4(lane_base + TM_D + ROT0 + 4 * sub, lo);
            tm_ld4(lane_base + TM_D + ROT0 + 32 + 4 * sub, hi);
            tm_ld_wait();
            const float2* rstep = reinterpret_cast<const float2*>(smem + SM_RSTEP) + 4 * sub;
#pragma unroll
            for (int mm = 0; mm < 4; ++mm) {
                const float k0 = __uint_as_float(lo[mm]), k1 = __uint_as_float(hi[mm]);
                lo[mm] = __float_as_uint(k0 * rc[mm] - k1 * rs[mm]);
                hi[mm] = __float_as_uint(k0 * rs[mm] + k1 * rc[mm]);
                const float2 st = rstep[mm];
                const float c = rc[mm] * st.x - rs[mm] * st.y, s = rs[mm] * st.x + rc[mm] * st.y;
                rc[mm] = c;
                rs[mm] = s;
            }
            tm_st4(lane_base + TM_D + ROT0 + 4 * sub, lo);
            tm_st4(lane_base + TM_D + ROT0 + 32 + 4 * sub, hi);
            tm_st_wait();
            tc_before();
        }
        __syncthreads();  // C
        // ---------------- V step, chunks 2 and 3 of tile i - 1 ---------------------------------------
        if (has_v) {
            const unsigned vc = vd0 + 2u * (unsigned)(i - 1) + 1u;
            wait_bar(&bars[W_VDONE], (vc - 1) & 1u, abortf);
            v_pair(i - 1, 1);
        }
        __syncthreads();  // D: the V part of the stage is free
        if (warp == 0) {
            if (has_v && lane == 0) {
                tc_after();
                issue_pv(i - 1, 1);
                mma_commit(&bars[W_PVDONE]);
            }
            __syncwarp();
            if (has_k && i >= 1) stage_tile(1, i);
        }
        // ---------------- S2 step: scores ---------------------------------------------------------------
        float sc = M_NONE, s1 = 0.0f, s2 = 0.0f;  // the row scalars are read before barrier E: the next K step rewrites them
        bool valid = false;
        const int par = i & 1;
        if (has_k && warp < 24) {
            tc_after();
            uint32_t pv[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) pv[k] = tm_ld1(lane_base + TM_D + NREP * k + sub);
            const float* qrot = reinterpret_cast<const float*>(smem + SM_QROT) + kvh * QROT_KVH + sub * 64;
            float acc = 0.0f;
#pragma unroll 1
            for (int c4 = 0; c4 < 4; ++c4) {
                uint32_t dv[16];
                tm_ld16(lane_base + TM_D + ROT0 + 16 * c4, dv);
                tm_ld_wait();
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const float4 qa = *reinterpret_cast<const float4*>(qrot + 16 * c4 + 4 * q4);
                    acc = fmaf(__uint_as_float(dv[4 * q4]), qa.x,
                               fmaf(__uint_as_float(dv[4 * q4 + 1]), qa.y,
                                    fmaf(__uint_as_float(dv[4 * q4 + 2]), qa.z, fmaf(__uint_as_float(dv[4 * q4 + 3]), qa.w, acc))));
                }
            }
            tc_before();  // every column of D this thread needs has been read
            const float pass = __uint_as_float(kvh == 0 ? pv[0] : (kvh == 1 ? pv[1] : (kvh == 2 ? pv[2] : pv[3])));
            const int tok = base + i * TILE_TOK + (r >> 2);
            valid = tok >= my_lo && tok < my_hi;
            sc = valid ? row_scalar(smem, 0)[r] * (pass + acc) : M_NONE;
            s1 = row_scalar(smem, 1)[r];
            s2 = row_scalar(smem, 2)[r];
            const bool need = valid && sc > soft->M[hd];
            if (__any_sync(0xFFFFFFFFu, need)) {
                if (need) {
                    atomicMax(&soft->tmax[hd], fkey(sc));
                    soft->grow[par] = 1;
                }
            }
        }
        __syncthreads();  // E
        if (has_k) {
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
                __syncthreads();
                if (tid == 0) soft->grow[par] = 0;
                if (warp < 24) lrun *= soft->fac[hd];
                if (i > 0 && warp < 2) {
                    // O holds earlier tiles of this item.  Rows: lane m < 24 = head m (dims 0..2 of the
                    // patches), 24..47 = head m - 24 (dim 3)
                    wait_bar(&bars[W_PVDONE], (g - 1) & 1u, abortf);
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
            if (warp < 24) {
                const float pw = valid ? ex2f(sc - soft->M[hd]) : 0.0f;
                lrun += pw;
                // P of the previous tile must have been consumed before it is overwritten
                if (g >= 1) wait_bar(&bars[W_PVDONE], (g - 1) & 1u, abortf);
                // rows outside the item write an exact zero: their row scalars are whatever the staging area held
                *reinterpret_cast<__half*>(smem + SM_P + p_off(hd, r)) = __float2half(valid ? pw * s1 : 0.0f);
                *reinterpret_cast<__half*>(smem + SM_P + p_off(24 + hd, r)) = __float2half(valid ? pw * s2 : 0.0f);
                fence_proxy_async();
            }
        }
        // the next iteration's barrier A orders these P writes before warp 0 issues the MMAs that read them
    }
    // ---------------- item epilogue: O and the running sums -> the first generation's state -----------
    {
        const unsigned glast = g0 + (unsigned)ntiles - 1u;
        wait_bar(&bars[W_PVDONE], glast & 1u, abortf);
        tc_after();
        if (warp < 24) {
            float v = lrun;
            v += __shfl_xor_sync(0xFFFFFFFFu, v, 4);
            v += __shfl_xor_sync(0xFFFFFFFFu, v, 8);
            v += __shfl_xor_sync(0xFFFFFFFFu, v, 16);
            if (lane < 4) atomicAdd(&soft->lsum[hd], v);  // lane = kv-head of this thread
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
        __syncthreads();
    }
    cn.tiles = g0 + (unsigned)ntiles;
    cn.vdone = vd0 + 2u * (unsigned)ntiles;
    return true;
}

// Persistent batched kernel, fourth generation (same contract as khq_decode_batched_kernel).
__global__ void __launch_bounds__(W_THREADS, 1)
khq_decode_batched_tc5w_kernel(const KhqSeqDesc* __restrict__ descs, const KhqTablesDesc* __restrict__ tables,
                               const KhqWorkItem* __restrict__ items, int n_items, int* __restrict__ counter,
                               float* __restrict__ partials, float scale, float rope_base, int ring_cap) {
    extern __shared__ __align__(1024) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM_BARS);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM_BARS + 15 * 8);
    Soft* soft = reinterpret_cast<Soft*>(smem + SM_SOFT);
    if ((smem_u32(smem) & 1023u) != 0) {  // the swizzled operand layouts need a 1024-byte aligned base
        if (tid == 0) atomicExch(&g_status, 2);
        return;
    }
    if (tid == 0) {
        for (int b = 0; b < W_COUNT; ++b) mbar_init(&bars[b], 1);
        fence_barrier_init();
        soft->abort_flag = 0;
        soft->all_alpha = 1;
    }
    // P starts as zeros: a row only ever writes the columns of its own kv-head's heads
    for (int e = tid; e < 2 * P_GROUP / 16; e += W_THREADS) reinterpret_cast<uint4*>(smem + SM_P)[e] = make_uint4(0u, 0u, 0u, 0u);
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "n"(TM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_before();
    __syncthreads();
    tc_after();
    const uint32_t tmem = *tmem_slot;

    int cur_table = -1;
    WCounters cn = {0u, 0u};
#pragma unroll 1
    while (true) {
        __syncthreads();  // previous item fully retired
        if (tid == 0) soft->next_item = soft->abort_flag ? n_items : atomicAdd(counter, 1);
        __syncthreads();
        const int it = soft->next_item;
        if (it >= n_items) break;
        const KhqWorkItem w = items[it];
        const KhqSeqDesc d = descs[w.desc];
        const int kvh = warp & 3;
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
                setup_layer<W_THREADS>(smem, P, tid);
                cur_table = d.table_id;
            }
            if (warp < 8) w_setup_item(smem, d.q_gate, (size_t)2 * D, P, tid);
            fence_proxy_async();  // B columns were written with ordinary stores, the tensor core reads them
            __syncthreads();
            const bool any = compressed_range_w(smem, tmem, P, w.lo, w.hi, scale, cn);
            if (warp < 4) w_item_store(smem, P, !any, ob);
        } else if (warp < 8) {
            w_window_item(d, w, smem, ring_cap, scale, ob);
        }
    }
    tc_before();
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(TM_COLS) : "memory");
    }
}

}  // namespace m3
}  // namespace khq
