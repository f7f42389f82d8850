// khq_prefill_tc5.cu -- causal GQA prefill attention with sigmoid output gate on the fifth
// generation tensor cores (tcgen05.mma, accumulators in tensor memory, operands staged by TMA).
//
// Same math and the same tensors as the warp-level kernel in khq_prefill.cu (the reference's
// fp16-KV attention, src/kernels/elementwise_sm75.mojo:1140-1231, applied to all prompt rows at
// once): out[t,h,:] = softmax_{u<=t}(q[t,h].K[u,h/6]*scale) V[u,h/6] * sigmoid(gate[t,h,:]).
//
// A work item = 128 query rows of one query head; key tiles of 128.  A CTA works through one item
// (long prompts: one CTA per item, left to the hardware scheduler) or through several (short
// prompts: one persistent CTA per SM; the producers and the MMA thread then run ahead into the
// next item while the softmax warps finish the epilogue of the current one).  Eleven warps:
//   warps 0-7  softmax, two threads per query row (warp w and warp w+4 share the tensor-memory
//              lane quarter w%4 and a scheduler): a row's S and O live in tensor-memory lane i,
//              so there are no shuffles; the two threads of a row take 64 keys of a tile each
//              and swap their half maxima (and, at the end, half sums) through shared memory.
//              Per tile a thread reads 64 S columns with tcgen05.ld and writes P (fp16 pairs, 32
//              columns) back over the S buffer with tcgen05.st; O is rescaled lazily (only when
//              the running max grew by more than 2^8); the epilogue normalises, gates, stores.
//   warps 8,10 producers: one thread each issues the TMA loads of Q and the K tiles (warp 8, a
//              K tile in two halves of 128 head dims, each released as soon as the Q K^T steps
//              that read it have completed) and of the V tiles (warp 10, two halves of 64 keys,
//              each released when the P V steps that read it have completed).
//   warp 9     MMA: one thread issues S = Q K^T (M128 N128 K256, A = Q from shared memory) for
//              tile j+1, then O += P V (M128 N256 K128, A = P from tensor memory) for tile j;
//              tcgen05.commit signals the mbarriers.
// Tensor memory columns: O [0,256), S/P ping [256,384), S/P pong [384,512).  An A operand in
// tensor memory is row = lane, 16 consecutive K elements = 8 columns of fp16 pairs.
// Why these shapes: one tcgen05.mma of M 128 costs the tensor pipe at least ~93 cycles whatever
// its N (measured: N 64 and N 128 both 93, N 256 138 with A in tensor memory; 107 / 171 for
// N 128 / 256 with A in shared memory), so 64-key tiles (N 64, ideal 32 cycles) run Q K^T at a
// third of the pipe's rate; tensor memory (512 columns) holds O plus two 128-key S buffers, which
// leaves no room for Q, so Q stays in shared memory.
//
// Shared-memory operand layout: the 128-byte-swizzle canonical layouts.  A 5-D tensor map
// {64 halfs, row, 64-column group, head, batch} with 128-byte swizzle makes TMA write a
// (rows x 256) tile as sub-tiles [group][row][128 bytes], 16-byte chunk c of row r at
// r*128 + ((c ^ (r & 7)) << 4).  Descriptors over it:
//   K-major  (Q, K): stride-dim byte offset (between 8-row groups) = 1024; a K step of 16 halfs
//                 advances the start address by 32 bytes inside a group, then to the next group;
//   MN-major (V as the B operand of P V, keys are the contraction dim): leading-dim byte offset
//                 (between 64-column groups) = rows*128, stride-dim byte offset (between 8-key
//                 groups) = 1024; a K step of 16 keys advances the start address by 2048 bytes.
// Every wait is bounded; a wait that runs out sets a status word the host can read and the CTA
// falls through to the teardown (tensor memory is always released).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "khq_common.cuh"

namespace khq_prefill5 {

using khq::smem_u32;

constexpr int D = 256;
constexpr int BR = 128;     // query rows per CTA
constexpr int BC = 128;     // keys per tile
constexpr int NSOFT = 256;  // softmax threads: two per query row, 64 of a tile's 128 keys each
constexpr int NTHREADS = NSOFT + 96;
constexpr int Q_BYTES = BR * D * 2;        // 64 KB
constexpr int KHALF_BYTES = BC * 128 * 2;  // 32 KB: 128 keys x 128 head dims (two 64-dim groups)
constexpr int VHALF_BYTES = 64 * D * 2;    // 32 KB: 64 keys x 256 head dims (four 64-dim groups)
constexpr int OFF_Q = 0;
constexpr int OFF_K = OFF_Q + Q_BYTES;
constexpr int OFF_V = OFF_K + 2 * KHALF_BYTES;
constexpr int OFF_XCHG = OFF_V + 2 * VHALF_BYTES;  // float [2 parities][2 halves][128 rows]
constexpr int OFF_BARS = OFF_XCHG + 2 * 2 * 128 * 4;
constexpr int SMEM_BYTES = OFF_BARS + 256;
constexpr uint32_t TM_COLS = 512, TM_O = 0, TM_S = 256;
constexpr float RESCALE_LOG2 = 8.0f;

enum Bar {
    B_KFULL = 0, B_VFULL = 2, B_KEMPTY = 4, B_VEMPTY = 6, B_SFULL = 8, B_QFULL = 10, B_PREADY = 11, B_PVDONE = 12,
    B_XCHG = 14, B_QEMPTY = 18, B_OFREE = 19, B_PREADY2 = 20, B_COUNT = 21
};
static_assert(B_COUNT * 8 <= 192, "barriers overlap the tensor-memory slot");

__device__ int g_prefill_status = 0;

// ---- descriptors ---------------------------------------------------------------------------------
// Shared-memory matrix descriptor (64 bits): start address, leading and stride byte offsets (all in
// 16-byte units; bits 0-13, 16-29, 32-45), descriptor version 1 in bits 46-47, layout type 2
// (128-byte swizzle) in bits 61-63.  It is assembled from a low and a high word, see desc_lo/desc_hi.
// Instruction descriptor for kind::f16: fp32 accumulate, fp16 A and B, A K-major, M = 128.
// (A/B format field: 0 = fp16, 1 = bf16, bits 7-9 and 10-12.)
__host__ __device__ constexpr uint32_t instr_desc(int n, bool b_mn_major, bool bf16) {
    return (1u << 4) | (bf16 ? ((1u << 7) | (1u << 10)) : 0u) | (b_mn_major ? (1u << 16) : 0u) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(128 >> 4) << 24);
}
// Two floats -> one 32-bit word of the 16-bit storage type (round to nearest even), and back.
template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    if (BF16) {
        const __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&t);
    }
    const __half2 t = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&t);
}
template <bool BF16>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
    if (BF16) return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
    return __half22float2(*reinterpret_cast<const __half2*>(&w));
}

// ---- tcgen05 / TMA wrappers ----------------------------------------------------------------------
// The issuing thread is on the critical path: the 64-bit descriptors are assembled from a
// precomputed low word (start address and leading offset; the caller adds the K-step offset, which
// never carries out of the 14-bit address field) and a constant high word.  umma_ss: A and B from
// shared memory; umma_ts: A from tensor memory (row = lane, fp16 pairs, 8 columns per K step of 16).
__device__ __forceinline__ uint32_t desc_lo(uint32_t addr, uint32_t lbo) {
    return ((addr & 0x3FFFFu) >> 4) | (((lbo >> 4) & 0x3FFFu) << 16);
}
__host__ __device__ constexpr uint32_t desc_hi(uint32_t sbo) {
    return ((sbo >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);  // version 1 (bit 46), 128-byte swizzle (bits 61-63)
}
template <int ACC>
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                        uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .b64 da, db;\n\t.reg .pred p;\n\t"
        "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
        "setp.ne.u32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}" ::"r"(d_tmem),
        "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "n"(ACC)
        : "memory");
}
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .b64 db;\n\t.reg .pred p;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "setp.ne.u32 p, %5, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
        "%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15};" ::"r"(r[0]),
        "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(taddr)
        : "memory");
}
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
        "%29,%30,%31};" ::"r"(r[0]),
        "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
        "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
        "r"(r[29]), "r"(r[30]), "r"(r[31]), "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// One 5-D tiled TMA load of a single CTA; coordinate 0 is always 0, so the 16-byte rule holds.
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, uint64_t* bar, int c1, int c2,
                                            int c3, int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, "
        "%6, %7}], [%2];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}

// Bounded wait on up to three barriers at once.  A satisfied mbarrier wait still costs a ~250-cycle
// round trip, so the MMA thread polls the barriers of a step together (the polls overlap) instead
// of one after the other; a barrier found complete stays "done" (its next phase cannot complete
// before this thread moves on).
__device__ __forceinline__ uint32_t mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok;
}
template <int N>
__device__ __forceinline__ bool mbar_wait_all_bounded(uint64_t* const (&bar)[N], const uint32_t (&parity)[N], int* status) {
    uint32_t done = 0;
    for (uint32_t it = 0; it < (1u << 22); ++it) {
        uint32_t got[N];
#pragma unroll
        for (int i = 0; i < N; ++i) got[i] = mbar_test(bar[i], parity[i]);
#pragma unroll
        for (int i = 0; i < N; ++i) done |= got[i] << i;
        if (done == (1u << N) - 1u) return true;
        bool parked = false;  // park (a blocking try_wait) on the first barrier that is still open
#pragma unroll
        for (int i = 0; i < N; ++i)
            if (!parked && !((done >> i) & 1u)) {
                if (khq::mbar_try_wait(bar[i], parity[i])) done |= 1u << i;
                parked = true;
            }
        if (done == (1u << N) - 1u) return true;
    }
    atomicExch(status, 1);
    return false;
}

// ---- the kernel ----------------------------------------------------------------------------------
// A work item = 128 query rows of one (batch, head); the last row block attends the most keys.  CTA c
// takes one item per round of `grid` items, the c-th of even rounds and the c-th from the end of odd
// rounds; with one CTA per item there is a single round and the item is the CTA index.
struct Item {
    int q0, h, b, kvh, n_tiles;
};
template <bool PERSIST>
__device__ __forceinline__ bool get_item(int ordinal, int T, int H_q, int H_kv, int batch, int group_major, Item& it) {
    if (!PERSIST && ordinal > 0) return false;  // one item per CTA: the item is the CTA index
    const int nqb = (T + BR - 1) / BR;
    const int per = H_q * batch;
    // boustrophedon over the item list: in odd rounds the CTAs take the items in reverse, so that
    // every CTA's share of the triangular workload stays within one round's spread
    const long long lane_in_round = (ordinal & 1) ? (long long)(gridDim.x - 1 - blockIdx.x) : (long long)blockIdx.x;
    const long long w = lane_in_round + (long long)ordinal * gridDim.x;
    if (w >= (long long)nqb * per) return false;
    int qb;
    if (group_major) {
        // one (batch, kv head) group after the other, heaviest row blocks first inside a group:
        // the CTAs in flight then stream the K/V rows of one or two groups, which stay in L2
        const int n_rep = H_q / H_kv, per_group = n_rep * nqb;
        const int grp = (int)(w / per_group), idx = (int)(w % per_group);
        qb = nqb - 1 - idx / n_rep;
        it.b = grp / H_kv;
        it.kvh = grp % H_kv;
        it.h = it.kvh * n_rep + idx % n_rep;
    } else {
        // heaviest first over everything: consecutive items have (almost) the same size
        qb = nqb - 1 - (int)(w / per);
        const int rem = (int)(w % per);
        it.h = rem % H_q;
        it.b = rem / H_q;
        it.kvh = it.h / (H_q / H_kv);
    }
    it.q0 = qb * BR;
    it.n_tiles = min((T + BC - 1) / BC, qb + 1);  // causal: key tiles 0..qb (BR == BC)
    return true;
}

// grid = min(items, SMs) persistent CTAs for short prompts, one CTA per item for long ones (the
// launcher decides; a CTA simply works through the items its index selects).  q_gate (B, T, H_q, 2D), out (B, T, H_q, D); Q, K and V
// operands come through their tensor maps.  Per-tile barriers are indexed by g, the running count of
// tiles this CTA has processed over all its items, so that the producers and the MMA thread run
// ahead into the next item while the softmax warps are still in the epilogue of the current one.
template <bool PERSIST, bool BF16>
__global__ void __launch_bounds__(NTHREADS, 1)
khq_gqa_prefill_tc5_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                           const __grid_constant__ CUtensorMap tm_v, const __half* __restrict__ q_gate,
                           __half* __restrict__ out, int T, int H_q, int H_kv, int batch, int group_major,
                           float scale_log2e, long long q_bs, long long o_bs) {
    extern __shared__ __align__(1024) unsigned char smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BARS);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + OFF_BARS + 192);
    float* xchg = reinterpret_cast<float*>(smem + OFF_XCHG);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    int* status = &g_prefill_status;
    if ((smem_u32(smem) & 1023u) != 0) {  // the swizzled layouts need a 1024-byte aligned base
        if (tid == 0) atomicExch(status, 2);
        return;
    }

    if (tid == 0) {
        for (int s = 0; s < 2; ++s) {
            khq::mbar_init(&bars[B_KFULL + s], 1);
            khq::mbar_init(&bars[B_VFULL + s], 1);
            khq::mbar_init(&bars[B_KEMPTY + s], 1);
            khq::mbar_init(&bars[B_VEMPTY + s], 1);
            khq::mbar_init(&bars[B_SFULL + s], 1);
            khq::mbar_init(&bars[B_PVDONE + s], 1);
        }
        khq::mbar_init(&bars[B_QFULL], 1);
        khq::mbar_init(&bars[B_QEMPTY], 1);
        // one elected arrival per softmax warp: 256 separate arrivals on one barrier serialise
        // Two "P ready" barriers, used alternately: a softmax warp may finish tile g+1 (its S is
        // computed ahead) before a slower warp has arrived for tile g, and its arrival must not be
        // counted for tile g.  It cannot get two tiles ahead: S of tile g+2 is issued after tile g's
        // barrier has completed.
        khq::mbar_init(&bars[B_PREADY], NSOFT / 32);
        khq::mbar_init(&bars[B_PREADY2], NSOFT / 32);
        khq::mbar_init(&bars[B_OFREE], NSOFT / 32);
        for (int q = 0; q < 4; ++q) khq::mbar_init(&bars[B_XCHG + q], 2);  // the two warps of a lane quarter
        khq::fence_barrier_init();
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "n"(TM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t sbase = smem_u32(smem);

    if (warp == 8) {
        // ================================ producer of Q and K ======================================
        // K tile = two halves by head dim (groups 0-1 and 2-3), each [2 groups][128 keys][128 B].
        // The Q buffer is reloaded for the next item once the MMA thread has committed the last
        // Q K^T of the current one.
        if (lane == 0) {
            int g = 0, items = 0, halves = 0;
            bool ok = true;
            Item it;
            for (int i = 0; ok && get_item<PERSIST>(i, T, H_q, H_kv, batch, group_major, it); ++i) {
                if (i > 0 && !khq::mbar_wait_bounded(&bars[B_QEMPTY], (uint32_t)((i - 1) & 1), status)) break;
                khq::mbar_arrive_expect_tx(&bars[B_QFULL], Q_BYTES);
                tma_load_5d(sbase + OFF_Q, &tm_q, &bars[B_QFULL], it.q0, 0, it.h, it.b);
                items = i + 1;
                for (int j = 0; ok && j < it.n_tiles; ++j, ++g) {
                    for (int hf = 0; hf < 2; ++hf) {
                        if (g >= 1 && !khq::mbar_wait_bounded(&bars[B_KEMPTY + hf], (uint32_t)((g - 1) & 1), status)) {
                            ok = false;
                            break;
                        }
                        khq::mbar_arrive_expect_tx(&bars[B_KFULL + hf], KHALF_BYTES);
                        tma_load_5d(sbase + OFF_K + hf * KHALF_BYTES, &tm_k, &bars[B_KFULL + hf], j * BC, 2 * hf, it.kvh, it.b);
                        halves = 2 * g + hf + 1;
                    }
                }
            }
            // nothing this thread started may still be in flight when the CTA leaves
            if (items > 0) khq::mbar_wait_bounded(&bars[B_QFULL], (uint32_t)((items - 1) & 1), status);
            for (int i = max(0, halves - 2); i < halves; ++i)
                khq::mbar_wait_bounded(&bars[B_KFULL + (i & 1)], (uint32_t)((i >> 1) & 1), status);
        }
    } else if (warp == 10) {
        // ================================ producer of V ============================================
        // V tile = two halves by key (64 keys each), each [4 groups][64 keys][128 B].
        if (lane == 0) {
            int g = 0, halves = 0;
            bool ok = true;
            Item it;
            for (int i = 0; ok && get_item<PERSIST>(i, T, H_q, H_kv, batch, group_major, it); ++i) {
                for (int j = 0; ok && j < it.n_tiles; ++j, ++g) {
                    for (int hf = 0; hf < 2; ++hf) {
                        if (g >= 1 && !khq::mbar_wait_bounded(&bars[B_VEMPTY + hf], (uint32_t)((g - 1) & 1), status)) {
                            ok = false;
                            break;
                        }
                        khq::mbar_arrive_expect_tx(&bars[B_VFULL + hf], VHALF_BYTES);
                        tma_load_5d(sbase + OFF_V + hf * VHALF_BYTES, &tm_v, &bars[B_VFULL + hf], j * BC + hf * 64, 0, it.kvh,
                                    it.b);
                        halves = 2 * g + hf + 1;
                    }
                }
            }
            for (int i = max(0, halves - 2); i < halves; ++i)
                khq::mbar_wait_bounded(&bars[B_VFULL + (i & 1)], (uint32_t)((i >> 1) & 1), status);
        }
    } else if (warp == 9) {
        // ================================ MMA issuer ==============================================
        if (lane == 0) {
            constexpr uint32_t IDESC_S = instr_desc(BC, false, BF16);
            constexpr uint32_t IDESC_O = instr_desc(D, true, BF16);
            constexpr uint32_t HI_K = desc_hi(1024);  // Q, K (K-major) and V (MN-major): 1024 bytes between 8-row groups
            const uint32_t q_lo = desc_lo(sbase + OFF_Q, 16), k_lo = desc_lo(sbase + OFF_K, 16);
            const uint32_t v_lo = desc_lo(sbase + OFF_V, 64 * 128);  // leading offset: the next 64-column group
            bool ok = true;
            auto issue_qk = [&](int g) {  // S[g & 1] = Q K^T of the tile with running index g
                const uint32_t s_tmem = tmem + TM_S + (uint32_t)(g & 1) * BC;
                uint64_t* const kb[2] = {&bars[B_KFULL], &bars[B_KFULL + 1]};
                const uint32_t kp[2] = {(uint32_t)(g & 1), (uint32_t)(g & 1)};
                ok = ok && mbar_wait_all_bounded(kb, kp, status);
                if (!ok) return;
                tc_fence_after();
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk) {
                        const int ks = hf * 8 + kk;
                        // byte offsets / 16: next 64-dim group = rows*128 bytes, next K step = 32 bytes
                        const uint32_t oa = (uint32_t)((ks >> 2) * (BR * 128) + (ks & 3) * 32) >> 4;
                        const uint32_t ob = (uint32_t)(hf * KHALF_BYTES + (kk >> 2) * (BC * 128) + (kk & 3) * 32) >> 4;
                        if (ks == 0) umma_ss<0>(s_tmem, q_lo + oa, HI_K, k_lo + ob, HI_K, IDESC_S);
                        else umma_ss<1>(s_tmem, q_lo + oa, HI_K, k_lo + ob, HI_K, IDESC_S);
                    }
                    umma_commit(&bars[B_KEMPTY + hf]);
                }
                umma_commit(&bars[B_SFULL + (g & 1)]);
            };
            Item it, nx;
            bool have = get_item<PERSIST>(0, T, H_q, H_kv, batch, group_major, it);
            int g = 0;
            if (have) {
                ok = khq::mbar_wait_bounded(&bars[B_QFULL], 0u, status);
                if (ok) issue_qk(0);
                if (PERSIST && ok && it.n_tiles == 1) umma_commit(&bars[B_QEMPTY]);
            }
            for (int i = 0; have && ok; ++i) {
                const bool have_nx = get_item<PERSIST>(i + 1, T, H_q, H_kv, batch, group_major, nx);
                for (int j = 0; ok && j < it.n_tiles; ++j, ++g) {
                    // run ahead: Q K^T of the next tile, which may be the first tile of the next item
                    const bool same_item = j + 1 < it.n_tiles;
                    if (same_item || have_nx) {
                        if (!same_item) ok = khq::mbar_wait_bounded(&bars[B_QFULL], (uint32_t)((i + 1) & 1), status);
                        if (ok) issue_qk(g + 1);
                        // once the last Q K^T of an item is out, its Q buffer may be reloaded
                        const bool last_qk = same_item ? (j + 2 == it.n_tiles) : (nx.n_tiles == 1);
                        if (PERSIST && ok && last_qk) umma_commit(&bars[B_QEMPTY]);
                    }
                    if (!ok) break;
                    uint64_t* const pb[3] = {&bars[(g & 1) ? B_PREADY2 : B_PREADY], &bars[B_VFULL], &bars[B_VFULL + 1]};
                    const uint32_t pp[3] = {(uint32_t)((g >> 1) & 1), (uint32_t)(g & 1), (uint32_t)(g & 1)};
                    ok = mbar_wait_all_bounded(pb, pp, status);
                    // the first P V of an item overwrites O: the previous item's epilogue must have read it
                    if (PERSIST && ok && j == 0 && i > 0)
                        ok = khq::mbar_wait_bounded(&bars[B_OFREE], (uint32_t)((i - 1) & 1), status);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t p_tmem = tmem + TM_S + (uint32_t)(g & 1) * BC;
#pragma unroll
                    for (int hf = 0; hf < 2; ++hf) {
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            const uint32_t ob = (uint32_t)(hf * VHALF_BYTES + kk * 2048) >> 4;  // 16 keys = 2048 bytes
                            umma_ts(tmem + TM_O, p_tmem + (hf * 4 + kk) * 8, v_lo + ob, HI_K, IDESC_O,
                                    (hf > 0 || kk > 0) ? 1u : (uint32_t)(j > 0));
                        }
                        if (hf == 1) umma_commit(&bars[B_PVDONE + (g & 1)]);
                        umma_commit(&bars[B_VEMPTY + hf]);
                    }
                }
                it = nx;
                have = have_nx;
            }
        }
    } else {
        // ================================ softmax + epilogue ======================================
        // Two threads per query row: half 0 (warps 0-3) takes keys 0-63 of a tile and columns 0-127
        // of O, half 1 (warps 4-7) keys 64-127 and columns 128-255.  Both warps of a row sit on the
        // same tensor-memory lane quarter (warp % 4) and on the same scheduler.
        const int half = warp >> 2, r = tid & 127;
        const long long q_row = (long long)H_q * 2 * D, o_row = (long long)H_q * D;
        const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        uint64_t* xbar = &bars[B_XCHG + (warp & 3)];
        int g = 0, x = 0;  // running tile index; running phase of the exchange barrier
        bool ok = true;
        Item it;
        for (int i = 0; ok && get_item<PERSIST>(i, T, H_q, H_kv, batch, group_major, it); ++i) {
            const int q0 = it.q0, row = q0 + r;
            const bool live = row < T;
            const __half* qrow = q_gate + it.b * q_bs + (long long)(live ? row : 0) * q_row + (long long)it.h * 2 * D;
            float m_used = -1e30f, l_run = 0.0f;
            for (int j = 0; j < it.n_tiles; ++j, ++g, ++x) {
                ok = __all_sync(0xFFFFFFFFu, khq::mbar_wait_bounded(&bars[B_SFULL + (g & 1)], (uint32_t)((g >> 1) & 1), status));
                if (!ok) break;
                tc_fence_after();
                const uint32_t s_addr = lane_base + TM_S + (uint32_t)(g & 1) * BC;
                uint32_t sr[2][32];
                tmem_ld32(s_addr + half * 64, sr[0]);
                tmem_ld32(s_addr + half * 64 + 32, sr[1]);
                tmem_ld_wait();
                const int k0 = j * BC + half * 64;
                // raw scores; masked entries (key after the row, or past the prompt) become -inf-like
                if ((k0 + 63 > q0) || (k0 + 64 > T)) {
#pragma unroll
                    for (int c = 0; c < 64; ++c)
                        if (k0 + c > row || k0 + c >= T) sr[c >> 5][c & 31] = __float_as_uint(-1e30f);
                }
                float mx4[4] = {-1e30f, -1e30f, -1e30f, -1e30f};
#pragma unroll
                for (int c = 0; c < 64; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(sr[c >> 5][c & 31]));
                float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
                // the row maximum over all 128 keys: swap half maxima with the partner thread
                xchg[((x & 1) * 2 + half) * 128 + r] = mx;
                __syncwarp();
                if (lane == 0) khq::mbar_arrive(xbar);
                ok = __all_sync(0xFFFFFFFFu, khq::mbar_wait_bounded(xbar, (uint32_t)(x & 1), status));
                if (!ok) break;
                mx = fmaxf(mx, xchg[((x & 1) * 2 + (half ^ 1)) * 128 + r]) * scale_log2e;  // scale > 0
                float factor = 1.0f;
                bool grow = false;
                if (j == 0) {
                    m_used = mx;
                } else if (mx > m_used + RESCALE_LOG2) {
                    factor = exp2f(m_used - mx);
                    m_used = mx;
                    grow = true;
                }
                // p = 2^(s*scale - m): one fused multiply-add and one ex2 per score
                float rs4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                uint32_t pk[32];
                const float neg_m = -m_used;
#pragma unroll
                for (int c = 0; c < 64; c += 2) {
                    const float p0 = ex2_approx(fmaf(__uint_as_float(sr[c >> 5][c & 31]), scale_log2e, neg_m));
                    const float p1 = ex2_approx(fmaf(__uint_as_float(sr[(c + 1) >> 5][(c + 1) & 31]), scale_log2e, neg_m));
                    rs4[(c >> 1) & 3] += p0 + p1;
                    pk[c >> 1] = pack2<BF16>(p0, p1);
                }
                const float rs = (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
                l_run = l_run * factor + rs;
                if (j > 0 && __any_sync(0xFFFFFFFFu, grow)) {
                    // O may only be touched between P V of the previous tile and P V of this one.  The
                    // completion barriers alternate between two mbarriers so that a thread may skip
                    // phases: barrier (g-1)&1 last completed for tile g-3 (certainly, since Q K^T of
                    // this tile was issued behind P V of tile g-2) and cannot complete for tile g+1
                    // before this thread's own arrival for that tile.
                    ok = __all_sync(0xFFFFFFFFu, khq::mbar_wait_bounded(&bars[B_PVDONE + ((g - 1) & 1)],
                                                                      (uint32_t)(((g - 1) >> 1) & 1), status));
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll 1
                    for (int c0 = half * 128; c0 < half * 128 + 128; c0 += 32) {
                        uint32_t orr[32];
                        tmem_ld32(lane_base + TM_O + c0, orr);
                        tmem_ld_wait();
#pragma unroll
                        for (int q = 0; q < 32; ++q) orr[q] = __float_as_uint(__uint_as_float(orr[q]) * factor);
                        tmem_st32(lane_base + TM_O + c0, orr);
                    }
                }
                // P (fp16 pairs) over the S buffer it came from: keys 64*half.. -> columns 32*half..
                // (the partner has read its S columns: it passed the exchange barrier after its load)
                tmem_st32(s_addr + half * 32, pk);
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) khq::mbar_arrive(&bars[(g & 1) ? B_PREADY2 : B_PREADY]);
            }
            if (!ok) break;
            // ---- epilogue of the item -------------------------------------------------------------
            // this thread's 128 gate values: all sixteen 16-byte loads go out together, ahead of the
            // final waits (issued one per use they cost a full memory latency each)
            const __half* gate = qrow + D + half * 128;
            uint4 g4[16];
#pragma unroll
            for (int q = 0; q < 16; ++q) g4[q] = live ? __ldg(reinterpret_cast<const uint4*>(gate) + q) : make_uint4(0u, 0u, 0u, 0u);
            // row sum over both halves (one more phase of the exchange barrier)
            xchg[((x & 1) * 2 + half) * 128 + r] = l_run;
            __syncwarp();
            if (lane == 0) khq::mbar_arrive(xbar);
            ok = khq::mbar_wait_bounded(xbar, (uint32_t)(x & 1), status);
            if (ok) l_run += xchg[((x & 1) * 2 + (half ^ 1)) * 128 + r];
            ++x;
            if (ok) ok = khq::mbar_wait_bounded(&bars[B_PVDONE + ((g - 1) & 1)], (uint32_t)(((g - 1) >> 1) & 1), status);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            tc_fence_after();
            const float inv = 1.0f / (l_run + 1e-9f);
            __half* op = out + it.b * o_bs + (long long)(live ? row : 0) * o_row + (long long)it.h * D + half * 128;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t orr[32];
                tmem_ld32(lane_base + TM_O + half * 128 + c * 32, orr);
                tmem_ld_wait();
                if (PERSIST && c == 3) {  // O has been read: the next item's first P V may overwrite it
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) khq::mbar_arrive(&bars[B_OFREE]);
                }
                if (live) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const uint4 gq = g4[c * 4 + q];
                        const uint32_t gw[4] = {gq.x, gq.y, gq.z, gq.w};
                        uint32_t ow[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 gf = unpack2<BF16>(gw[e]);
                            const float g0 = gf.x, g1 = gf.y;
                            const float x0 = __uint_as_float(orr[q * 8 + 2 * e]) * inv * __fdividef(1.0f, 1.0f + __expf(-g0));
                            const float x1 = __uint_as_float(orr[q * 8 + 2 * e + 1]) * inv * __fdividef(1.0f, 1.0f + __expf(-g1));
                            ow[e] = pack2<BF16>(x0, x1);
                        }
                        *reinterpret_cast<uint4*>(op + c * 32 + q * 8) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
                    }
                }
            }
        }
    }
    // ---- teardown: every thread arrives here, with or without a failed wait ----------------------
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(TM_COLS) : "memory");
    }
}

}  // namespace khq_prefill5

// ---- host side -----------------------------------------------------------------------------------
namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// Tensor map over a (batch, T, heads, row_halfs) fp16 tensor that exposes, per (head, batch), a
// T x 256 matrix as {64 halfs, T rows, 4 column groups}; a box is `box_rows` rows x `box_groups`
// column groups of one head.
int make_map(CUtensorMap* map, const void* base, int T, int heads, int batch, long long row_halfs,
             long long head_halfs, long long batch_halfs, int box_rows, int box_groups, bool bf16) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return -107;
    if (batch == 1) batch_halfs = (long long)T * row_halfs;
    const cuuint64_t dims[5] = {64, (cuuint64_t)T, 4, (cuuint64_t)heads, (cuuint64_t)batch};
    const cuuint64_t strides[4] = {(cuuint64_t)row_halfs * 2, 128, (cuuint64_t)head_halfs * 2, (cuuint64_t)batch_halfs * 2};
    const cuuint32_t box[5] = {64, (cuuint32_t)box_rows, (cuuint32_t)box_groups, 1, 1};
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    for (cuuint64_t st : strides)
        if (st % 16 != 0) return -104;
    const CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -108;
}

}  // namespace

static int g_tc5_items_per_cta = 0;

// 0 = choose by prompt length, 1 = one item per CTA, n > 1 = n items per CTA (a large n gives
// the fully persistent grid).  Returns -100 for a negative value.
extern "C" int khq_b200_prefill_tc5_items_per_cta(int n) {
    if (n < 0) return -100;
    g_tc5_items_per_cta = n;
    return 0;
}

namespace {
int launch_tc5(const void* q_gate, const void* k, const void* v, void* out, int batch, int T, int H_q, int H_kv, int d,
               float scale, long long q_batch_stride, long long kv_batch_stride, long long out_batch_stride,
               cudaStream_t stream, bool bf16) {
    using namespace khq_prefill5;
    if (batch <= 0 || T <= 0 || H_q <= 0 || H_kv <= 0) return -100;
    if (d != D || H_q % H_kv != 0) return -103;
    const void* ptrs[] = {q_gate, k, v, out};
    for (const void* p : ptrs)
        if ((reinterpret_cast<uintptr_t>(p) & 15) != 0) return -104;
    if (batch > 1 && ((q_batch_stride | kv_batch_stride | out_batch_stride) & 7) != 0) return -104;
    CUtensorMap mq, mk, mv;
    int rc = make_map(&mq, q_gate, T, H_q, batch, (long long)H_q * 2 * D, 2 * D, q_batch_stride, BR, 4, bf16);
    if (rc == 0) rc = make_map(&mk, k, T, H_kv, batch, (long long)H_kv * D, D, kv_batch_stride, BC, 2, bf16);
    if (rc == 0) rc = make_map(&mv, v, T, H_kv, batch, (long long)H_kv * D, D, kv_batch_stride, 64, 4, bf16);
    if (rc != 0) return rc;
    static bool attr_done[64] = {};
    static int sm_count[64] = {};
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return static_cast<int>(err);
    if (dev < 0 || dev >= 64) return -100;
    if (!attr_done[dev]) {
        const void* kernels[4] = {(const void*)khq_gqa_prefill_tc5_kernel<true, false>, (const void*)khq_gqa_prefill_tc5_kernel<false, false>,
                                  (const void*)khq_gqa_prefill_tc5_kernel<true, true>, (const void*)khq_gqa_prefill_tc5_kernel<false, true>};
        for (const void* kf : kernels) {
            err = cudaFuncSetAttribute(kf, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
            if (err != cudaSuccess) return static_cast<int>(err);
        }
        err = cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
        if (err != cudaSuccess) return static_cast<int>(err);
        attr_done[dev] = true;
    }
    const long long items = (long long)((T + BR - 1) / BR) * H_q * batch;
    // Short prompts (up to 24 row blocks): a persistent grid of one CTA per SM, each working through
    // its items and overlapping one item's epilogue with the next one's first tiles (32 x 512:
    // 0.26 ms against 0.31 ms; 8 x 2048: 0.49 against 0.53).  Longer prompts: one CTA per item, one
    // (batch, kv head) group after the other, heaviest first, which leaves the balancing of the
    // triangular workload to the hardware's dynamic CTA scheduler and runs the leaner instantiation
    // of the kernel (4 x 4096: 0.78 ms against 0.81; 4 x 8192: 2.72 against 2.99).
    // khq_b200_prefill_tc5_items_per_cta(n) or KHQ_PREFILL_ITEMS_PER_CTA (read once) force a mode:
    // 1 = one item per CTA, larger = that many items per CTA (the setter wins; 0 = automatic).
    static int env_forced = -1;
    if (env_forced < 0) {
        const char* e = getenv("KHQ_PREFILL_ITEMS_PER_CTA");
        env_forced = e ? atoi(e) : 0;
        if (env_forced < 0) env_forced = 0;
    }
    const int forced = g_tc5_items_per_cta > 0 ? g_tc5_items_per_cta : env_forced;
    const int nqb = (T + BR - 1) / BR;
    long long ctas;
    int group_major = 0;
    if (forced == 1 || (forced == 0 && nqb > 24)) {
        ctas = items;
        group_major = 1;
    } else if (forced > 1) {
        ctas = (items + forced - 1) / forced;
        if (ctas < sm_count[dev]) ctas = items < sm_count[dev] ? items : sm_count[dev];
    } else {
        ctas = items < sm_count[dev] ? items : sm_count[dev];
    }
    const unsigned grid = (unsigned)ctas;
    const __half* qp = static_cast<const __half*>(q_gate);  // 16-bit storage; the kernel converts per its type flag
    __half* op = static_cast<__half*>(out);
    const float sl2 = scale * 1.4426950408889634f;
#define KHQ_TC5_LAUNCH(PERSIST, BF16)                                                                                  \
    khq_gqa_prefill_tc5_kernel<PERSIST, BF16><<<grid, NTHREADS, SMEM_BYTES, stream>>>(                                  \
        mq, mk, mv, qp, op, T, H_q, H_kv, batch, group_major, sl2, q_batch_stride, out_batch_stride)
    if (ctas == items) {
        if (bf16) KHQ_TC5_LAUNCH(false, true);
        else KHQ_TC5_LAUNCH(false, false);
    } else {
        if (bf16) KHQ_TC5_LAUNCH(true, true);
        else KHQ_TC5_LAUNCH(true, false);
    }
#undef KHQ_TC5_LAUNCH
    err = cudaGetLastError();
    return (err == cudaSuccess) ? 0 : static_cast<int>(err);
}
}  // namespace

// Same arguments as launch_khq_gqa_prefill_fp16.  Returns -107 when the driver offers no tensor-map
// encoder and -108 when it refuses these shapes.
extern "C" int launch_khq_gqa_prefill_tc5_fp16(const void* q_gate, const void* k, const void* v, void* out, int batch,
                                               int T, int H_q, int H_kv, int d, float scale,
                                               long long q_batch_stride, long long kv_batch_stride,
                                               long long out_batch_stride, cudaStream_t stream) {
    return launch_tc5(q_gate, k, v, out, batch, T, H_q, H_kv, d, scale, q_batch_stride, kv_batch_stride, out_batch_stride,
                      stream, false);
}

// The same attention over bf16 tensors (bf16 operands and P, fp32 accumulation, bf16 output).
extern "C" int launch_khq_gqa_prefill_bf16(const void* q_gate, const void* k, const void* v, void* out, int batch, int T,
                                           int H_q, int H_kv, int d, float scale, long long q_batch_stride,
                                           long long kv_batch_stride, long long out_batch_stride, cudaStream_t stream) {
    return launch_tc5(q_gate, k, v, out, batch, T, H_q, H_kv, d, scale, q_batch_stride, kv_batch_stride, out_batch_stride,
                      stream, true);
}

// Reads and clears the status word of the tcgen05 prefill kernel on the current device
// (synchronises the device): 0 = clean, 1 = a bounded wait ran out, 2 = misaligned shared memory.
extern "C" int khq_b200_prefill_status(void) {
    int st = 0;
    if (cudaMemcpyFromSymbol(&st, khq_prefill5::g_prefill_status, sizeof(int)) != cudaSuccess) return -1;
    if (st != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(khq_prefill5::g_prefill_status, &zero, sizeof(int));
    }
    return st;
}
