// khq_prefill.cu -- causal GQA prefill attention with sigmoid output gate (fp16 in, fp32
// accumulate) for Bonsai-27B's attention shape: H_q 24, H_kv 4, head_dim 256.
//
// Math (the reference's fp16-KV attention, src/kernels/elementwise_sm75.mojo:1140-1231, applied
// to every prompt row at once instead of one launch per token as src/models/qwen3_5/layer.mojo:
// 630-641 does): out[t,h,:] = softmax_{u<=t}(q[t,h].K[u,g]*scale) V[u,g] * sigmoid(gate[t,h,:]),
// g = h/6, with the kernel's 1/(Z + 1e-9) denominator.  K is already RoPE'd.
//
// This generation runs the two contractions on the warp-level tensor path (mma.sync m16n8k16,
// ldmatrix, cp.async double buffering): one CTA = 64 query rows of one query head, 4 warps x 16
// rows, KV tiles of 64 keys, online softmax in registers, O (16 x 256 per warp) in registers.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace khq_prefill {

constexpr int D = 256;
constexpr int BR = 64;   // query rows per CTA
constexpr int BC = 64;   // keys per tile
constexpr int NTHREADS = 128;
constexpr int ROW_BYTES = D * 2;            // 512
constexpr int TILE_BYTES = BC * ROW_BYTES;  // 32 KB
constexpr int SMEM_BYTES = TILE_BYTES * 5;  // Q + 2 x (K, V)

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
// 16-byte chunk c (0..31) of row r inside a [rows][256] fp16 tile, XOR-swizzled so that the
// eight rows an ldmatrix phase touches fall in eight different bank groups.
__device__ __forceinline__ uint32_t tile_off(int r, int c) { return (uint32_t)(r * ROW_BYTES + ((c ^ (r & 7)) << 4)); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int sz = valid ? 16 : 0;  // src-size 0 => the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// Copies `rows` x 256 halfs (row stride `src_stride` halfs) into a swizzled tile; rows at or
// beyond `valid_rows` are zero-filled.
__device__ __forceinline__ void load_tile(unsigned char* tile, const __half* src, long long src_stride,
                                          int valid_rows, int tid) {
#pragma unroll 4
    for (int i = tid; i < BC * 32; i += NTHREADS) {
        const int r = i >> 5, c = i & 31;
        const bool ok = r < valid_rows;
        cp_async16(smem_u32(tile) + tile_off(r, c), src + (long long)(ok ? r : 0) * src_stride + c * 8, ok);
    }
}

// grid = (ceil(T/64), H_q, batch).  q_gate (B, T, H_q, 2D), k/v (B, T, H_kv, D), out (B, T, H_q, D).
__global__ void __launch_bounds__(NTHREADS, 1)
khq_gqa_prefill_kernel(const __half* __restrict__ q_gate, const __half* __restrict__ k,
                       const __half* __restrict__ v, __half* __restrict__ out, int T, int H_q, int H_kv,
                       float scale_log2e, long long q_bs, long long kv_bs, long long o_bs) {
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* sQ = smem;
    unsigned char* sK[2] = {smem + TILE_BYTES, smem + 3 * TILE_BYTES};
    unsigned char* sV[2] = {smem + 2 * TILE_BYTES, smem + 4 * TILE_BYTES};
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t4 = lane & 3;
    // heaviest row blocks first: the last query block attends the most keys
    const int qb = (int)gridDim.x - 1 - (int)blockIdx.x;
    const int h = blockIdx.y, b = blockIdx.z;
    const int kvh = h / (H_q / H_kv);
    const int q0 = qb * BR;
    const long long q_row = (long long)H_q * 2 * D, kv_row = (long long)H_kv * D, o_row = (long long)H_q * D;
    const __half* qp = q_gate + b * q_bs + (long long)q0 * q_row + (long long)h * 2 * D;
    const __half* kp = k + b * kv_bs + (long long)kvh * D;
    const __half* vp = v + b * kv_bs + (long long)kvh * D;

    const int n_tiles = qb + 1;  // causal: key tiles 0..qb (BR == BC)
    load_tile(sQ, qp, q_row, min(BR, T - q0), tid);
    load_tile(sK[0], kp, kv_row, min(BC, T), tid);
    load_tile(sV[0], vp, kv_row, min(BC, T), tid);
    cp_async_commit();

    float o[32][4];
#pragma unroll
    for (int i = 0; i < 32; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m_run[2] = {-1e30f, -1e30f}, l_run[2] = {0.0f, 0.0f};
    const int row_a = q0 + warp * 16 + g;  // this thread's two query rows: row_a and row_a + 8

#pragma unroll 1
    for (int j = 0; j < n_tiles; ++j) {
        const int buf = j & 1;
        if (j + 1 < n_tiles) {
            const int k0n = (j + 1) * BC;
            load_tile(sK[buf ^ 1], kp + (long long)k0n * kv_row, kv_row, min(BC, T - k0n), tid);
            load_tile(sV[buf ^ 1], vp + (long long)k0n * kv_row, kv_row, min(BC, T - k0n), tid);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();

        // ---- S = Q K^T : 16 rows x 64 keys per warp ------------------------------------------
        float s[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
        const uint32_t qbase = smem_u32(sQ), kbase = smem_u32(sK[buf]), vbase = smem_u32(sV[buf]);
#pragma unroll 4
        for (int kk = 0; kk < 16; ++kk) {
            uint32_t a[4];
            ldsm_x4(a, qbase + tile_off(warp * 16 + (lane & 15), kk * 2 + (lane >> 4)));
#pragma unroll
            for (int np = 0; np < 4; ++np) {  // two 8-key tiles per ldmatrix.x4
                uint32_t bb[4];
                ldsm_x4(bb, kbase + tile_off(np * 16 + (lane & 7) + ((lane >> 4) << 3), kk * 2 + ((lane >> 3) & 1)));
                mma16816(s[np * 2], a, bb[0], bb[1]);
                mma16816(s[np * 2 + 1], a, bb[2], bb[3]);
            }
        }
        // ---- scale, causal mask, online softmax -------------------------------------------------
        const int k0 = j * BC;
        const bool diag = (j == n_tiles - 1);
        float mx[2] = {m_run[0], m_run[1]};
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = k0 + nt * 8 + t4 * 2 + (e & 1);
                const int row = row_a + ((e >> 1) << 3);
                float x = s[nt][e] * scale_log2e;
                if ((diag && key > row) || key >= T) x = -1e30f;
                s[nt][e] = x;
                mx[e >> 1] = fmaxf(mx[e >> 1], x);
            }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xFFFFFFFFu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xFFFFFFFFu, mx[r], 2));
        }
        float corr[2], rs[2] = {0.0f, 0.0f};
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            corr[r] = exp2f(m_run[r] - mx[r]);
            m_run[r] = mx[r];
        }
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float p = exp2f(s[nt][e] - mx[e >> 1]);
                s[nt][e] = p;
                rs[e >> 1] += p;
            }
#pragma unroll
        for (int r = 0; r < 2; ++r) l_run[r] = l_run[r] * corr[r] + rs[r];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            o[i][0] *= corr[0];
            o[i][1] *= corr[0];
            o[i][2] *= corr[1];
            o[i][3] *= corr[1];
        }
        // ---- O += P V : keys are the contraction dim --------------------------------------------
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            uint32_t a[4];
            a[0] = pack_h2(s[2 * kk][0], s[2 * kk][1]);
            a[1] = pack_h2(s[2 * kk][2], s[2 * kk][3]);
            a[2] = pack_h2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            a[3] = pack_h2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int dp = 0; dp < 16; ++dp) {  // two 8-dim tiles per ldmatrix.x4.trans
                uint32_t bb[4];
                ldsm_x4_trans(bb, vbase + tile_off(kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), dp * 2 + (lane >> 4)));
                mma16816(o[dp * 2], a, bb[0], bb[1]);
                mma16816(o[dp * 2 + 1], a, bb[2], bb[3]);
            }
        }
        __syncthreads();  // all warps are done with this K/V buffer before it is refilled
    }

    // ---- normalise (quad sum of l), gate, store -------------------------------------------------
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xFFFFFFFFu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xFFFFFFFFu, l_run[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = row_a + r * 8;
        if (row >= T) continue;
        const float inv = 1.0f / (l_run[r] + 1e-9f);
        const __half* gate = q_gate + b * q_bs + (long long)row * q_row + (long long)h * 2 * D + D;
        __half* op = out + b * o_bs + (long long)row * o_row + (long long)h * D;
#pragma unroll
        for (int nt = 0; nt < 32; ++nt) {
            const int col = nt * 8 + t4 * 2;
            const __half2 gg = *reinterpret_cast<const __half2*>(gate + col);
            const float g0 = __half2float(__low2half(gg)), g1 = __half2float(__high2half(gg));
            const float x0 = o[nt][2 * r] * inv * (1.0f / (1.0f + __expf(-g0)));
            const float x1 = o[nt][2 * r + 1] * inv * (1.0f / (1.0f + __expf(-g1)));
            *reinterpret_cast<__half2*>(op + col) = __floats2half2_rn(x0, x1);
        }
    }
}

}  // namespace khq_prefill

extern "C" int launch_khq_gqa_prefill_mma_fp16(const void* q_gate, const void* k, const void* v, void* out,
                                               int batch, int T, int H_q, int H_kv, int d, float scale,
                                               long long q_batch_stride, long long kv_batch_stride,
                                               long long out_batch_stride, cudaStream_t stream) {
    using namespace khq_prefill;
    if (batch <= 0 || T <= 0 || H_q <= 0 || H_kv <= 0) return -100;
    if (d != D || H_q % H_kv != 0) return -103;
    const void* ptrs[] = {q_gate, k, v, out};
    for (const void* p : ptrs)
        if ((reinterpret_cast<uintptr_t>(p) & 15) != 0) return -104;
    static bool attr_done[64] = {};
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return static_cast<int>(err);
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        err = cudaFuncSetAttribute(khq_gqa_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (err != cudaSuccess) return static_cast<int>(err);
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    const dim3 grid((unsigned)((T + BR - 1) / BR), (unsigned)H_q, (unsigned)batch);
    khq_gqa_prefill_kernel<<<grid, NTHREADS, SMEM_BYTES, stream>>>(
        static_cast<const __half*>(q_gate), static_cast<const __half*>(k), static_cast<const __half*>(v),
        static_cast<__half*>(out), T, H_q, H_kv, scale * 1.4426950408889634f, q_batch_stride, kv_batch_stride,
        out_batch_stride);
    err = cudaGetLastError();
    return (err == cudaSuccess) ? 0 : static_cast<int>(err);
}

// ---- kernel selection -----------------------------------------------------------------------------
extern "C" int launch_khq_gqa_prefill_tc5_fp16(const void* q_gate, const void* k, const void* v, void* out,
                                               int batch, int T, int H_q, int H_kv, int d, float scale,
                                               long long q_batch_stride, long long kv_batch_stride,
                                               long long out_batch_stride, cudaStream_t stream);

static int g_prefill_kernel = 0;  // 0: tcgen05 / tensor-memory kernel, 1: warp-level mma.sync kernel

extern "C" int khq_b200_prefill_select(int which) {
    if (which != 0 && which != 1) return -100;
    g_prefill_kernel = which;
    return 0;
}

extern "C" int launch_khq_gqa_prefill_fp16(const void* q_gate, const void* k, const void* v, void* out,
                                           int batch, int T, int H_q, int H_kv, int d, float scale,
                                           long long q_batch_stride, long long kv_batch_stride,
                                           long long out_batch_stride, cudaStream_t stream) {
    return (g_prefill_kernel == 0 ? launch_khq_gqa_prefill_tc5_fp16 : launch_khq_gqa_prefill_mma_fp16)(
        q_gate, k, v, out, batch, T, H_q, H_kv, d, scale, q_batch_stride, kv_batch_stride, out_batch_stride, stream);
}
