// khq_prestep.cu -- the five launches that precede the KHQ decode step in the reference, as one:
//   per-head RMSNorm of q and k      (head_rmsnorm_sm75_gpu, src/kernels/elementwise_sm75.mojo:362-423;
//                                     called at src/models/qwen3_5/attention.mojo:329-336)
//   K un-RoPE'd -> ring_u[slot]      (khq_capture_unroped, src/khq/runtime.mojo:432-451)
//   half-split partial RoPE of q, k  (partial_rope_sm75_gpu, elementwise_sm75.mojo:1023-1061;
//                                     attention.mojo:348-353)
//   K RoPE'd, V -> ring_k/ring_v[slot] (khq_ring_dual_sm75_gpu, elementwise_sm75.mojo:293-312;
//                                     src/khq/runtime.mojo:486)
// One warp per head (24 query heads + 4 kv heads).  The arithmetic follows the reference kernels
// step by step (per-lane strided partial sums, shuffle-down tree, fp16 rounding between the norm
// and the rotation, fp32 angle pos*freq), so un-rotated dims are bit-identical to them.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace khq_prestep {

__device__ __forceinline__ void norm_head(__half* x, const float* w, int dim, float eps, int lane) {
    float sum_sq = 0.0f;
    for (int d = lane; d < dim; d += 32) {
        const float v = __half2float(x[d]);
        sum_sq += v * v;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum_sq += __shfl_down_sync(0xFFFFFFFFu, sum_sq, off);
    float rms = 0.0f;
    if (lane == 0) rms = 1.0f / sqrtf(sum_sq / (float)dim + eps);
    rms = __shfl_sync(0xFFFFFFFFu, rms, 0);
    for (int d = lane; d < dim; d += 32) {
        float n = __half2float(x[d]) * rms;
        if (w) n *= w[d];
        x[d] = __float2half(n);
    }
    __syncwarp();
}

__device__ __forceinline__ void rope_head(__half* x, int rotary_dim, int pos, float theta, int lane) {
    const int half_r = rotary_dim / 2;
    if (lane < half_r) {
        const float ex = -(float)(2 * lane) / (float)rotary_dim;
        const float freq = expf(logf(theta) * ex);
        const float ang = (float)pos * freq;
        const float c = cosf(ang), s = sinf(ang);
        const float x0 = __half2float(x[lane]), x1 = __half2float(x[lane + half_r]);
        x[lane] = __float2half(x0 * c - x1 * s);
        x[lane + half_r] = __float2half(x0 * s + x1 * c);
    }
    __syncwarp();
}

__device__ __forceinline__ void copy_head(__half* dst, const __half* src, int dim, int lane) {
    for (int d = lane * 8; d < dim; d += 256)
        *reinterpret_cast<uint4*>(dst + d) = *reinterpret_cast<const uint4*>(src + d);
}

// grid = H_q + H_kv warps (one block of 32 threads each).
__global__ void __launch_bounds__(32)
khq_prestep_kernel(__half* __restrict__ q_gate, __half* __restrict__ k, const __half* __restrict__ v,
                   const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w, __half* __restrict__ ring_k,
                   __half* __restrict__ ring_v, __half* __restrict__ ring_u, int H_q, int d, int rotary_dim, int pos,
                   float theta, float eps, int has_norms) {
    const int h = blockIdx.x, lane = threadIdx.x;
    if (h < H_q) {
        __half* x = q_gate + (size_t)h * 2 * d;
        norm_head(x, has_norms ? q_norm_w : nullptr, d, eps, lane);
        rope_head(x, rotary_dim, pos, theta, lane);
    } else {
        const int g = h - H_q;
        __half* x = k + (size_t)g * d;
        norm_head(x, has_norms ? k_norm_w : nullptr, d, eps, lane);
        if (ring_u) copy_head(ring_u + (size_t)g * d, x, d, lane);
        __syncwarp();
        rope_head(x, rotary_dim, pos, theta, lane);
        if (ring_k) copy_head(ring_k + (size_t)g * d, x, d, lane);
        if (ring_v) copy_head(ring_v + (size_t)g * d, v + (size_t)g * d, d, lane);
    }
}

// The same work for B sequences in one launch: grid = B * (H_q + H_kv) warps.  Sequence b reads
// q_gate + b * 2 * H_q * d, k / v + b * H_kv * d, appends to ring slot slots[b] of its own rings
// (ring base + b * ring_seq_stride halfs) and rotates at position positions[b].
__global__ void __launch_bounds__(32)
khq_prestep_batched_kernel(__half* __restrict__ q_gate, __half* __restrict__ k, const __half* __restrict__ v,
                           const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w,
                           __half* __restrict__ ring_k, __half* __restrict__ ring_v, __half* __restrict__ ring_u,
                           long long ring_seq_stride, const int* __restrict__ slots, const int* __restrict__ positions,
                           int H_q, int H_kv, int d, int rotary_dim, float theta, float eps, int has_norms) {
    const int per = H_q + H_kv;
    const int b = blockIdx.x / per, h = blockIdx.x % per, lane = threadIdx.x;
    const int pos = positions[b];
    if (h < H_q) {
        __half* x = q_gate + ((size_t)b * H_q + h) * 2 * d;
        norm_head(x, has_norms ? q_norm_w : nullptr, d, eps, lane);
        rope_head(x, rotary_dim, pos, theta, lane);
    } else {
        const int g = h - H_q;
        __half* x = k + ((size_t)b * H_kv + g) * d;
        const size_t slot_off = (size_t)b * ring_seq_stride + ((size_t)slots[b] * H_kv + g) * d;
        norm_head(x, has_norms ? k_norm_w : nullptr, d, eps, lane);
        if (ring_u) copy_head(ring_u + slot_off, x, d, lane);
        __syncwarp();
        rope_head(x, rotary_dim, pos, theta, lane);
        if (ring_k) copy_head(ring_k + slot_off, x, d, lane);
        if (ring_v) copy_head(ring_v + slot_off, v + ((size_t)b * H_kv + g) * d, d, lane);
    }
}

}  // namespace khq_prestep

extern "C" int launch_khq_prestep_fp16(void* q_gate, void* k, const void* v, const void* q_norm_w,
                                       const void* k_norm_w, void* ring_k_slot, void* ring_v_slot,
                                       void* ring_u_slot, int H_q, int H_kv, int d, int rotary_dim, int pos,
                                       float rope_theta, float rms_eps, int has_norms, cudaStream_t stream) {
    if (H_q <= 0 || H_kv <= 0 || d <= 0 || !q_gate || !k || !v) return -100;
    if (d % 8 != 0 || rotary_dim <= 0 || rotary_dim > 64 || rotary_dim > d || (rotary_dim & 1)) return -103;
    const void* ptrs[] = {q_gate, k, v, ring_k_slot, ring_v_slot, ring_u_slot};
    for (const void* p : ptrs)
        if ((reinterpret_cast<uintptr_t>(p) & 15) != 0) return -104;
    khq_prestep::khq_prestep_kernel<<<H_q + H_kv, 32, 0, stream>>>(
        static_cast<__half*>(q_gate), static_cast<__half*>(k), static_cast<const __half*>(v),
        static_cast<const float*>(q_norm_w), static_cast<const float*>(k_norm_w), static_cast<__half*>(ring_k_slot),
        static_cast<__half*>(ring_v_slot), static_cast<__half*>(ring_u_slot), H_q, d, rotary_dim, pos, rope_theta,
        rms_eps, has_norms);
    const cudaError_t err = cudaGetLastError();
    return (err == cudaSuccess) ? 0 : static_cast<int>(err);
}

// launch_khq_prestep_fp16 for `batch` sequences at once (no counterpart in the reference, which
// serves one sequence).  slots / positions: device int32 arrays of `batch` entries (ring slot of
// the new token, its absolute position); ring_seq_stride: halfs between two sequences' rings.
extern "C" int launch_khq_prestep_batched_fp16(void* q_gate, void* k, const void* v, const void* q_norm_w,
                                               const void* k_norm_w, void* ring_k, void* ring_v, void* ring_u,
                                               long long ring_seq_stride, const void* slots, const void* positions,
                                               int batch, int H_q, int H_kv, int d, int rotary_dim, float rope_theta,
                                               float rms_eps, int has_norms, cudaStream_t stream) {
    if (batch <= 0 || H_q <= 0 || H_kv <= 0 || d <= 0 || !q_gate || !k || !v || !slots || !positions) return -100;
    if (d % 8 != 0 || rotary_dim <= 0 || rotary_dim > 64 || rotary_dim > d || (rotary_dim & 1)) return -103;
    const void* ptrs[] = {q_gate, k, v, ring_k, ring_v, ring_u};
    for (const void* p : ptrs)
        if ((reinterpret_cast<uintptr_t>(p) & 15) != 0) return -104;
    if ((ring_seq_stride & 7) != 0) return -104;
    khq_prestep::khq_prestep_batched_kernel<<<(unsigned)(batch * (H_q + H_kv)), 32, 0, stream>>>(
        static_cast<__half*>(q_gate), static_cast<__half*>(k), static_cast<const __half*>(v),
        static_cast<const float*>(q_norm_w), static_cast<const float*>(k_norm_w), static_cast<__half*>(ring_k),
        static_cast<__half*>(ring_v), static_cast<__half*>(ring_u), ring_seq_stride, static_cast<const int*>(slots),
        static_cast<const int*>(positions), H_q, H_kv, d, rotary_dim, rope_theta, rms_eps, has_norms);
    const cudaError_t err = cudaGetLastError();
    return (err == cudaSuccess) ? 0 : static_cast<int>(err);
}
