// khq_common.cuh -- shared constants and device helpers for the sm_100a KHQ kernels.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace khq {

constexpr int D = 256;          // head_dim
constexpr int NP = 64;          // 4-dim patches per row
constexpr int HKV = 4;          // kv heads
constexpr int NREP = 6;         // query heads per kv head
constexpr int HQ = HKV * NREP;  // 24
constexpr int K_PAY = 40;       // bytes per K payload row
constexpr int V_PAY = 104;      // bytes per V payload row
constexpr int MAX_OUT = 50;     // outliers kept per K row
constexpr int PART = D + 2;     // floats per partial: acc[D], max, sum_exp
constexpr float NEG_BIG = -1e20f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier + 1-D bulk asynchronous copy (global -> shared), no multicast ----------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count)
                 : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after ~2^22 polls, records it in *status and returns false.  The
// caller carries on (its result is then meaningless, and the host can see why) instead of
// spinning for ever.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, int* status) {
    for (uint32_t it = 0; it < (1u << 22); ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if (it > 64) __nanosleep(32);
    }
    atomicExch(status, 1);
    return false;
}
// size must be a multiple of 16; both addresses 16-byte aligned.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes,
                                         uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
            "r"(smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// ---- small math helpers ---------------------------------------------------------------------
__device__ __forceinline__ float h2f(__half h) { return __half2float(h); }
__device__ __forceinline__ float hbits2f(uint16_t b) { return __half2float(__ushort_as_half(b)); }

// In-lane part of the unnormalised natural-order FWHT-256 when a lane holds the 8 consecutive
// elements 8*lane..8*lane+7 (stages 1, 2, 4), followed by the cross-lane stages 8..128.
// Each butterfly computes a+b and a-b exactly as a sequential implementation does.
__device__ __forceinline__ void fwht256_lane8(float (&v)[8], int lane) {
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
        float a = v[j], b = v[j + 1];
        v[j] = a + b;
        v[j + 1] = a - b;
    }
#pragma unroll
    for (int b4 = 0; b4 < 8; b4 += 4)
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            float a = v[b4 + k], b = v[b4 + k + 2];
            v[b4 + k] = a + b;
            v[b4 + k + 2] = a - b;
        }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float a = v[j], b = v[j + 4];
        v[j] = a + b;
        v[j + 4] = a - b;
    }
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
        const bool lower = (lane & m) == 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float other = __shfl_xor_sync(0xFFFFFFFFu, v[j], m);
            v[j] = lower ? (v[j] + other) : (other - v[j]);
        }
    }
}

// Online-softmax state of one query head held redundantly by every lane of a warp.
struct Softmax {
    float m, l;
};

}  // namespace khq
