// khq_calib.cu -- the one calibration step the decode path's tables depend on directly: the K-static
// fit (per-dim sigma of the projected sample -> threshold scale ts -> base centroid rows), i.e.
// cal_kstatic_p_kernel + cal_kstatic_f_kernel of the reference (src/csrc/qmv_sm75_kernel.cu:2645-2680,
// launched as op 2 of launch_cal_op, :4634-4643).  The rest of the calibration (PCA rotors, k-means,
// SVQ training) is offline work outside the attention path and is not built.
//
// Same arithmetic in the same order as the reference so that the tables come out bit-identical: per
// dim a serial mean, a serial sum of squared deviations, sigma = sqrt(v / rows); then one serial sum
// of the 256 partial terms, ts = 16 / sqrt(sum), centroid rows {0, -cb, +cb, +cb} with
// cb = 0.9350 * sigma * ts.  One block of 256 threads; nothing is allocated (the reference allocates
// and frees two scratch arrays per call and synchronises the stream).
#include <cuda_runtime.h>

namespace khq_calib {

__global__ void __launch_bounds__(256)
khq_cal_kstatic_kernel(const float* __restrict__ rot, int rows, float* __restrict__ cents, float* __restrict__ out_ts,
                       float* __restrict__ sigma_out) {
    __shared__ float psum[256];
    __shared__ float ts_s;
    const int i = threadIdx.x;
    float m = 0.0f;
    for (int r = 0; r < rows; r++) m += rot[(size_t)r * 256 + i];
    m /= (float)rows;
    float v = 0.0f;
    for (int r = 0; r < rows; r++) {
        float dv = rot[(size_t)r * 256 + i] - m;
        v += dv * dv;
    }
    const float sg = sqrtf(v / (float)rows);
    if (sigma_out) sigma_out[i] = sg;
    const float cb0 = 0.9350f * sg;
    psum[i] = 0.528756f * cb0 * cb0 + 0.464545f * sg * sg;
    __syncthreads();
    if (i == 0) {
        float se = 0.0f;
        for (int k = 0; k < 256; k++) se += psum[k];
        ts_s = 16.0f / sqrtf(se);
        out_ts[0] = ts_s;
    }
    __syncthreads();
    const float cb = 0.9350f * sg * ts_s;
    cents[0 * 256 + i] = 0.0f;
    cents[1 * 256 + i] = -cb;
    cents[2 * 256 + i] = cb;
    cents[3 * 256 + i] = cb;
}

}  // namespace khq_calib

// rot: (rows, 256) fp32 projected sample (device); cents: 4 x 256 fp32 (device); out_ts: 1 fp32
// (device); sigma_out: 256 fp32 (device) or NULL.  Returns -100 on bad arguments.
extern "C" int launch_khq_cal_kstatic_fp32(const void* rot, int rows, void* cents, void* out_ts, void* sigma_out,
                                           cudaStream_t stream) {
    if (!rot || !cents || !out_ts || rows <= 0) return -100;
    khq_calib::khq_cal_kstatic_kernel<<<1, 256, 0, stream>>>(static_cast<const float*>(rot), rows, static_cast<float*>(cents),
                                                             static_cast<float*>(out_ts), static_cast<float*>(sigma_out));
    const cudaError_t err = cudaGetLastError();
    return (err == cudaSuccess) ? 0 : static_cast<int>(err);
}
