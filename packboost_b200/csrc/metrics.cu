// Per-era Pearson correlation of predictions and targets on the device
// (packboost/booster.py:909-929 computes it with numpy on host copies of both arrays).
//
// Rows are ordered by era, so an era is a contiguous row range.  One CTA per era makes two passes
// over its rows in float64: means first, centred second moments next.  An era is skipped (NaN in
// the output) under the reference's rules: fewer than two rows, a standard deviation of either
// array at or below 1e-12, or a non-finite quotient.  The caller averages the eras that remain.

#include "common.cuh"

namespace pb {

namespace {

constexpr int kCorrThreads = 256;

__device__ __forceinline__ double block_sum(double v, double* scratch) {
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();  // scratch may still be read from the previous call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    double t = 0.0;
    for (int w = 0; w < kCorrThreads / 32; ++w) t += scratch[w];  // same order in every thread
    return t;
}

__global__ void __launch_bounds__(kCorrThreads) era_corr_kernel(const float* __restrict__ y,
                                                                const float* __restrict__ p,
                                                                const int32_t* __restrict__ era_offsets,
                                                                double* __restrict__ corr) {
    __shared__ double scratch[kCorrThreads / 32];
    const int e = blockIdx.x;
    const int r0 = era_offsets[e], r1 = era_offsets[e + 1];
    const int n = r1 - r0;
    if (n < 2) {
        if (threadIdx.x == 0) corr[e] = nan("");
        return;
    }
    double sy = 0.0, sp = 0.0;
    for (int r = r0 + threadIdx.x; r < r1; r += kCorrThreads) {
        sy += (double)y[r];
        sp += (double)p[r];
    }
    const double my = block_sum(sy, scratch) / n;
    const double mp = block_sum(sp, scratch) / n;
    double vyy = 0.0, vpp = 0.0, vyp = 0.0;
    for (int r = r0 + threadIdx.x; r < r1; r += kCorrThreads) {
        const double dy = (double)y[r] - my, dp = (double)p[r] - mp;
        vyy += dy * dy;
        vpp += dp * dp;
        vyp += dy * dp;
    }
    vyy = block_sum(vyy, scratch);
    vpp = block_sum(vpp, scratch);
    vyp = block_sum(vyp, scratch);
    if (threadIdx.x == 0) {
        const double std_y = sqrt(vyy / n), std_p = sqrt(vpp / n);
        double c = nan("");
        if (std_y > 1e-12 && std_p > 1e-12) {
            c = (vyp / n) / (std_y * std_p);
            if (!isfinite(c)) c = nan("");
        }
        corr[e] = c;
    }
}

}  // namespace

}  // namespace pb

extern "C" int pb_era_correlation(const float* y, const float* preds, const int32_t* era_offsets, int64_t n_eras,
                                  double* corr_out, void* stream) {
    PB_REQUIRE(y && preds && era_offsets && corr_out, "null argument");
    PB_REQUIRE(n_eras >= 1 && n_eras <= 32767, "n_eras=%lld outside [1,32767]", (long long)n_eras);
    pb::era_corr_kernel<<<(unsigned)n_eras, pb::kCorrThreads, 0, (cudaStream_t)stream>>>(y, preds, era_offsets,
                                                                                       corr_out);
    pb::count_launch(1);
    PB_LAUNCH_CHECK("era_corr_kernel");
    return PB_OK;
}
