// Float32 arithmetic of the per-era split gain, shared by the scorer kernels and by the
// histogram kernel's fused flush.  Every product, quotient and sum is a separately rounded
// round-to-nearest intrinsic (the compiler never contracts these), in the operation order of
// the tensor code it restates (packboost/booster.py:1828-1883), so that the same integer prefix
// sums give bit-identical gains wherever they are computed.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace pb {

__device__ __forceinline__ float f_add(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float f_sub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float f_mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float f_div(float a, float b) { return __fdiv_rn(a, b); }

// Era totals of one (node, era): float32 gradient total, hessian total (= count: the squared
// loss has unit hessians), the parent term 0.5 * G^2 / (H + lambda) and the era weight
// (packboost/booster.py:815-826: 1 when the era is present, count + alpha with era_alpha > 0).
struct EraTotals {
    uint32_t tc;
    float tg, th, parent, w_era;
};

__device__ __forceinline__ EraTotals era_totals(uint32_t tc, long long tgq, float inv_scale, float lam, float era_alpha) {
    EraTotals t;
    t.tc = tc;
    t.tg = f_mul(__ll2float_rn(tgq), inv_scale);
    t.th = (float)tc;
    t.parent = f_div(f_mul(0.5f, f_mul(t.tg, t.tg)), f_add(t.th, lam));
    t.w_era = (tc == 0) ? 0.f : ((era_alpha > 0.f) ? f_add((float)tc, era_alpha) : 1.f);
    return t;
}

// gain and validity weight of one threshold of one (node, era) from its integer prefix sums
__device__ __forceinline__ float2 gain_of(uint32_t lc, long long lgq, uint32_t tc, float tg, float th, float parent,
                                          float inv_scale, float lam, float w_era) {
    const float lg = f_mul(__ll2float_rn(lgq), inv_scale);
    const float lh = (float)lc;
    const float rg = f_sub(tg, lg);
    const float rh = f_sub(th, lh);
    const float dl = f_add(lh, lam);
    const float dr = f_add(rh, lam);
    const float g2 = f_mul(0.5f, f_add(f_div(f_mul(lg, lg), dl), f_div(f_mul(rg, rg), dr)));
    float2 out;
    out.x = f_sub(g2, parent);
    out.y = ((lc > 0) && (tc - lc > 0)) ? w_era : 0.f;
    return out;
}

// Position of (feature, node, threshold) in the era-summed left-count / left-gradient tables.
// Classic layout (lanes == 0): [feature][node][threshold].  Lane layout (written by the fused
// flush of the lane histogram kernel, where the 32 lanes of a warp hold 32 different features):
// [node][threshold][feature % fpl][feature / fpl], so that the atomics of a warp fall on
// consecutive addresses.
__host__ __device__ __forceinline__ size_t tot_index(int f, int node, int k, int node_stride, int n_thr, int fpl,
                                                     int lanes) {
    if (lanes == 0) return ((size_t)f * node_stride + node) * n_thr + k;
    return (((size_t)node * n_thr + k) * fpl + (f % fpl)) * lanes + (f / fpl);
}

}  // namespace pb
