// DES scorer: per-era split gains, sequential weighted Welford over eras, mean - lambda*std,
// optional directional agreement, global min-samples mask and the best threshold of every
// (sampled feature, frontier node) pair.
//
// The float32 arithmetic follows the order of the torch frontier it replaces operation by
// operation (every product, quotient and sum is rounded separately: this file is compiled
// with -fmad=false and uses the round-to-nearest intrinsics), so that candidates which
// describe the same partition of the rows receive bit-identical scores and ties resolve the
// same way.  Prefix sums over bins are exact integers; they are converted to float32 once.
//
// Two kernels:
//   gain_kernel   everything that is independent across eras, in parallel over
//                 (feature, era, node): prefix sums over bins, the per-era gain and validity
//                 weight of every threshold (written to a scratch table as float2), and the
//                 era-summed left counts / gradient sums (integer, accumulated per thread and
//                 merged with a few atomics).  A thread keeps one node and strides the eras.
//   chain_kernel  the order-dependent part: one thread per (feature, node, threshold) walks the
//                 eras in ascending order with the weighted Welford recursion, then the score,
//                 the global min_samples_leaf mask and the best threshold of the pair.

#include "common.cuh"

namespace pb {

namespace {

constexpr int kGainThreads = 256;
constexpr int kChainThreads = 256;
constexpr int kSmallBins = 8;

__device__ __forceinline__ float f_add(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float f_sub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float f_mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float f_div(float a, float b) { return __fdiv_rn(a, b); }

__device__ __forceinline__ float sign_of(float v) {
    // torch.sign: -1, 0, +1, NaN stays NaN (compares false to everything)
    if (v > 0.f) return 1.f;
    if (v < 0.f) return -1.f;
    return v;  // +-0 or NaN
}

// (score, left count, position) lexicographic "a is a better or equal-later candidate".
__device__ __forceinline__ bool takes_over(float s, uint32_t c, float bs, int64_t bc) {
    return (s > bs) || (s == bs && (int64_t)c >= bc);
}

struct GainArgs {
    ScoreLaunch s;
    int nodes_per_cta;  // small-bin kernel: power of two <= 32 dividing the block; wide kernel: warps per CTA
    int era_splits;
};

// gain and validity weight of threshold t of one (node, era) from its integer prefix sums
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

// ---- few bins: a thread scans the bins of its (era, node) in registers ---------------------------
__global__ void __launch_bounds__(kGainThreads) gain_kernel_small(GainArgs a) {
    const ScoreLaunch& s = a.s;
    __shared__ uint32_t s_lc[32 * kSmallBins];
    __shared__ unsigned long long s_lg[32 * kSmallBins];
    const int n_nodes = min(*s.n_nodes_ptr, s.n_nodes_max);
    const int npc = a.nodes_per_cta;
    const int node0 = blockIdx.y * npc;
    if (node0 >= n_nodes) return;
    const int f = blockIdx.x;
    const int E = s.n_eras, NB = s.max_bins, K = s.n_thr;
    const float inv_scale = *s.inv_scale_ptr;
    const float lam = s.lambda_l2;
    for (int i = threadIdx.x; i < npc * K; i += kGainThreads) {
        s_lc[i] = 0u;
        s_lg[i] = 0ull;
    }
    __syncthreads();

    const int nl = threadIdx.x % npc;  // node of this thread (fixed)
    const int node = node0 + nl;
    const int e_lane = threadIdx.x / npc;
    const int e_step = kGainThreads / npc;
    const int e_per = (E + a.era_splits - 1) / a.era_splits;
    const int e_begin = blockIdx.z * e_per;
    const int e_end = min(E, e_begin + e_per);
    int thr[kSmallBins];
#pragma unroll
    for (int k = 0; k < kSmallBins; ++k) thr[k] = (k < K) ? s.thr_ids[k] : 0;
    uint32_t lc_sum[kSmallBins];
    long long lg_sum[kSmallBins];
#pragma unroll
    for (int k = 0; k < kSmallBins; ++k) {
        lc_sum[k] = 0u;
        lg_sum[k] = 0ll;
    }

    if (node < n_nodes) {
        for (int e = e_begin + e_lane; e < e_end; e += e_step) {
            const size_t base = (((size_t)f * E + e) * s.node_stride + node) * NB;
            uint32_t pc[kSmallBins];
            long long pg[kSmallBins];
            uint32_t c = 0;
            long long g = 0;
#pragma unroll
            for (int b = 0; b < kSmallBins; ++b) {
                if (b < NB) {
                    c += s.cnt[base + b];
                    g += s.gsum[base + b];
                }
                pc[b] = c;
                pg[b] = g;
            }
            const uint32_t tc = c;
            const float tg = f_mul(__ll2float_rn(g), inv_scale);
            const float th = (float)tc;
            const float parent = f_div(f_mul(0.5f, f_mul(tg, tg)), f_add(th, lam));
            const float w_era = (tc == 0) ? 0.f : ((s.era_alpha > 0.f) ? f_add((float)tc, s.era_alpha) : 1.f);
            float2* out = s.gw + (((size_t)f * E + e) * s.node_stride + node) * K;
#pragma unroll
            for (int k = 0; k < kSmallBins; ++k) {
                if (k < K) {
                    uint32_t lc = 0;
                    long long lgq = 0;
#pragma unroll
                    for (int b = 0; b < kSmallBins; ++b)
                        if (b == thr[k]) {
                            lc = pc[b];
                            lgq = pg[b];
                        }
                    out[k] = gain_of(lc, lgq, tc, tg, th, parent, inv_scale, lam, w_era);
                    lc_sum[k] += lc;
                    lg_sum[k] += lgq;
                }
            }
        }
#pragma unroll
        for (int k = 0; k < kSmallBins; ++k) {
            if (k < K) {
                if (lc_sum[k]) atomicAdd(&s_lc[nl * K + k], lc_sum[k]);
                if (lg_sum[k]) atomicAdd(&s_lg[nl * K + k], (unsigned long long)lg_sum[k]);
            }
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < npc * K; i += kGainThreads) {
        const int n = node0 + i / K, k = i - (i / K) * K;
        if (n < n_nodes) {
            const size_t o = ((size_t)f * s.node_stride + n) * K + k;
            if (s_lc[i]) atomicAdd(s.lc_tot + o, s_lc[i]);
            if (s_lg[i]) atomicAdd(reinterpret_cast<unsigned long long*>(s.lg_tot + o), s_lg[i]);
        }
    }
}

// ---- many bins: a warp scans the bins of its (era, node); lane l owns bins l, l+32, ... ----------
__global__ void __launch_bounds__(kGainThreads) gain_kernel_wide(GainArgs a) {
    const ScoreLaunch& s = a.s;
    __shared__ int s_kof[256];  // threshold index of a bin, -1 when the bin is not a threshold
    const int n_nodes = min(*s.n_nodes_ptr, s.n_nodes_max);
    const int warps = kGainThreads / 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int node = blockIdx.y * warps + warp;
    const int f = blockIdx.x;
    const int E = s.n_eras, NB = s.max_bins, K = s.n_thr;
    for (int i = threadIdx.x; i < 256; i += kGainThreads) s_kof[i] = -1;
    __syncthreads();
    for (int k = threadIdx.x; k < K; k += kGainThreads) s_kof[s.thr_ids[k]] = k;
    __syncthreads();
    if (node >= n_nodes) return;
    const float inv_scale = *s.inv_scale_ptr;
    const float lam = s.lambda_l2;
    const int e_per = (E + a.era_splits - 1) / a.era_splits;
    const int e_begin = blockIdx.z * e_per;
    const int e_end = min(E, e_begin + e_per);
    const unsigned full = 0xFFFFFFFFu;
    const int iters = (NB + 31) / 32;  // <= 8
    uint32_t lc_sum[8];
    long long lg_sum[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        lc_sum[i] = 0u;
        lg_sum[i] = 0ll;
    }

    for (int e = e_begin; e < e_end; ++e) {
        const size_t base = (((size_t)f * E + e) * s.node_stride + node) * NB;
        uint32_t pc[8];
        long long pg[8];
        uint32_t carry_c = 0;
        long long carry_g = 0;
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            if (it < iters) {
                const int b = it * 32 + lane;
                uint32_t c = (b < NB) ? s.cnt[base + b] : 0u;
                long long g = (b < NB) ? s.gsum[base + b] : 0ll;
                for (int d = 1; d < 32; d <<= 1) {
                    const uint32_t c2 = __shfl_up_sync(full, c, d);
                    const long long g2 = __shfl_up_sync(full, g, d);
                    if (lane >= d) {
                        c += c2;
                        g += g2;
                    }
                }
                c += carry_c;
                g += carry_g;
                pc[it] = c;
                pg[it] = g;
                carry_c = __shfl_sync(full, c, 31);
                carry_g = __shfl_sync(full, g, 31);
            }
        }
        const uint32_t tc = carry_c;  // bins past NB add nothing: the carry is the era total
        const float tg = f_mul(__ll2float_rn(carry_g), inv_scale);
        const float th = (float)tc;
        const float parent = f_div(f_mul(0.5f, f_mul(tg, tg)), f_add(th, lam));
        const float w_era = (tc == 0) ? 0.f : ((s.era_alpha > 0.f) ? f_add((float)tc, s.era_alpha) : 1.f);
        float2* out = s.gw + (((size_t)f * E + e) * s.node_stride + node) * K;
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            if (it < iters) {
                const int b = it * 32 + lane;
                const int k = (b < NB) ? s_kof[b] : -1;
                if (k >= 0) {
                    out[k] = gain_of(pc[it], pg[it], tc, tg, th, parent, inv_scale, lam, w_era);
                    lc_sum[it] += pc[it];
                    lg_sum[it] += pg[it];
                }
            }
        }
    }
#pragma unroll
    for (int it = 0; it < 8; ++it) {
        if (it < iters) {
            const int b = it * 32 + lane;
            const int k = (b < NB) ? s_kof[b] : -1;
            if (k >= 0) {
                const size_t o = ((size_t)f * s.node_stride + node) * K + k;
                if (lc_sum[it]) atomicAdd(s.lc_tot + o, lc_sum[it]);
                if (lg_sum[it])
                    atomicAdd(reinterpret_cast<unsigned long long*>(s.lg_tot + o), (unsigned long long)lg_sum[it]);
            }
        }
    }
}

// ---- the era recursion -----------------------------------------------------------------------------
struct ChainArgs {
    ScoreLaunch s;
    int nodes_per_cta;
    int unit_weights;  // 1: era weights are 0/1 and n_eras fits the reciprocal table
};

constexpr int kInvTable = 4096;

__device__ __forceinline__ void welford_step(float gn, float w, float& wsum, float& mean, float& m2) {
    const float wsum_new = f_add(wsum, w);
    const float factor = (wsum_new > 0.f) ? f_div(w, wsum_new) : 0.f;
    const float delta = f_sub(gn, mean);
    mean = f_add(mean, f_mul(factor, delta));
    m2 = f_add(m2, f_mul(f_mul(w, delta), f_sub(gn, mean)));
    wsum = wsum_new;
}

__global__ void __launch_bounds__(kChainThreads) chain_kernel(ChainArgs a) {
    const ScoreLaunch& s = a.s;
    extern __shared__ unsigned char smem_raw[];
    const int n_nodes = min(*s.n_nodes_ptr, s.n_nodes_max);
    const int npc = a.nodes_per_cta;
    const int node0 = blockIdx.y * npc;
    if (node0 >= n_nodes) return;
    const int nn = min(npc, n_nodes - node0);
    const int f = blockIdx.x;
    const int E = s.n_eras, K = s.n_thr;
    const float lam = s.lambda_l2;
    const bool use_dir = (s.direction_weight != 0.f) && (*s.any_dir_ptr != 0);

    long long* res_lg = reinterpret_cast<long long*>(smem_raw);
    float* res_score = reinterpret_cast<float*>(res_lg + (size_t)npc * K);
    uint32_t* res_cnt = reinterpret_cast<uint32_t*>(res_score + (size_t)npc * K);
    float* s_inv = reinterpret_cast<float*>(res_cnt + (size_t)npc * K);  // s_inv[n] = 1/n, n <= n_eras
    if (a.unit_weights) {
        for (int n = threadIdx.x; n <= E; n += blockDim.x) s_inv[n] = (n > 0) ? f_div(1.f, (float)n) : 0.f;
        __syncthreads();
    }

    const int my_i = threadIdx.x / K;
    const int my_k = threadIdx.x - my_i * K;
    const bool scorer = (threadIdx.x < nn * K);
    if (scorer) {
        const int node = node0 + my_i;
        float wsum = 0.f, mean = 0.f, m2 = 0.f, a_num = 0.f, a_den = 0.f;
        const float2* gw = s.gw + ((size_t)f * E * s.node_stride + node) * K + my_k;
        const size_t e_stride = (size_t)s.node_stride * K;
        if (!use_dir && a.unit_weights) {
            // Every era weight is 0 or 1 (era_alpha == 0), so the running weight sum is a small
            // integer n and the Welford factor w / n is either 0 or the correctly rounded 1 / n,
            // which is read from a table built once per CTA: no division on the recursion.
            constexpr int kChunk = 16;
            float2 cur[kChunk], nxt[kChunk];
#pragma unroll
            for (int q = 0; q < kChunk; ++q)
                cur[q] = (q < E) ? gw[(size_t)q * e_stride] : make_float2(0.f, 0.f);
            int n_valid = 0;
            for (int e = 0; e < E; e += kChunk) {
#pragma unroll
                for (int q = 0; q < kChunk; ++q) {
                    const int en = e + kChunk + q;
                    nxt[q] = (en < E) ? gw[(size_t)en * e_stride] : make_float2(0.f, 0.f);
                }
#pragma unroll
                for (int q = 0; q < kChunk; ++q) {
                    const float gn = cur[q].x, w = cur[q].y;
                    const bool on = w > 0.f;
                    n_valid += on ? 1 : 0;
                    const float fac = on ? s_inv[n_valid] : 0.f;
                    const float delta = f_sub(gn, mean);
                    mean = f_add(mean, f_mul(fac, delta));
                    m2 = f_add(m2, f_mul(f_mul(w, delta), f_sub(gn, mean)));
                }
#pragma unroll
                for (int q = 0; q < kChunk; ++q) cur[q] = nxt[q];
            }
            wsum = (float)n_valid;
        } else if (!use_dir) {
            // Chunks of kChunk eras: the running weight sums are a short dependent chain of adds,
            // the kChunk divisions w / wsum are independent of each other (the scheduler overlaps
            // them), and only the mean / M2 updates form the long dependent chain.  The next
            // chunk's table entries are loaded while the current one is processed.
            constexpr int kChunk = 16;
            float2 cur[kChunk], nxt[kChunk];
#pragma unroll
            for (int q = 0; q < kChunk; ++q)
                cur[q] = (q < E) ? gw[(size_t)q * e_stride] : make_float2(0.f, 0.f);
            for (int e = 0; e < E; e += kChunk) {
#pragma unroll
                for (int q = 0; q < kChunk; ++q) {
                    const int en = e + kChunk + q;
                    nxt[q] = (en < E) ? gw[(size_t)en * e_stride] : make_float2(0.f, 0.f);
                }
                float wsn[kChunk], fac[kChunk];
                float ws = wsum;
#pragma unroll
                for (int q = 0; q < kChunk; ++q) {
                    ws = f_add(ws, cur[q].y);
                    wsn[q] = ws;
                }
                wsum = ws;
#pragma unroll
                for (int q = 0; q < kChunk; ++q) fac[q] = (wsn[q] > 0.f) ? f_div(cur[q].y, wsn[q]) : 0.f;
#pragma unroll
                for (int q = 0; q < kChunk; ++q) {
                    // entries past the last era carry weight 0 and gain 0: they leave the state unchanged
                    const float gn = cur[q].x, w = cur[q].y;
                    const float delta = f_sub(gn, mean);
                    mean = f_add(mean, f_mul(fac[q], delta));
                    m2 = f_add(m2, f_mul(f_mul(w, delta), f_sub(gn, mean)));
                }
#pragma unroll
                for (int q = 0; q < kChunk; ++q) cur[q] = nxt[q];
            }
        } else {
            // directional agreement needs the per-era left / right leaf directions: recompute them
            // from the histogram prefix of this threshold
            const long long gpar = s.frontier[node].gq;
            const float pa = (gpar > 0) ? -1.f : ((gpar < 0) ? 1.f : 0.f);  // sign(-G/(H+lambda)), H+lambda > 0
            const float inv_scale = *s.inv_scale_ptr;
            const int NB = s.max_bins;
            const int t = s.thr_ids[my_k];
            for (int e = 0; e < E; ++e) {
                const float2 v = gw[(size_t)e * e_stride];
                const float w = v.y;
                welford_step(v.x, w, wsum, mean, m2);
                const size_t base = (((size_t)f * E + e) * s.node_stride + node) * NB;
                uint32_t lc = 0, tc = 0;
                long long lgq = 0, tgq = 0;
                for (int b = 0; b < NB; ++b) {
                    const uint32_t cc = s.cnt[base + b];
                    const long long gg = s.gsum[base + b];
                    tc += cc;
                    tgq += gg;
                    if (b <= t) {
                        lc += cc;
                        lgq += gg;
                    }
                }
                if (tc == 0) continue;
                const float lg = f_mul(__ll2float_rn(lgq), inv_scale);
                const float tg = f_mul(__ll2float_rn(tgq), inv_scale);
                const float lh = (float)lc, th = (float)tc;
                const float vl = f_div(-lg, f_add(lh, lam));
                const float vr = f_div(-f_sub(tg, lg), f_add(f_sub(th, lh), lam));
                const float agree =
                    f_mul(0.5f, f_add((sign_of(vl) == pa) ? 1.f : 0.f, (sign_of(vr) == pa) ? 1.f : 0.f));
                a_num = f_add(a_num, f_mul(w, agree));
                a_den = f_add(a_den, w);
            }
        }
        // final score, global min_samples_leaf mask
        const float ws = (wsum < 1e-12f) ? 1e-12f : wsum;
        float var = f_div(m2, ws);
        if (var < 0.f) var = 0.f;  // NaN stays NaN
        float score = f_sub(mean, f_mul(s.lambda_dro, __fsqrt_rn(var)));
        if (use_dir) {
            const float agr = (a_den > 0.f) ? f_div(a_num, a_den) : 0.f;
            score = f_add(score, f_mul(s.direction_weight, agr));
        }
        const size_t o = ((size_t)f * s.node_stride + node) * K + my_k;
        const long long lc_all = s.lc_tot[o];
        const long long total = s.frontier[node].count;
        const bool ok = (lc_all >= s.min_samples_leaf) && (total - lc_all >= s.min_samples_leaf);
        res_score[my_i * K + my_k] = ok ? score : -INFINITY;
        res_cnt[my_i * K + my_k] = (uint32_t)lc_all;
        res_lg[my_i * K + my_k] = s.lg_tot[o];
    }
    __syncthreads();
    // best threshold of each node: max score, then max left count, then max k
    if (threadIdx.x < nn) {
        const int i = threadIdx.x;
        float bs = -INFINITY;
        int64_t bc = -1;
        int bk = -1;
        uint32_t flags = 0;
        for (int k = 0; k < K; ++k) {
            const float sc = res_score[i * K + k];
            if (sc != sc) {
                flags |= 1u;
                continue;
            }
            const uint32_t c = res_cnt[i * K + k];
            if (takes_over(sc, c, bs, bc)) {
                bs = sc;
                bc = c;
                bk = k;
            }
        }
        Cand out;
        out.score = bs;
        out.k = bk;
        out.left_count = (bk >= 0) ? (uint32_t)bc : 0u;
        out.flags = flags;
        out.left_gq = (bk >= 0) ? res_lg[i * K + bk] : 0ll;
        s.cand[(size_t)s.feat_pos[f] * s.node_stride + node0 + i] = out;
    }
}

}  // namespace

size_t score_scratch_bytes_per_feature(int node_stride, int n_eras, int n_thr) {
    return (size_t)node_stride * n_eras * n_thr * sizeof(float2) + (size_t)node_stride * n_thr * 12;
}

int launch_score(const ScoreLaunch& s, cudaStream_t stream) {
    if (s.n_feat <= 0 || s.n_nodes_max <= 0) return PB_OK;
    const int K = s.n_thr, NB = s.max_bins;
    if (K < 1 || K > kChainThreads) return fail_arg("n_thresholds=%d outside [1,%d]", K, kChainThreads);
    if (!s.gw || !s.lc_tot || !s.lg_tot) return fail_arg("scorer scratch is null");
    const size_t tot_cells = (size_t)s.n_feat * s.node_stride * K;
    PB_CUDA_TRY(cudaMemsetAsync(s.lc_tot, 0, tot_cells * sizeof(uint32_t), stream));
    PB_CUDA_TRY(cudaMemsetAsync(s.lg_tot, 0, tot_cells * sizeof(int64_t), stream));

    prof_begin(kProfScore, stream);
    GainArgs g;
    g.s = s;
    if (NB <= kSmallBins) {
        int npc = 1;
        while (npc < 32 && npc < s.n_nodes_max) npc *= 2;
        g.nodes_per_cta = npc;
        const int groups = (s.n_nodes_max + npc - 1) / npc;
        int splits = (600 + s.n_feat * groups - 1) / (s.n_feat * groups);
        const int max_splits = (s.n_eras * npc + kGainThreads - 1) / kGainThreads;
        if (splits > max_splits) splits = max_splits;
        if (splits < 1) splits = 1;
        g.era_splits = splits;
        dim3 grid((unsigned)s.n_feat, (unsigned)groups, (unsigned)splits);
        if (grid.y > 65535u) return fail_arg("scorer grid too large");
        gain_kernel_small<<<grid, kGainThreads, 0, stream>>>(g);
    } else {
        const int warps = kGainThreads / 32;
        const int groups = (s.n_nodes_max + warps - 1) / warps;
        int splits = (1200 + s.n_feat * groups - 1) / (s.n_feat * groups);
        if (splits > s.n_eras) splits = s.n_eras;
        if (splits < 1) splits = 1;
        g.nodes_per_cta = warps;
        g.era_splits = splits;
        dim3 grid((unsigned)s.n_feat, (unsigned)groups, (unsigned)splits);
        if (grid.y > 65535u) return fail_arg("scorer grid too large");
        gain_kernel_wide<<<grid, kGainThreads, 0, stream>>>(g);
    }
    PB_LAUNCH_CHECK("gain_kernel");

    ChainArgs c;
    c.s = s;
    int npc = kChainThreads / K;
    if (npc < 1) npc = 1;
    if (npc > s.n_nodes_max) npc = s.n_nodes_max;
    c.nodes_per_cta = npc;
    c.unit_weights = (s.era_alpha <= 0.f && s.n_eras < kInvTable) ? 1 : 0;
    const size_t smem = (size_t)npc * K * 16 + (c.unit_weights ? (size_t)(s.n_eras + 1) * 4 : 0);
    dim3 grid((unsigned)s.n_feat, (unsigned)((s.n_nodes_max + npc - 1) / npc));
    if (grid.y > 65535u) return fail_arg("scorer grid too large");
    const int threads = ((npc * K + 31) / 32) * 32;
    chain_kernel<<<grid, threads, smem, stream>>>(c);
    prof_end(kProfScore, stream);
    count_launch(2);
    PB_LAUNCH_CHECK("chain_kernel");
    return PB_OK;
}

}  // namespace pb
