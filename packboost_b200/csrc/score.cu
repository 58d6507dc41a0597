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
// One CTA handles one feature and a group of frontier nodes.  Eras are processed in chunks:
//   1. threads (or warps, for many bins) scan the bins of (era, node) pairs and leave inclusive
//      prefixes in shared memory,
//   2. all threads evaluate gain and validity weight of (node, era, threshold) triples in
//      parallel; one thread per (node, threshold) accumulates the running weight sum; all
//      threads turn it into the Welford factor w / wsum (the divisions run in parallel),
//   3. one thread per (node, threshold) runs the order-dependent mean / M2 recursion over the
//      chunk's eras (adds and multiplies only), carrying its state to the next chunk.

#include "common.cuh"

namespace pb {

namespace {

constexpr int kScoreThreads = 256;
constexpr int kScoreSmemBudget = 96 * 1024;

struct ScoreKernelArgs {
    ScoreLaunch s;
    int nodes_per_cta;
    int era_chunk;
    int lanes_per_item;  // 1 or 32
};

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

__global__ void __launch_bounds__(kScoreThreads) score_kernel(ScoreKernelArgs a) {
    const ScoreLaunch& s = a.s;
    extern __shared__ unsigned char smem_raw[];
    const int n_nodes = min(*s.n_nodes_ptr, s.n_nodes_max);
    const int node0 = blockIdx.y * a.nodes_per_cta;
    if (node0 >= n_nodes) return;
    const int nn = min(a.nodes_per_cta, n_nodes - node0);
    const int f = blockIdx.x;
    const int E = s.n_eras, NB = s.max_bins, K = s.n_thr, EC = a.era_chunk;
    const float inv_scale = *s.inv_scale_ptr;
    const float lam = s.lambda_l2;
    const bool use_dir = (s.direction_weight != 0.f) && (*s.any_dir_ptr != 0);

    // shared layout: Lg int64 [npc][EC][NB] | res_lg int64 [npc][K] | Lc uint32 [npc][EC][NB]
    //   | gain, weight, factor float [npc][EC][K] each | res_score float [npc][K] | res_cnt uint32 [npc][K]
    const int npc = a.nodes_per_cta;
    long long* Lg = reinterpret_cast<long long*>(smem_raw);
    long long* res_lg = Lg + (size_t)npc * EC * NB;
    uint32_t* Lc = reinterpret_cast<uint32_t*>(res_lg + (size_t)npc * K);
    float* gain = reinterpret_cast<float*>(Lc + (size_t)npc * EC * NB);
    float* wgt = gain + (size_t)npc * EC * K;
    float* fac = wgt + (size_t)npc * EC * K;
    float* res_score = fac + (size_t)npc * EC * K;
    uint32_t* res_cnt = reinterpret_cast<uint32_t*>(res_score + (size_t)npc * K);

    // state of thread (node i, threshold k)
    const int my_i = threadIdx.x / K;
    const int my_k = threadIdx.x - my_i * K;
    const bool scorer = (threadIdx.x < nn * K);
    const int my_t = scorer ? s.thr_ids[my_k] : 0;
    float wsum = 0.f, mean = 0.f, m2 = 0.f, a_num = 0.f, a_den = 0.f;
    long long lc_all = 0, lg_all = 0;
    float pa = 0.f;
    if (scorer && use_dir) {
        const long long g = s.frontier[node0 + my_i].gq;
        pa = (g > 0) ? -1.f : ((g < 0) ? 1.f : 0.f);  // sign(-G/(H+lambda)), H+lambda > 0
    }

    const int G = a.lanes_per_item;  // 1: a thread scans the bins of its (era, node); 32: a warp does
    const unsigned full = 0xFFFFFFFFu;

    for (int e0 = 0; e0 < E; e0 += EC) {
        const int ec = min(EC, E - e0);
        const int n_items = nn * ec;
        // ---- 1. inclusive prefix over bins of each (era, node); items run node-fastest so that
        //         neighbouring threads read neighbouring cells of the [era][node][bin] layout ----
        if (G == 1) {
            for (int it = threadIdx.x; it < n_items; it += kScoreThreads) {
                const int e = it / nn, i = it - e * nn;
                const size_t base = (((size_t)f * E + (e0 + e)) * s.node_stride + node0 + i) * NB;
                uint32_t c = 0;
                long long g = 0;
                for (int b = 0; b < NB; ++b) {
                    c += s.cnt[base + b];
                    g += s.gsum[base + b];
                    Lc[((size_t)i * EC + e) * NB + b] = c;
                    Lg[((size_t)i * EC + e) * NB + b] = g;
                }
            }
        } else {
            const int lane_in = threadIdx.x & 31;
            const int item0 = threadIdx.x >> 5;
            const int item_stride = kScoreThreads >> 5;
            // (every lane of a warp runs the same number of iterations: the shuffles need all of them)
            for (int itb = 0; itb < n_items; itb += item_stride) {
                const bool act = (itb + item0) < n_items;
                const int it = act ? (itb + item0) : 0;
                const int e = it / nn, i = it - e * nn;
                const size_t base = (((size_t)f * E + (e0 + e)) * s.node_stride + node0 + i) * NB;
                uint32_t carry_c = 0;
                long long carry_g = 0;
                for (int b0 = 0; b0 < NB; b0 += 32) {
                    const int b = b0 + lane_in;
                    const bool in = act && (b < NB);
                    uint32_t c = in ? s.cnt[base + b] : 0u;
                    long long g = in ? s.gsum[base + b] : 0ll;
                    for (int d = 1; d < 32; d <<= 1) {
                        const uint32_t c2 = __shfl_up_sync(full, c, d);
                        const long long g2 = __shfl_up_sync(full, g, d);
                        if (lane_in >= d) { c += c2; g += g2; }
                    }
                    c += carry_c;
                    g += carry_g;
                    if (in) {
                        Lc[((size_t)i * EC + e) * NB + b] = c;
                        Lg[((size_t)i * EC + e) * NB + b] = g;
                    }
                    carry_c = __shfl_sync(full, c, 31);
                    carry_g = __shfl_sync(full, g, 31);
                }
            }
        }
        __syncthreads();
        // ---- 2a. gain and validity weight of all (node, era, threshold) triples ----
        for (int it = threadIdx.x; it < nn * ec * K; it += kScoreThreads) {
            const int i = it / (ec * K);
            const int r = it - i * (ec * K);
            const int e = r / K, k = r - e * K;
            const int t = s.thr_ids[k];
            const size_t row = ((size_t)i * EC + e) * NB;
            const uint32_t lc = Lc[row + t], tc = Lc[row + NB - 1];
            const float lg = f_mul(__ll2float_rn(Lg[row + t]), inv_scale);
            const float tg = f_mul(__ll2float_rn(Lg[row + NB - 1]), inv_scale);
            const float lh = (float)lc;
            const float th = (float)tc;
            const float rg = f_sub(tg, lg);
            const float rh = f_sub(th, lh);
            const float dl = f_add(lh, lam);
            const float dr = f_add(rh, lam);
            const float parent = f_div(f_mul(0.5f, f_mul(tg, tg)), f_add(th, lam));
            const float g2 = f_mul(0.5f, f_add(f_div(f_mul(lg, lg), dl), f_div(f_mul(rg, rg), dr)));
            const size_t o = ((size_t)i * EC + e) * K + k;
            gain[o] = f_sub(g2, parent);
            // era weight: 1 (or count + alpha) when the era has rows in this node, masked by validity
            const float w_era = (tc == 0) ? 0.f : ((s.era_alpha > 0.f) ? f_add((float)tc, s.era_alpha) : 1.f);
            wgt[o] = ((lc > 0) && (tc - lc > 0)) ? w_era : 0.f;
        }
        __syncthreads();
        // ---- 2b. running weight sum (sequential, cheap) ----
        if (scorer) {
            float ws = wsum;
            for (int e = 0; e < ec; ++e) {
                const size_t o = ((size_t)my_i * EC + e) * K + my_k;
                ws = f_add(ws, wgt[o]);
                fac[o] = ws;
            }
            wsum = ws;
        }
        __syncthreads();
        // ---- 2c. Welford factor w / wsum_new of every triple, in parallel ----
        for (int it = threadIdx.x; it < nn * ec * K; it += kScoreThreads) {
            const int i = it / (ec * K);
            const int r = it - i * (ec * K);
            const int e = r / K, k = r - e * K;
            const size_t o = ((size_t)i * EC + e) * K + k;
            const float wsn = fac[o];
            fac[o] = (wsn > 0.f) ? f_div(wgt[o], wsn) : 0.f;
        }
        __syncthreads();
        // ---- 3. the order-dependent mean / M2 recursion over the chunk's eras ----
        if (scorer) {
            for (int e = 0; e < ec; ++e) {
                const size_t row = ((size_t)my_i * EC + e) * NB;
                const size_t o = ((size_t)my_i * EC + e) * K + my_k;
                const uint32_t tc = Lc[row + NB - 1];
                if (tc == 0) continue;  // era absent from this node: weight 0, nothing changes
                const float gn = gain[o], w = wgt[o], fc = fac[o];
                const float delta = f_sub(gn, mean);
                mean = f_add(mean, f_mul(fc, delta));
                m2 = f_add(m2, f_mul(f_mul(w, delta), f_sub(gn, mean)));
                const uint32_t lc = Lc[row + my_t];
                const long long lgq = Lg[row + my_t];
                if (use_dir) {
                    const float lg = f_mul(__ll2float_rn(lgq), inv_scale);
                    const float tg = f_mul(__ll2float_rn(Lg[row + NB - 1]), inv_scale);
                    const float lh = (float)lc, th = (float)tc;
                    const float vl = f_div(-lg, f_add(lh, lam));
                    const float vr = f_div(-f_sub(tg, lg), f_add(f_sub(th, lh), lam));
                    const float agree = f_mul(0.5f, f_add((sign_of(vl) == pa) ? 1.f : 0.f,
                                                          (sign_of(vr) == pa) ? 1.f : 0.f));
                    a_num = f_add(a_num, f_mul(w, agree));
                    a_den = f_add(a_den, w);
                }
                lc_all += lc;
                lg_all += lgq;
            }
        }
        __syncthreads();
    }

    // ---- final score, global min_samples_leaf mask ----
    if (scorer) {
        const float ws = (wsum < 1e-12f) ? 1e-12f : wsum;
        float var = f_div(m2, ws);
        if (var < 0.f) var = 0.f;  // NaN stays NaN
        float score = f_sub(mean, f_mul(s.lambda_dro, __fsqrt_rn(var)));
        if (use_dir) {
            const float agr = (a_den > 0.f) ? f_div(a_num, a_den) : 0.f;
            score = f_add(score, f_mul(s.direction_weight, agr));
        }
        const long long total = s.frontier[node0 + my_i].count;
        const bool ok = (lc_all >= s.min_samples_leaf) && (total - lc_all >= s.min_samples_leaf);
        res_score[my_i * K + my_k] = ok ? score : -INFINITY;
        res_cnt[my_i * K + my_k] = (uint32_t)lc_all;
        res_lg[my_i * K + my_k] = lg_all;
    }
    __syncthreads();
    // ---- best threshold of each node: max score, then max left count, then max k ----
    if (threadIdx.x < nn) {
        const int i = threadIdx.x;
        float bs = -INFINITY;
        int64_t bc = -1;
        int bk = -1;
        uint32_t flags = 0;
        for (int k = 0; k < K; ++k) {
            const float sc = res_score[i * K + k];
            if (sc != sc) { flags |= 1u; continue; }
            const uint32_t c = res_cnt[i * K + k];
            if (takes_over(sc, c, bs, bc)) { bs = sc; bc = c; bk = k; }
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

int launch_score(const ScoreLaunch& s, cudaStream_t stream) {
    if (s.n_feat <= 0 || s.n_nodes_max <= 0) return PB_OK;
    const int K = s.n_thr, NB = s.max_bins;
    if (K < 1 || K > kScoreThreads) return fail_arg("n_thresholds=%d outside [1,%d]", K, kScoreThreads);
    ScoreKernelArgs a;
    a.s = s;
    int npc = kScoreThreads / K;
    if (npc > 16) npc = 16;
    if (npc > s.n_nodes_max) npc = s.n_nodes_max;
    if (npc < 1) npc = 1;
    const size_t per_era = (size_t)npc * ((size_t)NB * 12 + (size_t)K * 12);
    const size_t fixed = (size_t)npc * K * 16 + 64;
    int ec = (int)((kScoreSmemBudget - fixed) / per_era);
    if (ec < 1) {
        npc = 1;
        ec = 1;
    }
    if (ec > s.n_eras) ec = s.n_eras;
    a.nodes_per_cta = npc;
    a.era_chunk = ec;
    a.lanes_per_item = (NB <= 8) ? 1 : 32;
    const size_t smem = (size_t)npc * ec * ((size_t)NB * 12 + (size_t)K * 12) + (size_t)npc * K * 16 + 64;
    if (smem > 200 * 1024) return fail_arg("scorer tile does not fit shared memory (bins=%d)", NB);
    if (smem > 48 * 1024)
        PB_CUDA_TRY(cudaFuncSetAttribute(score_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((unsigned)s.n_feat, (unsigned)((s.n_nodes_max + npc - 1) / npc));
    prof_begin(kProfScore, stream);
    score_kernel<<<grid, kScoreThreads, smem, stream>>>(a);
    prof_end(kProfScore, stream);
    count_launch(1);
    PB_LAUNCH_CHECK("score_kernel");
    return PB_OK;
}

}  // namespace pb
