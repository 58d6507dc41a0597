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
#include "des_math.cuh"

namespace pb {

namespace {

constexpr int kGainThreads = 256;
constexpr int kChainThreads = 256;
constexpr int kSmallBins = 8;

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

// ---- few bins: a thread scans the bins of its (era, node) in registers ---------------------------
template <int KT, int NBT>  // compile-time bounds of the threshold count and of the bin count
__global__ void __launch_bounds__(kGainThreads, (KT <= 4 && NBT <= 5) ? 3 : 2) gain_kernel_small(GainArgs a) {
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
    int thr[KT];
#pragma unroll
    const int32_t* thr_list = s.thr_ids + (s.thr_per_feature ? (size_t)f * K : 0);
#pragma unroll
    for (int k = 0; k < KT; ++k) thr[k] = (k < K) ? thr_list[k] : 0;
    uint32_t lc_sum[KT];
    long long lg_sum[KT];
#pragma unroll
    for (int k = 0; k < KT; ++k) {
        lc_sum[k] = 0u;
        lg_sum[k] = 0ll;
    }

    if (node < n_nodes) {
        // The histogram row of the next era is loaded while the current one is worked on: the rows
        // come from HBM and a thread has little else to overlap their latency with.
        uint32_t hc[NBT], hc_next[NBT];
        long long hg[NBT], hg_next[NBT];
        auto load_row = [&](int e, uint32_t (&rc)[NBT], long long (&rg)[NBT]) {
            const size_t base = (((size_t)f * E + e) * s.node_stride + node) * NB;
#pragma unroll
            for (int b = 0; b < NBT; ++b) {
                rc[b] = (b < NB) ? s.cnt[base + b] : 0u;
                rg[b] = (b < NB) ? s.gsum[base + b] : 0ll;
            }
        };
        if (e_begin + e_lane < e_end) load_row(e_begin + e_lane, hc, hg);
        for (int e = e_begin + e_lane; e < e_end; e += e_step) {
            if (e + e_step < e_end) load_row(e + e_step, hc_next, hg_next);
            // running prefix over the bins; threshold k keeps the prefix at its bin (selects with
            // static indices, so everything stays in registers)
            uint32_t lcs[KT];
            long long lgs[KT];
#pragma unroll
            for (int k = 0; k < KT; ++k) {
                lcs[k] = 0u;
                lgs[k] = 0ll;
            }
            uint32_t c = 0;
            long long g = 0;
#pragma unroll
            for (int b = 0; b < NBT; ++b) {
                if (b < NB) {
                    c += hc[b];
                    g += hg[b];
#pragma unroll
                    for (int k = 0; k < KT; ++k) {
                        const bool at = (k < K) && (thr[k] == b);
                        lcs[k] = at ? c : lcs[k];
                        lgs[k] = at ? g : lgs[k];
                    }
                }
            }
            const uint32_t tc = c;
            const float tg = f_mul(__ll2float_rn(g), inv_scale);
            const float th = (float)tc;
            const float parent = f_div(f_mul(0.5f, f_mul(tg, tg)), f_add(th, lam));
            const float w_era = (tc == 0) ? 0.f : ((s.era_alpha > 0.f) ? f_add((float)tc, s.era_alpha) : 1.f);
            float2* out = s.gw + (((size_t)f * E + e) * s.node_stride + node) * K;
            float2 gk[KT];
#pragma unroll
            for (int k = 0; k < KT; ++k) {
                if (k < K) {
                    const uint32_t lc = lcs[k];
                    const long long lgq = lgs[k];
                    gk[k] = gain_of(lc, lgq, tc, tg, th, parent, inv_scale, lam, w_era);
                    lc_sum[k] += lc;
                    lg_sum[k] += lgq;
                }
            }
            if ((K & 1) == 0) {  // rows of an even K start on 16 bytes
#pragma unroll
                for (int k = 0; k < KT; k += 2)
                    if (k < K)
                        reinterpret_cast<float4*>(out)[k >> 1] = make_float4(gk[k].x, gk[k].y, gk[k + 1].x, gk[k + 1].y);
            } else {
#pragma unroll
                for (int k = 0; k < KT; ++k)
                    if (k < K) out[k] = gk[k];
            }
#pragma unroll
            for (int b = 0; b < NBT; ++b) {
                hc[b] = hc_next[b];
                hg[b] = hg_next[b];
            }
        }
    }
    // threads of a warp that share a node (lanes a multiple of npc apart) are summed with shuffles
    // first, so that only npc lanes per warp touch the shared accumulators
#pragma unroll
    for (int k = 0; k < KT; ++k) {
        if (k < K) {
            uint32_t c = lc_sum[k];
            long long g = lg_sum[k];
            for (int off = 16; off >= npc; off >>= 1) {
                c += __shfl_xor_sync(0xFFFFFFFFu, c, off);
                g += __shfl_xor_sync(0xFFFFFFFFu, g, off);
            }
            if ((threadIdx.x & 31) < npc) {
                if (c) atomicAdd(&s_lc[nl * K + k], c);
                if (g) atomicAdd(&s_lg[nl * K + k], (unsigned long long)g);
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
    const int32_t* thr_list = s.thr_ids + (s.thr_per_feature ? (size_t)f * K : 0);
    for (int k = threadIdx.x; k < K; k += kGainThreads) s_kof[thr_list[k]] = k;
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

    // the histogram row of the next era is loaded while the current one is scanned and scored
    uint32_t rc[8], rc_next[8];
    long long rg[8], rg_next[8];
    auto load_row = [&](int e, uint32_t (&oc)[8], long long (&og)[8]) {
        const size_t base = (((size_t)f * E + e) * s.node_stride + node) * NB;
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int b = it * 32 + lane;
            const bool in = (it < iters) && (b < NB);
            oc[it] = in ? s.cnt[base + b] : 0u;
            og[it] = in ? s.gsum[base + b] : 0ll;
        }
    };
    if (e_begin < e_end) load_row(e_begin, rc, rg);
    for (int e = e_begin; e < e_end; ++e) {
        if (e + 1 < e_end) load_row(e + 1, rc_next, rg_next);
        uint32_t pc[8];
        long long pg[8];
        uint32_t carry_c = 0;
        long long carry_g = 0;
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            if (it < iters) {
                uint32_t c = rc[it];
                long long g = rg[it];
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
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            rc[it] = rc_next[it];
            rg[it] = rg_next[it];
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
    int era_chunk;     // eras per staged chunk of the (gain, weight) table
    int slot_pow2;     // unit kernel with fewer than 32 slots per CTA: slots rounded up to a power of two, else 0
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

__device__ __forceinline__ void cp_async8(void* smem_dst, const void* gmem_src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// Final score of every (node, threshold) slot of a CTA, the global min_samples_leaf mask and the
// best threshold of each node (max score, then max left count, then max k).  Called by all
// threads of the CTA; slot threads are the first nn * K.
__device__ __forceinline__ void finish_pairs(const ScoreLaunch& s, int f, int node0, int nn, bool scorer, int my_i,
                                             int my_k, float wsum, float mean, float m2, bool use_dir, float a_num,
                                             float a_den, float* res_score, uint32_t* res_cnt, long long* res_lg) {
    const int K = s.n_thr;
    const int node = node0 + (scorer ? my_i : 0);
    if (scorer) {
        const float ws = (wsum < 1e-12f) ? 1e-12f : wsum;
        float var = f_div(m2, ws);
        if (var < 0.f) var = 0.f;  // NaN stays NaN
        float score = f_sub(mean, f_mul(s.lambda_dro, __fsqrt_rn(var)));
        if (use_dir) {
            const float agr = (a_den > 0.f) ? f_div(a_num, a_den) : 0.f;
            score = f_add(score, f_mul(s.direction_weight, agr));
        }
        const size_t o = tot_index(f, node, my_k, s.node_stride, K, s.tot_fpl, s.tot_lanes);
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
        // the bin id of the chosen threshold travels with the candidate (the lists may differ per feature)
        const int thr_bin = (bk >= 0) ? s.thr_ids[(s.thr_per_feature ? (size_t)f * K : 0) + bk] : 0;
        out.flags = flags | ((uint32_t)thr_bin << 8);
        out.left_gq = (bk >= 0) ? res_lg[i * K + bk] : 0ll;
        s.cand[(size_t)s.feat_pos[f] * s.node_stride + node0 + i] = out;
    }
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
    // (the parent-agreement form drops the term when no frontier node has a direction at all; the
    // comparing form depends on the children only)
    const bool use_dir = (s.direction_weight != 0.f) && (s.direction_form == 1 || *s.any_dir_ptr != 0);

    // shared layout: res_lg int64 [npc*K] | staged table float2 [2][EC][npc*K] | res_score, res_cnt
    const int npck = npc * K;
    const int EC = a.era_chunk;
    long long* res_lg = reinterpret_cast<long long*>(smem_raw);
    float2* s_gw = reinterpret_cast<float2*>(res_lg + npck);
    float* res_score = reinterpret_cast<float*>(s_gw + (size_t)2 * EC * npck);
    uint32_t* res_cnt = reinterpret_cast<uint32_t*>(res_score + npck);

    const int my_i = threadIdx.x / K;
    const int my_k = threadIdx.x - my_i * K;
    const int slots = nn * K;
    const bool scorer = (threadIdx.x < slots);
    const int node = node0 + (scorer ? my_i : 0);
    float wsum = 0.f, mean = 0.f, m2 = 0.f, a_num = 0.f, a_den = 0.f;
    const float2* gw_cta = s.gw + ((size_t)f * E * s.node_stride + node0) * K;  // + e * e_stride + slot
    const size_t e_stride = (size_t)s.node_stride * K;

    if (!use_dir) {
        // The (gain, weight) table of this CTA is streamed through shared memory in chunks of EC
        // eras with asynchronous copies, the next chunk in flight while the current one is walked;
        // only the mean / M2 updates form the long dependent chain.
        auto prefetch = [&](int c) {
            const int e0 = c * EC, ec = min(EC, E - e0);
            float2* dst = s_gw + (size_t)(c & 1) * EC * npck;
            for (int i = threadIdx.x; i < ec * slots; i += blockDim.x) {
                const int e = i / slots, j = i - e * slots;
                cp_async8(dst + (size_t)e * npck + j, gw_cta + (size_t)(e0 + e) * e_stride + j);
            }
            cp_async_commit();
        };
        const int n_chunks = (E + EC - 1) / EC;
        prefetch(0);
        for (int c = 0; c < n_chunks; ++c) {
            if (c + 1 < n_chunks) {
                prefetch(c + 1);
                cp_async_wait<1>();
            } else {
                cp_async_wait<0>();
            }
            __syncthreads();
            if (scorer) {
                const int ec = min(EC, E - c * EC);
                const float2* src = s_gw + (size_t)(c & 1) * EC * npck + threadIdx.x;
                {
                    constexpr int kSub = 8;  // the kSub divisions of a sub-chunk are independent
                    for (int e0 = 0; e0 < ec; e0 += kSub) {
                        float2 v[kSub];
                        float fac[kSub];
                        float ws = wsum;
#pragma unroll
                        for (int q = 0; q < kSub; ++q) {
                            v[q] = (e0 + q < ec) ? src[(size_t)(e0 + q) * npck] : make_float2(0.f, 0.f);
                            ws = f_add(ws, v[q].y);
                            fac[q] = ws;
                        }
                        wsum = ws;
#pragma unroll
                        for (int q = 0; q < kSub; ++q) fac[q] = (fac[q] > 0.f) ? f_div(v[q].y, fac[q]) : 0.f;
#pragma unroll
                        for (int q = 0; q < kSub; ++q) {
                            // padding entries carry weight 0 and gain 0: they leave the state unchanged
                            const float delta = f_sub(v[q].x, mean);
                            mean = f_add(mean, f_mul(fac[q], delta));
                            m2 = f_add(m2, f_mul(f_mul(v[q].y, delta), f_sub(v[q].x, mean)));
                        }
                    }
                }
            }
            __syncthreads();
        }
    } else {
        __syncthreads();
        if (scorer) {
            // directional agreement needs the per-era left / right leaf directions: recompute them
            // from the histogram prefix of this threshold
            const float2* gw = gw_cta + threadIdx.x;
            const long long gpar = s.frontier[node].gq;
            const float pa = (gpar > 0) ? -1.f : ((gpar < 0) ? 1.f : 0.f);  // sign(-G/(H+lambda)), H+lambda > 0
            const float inv_scale = *s.inv_scale_ptr;
            const int NB = s.max_bins;
            const int t = s.thr_ids[(s.thr_per_feature ? (size_t)f * K : 0) + my_k];
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
                const float agree = (s.direction_form == 1)
                    ? ((vl > vr) ? 1.f : -1.f)
                    : f_mul(0.5f, f_add((sign_of(vl) == pa) ? 1.f : 0.f, (sign_of(vr) == pa) ? 1.f : 0.f));
                a_num = f_add(a_num, f_mul(w, agree));
                a_den = f_add(a_den, w);
            }
        }
    }

    finish_pairs(s, f, node0, nn, scorer, my_i, my_k, wsum, mean, m2, use_dir, a_num, a_den, res_score, res_cnt, res_lg);
}

// The era recursion when every era weight is 0 or 1 (era_alpha == 0, no directional term): the
// running weight sum is then a small integer n and the Welford factor is 0 or the correctly
// rounded 1 / n, read from a table.  The CTA is split into two halves of equal size:
//   consumers (first half)  one thread per (node, threshold) slot; per era only a shared load and
//                           the mean / M2 updates, so the dependent float chain sets the pace;
//   producers (second half) stream the (gain, weight) table of the CTA into a ring of three
//                           chunks with asynchronous copies (chunk c + 2, 16-byte units dealt over
//                           all producer threads), and rewrite chunk c + 1 in place to
//                           (gain, factor) while the consumers walk chunk c.
// The rewrite counts the valid eras seen so far per slot.  With 32 or more slots a producer thread
// owns a slot and walks the chunk's eras; with fewer there is a single producer warp, which is
// split into P era phases of S2 lanes (S2: slots rounded up to a power of two): each phase counts
// and rewrites a contiguous part of the chunk and a shuffle scan joins the counts.
// Chunks are walked in groups of eight eras without bounds checks: the rows between the end of the
// last chunk and the next multiple of eight are zero-filled (gain 0, weight 0 leave every state
// unchanged).  One block-wide barrier per chunk hands the buffers on.
constexpr int kUnitSlotsMax = 128;  // consumer threads per CTA
constexpr int kSub = 8;             // eras per unrolled group

__global__ void __launch_bounds__(2 * kUnitSlotsMax) chain_unit_kernel(ChainArgs a) {
    const ScoreLaunch& s = a.s;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int n_nodes = min(*s.n_nodes_ptr, s.n_nodes_max);
    const int npc = a.nodes_per_cta;
    const int node0 = blockIdx.y * npc;
    if (node0 >= n_nodes) return;
    const int nn = min(npc, n_nodes - node0);
    const int f = blockIdx.x;
    const int E = s.n_eras, K = s.n_thr;

    // shared layout: res_lg int64 [npck2] | ring float2 [3][EC][npck] | res_score, res_cnt, s_nv [npck] | s_inv [E+1]
    const int npck = npc * K;
    const int npck2 = (npck + 1) & ~1;  // keeps the ring on a 16-byte boundary
    const int EC = a.era_chunk;         // multiple of kSub
    long long* res_lg = reinterpret_cast<long long*>(smem_raw);
    float2* ring = reinterpret_cast<float2*>(res_lg + npck2);
    float* res_score = reinterpret_cast<float*>(ring + (size_t)3 * EC * npck);
    uint32_t* res_cnt = reinterpret_cast<uint32_t*>(res_score + npck);
    int* s_nv = reinterpret_cast<int*>(res_cnt + npck);
    float* s_inv = reinterpret_cast<float*>(s_nv + npck);  // s_inv[n] = 1/n, n <= n_eras
    for (int n = threadIdx.x; n <= E; n += blockDim.x) s_inv[n] = (n > 0) ? f_div(1.f, (float)n) : 0.f;

    const int half = blockDim.x >> 1;
    const bool producer = (threadIdx.x >= half);
    const int t = producer ? threadIdx.x - half : threadIdx.x;  // index of this thread in its half
    const int slots = nn * K;
    const bool active = (t < slots);
    const int my_i = t / K;
    const int my_k = t - my_i * K;
    const float2* gw_cta = s.gw + ((size_t)f * E * s.node_stride + node0) * K;  // + e * e_stride + slot
    const size_t e_stride = (size_t)s.node_stride * K;
    const int n_chunks = (E + EC - 1) / EC;

    // ---- producers ----
    // 16-byte copies need both sides on 16 bytes: an even slot count, row pitch and table row
    const bool wide = ((slots | npck | (int)(e_stride & 1) | (int)((node0 * K) & 1)) & 1) == 0;
    const int units = wide ? slots >> 1 : slots;  // copy units per era
    const int step_e = half / units, step_u = half - step_e * units;
    auto load_chunk = [&](int c) {  // always commits a group, possibly an empty one
        if (c < n_chunks) {
            const int e0 = c * EC, ec = min(EC, E - e0);
            float2* dst = ring + (size_t)(c % 3) * EC * npck;
            const float2* src = gw_cta + (size_t)e0 * e_stride;
            int e = t / units, u = t - e * units;
            while (e < ec) {
                if (wide) cp_async16(dst + (size_t)e * npck + 2 * u, src + (size_t)e * e_stride + 2 * u);
                else cp_async8(dst + (size_t)e * npck + u, src + (size_t)e * e_stride + u);
                e += step_e;
                u += step_u;
                if (u >= units) {
                    u -= units;
                    ++e;
                }
            }
            // rows up to the next multiple of kSub: zero
            const int ec8 = (ec + kSub - 1) / kSub * kSub;
            for (int i = t; i < (ec8 - ec) * slots; i += half)
                dst[(size_t)(ec + i / slots) * npck + (i % slots)] = make_float2(0.f, 0.f);
        }
        cp_async_commit();
    };
    // (a slot's column of a chunk is copied by several producers: each waits for its own copies,
    // then all meet at a barrier of the producer half before anyone rewrites)
    auto producers_sync = [&]() { asm volatile("bar.sync 1, %0;\n" ::"r"(half) : "memory"); };

    const int S2 = a.slot_pow2;              // 0: one producer thread per slot
    const int P = S2 ? 32 / S2 : 1;          // era phases of the single producer warp
    const int pj = S2 ? (t & (S2 - 1)) : t;  // slot of this producer thread
    const int pp = S2 ? t / S2 : 0;          // its era phase
    const bool col = producer && (pj < slots);
    int n_valid = 0;
    auto rewrite_chunk = [&](int c) {
        if (c >= n_chunks) return;
        const int ec = min(EC, E - c * EC);
        const int ec8 = (ec + kSub - 1) / kSub * kSub;
        float2* buf = ring + (size_t)(c % 3) * EC * npck + pj;
        const int L = EC / P;  // multiple of kSub (checked by the launcher)
        const int e_lo = min(ec8, pp * L), e_hi = min(ec8, e_lo + L);
        int base = n_valid;
        if (S2) {
            // valid eras of this phase's part, then an inclusive scan over the phases of the slot
            int cnt = 0;
            if (col)
                for (int e0 = e_lo; e0 < e_hi; e0 += kSub) {
                    float w[kSub];
#pragma unroll
                    for (int q = 0; q < kSub; ++q) w[q] = buf[(size_t)(e0 + q) * npck].y;
#pragma unroll
                    for (int q = 0; q < kSub; ++q) cnt += (w[q] > 0.f) ? 1 : 0;
                }
            int incl = cnt;
            for (int d = S2; d < 32; d <<= 1) {
                const int up = __shfl_up_sync(0xFFFFFFFFu, incl, d);
                if ((int)(threadIdx.x & 31) >= d) incl += up;
            }
            const int total = __shfl_sync(0xFFFFFFFFu, incl, (pj + (P - 1) * S2) & 31);
            base = n_valid + incl - cnt;
            n_valid += total;
        }
        if (!col) return;
        int n = base;
        for (int e0 = e_lo; e0 < e_hi; e0 += kSub) {
            float2 v[kSub];
#pragma unroll
            for (int q = 0; q < kSub; ++q) v[q] = buf[(size_t)(e0 + q) * npck];
#pragma unroll
            for (int q = 0; q < kSub; ++q) {
                const bool on = v[q].y > 0.f;
                n += on ? 1 : 0;
                v[q].y = on ? s_inv[n] : 0.f;
            }
#pragma unroll
            for (int q = 0; q < kSub; ++q) buf[(size_t)(e0 + q) * npck] = v[q];
        }
        if (!S2) n_valid = n;
    };

    if (producer) {
        load_chunk(0);
        load_chunk(1);
        cp_async_wait<1>();  // this thread's copies of chunk 0 have landed
    }
    __syncthreads();  // chunk 0 and the reciprocal table are visible
    if (producer) rewrite_chunk(0);
    __syncthreads();

    float mean = 0.f, m2 = 0.f;
    for (int c = 0; c < n_chunks; ++c) {
        if (producer) {
            load_chunk(c + 2);   // its buffer held chunk c - 1, released by the last barrier
            cp_async_wait<1>();  // this thread's copies of chunk c + 1 have landed
            producers_sync();
            rewrite_chunk(c + 1);
        } else if (active) {
            const int ec = min(EC, E - c * EC);
            const int ec8 = (ec + kSub - 1) / kSub * kSub;
            const float2* src = ring + (size_t)(c % 3) * EC * npck + t;
            for (int e0 = 0; e0 < ec8; e0 += kSub) {
                float2 v[kSub];
#pragma unroll
                for (int q = 0; q < kSub; ++q) v[q] = src[(size_t)(e0 + q) * npck];
#pragma unroll
                for (int q = 0; q < kSub; ++q) {
                    // padding and invalid eras carry factor 0 and weight 0: the state is unchanged
                    const float w = (v[q].y > 0.f) ? 1.f : 0.f;
                    const float delta = f_sub(v[q].x, mean);
                    mean = f_add(mean, f_mul(v[q].y, delta));
                    m2 = f_add(m2, f_mul(f_mul(w, delta), f_sub(v[q].x, mean)));
                }
            }
        }
        __syncthreads();
    }
    if (col && pp == 0) s_nv[pj] = n_valid;
    __syncthreads();
    const bool scorer = !producer && active;
    const float wsum = scorer ? (float)s_nv[t] : 0.f;
    finish_pairs(s, f, node0, nn, scorer, my_i, my_k, wsum, mean, m2, false, 0.f, 0.f, res_score, res_cnt, res_lg);
}

}  // namespace

// ---- mass K-cuts -----------------------------------------------------------------------------------
// Thresholds of one feature at the quantiles of its bin masses over all frontier rows (every node,
// every era), as the reference's compiled split finder takes them
// (packboost/backends/cpu/frontier_cpu.cpp:59-109; its evenly spaced fallback :35-57): the target
// masses are i / (k - 1) of total * (1 - 1e-12) in float64, a threshold is one below the first bin
// whose cumulative mass reaches the target, duplicates are dropped, evenly spaced ids fill up, and
// the k smallest ids are kept.
namespace {

__global__ void __launch_bounds__(256) mass_thr_kernel(const uint32_t* __restrict__ cnt, const int32_t* n_nodes_ptr,
                                                       int n_nodes_max, int node_stride, int E, int nb, int K,
                                                       int32_t* __restrict__ thr_out) {
    __shared__ unsigned int s_m[256];
    __shared__ int s_set[256];
    const int f = blockIdx.x;
    const int n_nodes = min(*n_nodes_ptr, n_nodes_max);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    for (int i = threadIdx.x; i < 256; i += blockDim.x) { s_m[i] = 0u; s_set[i] = 0; }
    __syncthreads();
    // a warp takes (era, node) pairs in turn; lane l sums bins l, l + 32, ...
    unsigned int acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0u;
    for (int pair = warp; pair < E * n_nodes; pair += n_warps) {
        const int e = pair / n_nodes, n = pair - e * n_nodes;
        const uint32_t* row = cnt + (((size_t)f * E + e) * node_stride + n) * nb;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int b = j * 32 + lane;
            if (b < nb) acc[j] += row[b];
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int b = j * 32 + lane;
        if (b < nb && acc[j]) atomicAdd(&s_m[b], acc[j]);
    }
    __syncthreads();
    if (threadIdx.x != 0) return;
    const int max_thr = max(1, nb - 1);
    const int kk = max(1, min(K, max_thr));
    auto even_into_set = [&]() {  // evenly spaced ids, round half away from zero
        if (kk == 1) { s_set[0] = 1; return; }
        const double step = (double)(max_thr - 1) / (double)(kk - 1);
        for (int i = 0; i < kk; ++i) {
            long long idx = llround(round((double)i * step));
            idx = max(0ll, min(idx, (long long)max_thr - 1));
            s_set[(int)idx] = 1;
        }
    };
    long long total = 0;
    for (int b = 0; b < nb; ++b) total += s_m[b];
    int have = 0;
    if (total <= 0) {
        even_into_set();
    } else {
        const double upper = (double)total * (1.0 - 1e-12);
        for (int i = 0; i < kk; ++i) {
            const double alpha = (kk == 1) ? 0.0 : (double)i / (double)(kk - 1);
            const double target = upper * alpha;
            long long run = 0;
            int idx = nb - 1;
            for (int b = 0; b < nb; ++b) {  // first bin whose cumulative mass is not below the target
                run += s_m[b];
                if (!((double)run < target)) { idx = b; break; }
            }
            const int thr = max(0, min(idx - 1, max_thr - 1));
            if (!s_set[thr]) { s_set[thr] = 1; ++have; }
        }
        if (have < kk) even_into_set();
    }
    int w = 0, last = 0;
    for (int b = 0; b < max_thr && w < kk; ++b)
        if (s_set[b]) { thr_out[(size_t)f * K + w] = b; last = b; ++w; }
    for (; w < K; ++w) thr_out[(size_t)f * K + w] = last;  // (not reached: kk distinct ids always exist)
}

}  // namespace

int launch_mass_thresholds(const uint32_t* cnt, int n_feat, const int32_t* n_nodes_ptr, int n_nodes_max, int node_stride,
                           int n_eras, int max_bins, int n_thr, int32_t* thr_out, cudaStream_t stream) {
    if (n_feat <= 0) return PB_OK;
    if (max_bins > 256 || n_thr < 1 || n_thr > 255) return fail_arg("mass thresholds: bin or threshold count out of range");
    mass_thr_kernel<<<(unsigned)n_feat, 256, 0, stream>>>(cnt, n_nodes_ptr, n_nodes_max, node_stride, n_eras, max_bins,
                                                           n_thr, thr_out);
    count_launch(1);
    PB_LAUNCH_CHECK("mass_thr_kernel");
    return PB_OK;
}

// ---- one node, general hessians -------------------------------------------------------------------
// The reference's single-node entry (`_find_best_split`, packboost/booster.py:1010-1290 via the
// batched frontier) accepts arbitrary per-row hessians; the training loop never produces any (the
// squared loss has unit hessians), so this form is a kernel of its own instead of a mode of the fast
// path.  One CTA per feature, one thread per threshold: prefix sums over the bins of every era from
// the three histograms (counts, fixed-point gradient sums, fixed-point hessian sums), the per-era
// gain with H = sum of hessians, the weighted Welford recursion over the eras in ascending order,
// either directional term, the min_samples_leaf mask, and the best threshold of the feature under
// (score, left count, threshold index).  Same separately rounded float32 operations as the rest of
// this file.
namespace {

struct NodeGeneralArgs {
    const uint32_t* cnt;   // [n_feat][E][nb]
    const int64_t* gsum;
    const int64_t* hsum;
    int E, nb, K;
    const int32_t* thr_ids;
    float inv_g, inv_h, lambda_l2, lambda_dro, direction_weight, era_alpha;
    int direction_form, min_samples_leaf;
    long long total_count, total_gq;
    pb_split_general* out;  // [n_feat]
};

__global__ void __launch_bounds__(256) score_node_general_kernel(NodeGeneralArgs a) {
    __shared__ float s_score[256];
    __shared__ long long s_lc[256], s_lg[256], s_lh[256];
    __shared__ int s_nan;
    const int f = blockIdx.x, k = threadIdx.x;
    if (k == 0) s_nan = 0;
    __syncthreads();
    const float lam = a.lambda_l2;
    const bool use_dir = (a.direction_weight != 0.f) && (a.direction_form == 1 || a.total_gq != 0);
    const float pa = (a.total_gq > 0) ? -1.f : ((a.total_gq < 0) ? 1.f : 0.f);
    if (k < a.K) {
        const int thr = a.thr_ids[k];
        float wsum = 0.f, mean = 0.f, m2 = 0.f, a_num = 0.f, a_den = 0.f;
        long long lc_all = 0, lg_all = 0, lh_all = 0;
        for (int e = 0; e < a.E; ++e) {
            const size_t base = ((size_t)f * a.E + e) * a.nb;
            long long tc = 0, tgq = 0, thq = 0, lc = 0, lgq = 0, lhq = 0;
            for (int b = 0; b < a.nb; ++b) {
                const long long c = a.cnt[base + b], g = a.gsum[base + b], h = a.hsum[base + b];
                tc += c; tgq += g; thq += h;
                if (b <= thr) { lc += c; lgq += g; lhq += h; }
            }
            if (tc == 0) continue;  // era absent from the node: weight 0
            const float w_e = (a.era_alpha > 0.f) ? f_add((float)tc, a.era_alpha) : 1.f;
            const float w = (lc > 0 && tc - lc > 0) ? w_e : 0.f;
            const float lg = f_mul(__ll2float_rn(lgq), a.inv_g), tg = f_mul(__ll2float_rn(tgq), a.inv_g);
            const float lh = f_mul(__ll2float_rn(lhq), a.inv_h), th = f_mul(__ll2float_rn(thq), a.inv_h);
            const float rg = f_sub(tg, lg), rh = f_sub(th, lh);
            const float dl = f_add(lh, lam), dr = f_add(rh, lam);
            const float parent = f_div(f_mul(0.5f, f_mul(tg, tg)), f_add(th, lam));
            const float gain = f_sub(f_mul(0.5f, f_add(f_div(f_mul(lg, lg), dl), f_div(f_mul(rg, rg), dr))), parent);
            welford_step(gain, w, wsum, mean, m2);
            if (use_dir) {
                const float vl = f_div(-lg, dl), vr = f_div(-rg, dr);
                const float agree = (a.direction_form == 1)
                    ? ((vl > vr) ? 1.f : -1.f)
                    : f_mul(0.5f, f_add((sign_of(vl) == pa) ? 1.f : 0.f, (sign_of(vr) == pa) ? 1.f : 0.f));
                a_num = f_add(a_num, f_mul(w, agree));
                a_den = f_add(a_den, w);
            }
            lc_all += lc; lg_all += lgq; lh_all += lhq;
        }
        const float ws = (wsum < 1e-12f) ? 1e-12f : wsum;
        float var = f_div(m2, ws);
        if (var < 0.f) var = 0.f;
        float score = f_sub(mean, f_mul(a.lambda_dro, __fsqrt_rn(var)));
        if (use_dir) score = f_add(score, f_mul(a.direction_weight, (a_den > 0.f) ? f_div(a_num, a_den) : 0.f));
        const bool ok = (lc_all >= a.min_samples_leaf) && (a.total_count - lc_all >= a.min_samples_leaf);
        if (score != score) s_nan = 1;
        s_score[k] = ok ? score : -INFINITY;
        s_lc[k] = lc_all; s_lg[k] = lg_all; s_lh[k] = lh_all;
    }
    __syncthreads();
    if (k == 0) {
        float bs = -INFINITY;
        long long bc = -1;
        int bk = -1;
        for (int j = 0; j < a.K; ++j) {
            const float sc = s_score[j];
            if (sc != sc) continue;
            if (sc > bs || (sc == bs && s_lc[j] >= bc)) { bs = sc; bc = s_lc[j]; bk = j; }
        }
        pb_split_general o;
        o.score = bs;
        o.k = bk;
        o.threshold = (bk >= 0) ? a.thr_ids[bk] : -1;
        o.has_nan = s_nan;
        o.left_count = (bk >= 0) ? s_lc[bk] : 0;
        o.left_gq = (bk >= 0) ? s_lg[bk] : 0;
        o.left_hq = (bk >= 0) ? s_lh[bk] : 0;
        a.out[f] = o;
    }
}

}  // namespace

}  // namespace pb

extern "C" int pb_score_node_general(const uint32_t* cnt, const int64_t* gsum, const int64_t* hsum, int64_t n_feat,
                                     int64_t n_eras, int64_t max_bins, const int32_t* thr_ids, int64_t n_thresholds,
                                     float inv_scale_g, float inv_scale_h, float lambda_l2, float lambda_dro,
                                     float direction_weight, float era_alpha, int64_t direction_form,
                                     int64_t min_samples_leaf, int64_t total_count, int64_t total_gq,
                                     pb_split_general* out, void* stream) {
    using namespace pb;
    PB_REQUIRE(cnt && gsum && hsum && thr_ids && out, "null buffer");
    PB_REQUIRE(n_feat >= 1 && n_eras >= 1 && max_bins >= 2 && max_bins <= 256, "bad shape");
    PB_REQUIRE(n_thresholds >= 1 && n_thresholds < max_bins, "n_thresholds out of range");
    PB_REQUIRE(lambda_l2 > 0.f, "lambda_l2 must be positive");
    NodeGeneralArgs a{cnt, gsum, hsum, (int)n_eras, (int)max_bins, (int)n_thresholds, thr_ids, inv_scale_g, inv_scale_h,
                      lambda_l2, lambda_dro, direction_weight, era_alpha > 0.f ? era_alpha : 0.f, direction_form ? 1 : 0,
                      (int)min_samples_leaf, (long long)total_count, (long long)total_gq, out};
    score_node_general_kernel<<<(unsigned)n_feat, 256, 0, (cudaStream_t)stream>>>(a);
    count_launch(1);
    PB_LAUNCH_CHECK("score_node_general_kernel");
    return PB_OK;
}

namespace pb {

size_t score_scratch_bytes_per_feature(int node_stride, int n_eras, int n_thr) {
    return (size_t)node_stride * n_eras * n_thr * sizeof(float2) + (size_t)node_stride * n_thr * 12;
}

int launch_score(const ScoreLaunch& s, cudaStream_t stream) {
    if (s.n_feat <= 0 || s.n_nodes_max <= 0) return PB_OK;
    const int K = s.n_thr, NB = s.max_bins;
    if (K < 1 || K > kChainThreads) return fail_arg("n_thresholds=%d outside [1,%d]", K, kChainThreads);
    if (!s.gw || !s.lc_tot || !s.lg_tot) return fail_arg("scorer scratch is null");
    const size_t tot_cells = (size_t)s.n_feat * s.node_stride * K;
    if (!s.fused) {
        PB_CUDA_TRY(cudaMemsetAsync(s.lc_tot, 0, tot_cells * sizeof(uint32_t), stream));
        PB_CUDA_TRY(cudaMemsetAsync(s.lg_tot, 0, tot_cells * sizeof(int64_t), stream));
    }

    prof_begin(s.prof, kProfScore, stream);
    GainArgs g;
    g.s = s;
    if (s.fused) {
        // the histogram kernel's flush already wrote the (gain, weight) table and the era-summed
        // totals: only the era recursion is left
        if (s.direction_weight != 0.f) return fail_arg("the fused flush cannot serve the directional term");
    } else if (NB <= kSmallBins) {
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
        if (K <= 4 && NB <= 5) gain_kernel_small<4, 5><<<grid, kGainThreads, 0, stream>>>(g);
        else gain_kernel_small<kSmallBins, kSmallBins><<<grid, kGainThreads, 0, stream>>>(g);
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
    if (!s.fused) PB_LAUNCH_CHECK("gain_kernel");

    ChainArgs c;
    c.s = s;
    const bool unit = (s.era_alpha <= 0.f && s.direction_weight == 0.f && s.n_eras < kInvTable && K <= kUnitSlotsMax);
    c.unit_weights = unit ? 1 : 0;
    if (unit) {
        int npc = kUnitSlotsMax / K;
        if (npc > s.n_nodes_max) npc = s.n_nodes_max;
        // A feature shard of a multi-GPU run has fewer features than the GPU has SMs: spread the nodes
        // over more CTAs until every SM has one (a CTA with many slots is bound by its own issue rate)
        while (npc > 2 && (int64_t)s.n_feat * ((s.n_nodes_max + npc - 1) / npc) < 148) npc >>= 1;
        c.nodes_per_cta = npc;
        int ec = (int)((16 * 1024) / ((size_t)npc * K * sizeof(float2))) / 8 * 8;  // multiple of the unrolled group
        if (ec < 8) ec = 8;
        if (ec > 64) ec = 64;
        c.era_chunk = ec;
        // fewer than 32 slots: the single producer warp works in 32 / S2 era phases of ec / P eras
        c.slot_pow2 = 0;
        if (npc * K < 32) {
            int s2 = 1;
            while (s2 < npc * K) s2 *= 2;
            if (ec % (8 * (32 / s2)) == 0) c.slot_pow2 = s2;
        }
        const int npck2 = (npc * K + 1) & ~1;
        const size_t smem = (size_t)npck2 * 8 + (size_t)npc * K * 12 + (size_t)3 * ec * npc * K * sizeof(float2) +
                            (size_t)(s.n_eras + 1) * 4;
        if (smem > 48 * 1024)
            PB_CUDA_TRY(cudaFuncSetAttribute(chain_unit_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        dim3 grid((unsigned)s.n_feat, (unsigned)((s.n_nodes_max + npc - 1) / npc));
        if (grid.y > 65535u) return fail_arg("scorer grid too large");
        const int half = ((npc * K + 31) / 32) * 32;
        chain_unit_kernel<<<grid, 2 * half, smem, stream>>>(c);
    } else {
        int npc = kChainThreads / K;
        if (npc < 1) npc = 1;
        if (npc > s.n_nodes_max) npc = s.n_nodes_max;
        c.nodes_per_cta = npc;
        int ec = (int)((24 * 1024) / ((size_t)npc * K * sizeof(float2)));
        if (ec < 8) ec = 8;
        if (ec > 64) ec = 64;
        if (ec > s.n_eras) ec = s.n_eras;
        c.era_chunk = ec;
        const size_t smem = (size_t)npc * K * 16 + (size_t)2 * ec * npc * K * sizeof(float2);
        if (smem > 48 * 1024)
            PB_CUDA_TRY(cudaFuncSetAttribute(chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        dim3 grid((unsigned)s.n_feat, (unsigned)((s.n_nodes_max + npc - 1) / npc));
        if (grid.y > 65535u) return fail_arg("scorer grid too large");
        const int threads = ((npc * K + 31) / 32) * 32;
        chain_kernel<<<grid, threads, smem, stream>>>(c);
    }
    prof_end(s.prof, kProfScore, stream);
    count_launch(s.fused ? 1 : 2);
    PB_LAUNCH_CHECK("chain_kernel");
    return PB_OK;
}

}  // namespace pb
