// Per-(feature, node, era, bin) histograms of counts and fixed-point gradient sums.
//
// Rows are ordered by era, so an era is a contiguous row range.  One CTA owns one row tile of
// one era (at most kTileRowsMax rows) and a contiguous range of the sampled features.  Every
// thread owns one 16-byte chunk of codes per feature (32 rows of 4-bit codes, 16 rows of 8-bit
// codes); the slot and gradient of those rows are loaded once and stay in registers while the
// thread walks the CTA's features, prefetching the next feature's chunk while it accumulates
// the current one.  Features are accumulated in groups in shared memory and each group is
// written (or, when an era is cut into several tiles, atomically added) to the global
// histogram.  Every cell is an integer, so the result does not depend on the order of the
// additions.
//
// Shared-memory cell: two 32-bit words updated with one native 32-bit shared atomic each
// (64-bit shared atomics are an order of magnitude slower on this part):
//   A = (sum of lo) << CB | count        lo = gq & (2^LB - 1)
//   B = sum of hi                        hi = gq >> LB (arithmetic)
// With fewer than 2^CB rows per tile, LB = 32 - 2*CB and |gq| <= 2^(63 - 3*CB) (capped at
// 2^30) neither word can overflow; pb_train_prepare derives CB/LB and the gradient scale from
// the largest tile.  When a feature has few cells they are replicated ("copies") so that the
// lanes of a warp rarely hit the same address.

#include "common.cuh"

namespace pb {

namespace {

constexpr int kMaxGroup = 8;            // features accumulated together in shared memory
constexpr int kSmemCellBudget = 24576;  // 192 KB of 2-word cells

struct HistKernelArgs {
    const uint8_t* codes;
    int64_t pitch;
    const int32_t* feat_rows;
    int n_feat;
    const int32_t* gq;
    const uint16_t* slot;
    const int32_t* era_offsets;
    int n_eras;
    int max_bins;
    int tiles_per_era;
    int tile_rows;
    const int32_t* n_nodes_ptr;
    int n_nodes;
    int node_stride;
    int nodes_per_chunk;
    int feats_per_cta;
    int group;       // features per shared-memory pass
    int copies;      // power of two, <= 32
    int use_atomics; // 1: several tiles per era -> global atomics onto a zeroed histogram
    int count_bits;  // CB
    int lo_bits;     // LB
    uint32_t* cnt;
    int64_t* gsum;
};

template <int BITS, int THREADS>
__global__ void __launch_bounds__(THREADS) hist_kernel(HistKernelArgs a) {
    constexpr int RPI = (BITS == 4) ? 32 : 16;  // rows per thread (16 bytes of codes)
    extern __shared__ uint32_t cells[];         // [group][cells_per_feat][copies][2]
    __shared__ int s_frow[256];

    const int n_nodes = a.n_nodes_ptr ? min(*a.n_nodes_ptr, a.n_nodes) : a.n_nodes;
    const int node_lo = blockIdx.z * a.nodes_per_chunk;
    if (node_lo >= n_nodes) return;
    const int node_hi = min(n_nodes, node_lo + a.nodes_per_chunk);
    const int era = blockIdx.x / a.tiles_per_era;
    const int tile = blockIdx.x - era * a.tiles_per_era;
    const int era_begin = a.era_offsets[era];
    const int era_end = a.era_offsets[era + 1];
    const int r0 = era_begin + tile * a.tile_rows;
    const int r1 = min(era_end, r0 + a.tile_rows);
    if (r0 >= r1 && a.use_atomics) return;  // (without atomics an empty tile still writes its zeros)

    const int fa = blockIdx.y * a.feats_per_cta;
    const int fb = min(a.n_feat, fa + a.feats_per_cta);
    for (int i = threadIdx.x; i < fb - fa; i += blockDim.x) s_frow[i] = a.feat_rows[fa + i];

    const int nb = a.max_bins;
    const int cells_per_feat = (node_hi - node_lo) * nb;
    const int copies = a.copies;
    const int lane_copy = threadIdx.x & (copies - 1);
    const int CB = a.count_bits, LB = a.lo_bits;
    const uint32_t lo_mask = (1u << LB) - 1u;

    // ---- row state of this thread's chunk, kept in registers for the whole CTA ----
    const int c = r0 / RPI + threadIdx.x;
    const bool has = (r0 < r1) && (c * RPI < r1);
    int32_t g[RPI];
    uint32_t cb2[RPI / 2];  // two 16-bit cell bases per word; 0xFFFF: row not accumulated here
    if (has) {
        const int row_base = c * RPI;
        const uint4* sp = reinterpret_cast<const uint4*>(a.slot + row_base);
        const int4* gp = reinterpret_cast<const int4*>(a.gq + row_base);
#pragma unroll
        for (int q = 0; q < RPI / 8; ++q) {
            const uint4 sv = __ldg(sp + q);
            const uint32_t w[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t packed = 0;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int s = (w[j] >> (h * 16)) & 0xFFFF;
                    const int r = row_base + q * 8 + j * 2 + h;
                    const bool ok = (r >= r0) & (r < r1) & (s >= node_lo) & (s < node_hi);
                    packed |= (ok ? (uint32_t)((s - node_lo) * nb) : 0xFFFFu) << (h * 16);
                }
                cb2[q * 4 + j] = packed;
            }
        }
#pragma unroll
        for (int q = 0; q < RPI / 4; ++q) {
            const int4 gv = __ldg(gp + q);
            g[q * 4 + 0] = gv.x;
            g[q * 4 + 1] = gv.y;
            g[q * 4 + 2] = gv.z;
            g[q * 4 + 3] = gv.w;
        }
    } else {
#pragma unroll
        for (int j = 0; j < RPI / 2; ++j) cb2[j] = 0xFFFFFFFFu;
#pragma unroll
        for (int j = 0; j < RPI; ++j) g[j] = 0;
    }
    __syncthreads();  // s_frow

    uint4 cur = make_uint4(0, 0, 0, 0);
    if (has && fa < fb) cur = __ldg(reinterpret_cast<const uint4*>(a.codes + (int64_t)s_frow[0] * a.pitch) + c);

    for (int g0 = fa; g0 < fb; g0 += a.group) {
        const int nf = min(a.group, fb - g0);
        const int total_words = nf * cells_per_feat * copies * 2;
        for (int i = threadIdx.x; i < total_words; i += blockDim.x) cells[i] = 0u;
        __syncthreads();

        for (int fi = 0; fi < nf; ++fi) {
            uint4 nxt = make_uint4(0, 0, 0, 0);
            const int fnext = g0 + fi + 1;
            if (has && fnext < fb)
                nxt = __ldg(reinterpret_cast<const uint4*>(a.codes + (int64_t)s_frow[fnext - fa] * a.pitch) + c);
            if (has) {
                const uint32_t w[4] = {cur.x, cur.y, cur.z, cur.w};
                uint32_t* fc = cells + ((size_t)fi * cells_per_feat * copies + lane_copy) * 2;
#pragma unroll
                for (int j = 0; j < RPI; ++j) {
                    int code;
                    if (BITS == 4) {
                        code = (w[j >> 3] >> ((j & 7) * 4)) & 0xF;
                    } else {
                        code = (w[j >> 2] >> ((j & 3) * 8)) & 0xFF;
                    }
                    const uint32_t base = (cb2[j >> 1] >> ((j & 1) * 16)) & 0xFFFFu;
                    if (base != 0xFFFFu) {
                        uint32_t* cell = fc + (size_t)(base + code) * copies * 2;
                        atomicAdd(cell, (((uint32_t)g[j] & lo_mask) << CB) + 1u);
                        atomicAdd(reinterpret_cast<int*>(cell) + 1, g[j] >> LB);
                    }
                }
            }
            cur = nxt;
        }
        __syncthreads();

        // flush: fold the copies, rebuild count and gradient sum, write [feature][node][era][bin]
        const int out_cells = nf * cells_per_feat;
        for (int i = threadIdx.x; i < out_cells; i += blockDim.x) {
            const int fi = i / cells_per_feat;
            const int rem = i - fi * cells_per_feat;
            const int node = node_lo + rem / nb;
            const int bin = rem - (rem / nb) * nb;
            const uint32_t* src = cells + (size_t)i * copies * 2;
            uint32_t count = 0;
            long long lo_sum = 0, hi_sum = 0;
            for (int k = 0; k < copies; ++k) {
                const uint32_t A = src[2 * k];
                count += A & ((1u << CB) - 1u);
                lo_sum += (long long)(A >> CB);
                hi_sum += (long long)(int32_t)src[2 * k + 1];
            }
            const long long gs = hi_sum * (1ll << LB) + lo_sum;
            const size_t o = (((size_t)(g0 + fi) * a.node_stride + node) * a.n_eras + era) * nb + bin;
            if (a.use_atomics) {
                if (count) atomicAdd(a.cnt + o, count);
                if (gs) atomicAdd(reinterpret_cast<unsigned long long*>(a.gsum + o), (unsigned long long)gs);
            } else {
                a.cnt[o] = count;
                a.gsum[o] = gs;
            }
        }
        __syncthreads();
    }
}

}  // namespace

int launch_hist(const HistLaunch& h, cudaStream_t stream) {
    if (h.n_feat <= 0 || h.n_nodes <= 0) return PB_OK;
    HistKernelArgs a;
    a.codes = h.codes;
    a.pitch = h.pitch;
    a.feat_rows = h.feat_rows;
    a.n_feat = h.n_feat;
    a.gq = h.gq;
    a.slot = h.slot;
    a.era_offsets = h.era_offsets;
    a.n_eras = h.n_eras;
    a.max_bins = h.max_bins;
    a.n_nodes_ptr = h.n_nodes_ptr;
    a.n_nodes = h.n_nodes;
    a.node_stride = h.node_stride;
    a.cnt = h.cnt;
    a.gsum = h.gsum;
    a.count_bits = h.count_bits;
    a.lo_bits = h.lo_bits;

    const int rpi = (h.code_bits == 4) ? 32 : 16;
    a.tile_rows = kTileRowsMax;
    if (h.max_era_rows <= kTileRowsMax) {
        a.tiles_per_era = 1;
        a.use_atomics = 0;
    } else {
        a.tiles_per_era = (h.max_era_rows + kTileRowsMax - 1) / kTileRowsMax;
        a.use_atomics = 1;
    }
    const int max_tile = (h.max_era_rows < kTileRowsMax) ? h.max_era_rows : kTileRowsMax;
    int threads = (max_tile + rpi - 1) / rpi + 1;  // +1: a tile may straddle one extra chunk
    threads = (threads + 31) / 32 * 32;
    const int thread_cap = (h.code_bits == 4) ? 256 : 512;
    if (threads > thread_cap) return fail_arg("histogram tile of %d rows exceeds the thread block", max_tile);

    // shared-memory plan: cells per feature, node chunks, feature group, copies
    const int64_t per_feat_all = (int64_t)h.n_nodes * h.max_bins;
    int nodes_per_chunk = h.n_nodes;
    if (per_feat_all > kSmemCellBudget) {
        nodes_per_chunk = kSmemCellBudget / h.max_bins;
        if (nodes_per_chunk < 1) return fail_arg("max_bins=%d does not fit the histogram tile", h.max_bins);
    }
    const int chunks = (h.n_nodes + nodes_per_chunk - 1) / nodes_per_chunk;
    const int64_t per_feat = (int64_t)nodes_per_chunk * h.max_bins;
    if (per_feat > 65534) return fail_arg("node chunk too large");
    int copies = 1;
    while (copies < 32 && per_feat * copies * 2 <= 256) copies *= 2;
    int group = (int)(2048 / (per_feat * copies));
    if (group < 1) group = 1;
    if (group > kMaxGroup) group = kMaxGroup;
    if (group > h.n_feat) group = h.n_feat;
    a.nodes_per_chunk = nodes_per_chunk;
    a.group = group;
    a.copies = copies;

    // feature ranges: enough CTAs for several waves, each amortising its row-state load
    const int n_tiles = h.n_eras * a.tiles_per_era;
    const int n_groups = (h.n_feat + group - 1) / group;
    int split = (2400 + n_tiles * chunks - 1) / (n_tiles * chunks);
    if (split < 1) split = 1;
    if (split > n_groups) split = n_groups;
    int feats_per_cta = ((n_groups + split - 1) / split) * group;
    if (feats_per_cta > 256) feats_per_cta = 256 / group * group;
    a.feats_per_cta = feats_per_cta;

    const size_t smem = (size_t)group * per_feat * copies * 2 * sizeof(uint32_t);
    const size_t out_cells = (size_t)h.n_feat * h.node_stride * h.n_eras * h.max_bins;
    if (a.use_atomics) {
        PB_CUDA_TRY(cudaMemsetAsync(h.cnt, 0, out_cells * sizeof(uint32_t), stream));
        PB_CUDA_TRY(cudaMemsetAsync(h.gsum, 0, out_cells * sizeof(int64_t), stream));
    }
    dim3 grid((unsigned)n_tiles, (unsigned)((h.n_feat + feats_per_cta - 1) / feats_per_cta), (unsigned)chunks);
    if (grid.y > 65535u || grid.z > 65535u) return fail_arg("histogram grid too large");
    prof_begin(kProfHist, stream);
    if (h.code_bits == 4) {
        if (smem > 48 * 1024)
            PB_CUDA_TRY(cudaFuncSetAttribute(hist_kernel<4, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        hist_kernel<4, 256><<<grid, threads, smem, stream>>>(a);
    } else {
        if (smem > 48 * 1024)
            PB_CUDA_TRY(cudaFuncSetAttribute(hist_kernel<8, 512>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        hist_kernel<8, 512><<<grid, threads, smem, stream>>>(a);
    }
    prof_end(kProfHist, stream);
    count_launch(1);
    PB_LAUNCH_CHECK("hist_kernel");
    return PB_OK;
}

}  // namespace pb
