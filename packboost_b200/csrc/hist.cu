// Per-(feature, node, era, bin) histograms of counts and fixed-point gradient sums.
//
// Rows are ordered by era, so an era is a contiguous row range.  One CTA accumulates one row
// tile of one era for a small group of features in shared memory and then writes (or, when an
// era is cut into several tiles, atomically adds) its cells to the global histogram.  Because
// every cell is an integer, the result does not depend on the order of the additions.
//
// Shared-memory cell: one 64-bit word holding (gq_sum << 16) + count.  A tile has fewer than
// 65536 rows, so the count never carries into the gradient field, and |gq| <= 2^30 keeps the
// gradient field inside 48 bits.  One 64-bit shared atomic per (row, feature) updates both.
// When the number of cells per feature is small the cells are replicated per lane group
// ("copies") so that lanes of a warp rarely hit the same address.
//
// Global loads: a thread owns 32 consecutive rows (4-bit codes: one 128-bit load per feature)
// or 16 consecutive rows (8-bit codes).  The slot and gradient of those rows are loaded once
// with 128-bit loads and kept in registers while the thread walks the features of the group.

#include "common.cuh"

namespace pb {

namespace {

constexpr int kHistThreads = 256;
constexpr int kMaxGroup = 8;            // features per CTA
constexpr int kSmemCellBudget = 24576;  // 192 KB of 64-bit cells

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
    int group;       // features per CTA
    int copies;      // power of two, <= 32
    int use_atomics; // 1: several tiles per era -> global atomics onto a zeroed histogram
    uint32_t* cnt;
    int64_t* gsum;
};

template <int BITS>
__global__ void __launch_bounds__(kHistThreads) hist_kernel(HistKernelArgs a) {
    constexpr int RPI = (BITS == 4) ? 32 : 16;  // rows per thread iteration (16 bytes of codes)
    extern __shared__ unsigned long long cells[];

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

    const int f0 = blockIdx.y * a.group;
    const int nf = min(a.group, a.n_feat - f0);
    const int nb = a.max_bins;
    const int cells_per_feat = (node_hi - node_lo) * nb;
    const int copies = a.copies;
    const int total_cells = nf * cells_per_feat * copies;
    for (int i = threadIdx.x; i < total_cells; i += kHistThreads) cells[i] = 0ull;
    __syncthreads();

    const int lane_copy = threadIdx.x & (copies - 1);
    const int c0 = r0 / RPI;
    const int c1 = (r1 + RPI - 1) / RPI;

    for (int c = c0 + threadIdx.x; c < c1; c += kHistThreads) {
        const int row_base = c * RPI;
        // slot (uint16) and gq (int32) of RPI rows
        int32_t g[RPI];
        int cellbase[RPI];  // (slot - node_lo) * nb, or -1 when the row is not accumulated here
        {
            const uint4* sp = reinterpret_cast<const uint4*>(a.slot + row_base);
            const int4* gp = reinterpret_cast<const int4*>(a.gq + row_base);
#pragma unroll
            for (int q = 0; q < RPI / 8; ++q) {
                const uint4 sv = __ldg(sp + q);
                const uint32_t w[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int s = (w[j >> 1] >> ((j & 1) * 16)) & 0xFFFF;
                    const int r = row_base + q * 8 + j;
                    const bool ok = (r >= r0) & (r < r1) & (s >= node_lo) & (s < node_hi);
                    cellbase[q * 8 + j] = ok ? (s - node_lo) * nb : -1;
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
        }
        for (int fi = 0; fi < nf; ++fi) {
            const int frow = __ldg(a.feat_rows + f0 + fi);
            const uint4 cv = __ldg(reinterpret_cast<const uint4*>(a.codes + (int64_t)frow * a.pitch) + c);
            const uint32_t w[4] = {cv.x, cv.y, cv.z, cv.w};
            unsigned long long* fc = cells + (size_t)fi * cells_per_feat * copies + lane_copy;
#pragma unroll
            for (int j = 0; j < RPI; ++j) {
                int code;
                if (BITS == 4) {
                    code = (w[j >> 3] >> ((j & 7) * 4)) & 0xF;
                } else {
                    code = (w[j >> 2] >> ((j & 3) * 8)) & 0xFF;
                }
                if (cellbase[j] >= 0) {
                    const long long v = ((long long)g[j] << 16) + 1ll;
                    atomicAdd(fc + (size_t)(cellbase[j] + code) * copies, (unsigned long long)v);
                }
            }
        }
    }
    __syncthreads();

    // flush: fold the copies, split the packed word, write [feature][node][era][bin]
    const int out_cells = nf * cells_per_feat;
    for (int i = threadIdx.x; i < out_cells; i += kHistThreads) {
        const int fi = i / cells_per_feat;
        const int rem = i - fi * cells_per_feat;
        const int node = node_lo + rem / nb;
        const int bin = rem - (rem / nb) * nb;
        long long acc = 0;
        const unsigned long long* src = cells + (size_t)i * copies;
        for (int k = 0; k < copies; ++k) acc += (long long)src[k];
        const uint32_t count = (uint32_t)(acc & 0xFFFF);
        const long long gs = (acc - (long long)count) >> 16;
        const size_t o = (((size_t)(f0 + fi) * a.node_stride + node) * a.n_eras + era) * nb + bin;
        if (a.use_atomics) {
            if (count) atomicAdd(a.cnt + o, count);
            if (gs) atomicAdd(reinterpret_cast<unsigned long long*>(a.gsum + o), (unsigned long long)gs);
        } else {
            a.cnt[o] = count;
            a.gsum[o] = gs;
        }
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

    if (h.max_era_rows <= kSingleTileRows) {
        a.tiles_per_era = 1;
        a.tile_rows = kSingleTileRows;
        a.use_atomics = 0;
    } else {
        a.tile_rows = kSplitTileRows;
        a.tiles_per_era = (h.max_era_rows + kSplitTileRows - 1) / kSplitTileRows;
        a.use_atomics = 1;
    }

    // shared-memory plan: cells per feature, node chunks, feature group, copies
    const int64_t per_feat_all = (int64_t)h.n_nodes * h.max_bins;
    int nodes_per_chunk = h.n_nodes;
    if (per_feat_all > kSmemCellBudget) {
        nodes_per_chunk = kSmemCellBudget / h.max_bins;
        if (nodes_per_chunk < 1) return fail_arg("max_bins=%d does not fit the histogram tile", h.max_bins);
    }
    const int chunks = (h.n_nodes + nodes_per_chunk - 1) / nodes_per_chunk;
    const int64_t per_feat = (int64_t)nodes_per_chunk * h.max_bins;
    int copies = 1;
    while (copies < 32 && per_feat * copies * 2 <= 256) copies *= 2;
    // keep a CTA near 32 KB of cells so that several CTAs share an SM
    int group = (int)(4096 / (per_feat * copies));
    if (group < 1) group = 1;
    if (group > kMaxGroup) group = kMaxGroup;
    if (group > h.n_feat) group = h.n_feat;
    a.nodes_per_chunk = nodes_per_chunk;
    a.group = group;
    a.copies = copies;

    const size_t smem = (size_t)group * per_feat * copies * sizeof(unsigned long long);
    const size_t out_cells = (size_t)h.n_feat * h.node_stride * h.n_eras * h.max_bins;
    if (a.use_atomics) {
        PB_CUDA_TRY(cudaMemsetAsync(h.cnt, 0, out_cells * sizeof(uint32_t), stream));
        PB_CUDA_TRY(cudaMemsetAsync(h.gsum, 0, out_cells * sizeof(int64_t), stream));
    }
    dim3 grid((unsigned)(h.n_eras * a.tiles_per_era), (unsigned)((h.n_feat + group - 1) / group), (unsigned)chunks);
    if (grid.y > 65535u || grid.z > 65535u) return fail_arg("histogram grid too large");
    prof_begin(kProfHist, stream);
    if (h.code_bits == 4) {
        if (smem > 48 * 1024)
            PB_CUDA_TRY(cudaFuncSetAttribute(hist_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        hist_kernel<4><<<grid, kHistThreads, smem, stream>>>(a);
    } else {
        if (smem > 48 * 1024)
            PB_CUDA_TRY(cudaFuncSetAttribute(hist_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        hist_kernel<8><<<grid, kHistThreads, smem, stream>>>(a);
    }
    prof_end(kProfHist, stream);
    count_launch(1);
    PB_LAUNCH_CHECK("hist_kernel");
    return PB_OK;
}

}  // namespace pb
