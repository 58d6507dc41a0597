// Tree routing: a row goes left when its code is <= the node's threshold.
//
// Every walk is bounded: it takes at most as many steps as its tree has nodes, a child index must
// stay inside the tree and a feature index inside the row, and a tree that breaks one of these
// rules contributes 0 for that row (the guards of packboost/backends/cuda/frontier_cuda.cu:214-231
// and 953-966).  A malformed ensemble therefore cannot hang the device or read outside its buffers.

#include "common.cuh"

namespace pb {

namespace {

struct PredictRowsArgs {
    const uint8_t* codes;
    int64_t n_rows;
    int64_t pitch_row;
    const int32_t* feature;
    const int32_t* threshold;
    const int32_t* left;
    const int32_t* right;
    const float* value;
    const uint8_t* is_leaf;
    const int32_t* tree_offsets;
    const int32_t* repeat;
    int n_trees;
    float weight;
    float* out;
    const float* init;
    int rows_per_cta;
    int stage;  // 1: the CTA's rows are staged in shared memory
    int n_codes;  // codes held by one row (pitch_row * 8 / code_bits): bound of a feature index
};

template <int BITS>
__device__ __forceinline__ int code_at(const uint8_t* row, int f) {
    if (BITS == 4) return (row[f >> 1] >> ((f & 1) * 4)) & 0xF;
    return row[f];
}

// One thread per row; the ensemble is walked in tree order and the prediction is accumulated
// as out = out + weight * leaf with separately rounded product and sum, which is what a loop
// of float32 tensor operations over the trees produces.
template <int BITS>
__global__ void __launch_bounds__(128) predict_rows_kernel(PredictRowsArgs a) {
    extern __shared__ __align__(16) uint8_t s_rows[];
    const int64_t row0 = (int64_t)blockIdx.x * a.rows_per_cta;
    const int nr = (int)min((int64_t)a.rows_per_cta, a.n_rows - row0);
    if (nr <= 0) return;
    if (a.stage) {
        const int64_t n16 = (int64_t)nr * a.pitch_row / 16;
        const uint4* src = reinterpret_cast<const uint4*>(a.codes + row0 * a.pitch_row);
        uint4* dst = reinterpret_cast<uint4*>(s_rows);
        for (int64_t i = threadIdx.x; i < n16; i += blockDim.x) dst[i] = __ldg(src + i);
        __syncthreads();
    }
    for (int lr = threadIdx.x; lr < nr; lr += blockDim.x) {
        const uint8_t* row = a.stage ? (s_rows + (int64_t)lr * a.pitch_row) : (a.codes + (row0 + lr) * a.pitch_row);
        float acc = a.init ? a.init[row0 + lr] : 0.f;
        for (int t = 0; t < a.n_trees; ++t) {
            const int base = __ldg(a.tree_offsets + t);
            const int n_t = __ldg(a.tree_offsets + t + 1) - base;  // nodes of this tree
            int node = 0, steps = 0;
            bool good = n_t > 0;
            while (good && !__ldg(a.is_leaf + base + node)) {
                const int f = __ldg(a.feature + base + node);
                const int thr = __ldg(a.threshold + base + node);
                if ((unsigned)f >= (unsigned)a.n_codes || ++steps > n_t) { good = false; break; }
                node = (code_at<BITS>(row, f) <= thr) ? __ldg(a.left + base + node) : __ldg(a.right + base + node);
                good = (unsigned)node < (unsigned)n_t;
            }
            const float term = good ? __fmul_rn(a.weight, __ldg(a.value + base + node)) : 0.f;
            const int rep = a.repeat ? __ldg(a.repeat + t) : 1;
            for (int k = 0; k < rep; ++k) acc = __fadd_rn(acc, term);
        }
        a.out[row0 + lr] = acc;
    }
}

// Packed ensemble: one 8-byte word pair per node,
//   x = feature (bits 0-15) | threshold (bits 16-23) | leaf flag (bit 31)
//   y = tree-relative index of the left child (the right child is the next node, which is how
//       the trees are numbered when they are grown) or, for a leaf, the bits of its float value.
// A thread owns one row and walks kWay trees at a time so that their dependent node loads
// overlap; the leaf terms are still added in tree order.
struct PredictPackedArgs {
    const uint8_t* codes;
    int64_t n_rows;
    int64_t pitch_row;
    const uint2* nodes;
    const int32_t* tree_offsets;
    const int32_t* repeat;
    int n_trees;
    float weight;
    float* out;
    const float* init;
    int rows_per_cta;
    int stage;
    int trees_per_batch;
    int n_codes;         // codes held by one row: bound of a feature index
    int max_tree_nodes;  // node count of the largest tree: bound of a walk
};

// kTpr threads share a row (they sit in the same warp): thread q walks trees t0+q, t0+kTpr+q, ...
// of each group of kTpr*kWay consecutive trees, kWay at a time so that their dependent node
// loads overlap, and the leaf terms are then added in tree order by passing them to the row's
// first thread with shuffles — the float32 sum stays the sequential one.
constexpr int kTpr = 4;
constexpr int kWay = 4;

constexpr int kStageNodes = 4096;  // nodes per staged batch of trees (32 KB), two buffers

__device__ __forceinline__ void cp_async8(void* smem_dst, const void* gmem_src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// The CTA keeps its rows' codes in shared memory and streams the ensemble through two
// shared-memory buffers in batches of `trees_per_batch` trees (asynchronous 8-byte copies, the
// next batch in flight while the current one is walked), so a node visit is two shared-memory
// loads instead of a cache-line lookup per lane.
template <int BITS>
__global__ void __launch_bounds__(512) predict_rows_packed_kernel(PredictPackedArgs a) {
    extern __shared__ __align__(16) uint8_t s_rows[];
    const int64_t row0 = (int64_t)blockIdx.x * a.rows_per_cta;
    const int nr = (int)min((int64_t)a.rows_per_cta, a.n_rows - row0);
    if (nr <= 0) return;
    uint2* s_nodes = reinterpret_cast<uint2*>(s_rows + (size_t)a.rows_per_cta * a.pitch_row * (a.stage ? 1 : 0));
    if (a.stage) {
        const int64_t n16 = (int64_t)nr * a.pitch_row / 16;
        const uint4* src = reinterpret_cast<const uint4*>(a.codes + row0 * a.pitch_row);
        uint4* dst = reinterpret_cast<uint4*>(s_rows);
        for (int64_t i = threadIdx.x; i < n16; i += blockDim.x) dst[i] = __ldg(src + i);
    }
    const int TB = a.trees_per_batch;  // 0: trees too large to stage, nodes are read from global memory
    const int q = threadIdx.x % kTpr;
    const int lane = threadIdx.x & 31;
    const int quad_base = lane - q;  // lane of the row's first thread
    const int rows_per_pass = blockDim.x / kTpr;
    const int n_batches = TB ? (a.n_trees + TB - 1) / TB : 1;

    auto prefetch = [&](int b) {
        const int ta = b * TB, tb = min(a.n_trees, ta + TB);
        const int o0 = __ldg(a.tree_offsets + ta), o1 = __ldg(a.tree_offsets + tb);
        uint2* dst = s_nodes + (size_t)(b & 1) * kStageNodes;
        const int n_copy = min(o1 - o0, kStageNodes);
        for (int i = threadIdx.x; i < n_copy; i += blockDim.x) cp_async8(dst + i, a.nodes + o0 + i);
        cp_async_commit();
    };

    // every warp runs the same number of passes, batches and tree groups, so the shuffles below
    // always see all 32 lanes; threads whose row is past the end compute on row 0 and do not store
    for (int lr0 = 0; lr0 < nr; lr0 += rows_per_pass) {
        const int lr_raw = lr0 + threadIdx.x / kTpr;
        const bool has_row = lr_raw < nr;
        const int lr = has_row ? lr_raw : 0;
        const uint8_t* row = a.stage ? (s_rows + (int64_t)lr * a.pitch_row) : (a.codes + (row0 + lr) * a.pitch_row);
        float acc = a.init ? a.init[row0 + lr] : 0.f;
        if (TB) prefetch(0);
        for (int b = 0; b < n_batches; ++b) {
            const int ta = TB ? b * TB : 0, tb = TB ? min(a.n_trees, ta + TB) : a.n_trees;
            const uint2* node_base = a.nodes;
            int off_shift = 0;
            if (TB) {
                if (b + 1 < n_batches) {
                    prefetch(b + 1);
                    cp_async_wait<1>();
                } else {
                    cp_async_wait<0>();
                }
                __syncthreads();  // batch b (and, on the first batch, the rows) are in shared memory
                node_base = s_nodes + (size_t)(b & 1) * kStageNodes;
                off_shift = __ldg(a.tree_offsets + ta);
            } else {
                __syncthreads();
            }
            for (int t0 = ta; t0 < tb; t0 += kTpr * kWay) {
                const uint2* base[kWay];
                uint2 nd[kWay];
                uint32_t lim[kWay];  // nodes of the tree
#pragma unroll
                for (int u = 0; u < kWay; ++u) {
                    const int t = min(t0 + u * kTpr + q, tb - 1);
                    const int o = __ldg(a.tree_offsets + t);
                    lim[u] = (uint32_t)max(__ldg(a.tree_offsets + t + 1) - o, 0);
                    if (TB && ((unsigned)(o - off_shift) > (unsigned)kStageNodes ||
                               lim[u] > (uint32_t)kStageNodes - (uint32_t)(o - off_shift)))
                        lim[u] = 0u;  // not wholly inside the staged batch
                    base[u] = node_base + (o - off_shift);
                    nd[u] = lim[u] ? base[u][0] : make_uint2(0x80000000u, 0u);
                }
                bool any = true;
                for (int steps = 0; any && steps <= a.max_tree_nodes; ++steps) {
                    any = false;
#pragma unroll
                    for (int u = 0; u < kWay; ++u) {
                        if (!(nd[u].x >> 31)) {
                            const int f = nd[u].x & 0xFFFF;
                            const int thr = (nd[u].x >> 16) & 0xFF;
                            const uint32_t child = nd[u].y + ((f < a.n_codes && code_at<BITS>(row, min(f, a.n_codes - 1)) > thr) ? 1u : 0u);
                            // a child outside the tree or a feature outside the row ends the walk with 0
                            const bool good = (child < lim[u]) & (f < a.n_codes);
                            nd[u] = good ? base[u][child] : make_uint2(0x80000000u, 0u);
                            any = true;
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < kWay; ++u)
                    if (!(nd[u].x >> 31)) nd[u] = make_uint2(0x80000000u, 0u);  // step cap reached: 0
                // ordered accumulation: tree t0 + u*kTpr + qq for u, then qq, ascending
#pragma unroll
                for (int u = 0; u < kWay; ++u) {
                    const float mine = __fmul_rn(a.weight, __uint_as_float(nd[u].y));
#pragma unroll
                    for (int qq = 0; qq < kTpr; ++qq) {
                        const float term = __shfl_sync(0xFFFFFFFFu, mine, quad_base + qq);
                        const int t = t0 + u * kTpr + qq;
                        if (t < tb) {
                            const int rep = a.repeat ? __ldg(a.repeat + t) : 1;
                            for (int k = 0; k < rep; ++k) acc = __fadd_rn(acc, term);
                        }
                    }
                }
            }
            __syncthreads();  // the buffer of batch b may be overwritten by the prefetch of batch b + 2
        }
        if (has_row && q == 0) a.out[row0 + lr] = acc;
    }
}

// The common case of the packed predictor — rows and tree batches both staged in shared memory —
// with every address a 32-bit shared-memory address (the generic form above resolves the address
// space on each of its two loads per node visit and carries 64-bit pointers) and the tree offsets
// of a batch staged next to its nodes, so that a node visit is two shared loads and a handful of
// integer instructions.  Same traversal and the same ordered accumulation as above.
__device__ __forceinline__ uint32_t lds_u8(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];\n" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds_v2(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gmem_src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d), "l"(gmem_src) : "memory");
}

constexpr int kStageTrees = 1024;  // most trees of one staged batch (their offsets are staged too)

template <int BITS>
__global__ void __launch_bounds__(512) predict_rows_packed_smem_kernel(PredictPackedArgs a) {
    extern __shared__ __align__(16) uint8_t s_rows[];  // rows | nodes [2][kStageNodes] | offsets [2][kStageTrees + 1]
    const int64_t row0 = (int64_t)blockIdx.x * a.rows_per_cta;
    const int nr = (int)min((int64_t)a.rows_per_cta, a.n_rows - row0);
    if (nr <= 0) return;
    uint2* s_nodes = reinterpret_cast<uint2*>(s_rows + (size_t)a.rows_per_cta * a.pitch_row);
    int32_t* s_offs = reinterpret_cast<int32_t*>(s_nodes + 2 * kStageNodes);
    uint2* s_zero = reinterpret_cast<uint2*>(s_offs + 2 * (kStageTrees + 1));  // a leaf of value 0
    if (threadIdx.x == 0) *s_zero = make_uint2(0x80000000u, 0u);
    {
        const int64_t n16 = (int64_t)nr * a.pitch_row / 16;
        const uint4* src = reinterpret_cast<const uint4*>(a.codes + row0 * a.pitch_row);
        uint4* dst = reinterpret_cast<uint4*>(s_rows);
        for (int64_t i = threadIdx.x; i < n16; i += blockDim.x) dst[i] = __ldg(src + i);
    }
    const uint32_t rows_addr = (uint32_t)__cvta_generic_to_shared(s_rows);
    const uint32_t nodes_addr = (uint32_t)__cvta_generic_to_shared(s_nodes);
    const uint32_t offs_addr = (uint32_t)__cvta_generic_to_shared(s_offs);
    const uint32_t zero_leaf = (uint32_t)__cvta_generic_to_shared(s_zero);
    const uint32_t fmax = (uint32_t)a.n_codes - 1u;
    const int TB = a.trees_per_batch;
    const int q = threadIdx.x % kTpr;
    const int lane = threadIdx.x & 31;
    const int quad_base = lane - q;
    const int rows_per_pass = blockDim.x / kTpr;
    const int n_batches = (a.n_trees + TB - 1) / TB;

    auto prefetch = [&](int b) {
        const int ta = b * TB, tb = min(a.n_trees, ta + TB);
        const int o0 = __ldg(a.tree_offsets + ta), o1 = __ldg(a.tree_offsets + tb);
        uint2* dst = s_nodes + (size_t)(b & 1) * kStageNodes;
        const int n_copy = min(o1 - o0, kStageNodes);  // (a batch larger than the buffer: its tail trees yield 0)
        for (int i = threadIdx.x; i < n_copy; i += blockDim.x) cp_async8(dst + i, a.nodes + o0 + i);
        int32_t* od = s_offs + (size_t)(b & 1) * (kStageTrees + 1);
        for (int i = threadIdx.x; i <= tb - ta; i += blockDim.x) cp_async4(od + i, a.tree_offsets + ta + i);
        cp_async_commit();
    };

    for (int lr0 = 0; lr0 < nr; lr0 += rows_per_pass) {
        const int lr_raw = lr0 + threadIdx.x / kTpr;
        const bool has_row = lr_raw < nr;
        const int lr = has_row ? lr_raw : 0;
        const uint32_t row = rows_addr + (uint32_t)lr * (uint32_t)a.pitch_row;
        float acc = a.init ? a.init[row0 + lr] : 0.f;
        prefetch(0);
        for (int b = 0; b < n_batches; ++b) {
            const int ta = b * TB, tb = min(a.n_trees, ta + TB);
            if (b + 1 < n_batches) {
                prefetch(b + 1);
                cp_async_wait<1>();
            } else {
                cp_async_wait<0>();
            }
            __syncthreads();  // batch b (and, on the first batch, the rows) are in shared memory
            const uint32_t nbase = nodes_addr + (uint32_t)(b & 1) * (kStageNodes * 8u);
            const uint32_t obase = offs_addr + (uint32_t)(b & 1) * ((kStageTrees + 1) * 4u);
            const uint32_t off_shift = lds_u32(obase);
            for (int t0 = ta; t0 < tb; t0 += kTpr * kWay) {
                uint32_t base[kWay];
                uint2 nd[kWay];
                uint32_t lim[kWay];  // nodes of the tree
#pragma unroll
                for (int u = 0; u < kWay; ++u) {
                    const int t = min(t0 + u * kTpr + q, tb - 1);
                    const uint32_t o = lds_u32(obase + (uint32_t)(t - ta) * 4u);
                    const uint32_t rel = o - off_shift;
                    lim[u] = lds_u32(obase + (uint32_t)(t - ta) * 4u + 4u) - o;
                    // a tree that is empty or not wholly inside the staged batch yields 0
                    if (rel > (uint32_t)kStageNodes || lim[u] > (uint32_t)kStageNodes - rel) lim[u] = 0u;
                    base[u] = nbase + rel * 8u;
                    nd[u] = lds_v2(lim[u] ? base[u] : zero_leaf);
                }
                bool any = true;
                for (int steps = 0; any && steps <= a.max_tree_nodes; ++steps) {
                    any = false;
#pragma unroll
                    for (int u = 0; u < kWay; ++u) {
                        if (!(nd[u].x >> 31)) {
                            // a feature index past the row reads the row's last code and ends the walk
                            const uint32_t f = min(nd[u].x & 0xFFFFu, fmax);
                            const uint32_t thr = (nd[u].x >> 16) & 0xFFu;
                            uint32_t code;
                            if (BITS == 4) code = (lds_u8(row + (f >> 1)) >> ((f & 1u) * 4u)) & 0xFu;
                            else code = lds_u8(row + f);
                            const uint32_t child = nd[u].y + ((code > thr) ? 1u : 0u);
                            // a child outside the tree (or a bad feature) ends the walk at the zero leaf
                            const bool good = (child < lim[u]) & ((nd[u].x & 0xFFFFu) <= fmax);
                            nd[u] = lds_v2(good ? base[u] + child * 8u : zero_leaf);
                            any = true;
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < kWay; ++u)
                    if (!(nd[u].x >> 31)) nd[u] = make_uint2(0x80000000u, 0u);  // step cap reached: 0
#pragma unroll
                for (int u = 0; u < kWay; ++u) {
                    const float mine = __fmul_rn(a.weight, __uint_as_float(nd[u].y));
#pragma unroll
                    for (int qq = 0; qq < kTpr; ++qq) {
                        const float term = __shfl_sync(0xFFFFFFFFu, mine, quad_base + qq);
                        const int t = t0 + u * kTpr + qq;
                        if (t < tb) {
                            if (a.repeat) {
                                const int rep = __ldg(a.repeat + t);
                                for (int k = 0; k < rep; ++k) acc = __fadd_rn(acc, term);
                            } else {
                                acc = __fadd_rn(acc, term);
                            }
                        }
                    }
                }
            }
            __syncthreads();  // the buffers of batch b may be overwritten by the prefetch of batch b + 2
        }
        if (has_row && q == 0) a.out[row0 + lr] = acc;
    }
}


__global__ void __launch_bounds__(256) predict_bins_fm_kernel(
    const uint8_t* __restrict__ bins, int n_features, int64_t n_rows, const int32_t* __restrict__ feature,
    const int32_t* __restrict__ threshold, const int32_t* __restrict__ left, const int32_t* __restrict__ right,
    const float* __restrict__ value, const uint8_t* __restrict__ is_leaf, int n_nodes, float* __restrict__ out) {
    for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < n_rows; r += (int64_t)gridDim.x * blockDim.x) {
        int node = 0, steps = 0;
        bool good = true;
        while (!__ldg(is_leaf + node)) {
            const int f = __ldg(feature + node);
            if ((unsigned)f >= (unsigned)n_features || ++steps > n_nodes) { good = false; break; }
            node = ((int)bins[(int64_t)f * n_rows + r] <= __ldg(threshold + node)) ? __ldg(left + node) : __ldg(right + node);
            if ((unsigned)node >= (unsigned)n_nodes) { good = false; break; }
        }
        out[r] = good ? __ldg(value + node) : 0.f;
    }
}

__global__ void __launch_bounds__(256) predict_pack_fm_kernel(
    const uint8_t* __restrict__ bins, int n_features, int64_t n_rows, const int32_t* __restrict__ feature,
    const int32_t* __restrict__ threshold, const int32_t* __restrict__ left_abs, const int32_t* __restrict__ right_abs,
    const float* __restrict__ value, const uint8_t* __restrict__ is_leaf, const int32_t* __restrict__ offsets,
    int n_trees, float tree_weight, float* __restrict__ out) {
    for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < n_rows; r += (int64_t)gridDim.x * blockDim.x) {
        float sum = 0.f;
        for (int t = 0; t < n_trees; ++t) {
            int node = __ldg(offsets + t);
            const int end = __ldg(offsets + t + 1);
            if (node >= end) continue;
            const int begin = node;
            int steps = 0;
            bool good = true;
            while (!__ldg(is_leaf + node)) {
                const int f = __ldg(feature + node);
                if ((unsigned)f >= (unsigned)n_features || ++steps > end - begin) { good = false; break; }
                node = ((int)bins[(int64_t)f * n_rows + r] <= __ldg(threshold + node)) ? __ldg(left_abs + node)
                                                                                       : __ldg(right_abs + node);
                if (node < begin || node >= end) { good = false; break; }
            }
            if (good) sum = __fadd_rn(sum, __ldg(value + node));
        }
        out[r] = __fmul_rn(tree_weight, sum);
    }
}

}  // namespace
}  // namespace pb

using namespace pb;

extern "C" int pb_predict_rows(const uint8_t* codes, int64_t n_rows, int64_t pitch_row, int64_t code_bits,
                               const int32_t* feature, const int32_t* threshold, const int32_t* left,
                               const int32_t* right, const float* value, const uint8_t* is_leaf,
                               const int32_t* tree_offsets, const int32_t* repeat, int64_t n_trees, float weight,
                               float* out, const float* init, void* stream_) {
    PB_REQUIRE(codes && feature && threshold && left && right && value && is_leaf && tree_offsets && out,
               "null buffer");
    PB_REQUIRE(code_bits == 4 || code_bits == 8, "code_bits must be 4 or 8");
    PB_REQUIRE(pitch_row >= 16 && pitch_row % 16 == 0, "pitch_row must be a positive multiple of 16");
    PB_REQUIRE(((uintptr_t)codes % 16) == 0, "codes must be 16-byte aligned");
    PB_REQUIRE(n_trees >= 0 && n_trees < (1ll << 31), "n_trees out of range");
    if (n_rows <= 0) return PB_OK;
    cudaStream_t stream = (cudaStream_t)stream_;
    PredictRowsArgs a{codes, n_rows, pitch_row, feature, threshold, left, right, value, is_leaf,
                      tree_offsets, repeat, (int)n_trees, weight, out, init, 128, 1,
                      (int)((pitch_row < (1 << 27) ? pitch_row : (1 << 27)) * (code_bits == 4 ? 2 : 1))};
    const int64_t budget = 160 * 1024;
    int rows = (int)(budget / pitch_row);
    if (rows >= 128) rows = 128;
    else rows = rows / 32 * 32;
    size_t smem = 0;
    if (rows < 32) {
        a.stage = 0;
        a.rows_per_cta = 128;
    } else {
        a.rows_per_cta = rows;
        smem = (size_t)rows * pitch_row;
    }
    const unsigned grid = (unsigned)((n_rows + a.rows_per_cta - 1) / a.rows_per_cta);
    if (code_bits == 4) {
        if (smem > 48 * 1024)
            PB_CUDA_TRY(cudaFuncSetAttribute(predict_rows_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        predict_rows_kernel<4><<<grid, 128, smem, stream>>>(a);
    } else {
        if (smem > 48 * 1024)
            PB_CUDA_TRY(cudaFuncSetAttribute(predict_rows_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        predict_rows_kernel<8><<<grid, 128, smem, stream>>>(a);
    }
    count_launch(1);
    PB_LAUNCH_CHECK("predict_rows_kernel");
    return PB_OK;
}

static unsigned row_blocks(int64_t n) {
    int64_t b = (n + 255) / 256;
    if (b > 148 * 16) b = 148 * 16;
    return (unsigned)(b < 1 ? 1 : b);
}

extern "C" int pb_predict_bins_fm(const uint8_t* bins, int64_t n_features, int64_t n_rows, const int32_t* feature,
                                  const int32_t* threshold, const int32_t* left, const int32_t* right,
                                  const float* value, const uint8_t* is_leaf, int64_t n_nodes, float* out,
                                  void* stream) {
    PB_REQUIRE(bins && feature && threshold && left && right && value && is_leaf && out, "null buffer");
    PB_REQUIRE(n_features >= 1 && n_nodes >= 1, "bad shape");
    if (n_rows <= 0) return PB_OK;
    PB_REQUIRE(n_features < (1ll << 31) && n_nodes < (1ll << 31), "bad shape");
    predict_bins_fm_kernel<<<row_blocks(n_rows), 256, 0, (cudaStream_t)stream>>>(
        bins, (int)n_features, n_rows, feature, threshold, left, right, value, is_leaf, (int)n_nodes, out);
    count_launch(1);
    PB_LAUNCH_CHECK("predict_bins_fm_kernel");
    return PB_OK;
}

extern "C" int pb_predict_pack_fm(const uint8_t* bins, int64_t n_features, int64_t n_rows, const int32_t* feature,
                                  const int32_t* threshold, const int32_t* left_abs, const int32_t* right_abs,
                                  const float* value, const uint8_t* is_leaf, const int32_t* offsets, int64_t n_trees,
                                  float tree_weight, float* out, void* stream) {
    PB_REQUIRE(bins && feature && threshold && left_abs && right_abs && value && is_leaf && offsets && out,
               "null buffer");
    PB_REQUIRE(n_features >= 1 && n_trees >= 0, "bad shape");
    if (n_rows <= 0) return PB_OK;
    PB_REQUIRE(n_features < (1ll << 31) && n_trees < (1ll << 31), "bad shape");
    predict_pack_fm_kernel<<<row_blocks(n_rows), 256, 0, (cudaStream_t)stream>>>(
        bins, (int)n_features, n_rows, feature, threshold, left_abs, right_abs, value, is_leaf, offsets, (int)n_trees, tree_weight, out);
    count_launch(1);
    PB_LAUNCH_CHECK("predict_pack_fm_kernel");
    return PB_OK;
}

extern "C" int pb_predict_rows_packed(const uint8_t* codes, int64_t n_rows, int64_t pitch_row, int64_t code_bits,
                                      const void* nodes, const int32_t* tree_offsets, const int32_t* repeat,
                                      int64_t n_trees, int64_t max_tree_nodes, float weight, float* out,
                                      const float* init, void* stream_) {
    PB_REQUIRE(codes && nodes && tree_offsets && out, "null buffer");
    PB_REQUIRE(code_bits == 4 || code_bits == 8, "code_bits must be 4 or 8");
    PB_REQUIRE(pitch_row >= 16 && pitch_row % 16 == 0, "pitch_row must be a positive multiple of 16");
    PB_REQUIRE(((uintptr_t)codes % 16) == 0 && ((uintptr_t)nodes % 8) == 0, "codes / nodes are misaligned");
    PB_REQUIRE(n_trees >= 0 && n_trees < (1ll << 31) && max_tree_nodes >= 1, "tree counts out of range");
    if (n_rows <= 0 || n_trees == 0) {
        if (n_rows > 0) {
            if (init) PB_CUDA_TRY(cudaMemcpyAsync(out, init, (size_t)n_rows * 4, cudaMemcpyDeviceToDevice, (cudaStream_t)stream_));
            else PB_CUDA_TRY(cudaMemsetAsync(out, 0, (size_t)n_rows * 4, (cudaStream_t)stream_));
        }
        return PB_OK;
    }
    cudaStream_t stream = (cudaStream_t)stream_;
    PredictPackedArgs a{codes, n_rows, pitch_row, static_cast<const uint2*>(nodes), tree_offsets, repeat,
                        (int)n_trees, weight, out, init, 128, 1, 0,
                        (int)((pitch_row < (1 << 27) ? pitch_row : (1 << 27)) * (code_bits == 4 ? 2 : 1)),
                        (int)(max_tree_nodes < (1 << 30) ? max_tree_nodes : (1 << 30))};
    // trees per staged batch: a multiple of the group walked at once, as many as the buffer holds
    const int group = kTpr * kWay;
    int tb = (int)(kStageNodes / max_tree_nodes) / group * group;
    if (tb > kStageTrees) tb = kStageTrees / group * group;
    a.trees_per_batch = tb;  // 0: no staging
    const size_t stage_bytes = tb ? (size_t)2 * kStageNodes * sizeof(uint2) + (size_t)2 * (kStageTrees + 1) * 4 + 8 : 0;
    const int64_t budget = 224 * 1024 - (int64_t)stage_bytes;
    int rows = (int)(budget / pitch_row);
    if (rows > 128) rows = 128;
    rows = rows / 8 * 8;
    size_t smem = stage_bytes;
    if (rows < 8) {
        a.stage = 0;
        a.rows_per_cta = 128;
    } else {
        a.rows_per_cta = rows;
        smem += (size_t)rows * pitch_row;
    }
    const unsigned grid = (unsigned)((n_rows + a.rows_per_cta - 1) / a.rows_per_cta);
    const int threads = (a.rows_per_cta * kTpr + 31) / 32 * 32;
    if (a.stage && tb > 0) {  // rows and trees both staged: the all-shared-memory form
        if (code_bits == 4) {
            if (smem > 48 * 1024)
                PB_CUDA_TRY(cudaFuncSetAttribute(predict_rows_packed_smem_kernel<4>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            predict_rows_packed_smem_kernel<4><<<grid, threads, smem, stream>>>(a);
        } else {
            if (smem > 48 * 1024)
                PB_CUDA_TRY(cudaFuncSetAttribute(predict_rows_packed_smem_kernel<8>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            predict_rows_packed_smem_kernel<8><<<grid, threads, smem, stream>>>(a);
        }
    } else if (code_bits == 4) {
        if (smem > 48 * 1024)
            PB_CUDA_TRY(cudaFuncSetAttribute(predict_rows_packed_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        predict_rows_packed_kernel<4><<<grid, threads, smem, stream>>>(a);
    } else {
        if (smem > 48 * 1024)
            PB_CUDA_TRY(cudaFuncSetAttribute(predict_rows_packed_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        predict_rows_packed_kernel<8><<<grid, threads, smem, stream>>>(a);
    }
    count_launch(1);
    PB_LAUNCH_CHECK("predict_rows_packed_kernel");
    return PB_OK;
}
