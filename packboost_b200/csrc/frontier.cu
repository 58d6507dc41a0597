// Round bookkeeping that stays on the device: gradient update and quantisation, winner
// selection with the reference's tie-break, child numbering, leaf values, the row -> node
// map update and the leaf-delta table for the prediction update.

#include <mutex>

#include "common.cuh"

namespace pb {

namespace {

constexpr int kRowThreads = 256;

__device__ __forceinline__ float scale_from_max(float max_abs, int gq_bits, float* inv) {
    // power of two with max_abs * scale < 2^gq_bits
    if (!(max_abs > 0.f) || !isfinite(max_abs)) {
        *inv = 1.f;
        return 1.f;
    }
    int ex;
    frexpf(max_abs, &ex);  // max_abs = m * 2^ex, m in [0.5, 1)
    int sh = gq_bits - ex;
    sh = max(-100, min(100, sh));
    *inv = ldexpf(1.f, -sh);
    return ldexpf(1.f, sh);
}

__global__ void round_reset_kernel(Ctl c) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        c.head->max_abs_bits = 0u;
        c.head->root_gq = 0;
        c.head->n_tree_nodes = 1;
        c.head->select_ticket = 0u;
        for (int i = 0; i < kMaxDepth + 2; ++i) {
            c.head->n_ctx[i] = 0;
            c.head->any_dir[i] = 0;
        }
    }
}

// preds += delta[leaf] (optional), track max |preds - y|.  Four rows per thread and step (all row
// arrays are 16-byte aligned; y and preds hold n rows, so their last group is read row by row).
__global__ void __launch_bounds__(kRowThreads) preds_absmax_kernel(
    float* __restrict__ preds, const float* __restrict__ y, const uint16_t* __restrict__ leaf,
    const float* __restrict__ delta, int64_t n, int apply, CtlHead* head) {
    float m = 0.f;
    const int64_t n4 = (n + 3) >> 2;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i << 2;
        float p[4] = {0.f, 0.f, 0.f, 0.f}, yy[4] = {0.f, 0.f, 0.f, 0.f};
        if (r + 3 < n) {
            const float4 pv = *reinterpret_cast<const float4*>(preds + r);
            const float4 yv = *reinterpret_cast<const float4*>(y + r);
            p[0] = pv.x; p[1] = pv.y; p[2] = pv.z; p[3] = pv.w;
            yy[0] = yv.x; yy[1] = yv.y; yy[2] = yv.z; yy[3] = yv.w;
        } else {  // (y and preds hold n rows, not the padded count)
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (r + u < n) {
                    p[u] = preds[r + u];
                    yy[u] = y[r + u];
                }
        }
        if (apply) {
            const uint2 lv = *reinterpret_cast<const uint2*>(leaf + r);
            const uint32_t l[4] = {lv.x & 0xFFFFu, lv.x >> 16, lv.y & 0xFFFFu, lv.y >> 16};
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (r + u < n) p[u] = __fadd_rn(p[u], delta[l[u]]);
            if (r + 3 < n) {
                *reinterpret_cast<float4*>(preds + r) = make_float4(p[0], p[1], p[2], p[3]);
            } else {
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (r + u < n) preds[r + u] = p[u];
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (r + u < n) m = fmaxf(m, fabsf(__fsub_rn(p[u], yy[u])));
    }
    for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, d));
    __shared__ float wm[kRowThreads / 32];
    if ((threadIdx.x & 31) == 0) wm[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < kRowThreads / 32; ++i) m = fmaxf(m, wm[i]);
        atomicMax(&head->max_abs_bits, __float_as_uint(m));  // non-negative floats order like their bits
    }
}

// gq = rint((preds - y) * scale); rows back to the root; sum of gq.  Four rows per thread and step.
__global__ void __launch_bounds__(kRowThreads) quantise_kernel(
    const float* __restrict__ preds, const float* __restrict__ y, int32_t* __restrict__ gq,
    uint16_t* __restrict__ slot, uint16_t* __restrict__ leaf, int64_t n, int64_t n_pad, CtlHead* head, int gq_bits) {
    float inv;
    const float scale = scale_from_max(__uint_as_float(head->max_abs_bits), gq_bits, &inv);
    long long acc = 0;
    const int64_t n4 = n_pad >> 2;  // n_pad is a multiple of 256
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i << 2;
        int q[4] = {0, 0, 0, 0};
        uint32_t sl[4] = {kSlotNone, kSlotNone, kSlotNone, kSlotNone};
        if (r < n) {
            float p[4] = {0.f, 0.f, 0.f, 0.f}, yy[4] = {0.f, 0.f, 0.f, 0.f};
            if (r + 3 < n) {
                const float4 pv = *reinterpret_cast<const float4*>(preds + r);
                const float4 yv = *reinterpret_cast<const float4*>(y + r);
                p[0] = pv.x; p[1] = pv.y; p[2] = pv.z; p[3] = pv.w;
                yy[0] = yv.x; yy[1] = yv.y; yy[2] = yv.z; yy[3] = yv.w;
            } else {  // (y and preds hold n rows, not the padded count)
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (r + u < n) {
                        p[u] = preds[r + u];
                        yy[u] = y[r + u];
                    }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (r + u < n) {
                    q[u] = __float2int_rn(__fmul_rn(__fsub_rn(p[u], yy[u]), scale));
                    sl[u] = 0u;
                    acc += q[u];
                }
        }
        *reinterpret_cast<int4*>(gq + r) = make_int4(q[0], q[1], q[2], q[3]);
        *reinterpret_cast<uint2*>(slot + r) = make_uint2(sl[0] | (sl[1] << 16), sl[2] | (sl[3] << 16));
        *reinterpret_cast<uint2*>(leaf + r) = make_uint2(0u, 0u);
    }
    for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, d);
    __shared__ long long ws[kRowThreads / 32];
    if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < kRowThreads / 32; ++i) acc += ws[i];
        atomicAdd(reinterpret_cast<unsigned long long*>(&head->root_gq), (unsigned long long)acc);
    }
}

__global__ void root_kernel(Ctl c, int64_t n, int min_leaf, double lambda, int gq_bits) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    float inv;
    const float scale = scale_from_max(__uint_as_float(c.head->max_abs_bits), gq_bits, &inv);
    c.head->scale = scale;
    c.head->inv_scale = inv;
    const long long g = c.head->root_gq;
    FrontierNode fn;
    fn.tree_node = 0;
    fn.count = (int32_t)n;
    fn.gq = g;
    c.frontier[0][0] = fn;
    c.head->n_ctx[0] = (n >= 2 * (int64_t)min_leaf) ? 1 : 0;
    c.head->any_dir[0] = (g != 0) ? 1 : 0;
    const float g32 = __fmul_rn(__ll2float_rn(g), inv);
    const double v = (n > 0) ? (-(double)g32 / ((double)(float)n + lambda)) : 0.0;
    c.node_value[0] = v;
    pb_round_log_header* h = c.log_head;
    h->root_value = v;
    h->scale = scale;
    h->max_abs_grad = __uint_as_float(c.head->max_abs_bits);
    h->root_gq = g;
    for (int i = 0; i <= kMaxDepth; ++i) h->n_ctx[i] = 0;
    h->n_ctx[0] = c.head->n_ctx[0];
    h->n_tree_nodes = 1;
}

// ---- winner selection --------------------------------------------------------------------

struct SelectArgs {
    Ctl c;
    int depth;
    int max_depth;
    const Cand* cand;
    int node_stride;
    const int32_t* sampled;  // global feature ids in sampled order
    int n_sampled;
    int block_size;
    const int32_t* thr_ids;
    int n_thr;
    int min_leaf;
    double lambda;
};

// Candidate order inside a feature block: higher score, then larger left count, then the later
// position (exact float equality decides ties, as in the tensor code this replaces).
struct BlockBest {
    float s;
    long long c;
    long long lg;
    int p;
    int k;
    int f;  // global feature id of the candidate
};

__device__ __forceinline__ bool block_better(const BlockBest& x, const BlockBest& y) {
    // true when x beats y
    if (x.p < 0) return false;
    if (y.p < 0) return true;
    if (x.s != y.s) return x.s > y.s;
    if (x.c != y.c) return x.c > y.c;
    return x.p > y.p;
}

// One CTA per frontier node picks the node's winner: its warps take the feature blocks of the
// sampled order in turn (a lane per candidate, butterfly inside the block), thread 0 merges the
// block winners in block order.  The CTA that finishes last (a ticket counter in the control
// block; nobody waits for anybody) then numbers the children of all nodes, builds the next
// frontier and the partition table.
constexpr int kSelThreads = 256;
constexpr int kSelChunk = 64;  // block winners merged per pass

__global__ void __launch_bounds__(kSelThreads) select_kernel(SelectArgs a) {
    Ctl& c = a.c;
    __shared__ BlockBest s_best[kSelChunk];
    __shared__ int s_nan[kSelChunk];
    __shared__ int s_last;
    const int n_ctx = c.head->n_ctx[a.depth];
    const int n = blockIdx.x;
    if (n >= n_ctx) return;
    const FrontierNode* cur = c.frontier[a.depth & 1];
    FrontierNode* nxt = c.frontier[(a.depth + 1) & 1];
    pb_winner* win = c.winners + ((1 << a.depth) - 1);
    const float inv = c.head->inv_scale;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const bool keep_frontier = (a.depth + 1) < a.max_depth;

    // ---- A. this node: in-block winners by the warps, cross-block merge by thread 0 ----
    float best_s = -INFINITY;
    long long best_c = -1, best_lg = 0;
    int best_f = -1, best_t = -1;
    const int n_blocks = (a.n_sampled + a.block_size - 1) / a.block_size;
    for (int blk0 = 0; blk0 < n_blocks; blk0 += kSelChunk) {
        const int blk1 = min(n_blocks, blk0 + kSelChunk);
        for (int blk = blk0 + warp; blk < blk1; blk += n_warps) {
            const int b0 = blk * a.block_size, b1 = min(a.n_sampled, b0 + a.block_size);
            BlockBest mine{-INFINITY, -1, 0, -1, -1, -1};
            bool has_nan = false;
            for (int p = b0 + lane; p < b1; p += 32) {
                const Cand cd = a.cand[(size_t)p * a.node_stride + n];
                if (cd.flags & 1u) has_nan = true;
                if (cd.k < 0) continue;
                // (the k field of a block winner carries the candidate's threshold bin id from here on)
                const BlockBest x{cd.score, (long long)cd.left_count, cd.left_gq, p, (int)((cd.flags >> 8) & 0xFFu), a.sampled[p]};
                if (block_better(x, mine)) mine = x;
            }
            has_nan = __any_sync(0xFFFFFFFFu, has_nan);
            for (int d = 16; d > 0; d >>= 1) {
                BlockBest o;
                o.s = __shfl_xor_sync(0xFFFFFFFFu, mine.s, d);
                o.c = __shfl_xor_sync(0xFFFFFFFFu, mine.c, d);
                o.lg = __shfl_xor_sync(0xFFFFFFFFu, mine.lg, d);
                o.p = __shfl_xor_sync(0xFFFFFFFFu, mine.p, d);
                o.k = __shfl_xor_sync(0xFFFFFFFFu, mine.k, d);
                o.f = __shfl_xor_sync(0xFFFFFFFFu, mine.f, d);
                if (block_better(o, mine)) mine = o;
            }
            if (lane == 0) {
                s_best[blk - blk0] = mine;
                s_nan[blk - blk0] = has_nan ? 1 : 0;
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            // across blocks, in block order: strictly better on (score, left count, feature id, threshold)
            for (int j = 0; j < blk1 - blk0; ++j) {
                const BlockBest& m = s_best[j];
                if (s_nan[j] || m.p < 0) continue;
                const int feat = m.f;
                const int thr = m.k;
                const bool upd = (m.s > best_s) ||
                                 (m.s == best_s && ((m.c > best_c) ||
                                                    (m.c == best_c && ((feat > best_f) || (feat == best_f && thr > best_t)))));
                if (upd) { best_s = m.s; best_c = m.c; best_lg = m.lg; best_f = feat; best_t = thr; }
            }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        const FrontierNode fn = cur[n];
        pb_winner w;
        w.feature = best_f;
        w.threshold = best_t;
        w.score = best_s;
        w.tree_node = fn.tree_node;
        w.left_count = (best_f >= 0) ? best_c : 0;
        w.total_count = fn.count;
        w.left_gq = (best_f >= 0) ? best_lg : 0;
        w.total_gq = fn.gq;
        w.left_id = -1;
        w.right_id = -1;
        const float tg32 = __fmul_rn(__ll2float_rn(fn.gq), inv);
        const float lg32 = __fmul_rn(__ll2float_rn(w.left_gq), inv);
        const float th32 = (float)fn.count;
        const float lh32 = (float)w.left_count;
        w.left_grad = lg32;
        w.total_grad = tg32;
        int flag = 0;
        if (best_f >= 0) {
            w.left_value = -(double)lg32 / ((double)lh32 + a.lambda);
            const double rg = (double)tg32 - (double)lg32;
            const double rh = (double)th32 - (double)lh32;
            w.right_value = -rg / (rh + a.lambda);
            flag = 1;
            if (keep_frontier && w.left_count >= 2ll * a.min_leaf) flag |= 2;
            if (keep_frontier && (w.total_count - w.left_count) >= 2ll * a.min_leaf) flag |= 4;
        } else {
            // no usable candidate: the node stays a leaf with its Newton value
            w.left_value = -(double)tg32 / ((double)th32 + a.lambda);
            w.right_value = w.left_value;
        }
        win[n] = w;
        c.sel_flag[n] = flag;
        __threadfence();  // the winner and the flag are visible before the ticket is
        const unsigned ticket = atomicAdd(&c.head->select_ticket, 1u);
        s_last = (ticket == (unsigned)n_ctx - 1u) ? 1 : 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (threadIdx.x == 0) c.head->select_ticket = 0u;  // ready for the next launch

    // ---- B. (last CTA) exclusive prefix counts of splits and of active children, one warp ----
    // (other CTAs wrote the flags and winners: they are read past the L1 of this SM)
    const volatile int32_t* flags = c.sel_flag;
    __shared__ int s_first_id, s_any_dir;
    if (threadIdx.x == 0) s_any_dir = 0;
    // per 32-node group the number of splits / active children, then their exclusive prefix
    __shared__ int s_grp_id[kMaxCtx / 32 + 1], s_grp_slot[kMaxCtx / 32 + 1];
    const int n_groups = (n_ctx + 31) / 32;
    for (int g = warp; g < n_groups; g += n_warps) {
        const int i = g * 32 + lane;
        const int fl = (i < n_ctx) ? flags[i] : 0;
        int v_id = fl & 1, v_slot = ((fl >> 1) & 1) + ((fl >> 2) & 1);
        for (int d = 16; d > 0; d >>= 1) {
            v_id += __shfl_xor_sync(0xFFFFFFFFu, v_id, d);
            v_slot += __shfl_xor_sync(0xFFFFFFFFu, v_slot, d);
        }
        if (lane == 0) { s_grp_id[g] = v_id; s_grp_slot[g] = v_slot; }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run_id = 0, run_slot = 0;
        for (int g = 0; g < n_groups; ++g) {
            const int t1 = s_grp_id[g], t2 = s_grp_slot[g];
            s_grp_id[g] = run_id;
            s_grp_slot[g] = run_slot;
            run_id += t1;
            run_slot += t2;
        }
        s_first_id = c.head->n_tree_nodes;
        const int next_id = s_first_id + 2 * run_id;
        c.head->n_tree_nodes = next_id;
        c.head->n_ctx[a.depth + 1] = run_slot;
        c.log_head->n_ctx[a.depth] = n_ctx;
        if (a.depth + 1 <= kMaxDepth) c.log_head->n_ctx[a.depth + 1] = run_slot;
        c.log_head->n_tree_nodes = next_id;
    }
    __syncthreads();
    const int first_id = s_first_id;

    // ---- C. (last CTA) child ids, next frontier, partition table: a warp per 32-node group ----
    int any_dir = 0;
    for (int g = warp; g < n_groups; g += n_warps) {
        const int i = g * 32 + lane;
        const int fl = (i < n_ctx) ? flags[i] : 0;
        int v_id = fl & 1, v_slot = ((fl >> 1) & 1) + ((fl >> 2) & 1);
        const int own_id = v_id, own_slot = v_slot;
        for (int d = 1; d < 32; d <<= 1) {
            const int t1 = __shfl_up_sync(0xFFFFFFFFu, v_id, d);
            const int t2 = __shfl_up_sync(0xFFFFFFFFu, v_slot, d);
            if (lane >= d) { v_id += t1; v_slot += t2; }
        }
        if (i >= n_ctx) continue;
        const int ids_before = s_grp_id[g] + v_id - own_id;
        int slot = s_grp_slot[g] + v_slot - own_slot;
        pb_winner w;
        {
            const volatile pb_winner* src = win + i;
            w.feature = src->feature; w.threshold = src->threshold; w.tree_node = src->tree_node;
            w.left_count = src->left_count; w.total_count = src->total_count;
            w.left_gq = src->left_gq; w.total_gq = src->total_gq;
            w.left_value = src->left_value; w.right_value = src->right_value;
        }
        PartEntry pe;
        pe.feature = w.feature;
        pe.threshold = w.threshold;
        pe.slot_left = pe.slot_right = kSlotNone;
        pe.leaf_left = pe.leaf_right = (uint16_t)w.tree_node;
        if (fl & 1) {
            const int lid = first_id + 2 * ids_before;
            win[i].left_id = lid;
            win[i].right_id = lid + 1;
            pe.leaf_left = (uint16_t)lid;
            pe.leaf_right = (uint16_t)(lid + 1);
            c.node_value[lid] = w.left_value;
            c.node_value[lid + 1] = w.right_value;
            if (fl & 2) {
                FrontierNode fn; fn.tree_node = lid; fn.count = (int32_t)w.left_count; fn.gq = w.left_gq;
                nxt[slot] = fn;
                pe.slot_left = (uint16_t)slot++;
                any_dir |= (w.left_gq != 0);
            }
            if (fl & 4) {
                FrontierNode fn; fn.tree_node = lid + 1; fn.count = (int32_t)(w.total_count - w.left_count);
                fn.gq = w.total_gq - w.left_gq;
                nxt[slot] = fn;
                pe.slot_right = (uint16_t)slot;
                any_dir |= (fn.gq != 0);
            }
        } else {
            c.node_value[w.tree_node] = w.left_value;
        }
        c.part[i] = pe;
    }
    if (any_dir) atomicOr(&s_any_dir, 1);
    __syncthreads();
    if (threadIdx.x == 0) c.head->any_dir[a.depth + 1] = s_any_dir;
}

// ---- row -> node map ------------------------------------------------------------------------

template <int BITS>
__device__ __forceinline__ int load_code(const uint8_t* codes, int64_t pitch, int frow, int64_t r) {
    if (BITS == 4) {
        const uint8_t b = codes[(int64_t)frow * pitch + (r >> 1)];
        return (b >> ((r & 1) * 4)) & 0xF;
    }
    return codes[(int64_t)frow * pitch + r];
}

struct PartArgs {
    Ctl c;
    int depth;
    const uint8_t* codes;
    int64_t pitch;
    const int32_t* feat_local;
    uint16_t* slot;
    uint16_t* leaf;
    int64_t n;
    uint32_t* bits;        // goleft_bits output
    const uint32_t* bits_in;  // apply_bits input
    int n_features_total, n_features_local;
};

// mode 0: fused (decide + apply); mode 1: write go-left bits for locally held features;
// mode 2: apply bits
template <int BITS, int MODE>
__global__ void __launch_bounds__(kRowThreads) partition_kernel(PartArgs a) {
    extern __shared__ PartEntry tab[];
    const int n_ctx = a.c.head->n_ctx[a.depth];
    if (n_ctx <= 0) return;
    for (int i = threadIdx.x; i < n_ctx; i += blockDim.x) tab[i] = a.c.part[i];
    __syncthreads();
    // A thread owns eight consecutive rows: their slots and leaves move as one 16-byte word each
    // way, and rows that share a node share code bytes.  (The row arrays are padded past n with
    // slot "none", so the last group needs no special case.)
    constexpr int kRows = 8;
    const int64_t n_groups = (a.n + kRows - 1) / kRows;
    const int64_t n_groups_round = (n_groups + 31) / 32 * 32;  // whole warps: MODE 1 shuffles
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_groups_round; i += stride) {
        const int64_t r8 = i * kRows;
        const bool in = i < n_groups;
        uint4 sv = make_uint4(0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu);
        uint4 lv = make_uint4(0u, 0u, 0u, 0u);
        if (in) {
            sv = *reinterpret_cast<const uint4*>(a.slot + r8);
            if (MODE != 1) lv = *reinterpret_cast<const uint4*>(a.leaf + r8);
        }
        const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
        uint32_t lw[4] = {lv.x, lv.y, lv.z, lv.w};
        uint32_t nsw[4];
        uint32_t in_byte = 0u;
        if (MODE == 2 && in) in_byte = reinterpret_cast<const uint8_t*>(a.bits_in)[i];
        uint32_t left_mask = 0u;
#pragma unroll
        for (int u = 0; u < kRows; ++u) {
            const uint32_t sl = (sw[u >> 1] >> ((u & 1) * 16)) & 0xFFFFu;
            uint32_t new_slot = sl, new_leaf = (lw[u >> 1] >> ((u & 1) * 16)) & 0xFFFFu;
            if (sl != kSlotNone) {
                new_slot = kSlotNone;  // a slot past the frontier, or a node that does not split
                if ((int)sl < n_ctx) {
                    const PartEntry pe = tab[sl];
#ifdef PB_DEBUG_BOUNDS
                    if (pe.feature >= a.n_features_total ||
                        (MODE != 2 && pe.feature >= 0 && a.feat_local[pe.feature] >= a.n_features_local)) {
                        atomicOr(&a.c.head->debug_flags, kDbgFeature);
                        continue;
                    }
#endif
                    if (pe.feature >= 0) {
                        bool left = false;
                        if (MODE == 2) {
                            left = (in_byte >> u) & 1u;
                        } else {
                            const int frow = a.feat_local[pe.feature];
                            if (frow >= 0) left = load_code<BITS>(a.codes, a.pitch, frow, r8 + u) <= pe.threshold;
                        }
                        left_mask |= (left ? 1u : 0u) << u;
                        new_slot = left ? pe.slot_left : pe.slot_right;
                        new_leaf = left ? pe.leaf_left : pe.leaf_right;
                    }
                }
            }
            if ((u & 1) == 0) {
                nsw[u >> 1] = new_slot;
                lw[u >> 1] = (lw[u >> 1] & 0xFFFF0000u) | new_leaf;
            } else {
                nsw[u >> 1] |= new_slot << 16;
                lw[u >> 1] = (lw[u >> 1] & 0x0000FFFFu) | (new_leaf << 16);
            }
        }
        if (MODE == 1) {
            // four threads hold the 32 go-left bits of one word
            const int lane = threadIdx.x & 31;
            uint32_t word = left_mask << ((lane & 3) * 8);
            word |= __shfl_xor_sync(0xFFFFFFFFu, word, 1);
            word |= __shfl_xor_sync(0xFFFFFFFFu, word, 2);
            if ((lane & 3) == 0 && in) a.bits[i >> 2] = word;
        } else if (in) {
            *reinterpret_cast<uint4*>(a.slot + r8) = make_uint4(nsw[0], nsw[1], nsw[2], nsw[3]);
            *reinterpret_cast<uint4*>(a.leaf + r8) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
        }
    }
}

__global__ void delta_kernel(Ctl c, int pack_size, float lr) {
    const int n = c.head->n_tree_nodes;
    for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < n; t += gridDim.x * blockDim.x) {
        const float v = (float)c.node_value[t];
        float acc = 0.f;
        for (int b = 0; b < pack_size; ++b) acc = __fadd_rn(acc, v);
        c.delta[t] = __fmul_rn(lr, acc);
    }
}

__global__ void __launch_bounds__(kRowThreads) apply_delta_kernel(float* preds, const uint16_t* leaf,
                                                                  const float* delta, int64_t n) {
    for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < n; r += (int64_t)gridDim.x * blockDim.x)
        preds[r] = __fadd_rn(preds[r], delta[leaf[r]]);
}

int row_grid(int64_t n) {
    int64_t b = (n + kRowThreads - 1) / kRowThreads;
    const int64_t cap = 148 * 16;
    if (b > cap) b = cap;
    if (b < 1) b = 1;
    return (int)b;
}

}  // namespace

// Candidate table of a depth lives at the start of the workspace: [n_sampled][node_stride].
static inline int node_stride_of(int64_t depth) { return 1 << depth; }

}  // namespace pb

using namespace pb;

static int check_state(const pb_train_state* st) {
    PB_REQUIRE(st != nullptr, "state is null");
    PB_REQUIRE(st->n_rows > 0 && st->n_rows < (1ll << 31) - 512, "n_rows=%lld out of range", (long long)st->n_rows);
    PB_REQUIRE(st->code_bits == 4 || st->code_bits == 8, "code_bits must be 4 or 8");
    PB_REQUIRE(st->max_bins >= 2 && st->max_bins <= 256, "max_bins=%lld outside [2,256]", (long long)st->max_bins);
    PB_REQUIRE(st->code_bits == 8 || st->max_bins <= 16, "4-bit codes need max_bins <= 16");
    PB_REQUIRE(st->max_depth >= 1 && st->max_depth <= PB_MAX_DEPTH, "max_depth=%lld outside [1,%d]",
               (long long)st->max_depth, PB_MAX_DEPTH);
    PB_REQUIRE(st->n_eras >= 1 && st->n_eras <= 32767, "n_eras=%lld outside [1,32767]", (long long)st->n_eras);
    PB_REQUIRE(st->pitch % 128 == 0 && st->pitch * (st->code_bits == 4 ? 2 : 1) >= rows_padded(st->n_rows),
               "pitch=%lld does not cover the padded rows", (long long)st->pitch);
    PB_REQUIRE(st->n_thresholds >= 1 && st->n_thresholds < st->max_bins, "n_thresholds out of range");
    PB_REQUIRE(st->codes && st->era_offsets && st->thr_ids && st->feat_local && st->y && st->preds && st->gq &&
                   st->slot && st->leaf && st->ctl,
               "a device buffer of the training state is null");
    // (`workspace` may be null: only the entries that use it ask for it, see need_workspace)
    PB_REQUIRE(st->workspace != nullptr || st->workspace_bytes == 0, "workspace is null but workspace_bytes is not 0");
    PB_REQUIRE(st->lambda_l2 > 0.0, "lambda_l2 must be positive");
    PB_REQUIRE(st->count_bits >= 1 && st->count_bits <= 13 && st->lo_bits == 32 - 2 * st->count_bits &&
                   st->gq_bits >= st->lo_bits && st->gq_bits <= kGqBitsMax && st->gq_bits <= 63 - 3 * st->count_bits,
               "accumulator widths are not set: call pb_train_prepare first");
    // (the lane histogram kernel reads a 32-byte sector of codes with one 256-bit load)
    PB_REQUIRE((uintptr_t)st->codes % 32 == 0, "codes must be 32-byte aligned");
    PB_REQUIRE(((uintptr_t)st->gq % 16 == 0) && ((uintptr_t)st->slot % 16 == 0) && ((uintptr_t)st->leaf % 16 == 0),
               "gq, slot and leaf must be 16-byte aligned");
    PB_REQUIRE(((uintptr_t)st->y % 16 == 0) && ((uintptr_t)st->preds % 16 == 0), "y and preds must be 16-byte aligned");
    return PB_OK;
}


// Entries that keep their tables in the caller's workspace.  A host that cannot allocate one
// leaves it null and uses pb_depth_hist_score_static + pb_depth_select_cand instead.
static int need_workspace(const pb_train_state* st, const char* who) {
    PB_REQUIRE(st->workspace != nullptr, "%s needs pb_train_state.workspace (hosts without one: "
               "pb_depth_hist_score_static and pb_depth_select_cand)", who);
    return PB_OK;
}

// Carving of the scratch that one block of features needs between the histogram pass and the
// scorer: gsum | cnt | gain-weight table | era-summed gradient sums | era-summed counts.
struct BlockPlan {
    int64_t fb;  // features per block
    bool fused;  // the histogram is never stored (fused flush): no gsum / cnt arrays
    size_t off_gsum, off_cnt, off_gw, off_lg, off_lc, off_thr;
};

// The era-summed tables of the fused flush are laid out per lane of the histogram kernel and so
// cover the features of the last CTA in full: up to this many features more than the block has.
constexpr int64_t kTotPad = 256;

static bool plan_block(size_t avail, int stride, int64_t n_eras, int64_t max_bins, int64_t n_thr, int64_t n_feat,
                       bool fused, BlockPlan* p) {
    const size_t cells = fused ? 0 : (size_t)stride * n_eras * max_bins;
    const size_t per_feat = cells * 12 + score_scratch_bytes_per_feature(stride, (int)n_eras, (int)n_thr) + (size_t)n_thr * 4;
    const size_t fixed = 6 * 256 + (fused ? (size_t)kTotPad * stride * n_thr * 12 : 0);
    if (avail < per_feat + fixed) return false;
    int64_t fb = (int64_t)((avail - fixed) / per_feat);
    if (fb > n_feat) fb = n_feat;
    if (fb < 1) return false;
    p->fb = fb;
    p->fused = fused;
    const size_t tot_feats = (size_t)fb + (fused ? kTotPad : 0);
    size_t o = 0;
    p->off_gsum = o;
    o += align_up((size_t)fb * cells * 8, 256);
    p->off_cnt = o;
    o += align_up((size_t)fb * cells * 4, 256);
    p->off_gw = o;
    o += align_up((size_t)fb * stride * n_eras * n_thr * 8, 256);
    p->off_lg = o;
    o += align_up(tot_feats * stride * n_thr * 8, 256);
    p->off_lc = o;
    o += align_up(tot_feats * stride * n_thr * 4, 256);
    p->off_thr = o;  // per-feature threshold lists (mass cuts): fb * n_thr * 4 bytes
    return true;
}

// The histogram launch of one depth, up to the feature list and the output arrays.
static HistLaunch hist_launch_of(const pb_train_state* st, int64_t depth, const Ctl& c) {
    const int stride = node_stride_of(depth);
    HistLaunch h;
    h.codes = st->codes;
    h.pitch = st->pitch;
    h.code_bits = (int)st->code_bits;
    h.feat_rows = nullptr;
    h.n_feat = 1;
    h.gq = st->gq;
    h.slot = st->slot;
    h.era_offsets = st->era_offsets;
    h.n_eras = (int)st->n_eras;
    h.max_bins = (int)st->max_bins;
    h.max_era_rows = (int)st->max_era_rows;
    h.n_nodes_ptr = &c.head->n_ctx[depth];
    h.n_nodes = stride;
    h.node_stride = stride;
    h.count_bits = (int)st->count_bits;
    h.lo_bits = (int)st->lo_bits;
    h.max_arity = hist_max_arity();
    h.cnt = nullptr;
    h.gsum = nullptr;
    h.fuse = nullptr;
    h.prof = st->profile;
    h.debug_flags = &c.head->debug_flags;
    return h;
}

// The flush of the histogram kernel does the per-era gain step itself when a CTA holds a whole era
// of few-bin cells and no directional term needs the stored histogram (PACKBOOST_FUSED_FLUSH=0
// keeps the separate gain kernel, for comparisons).
static bool use_fused_flush(const pb_train_state* st, int64_t depth) {
    static const bool enabled = [] {
        const char* e = getenv("PACKBOOST_FUSED_FLUSH");
        return !(e && e[0] == '0' && e[1] == 0);
    }();
    if (!enabled || st->direction_weight != 0.0 || st->cut_mass) return false;  // (mass cuts need the stored histogram)
    Ctl c = ctl_view(st->ctl);
    return hist_can_fuse(hist_launch_of(st, depth, c));
}

static int hist_score_blocks(const pb_train_state* st, int64_t depth, const int32_t* feat_rows, const int32_t* feat_pos,
                             int64_t n_feat, char* scratch, const BlockPlan& plan, Cand* cand, cudaStream_t stream) {
    Ctl c = ctl_view(st->ctl);
    const int stride = node_stride_of(depth);
    int64_t* gsum = reinterpret_cast<int64_t*>(scratch + plan.off_gsum);
    uint32_t* cnt = reinterpret_cast<uint32_t*>(scratch + plan.off_cnt);
    for (int64_t f0 = 0; f0 < n_feat; f0 += plan.fb) {
        const int nf = (int)((n_feat - f0 < plan.fb) ? (n_feat - f0) : plan.fb);
        HistLaunch h = hist_launch_of(st, depth, c);
        h.feat_rows = feat_rows + f0;
        h.n_feat = nf;
        h.cnt = cnt;   // the histogram kernel overwrites (or zeroes, then adds to) every cell that is read later
        h.gsum = gsum;
        HistFuse fz;
        memset(&fz, 0, sizeof(fz));
        if (plan.fused) {
            fz.gw = reinterpret_cast<float2*>(scratch + plan.off_gw);
            fz.lg_tot = reinterpret_cast<int64_t*>(scratch + plan.off_lg);
            fz.lc_tot = reinterpret_cast<uint32_t*>(scratch + plan.off_lc);
            fz.thr_ids = st->thr_ids;
            fz.n_thr = (int)st->n_thresholds;
            // ascending distinct bin ids below max_bins - 1: as many as there are means all of them
            fz.full_sweep = (st->n_thresholds == st->max_bins - 1) ? 1 : 0;
            fz.inv_scale_ptr = &c.head->inv_scale;
            fz.lambda_l2 = (float)st->lambda_l2;
            fz.era_alpha = (float)(st->era_alpha > 0.0 ? st->era_alpha : 0.0);
            h.fuse = &fz;
            h.cnt = nullptr;
            h.gsum = nullptr;
        }
        int rc = launch_hist(h, stream);
        if (rc) return rc;
        const int32_t* thr_ids = st->thr_ids;
        if (st->cut_mass) {
            int32_t* thr_tab = reinterpret_cast<int32_t*>(scratch + plan.off_thr);
            rc = launch_mass_thresholds(cnt, nf, &c.head->n_ctx[depth], stride, stride, (int)st->n_eras, (int)st->max_bins,
                                        (int)st->n_thresholds, thr_tab, stream);
            if (rc) return rc;
            thr_ids = thr_tab;
        }
        ScoreLaunch s;
        s.cnt = cnt;
        s.gsum = gsum;
        s.n_feat = nf;
        s.feat_pos = feat_pos + f0;
        s.node_stride = stride;
        s.n_nodes_max = stride;
        s.n_nodes_ptr = &c.head->n_ctx[depth];
        s.frontier = c.frontier[depth & 1];
        s.any_dir_ptr = &c.head->any_dir[depth];
        s.inv_scale_ptr = &c.head->inv_scale;
        s.n_eras = (int)st->n_eras;
        s.max_bins = (int)st->max_bins;
        s.n_thr = (int)st->n_thresholds;
        s.thr_ids = thr_ids;
        s.thr_per_feature = st->cut_mass ? 1 : 0;
        s.lambda_l2 = (float)st->lambda_l2;
        s.lambda_dro = (float)st->lambda_dro;
        s.direction_weight = (float)st->direction_weight;
        s.direction_form = st->direction_form ? 1 : 0;
        s.era_alpha = (float)(st->era_alpha > 0.0 ? st->era_alpha : 0.0);
        s.min_samples_leaf = (int)st->min_samples_leaf;
        s.cand = cand;
        s.gw = reinterpret_cast<float2*>(scratch + plan.off_gw);
        s.lg_tot = reinterpret_cast<int64_t*>(scratch + plan.off_lg);
        s.lc_tot = reinterpret_cast<uint32_t*>(scratch + plan.off_lc);
        s.prof = st->profile;
        s.fused = plan.fused ? 1 : 0;
        s.tot_fpl = plan.fused ? fz.tot_fpl : 0;
        s.tot_lanes = plan.fused ? fz.tot_lanes : 0;
        rc = launch_score(s, stream);
        if (rc) return rc;
    }
    return PB_OK;
}

extern "C" int64_t pb_ctl_bytes(void) { return (int64_t)kCtlBytes; }

extern "C" int64_t pb_workspace_min_bytes(const pb_train_state* st) {
    if (!st) return 0;
    // candidate table at the deepest level for every feature + one feature of histogram
    const int64_t stride = 1ll << (st->max_depth - 1);
    const int64_t cand = (int64_t)sizeof(Cand) * st->n_features_total * stride;
    const int64_t hist_one = stride * st->n_eras * st->max_bins * 12 +
                             (int64_t)score_scratch_bytes_per_feature((int)stride, (int)st->n_eras, (int)st->n_thresholds);
    return align_up((size_t)cand, 256) + hist_one + 8192;
}

extern "C" int pb_train_prepare(pb_train_state* st, const int32_t* era_offsets_host) {
    PB_REQUIRE(st && era_offsets_host, "null argument");
    int64_t mx = 0;
    PB_REQUIRE(era_offsets_host[0] == 0, "era_offsets[0] must be 0");
    for (int64_t e = 0; e < st->n_eras; ++e) {
        const int64_t len = (int64_t)era_offsets_host[e + 1] - era_offsets_host[e];
        PB_REQUIRE(len >= 0, "era_offsets must be non-decreasing");
        if (len > mx) mx = len;
    }
    PB_REQUIRE(era_offsets_host[st->n_eras] == st->n_rows, "era_offsets[E] must equal n_rows");
    st->max_era_rows = mx;
    st->hist_rows_per_tile = kTileRowsMax;
    // widths of the 32-bit shared-memory accumulators of the histogram kernel
    const int64_t tile = (mx < kTileRowsMax) ? mx : kTileRowsMax;
    int cb = 1;
    while ((1ll << cb) <= tile) ++cb;  // tile < 2^cb
    if (cb < 11) cb = 11;  // (costs no gradient bits; the lane kernel keeps a cell index below the count field)
    st->count_bits = cb;
    st->lo_bits = 32 - 2 * cb;
    st->gq_bits = (63 - 3 * cb < kGqBitsMax) ? (63 - 3 * cb) : kGqBitsMax;
    int rc = check_state(st);
    if (rc) return rc;
    if (st->workspace != nullptr)
        PB_REQUIRE(st->workspace_bytes >= pb_workspace_min_bytes(st), "workspace too small: %lld < %lld",
                   (long long)st->workspace_bytes, (long long)pb_workspace_min_bytes(st));
    return PB_OK;
}

extern "C" int pb_round_begin(const pb_train_state* st, int64_t apply_previous, void* stream_) {
    NvtxRange nvtx("pb.round_begin apply=%lld", (long long)apply_previous);
    int rc = check_state(st);
    if (rc) return rc;
    cudaStream_t stream = (cudaStream_t)stream_;
    Ctl c = ctl_view(st->ctl);
    const int g = row_grid(st->n_rows);
    prof_begin(st->profile, kProfRound, stream);
    round_reset_kernel<<<1, 32, 0, stream>>>(c);
    preds_absmax_kernel<<<g, kRowThreads, 0, stream>>>(st->preds, st->y, st->leaf, c.delta, st->n_rows,
                                                        apply_previous ? 1 : 0, c.head);
    quantise_kernel<<<g, kRowThreads, 0, stream>>>(st->preds, st->y, st->gq, st->slot, st->leaf, st->n_rows,
                                                    rows_padded(st->n_rows), c.head, (int)st->gq_bits);
    root_kernel<<<1, 32, 0, stream>>>(c, st->n_rows, (int)st->min_samples_leaf, st->lambda_l2, (int)st->gq_bits);
    prof_end(st->profile, kProfRound, stream);
    count_launch(4);
    PB_LAUNCH_CHECK("round_begin");
    return PB_OK;
}

extern "C" int pb_candidates_buffer(const pb_train_state* st, int64_t depth, int64_t n_sampled, void** ptr,
                                    int64_t* bytes) {
    PB_REQUIRE(st && ptr && bytes, "null argument");
    PB_REQUIRE(depth >= 0 && depth < st->max_depth, "depth out of range");
    int rc = need_workspace(st, "pb_candidates_buffer");
    if (rc) return rc;
    *ptr = st->workspace;
    *bytes = (int64_t)sizeof(Cand) * n_sampled * node_stride_of(depth);
    return PB_OK;
}

extern "C" int pb_depth_clear_candidates(const pb_train_state* st, int64_t depth, int64_t n_sampled, void* stream) {
    void* p;
    int64_t b;
    int rc = pb_candidates_buffer(st, depth, n_sampled, &p, &b);
    if (rc) return rc;
    PB_CUDA_TRY(cudaMemsetAsync(p, 0, (size_t)b, (cudaStream_t)stream));
    return PB_OK;
}

extern "C" int pb_depth_hist_score(const pb_train_state* st, int64_t depth, const int32_t* feat_rows,
                                   const int32_t* feat_pos, int64_t n_feat, int64_t n_sampled, void* stream_) {
    NvtxRange nvtx("pb.hist_score d=%lld", (long long)depth);
    int rc = check_state(st);
    if (rc) return rc;
    rc = need_workspace(st, "pb_depth_hist_score");
    if (rc) return rc;
    PB_REQUIRE(depth >= 0 && depth < st->max_depth, "depth out of range");
    PB_REQUIRE(n_feat >= 0 && n_feat <= n_sampled && n_sampled <= st->n_features_total, "feature counts out of range");
    if (n_feat == 0) return PB_OK;
    PB_REQUIRE(feat_rows && feat_pos, "null feature list");
    const int stride = node_stride_of(depth);
    const size_t cand_bytes = align_up(sizeof(Cand) * (size_t)n_sampled * stride, 256);
    PB_REQUIRE((int64_t)cand_bytes < st->workspace_bytes, "workspace too small for the candidate table");
    char* ws = static_cast<char*>(st->workspace);
    BlockPlan plan;
    PB_REQUIRE(plan_block((size_t)st->workspace_bytes - cand_bytes, stride, st->n_eras, st->max_bins, st->n_thresholds,
                          n_feat, use_fused_flush(st, depth), &plan),
               "workspace too small for one feature of histogram at depth %lld", (long long)depth);
    return hist_score_blocks(st, depth, feat_rows, feat_pos, n_feat, ws + cand_bytes, plan, reinterpret_cast<Cand*>(ws),
                             (cudaStream_t)stream_);
}

extern "C" int pb_depth_select(const pb_train_state* st, int64_t depth, const int32_t* sampled_features,
                               int64_t n_sampled, void* stream_) {
    int rc = check_state(st);
    if (rc) return rc;
    rc = need_workspace(st, "pb_depth_select");
    if (rc) return rc;
    return pb_depth_select_cand(st, depth, sampled_features, n_sampled, st->workspace, stream_);
}

extern "C" int pb_depth_select_cand(const pb_train_state* st, int64_t depth, const int32_t* sampled_features,
                                    int64_t n_sampled, const void* cand, void* stream_) {
    NvtxRange nvtx("pb.select d=%lld", (long long)depth);
    int rc = check_state(st);
    if (rc) return rc;
    PB_REQUIRE(depth >= 0 && depth < st->max_depth, "depth out of range");
    PB_REQUIRE(sampled_features && n_sampled >= 1, "empty feature subset");
    PB_REQUIRE(cand != nullptr && ((uintptr_t)cand % 8) == 0, "candidate table must be a non-null 8-byte aligned buffer");
    SelectArgs a;
    a.c = ctl_view(st->ctl);
    a.depth = (int)depth;
    a.max_depth = (int)st->max_depth;
    a.cand = reinterpret_cast<const Cand*>(cand);
    a.node_stride = node_stride_of(depth);
    a.sampled = sampled_features;
    a.n_sampled = (int)n_sampled;
    int blk = (int)st->feature_block_size;
    if (blk <= 0 || blk > n_sampled) blk = (int)n_sampled;
    a.block_size = blk;
    a.thr_ids = st->thr_ids;
    a.n_thr = (int)st->n_thresholds;
    a.min_leaf = (int)st->min_samples_leaf;
    a.lambda = st->lambda_l2;
    prof_begin(st->profile, kProfSelect, (cudaStream_t)stream_);
    select_kernel<<<(unsigned)a.node_stride, kSelThreads, 0, (cudaStream_t)stream_>>>(a);
    prof_end(st->profile, kProfSelect, (cudaStream_t)stream_);
    count_launch(1);
    PB_LAUNCH_CHECK("select_kernel");
    return PB_OK;
}

template <int MODE>
static int launch_partition(const pb_train_state* st, int64_t depth, uint32_t* bits, const uint32_t* bits_in,
                            void* stream_) {
    NvtxRange nvtx("pb.partition d=%lld", (long long)depth);
    int rc = check_state(st);
    if (rc) return rc;
    PB_REQUIRE(depth >= 0 && depth < st->max_depth, "depth out of range");
    PartArgs a;
    a.c = ctl_view(st->ctl);
    a.depth = (int)depth;
    a.codes = st->codes;
    a.pitch = st->pitch;
    a.feat_local = st->feat_local;
    a.slot = st->slot;
    a.leaf = st->leaf;
    a.n = st->n_rows;
    a.bits = bits;
    a.bits_in = bits_in;
    a.n_features_total = (int)st->n_features_total;
    a.n_features_local = (int)st->n_features_local;
    const size_t smem = sizeof(PartEntry) * (size_t)(1 << depth);
    const int g = row_grid((st->n_rows + 7) / 8);  // a thread takes eight rows
    cudaStream_t stream = (cudaStream_t)stream_;
    prof_begin(st->profile, kProfPartition, stream);
    if (st->code_bits == 4)
        partition_kernel<4, MODE><<<g, kRowThreads, smem, stream>>>(a);
    else
        partition_kernel<8, MODE><<<g, kRowThreads, smem, stream>>>(a);
    prof_end(st->profile, kProfPartition, stream);
    count_launch(1);
    PB_LAUNCH_CHECK("partition_kernel");
    return PB_OK;
}

extern "C" int pb_depth_partition(const pb_train_state* st, int64_t depth, void* stream) {
    return launch_partition<0>(st, depth, nullptr, nullptr, stream);
}

extern "C" int pb_depth_goleft_bits(const pb_train_state* st, int64_t depth, uint32_t* bits, void* stream) {
    PB_REQUIRE(bits, "bits is null");
    return launch_partition<1>(st, depth, bits, nullptr, stream);
}

extern "C" int pb_depth_apply_bits(const pb_train_state* st, int64_t depth, const uint32_t* bits, void* stream) {
    PB_REQUIRE(bits, "bits is null");
    return launch_partition<2>(st, depth, nullptr, bits, stream);
}

extern "C" int pb_round_end(const pb_train_state* st, void* stream) {
    NvtxRange nvtx("pb.round_end (pack of %lld)", st ? (long long)st->pack_size : 0ll);
    int rc = check_state(st);
    if (rc) return rc;
    delta_kernel<<<8, 256, 0, (cudaStream_t)stream>>>(ctl_view(st->ctl), (int)st->pack_size, (float)st->learning_rate);
    count_launch(1);
    PB_LAUNCH_CHECK("delta_kernel");
    return PB_OK;
}

extern "C" int pb_apply_leaf_delta(const pb_train_state* st, void* stream) {
    int rc = check_state(st);
    if (rc) return rc;
    Ctl c = ctl_view(st->ctl);
    apply_delta_kernel<<<row_grid(st->n_rows), kRowThreads, 0, (cudaStream_t)stream>>>(st->preds, st->leaf, c.delta,
                                                                                      st->n_rows);
    count_launch(1);
    PB_LAUNCH_CHECK("apply_delta_kernel");
    return PB_OK;
}

extern "C" int pb_debug_bounds_enabled(void) {
#ifdef PB_DEBUG_BOUNDS
    return 1;
#else
    return 0;
#endif
}

extern "C" int pb_debug_flags(const pb_train_state* st, uint32_t* flags_out) {
    PB_REQUIRE(st && st->ctl && flags_out, "null argument");
    Ctl c = ctl_view(st->ctl);
    PB_CUDA_TRY(cudaMemcpy(flags_out, &c.head->debug_flags, sizeof(uint32_t), cudaMemcpyDeviceToHost));
    return PB_OK;
}

extern "C" int pb_round_log_buffer(const pb_train_state* st, void** ptr, int64_t* bytes) {
    PB_REQUIRE(st && ptr && bytes && st->ctl, "null argument");
    Ctl c = ctl_view(st->ctl);
    *ptr = c.log_head;
    *bytes = (int64_t)(sizeof(pb_round_log_header) + sizeof(pb_winner) * ((1ll << st->max_depth) - 1));
    return PB_OK;
}

extern "C" int pb_hist_build(const pb_train_state* st, const int32_t* feat_rows, int64_t n_feat, int64_t n_nodes,
                             int64_t node_stride, uint32_t* cnt, int64_t* gsum, void* stream) {
    int rc = check_state(st);
    if (rc) return rc;
    PB_REQUIRE(feat_rows && cnt && gsum, "null argument");
    PB_REQUIRE(n_nodes >= 1 && n_nodes <= node_stride && node_stride < 65535, "node counts out of range");
    HistLaunch h;
    h.codes = st->codes;
    h.pitch = st->pitch;
    h.code_bits = (int)st->code_bits;
    h.feat_rows = feat_rows;
    h.n_feat = (int)n_feat;
    h.gq = st->gq;
    h.slot = st->slot;
    h.era_offsets = st->era_offsets;
    h.n_eras = (int)st->n_eras;
    h.max_bins = (int)st->max_bins;
    h.max_era_rows = (int)st->max_era_rows;
    h.n_nodes_ptr = nullptr;
    h.n_nodes = (int)n_nodes;
    h.node_stride = (int)node_stride;
    h.count_bits = (int)st->count_bits;
    h.lo_bits = (int)st->lo_bits;
    h.max_arity = hist_max_arity();
    h.cnt = cnt;
    h.gsum = gsum;
    h.fuse = nullptr;
    h.prof = st->profile;
    h.debug_flags = &ctl_view(st->ctl).head->debug_flags;
    return launch_hist(h, (cudaStream_t)stream);
}

// ---- histogram + score without a caller-provided workspace -------------------------------------
//
// Some hosts of this library cannot hand it a workspace: their device memory is reserved in full
// by another component's pool when the process starts (an inference server, a framework allocator
// configured to take the whole device), or their deployment forbids device allocation after
// start-up, so nothing can call cudaMalloc for the tens of megabytes pb_depth_hist_score wants.
// For them the per-block histograms live in the fixed array below, which is part of the library
// image: every GPU that loads the library holds these bytes until the process exits.
constexpr size_t kStaticScratchBytes = 64ull << 20;  // 64 MiB
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` is only a handle for the symbol, not an address a kernel can use;
// the device address is looked up once per device (with that device current) and cached.
static std::mutex g_static_mu;
static void* g_static_ptr[64] = {nullptr};

static int static_scratch_ptr(void** out) {
    int dev = -1;
    PB_CUDA_TRY(cudaGetDevice(&dev));
    PB_REQUIRE(dev >= 0 && dev < 64, "device ordinal %d not supported by the static scratch", dev);
    std::lock_guard<std::mutex> lk(g_static_mu);
    if (!g_static_ptr[dev]) {
        void* p = nullptr;
        PB_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
        PB_REQUIRE(p != nullptr && ((uintptr_t)p % 256) == 0, "static scratch has no usable device address");
        g_static_ptr[dev] = p;
    }
    *out = g_static_ptr[dev];
    return PB_OK;
}

extern "C" int64_t pb_static_scratch_bytes(void) { return (int64_t)kStaticScratchBytes; }

extern "C" int pb_depth_hist_score_static(const pb_train_state* st, int64_t depth, const int32_t* feat_rows,
                                          const int32_t* feat_pos, int64_t n_feat, int64_t n_sampled,
                                          void* cand_out, void* stream_) {
    NvtxRange nvtx("pb.hist_score_static d=%lld", (long long)depth);
    int rc = check_state(st);
    if (rc) return rc;
    PB_REQUIRE(depth >= 0 && depth < st->max_depth, "depth out of range");
    PB_REQUIRE(n_feat >= 0 && n_feat <= n_sampled && n_sampled <= st->n_features_total, "feature counts out of range");
    PB_REQUIRE(cand_out != nullptr && ((uintptr_t)cand_out % 8) == 0, "cand_out must be a non-null 8-byte aligned buffer");
    if (n_feat == 0) return PB_OK;
    PB_REQUIRE(feat_rows && feat_pos, "null feature list");
    const int stride = node_stride_of(depth);
    BlockPlan plan;
    PB_REQUIRE(plan_block(kStaticScratchBytes, stride, st->n_eras, st->max_bins, st->n_thresholds, n_feat,
                          use_fused_flush(st, depth), &plan),
               "static scratch too small: one feature of histogram and scorer tables at depth %lld needs %llu bytes, "
               "the fixed array holds %llu; use pb_depth_hist_score with a workspace",
               (long long)depth,
               (unsigned long long)((size_t)stride * st->n_eras * st->max_bins * 12 +
                                    score_scratch_bytes_per_feature(stride, (int)st->n_eras, (int)st->n_thresholds)),
               (unsigned long long)kStaticScratchBytes);
    void* base = nullptr;
    rc = static_scratch_ptr(&base);
    if (rc) return rc;
    return hist_score_blocks(st, depth, feat_rows, feat_pos, n_feat, static_cast<char*>(base), plan,
                             static_cast<Cand*>(cand_out), (cudaStream_t)stream_);
}
