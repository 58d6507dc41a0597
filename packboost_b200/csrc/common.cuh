// Internal declarations shared by the kernels of libpackboost_b200.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/packboost_b200.h"

namespace pb {

// ---- error reporting --------------------------------------------------------------------

void set_error(const char* fmt, ...);
int fail_arg(const char* fmt, ...);
int fail_cuda(cudaError_t e, const char* what);

#define PB_CUDA_TRY(expr)                                   \
    do {                                                    \
        cudaError_t _e = (expr);                            \
        if (_e != cudaSuccess) return pb::fail_cuda(_e, #expr); \
    } while (0)

#define PB_LAUNCH_CHECK(what)                               \
    do {                                                    \
        cudaError_t _e = cudaGetLastError();                \
        if (_e != cudaSuccess) return pb::fail_cuda(_e, what); \
    } while (0)

// ---- optional in-stream timing of the kernel families and a launch counter -----------------

enum ProfKind { kProfHist = 0, kProfScore = 1, kProfSelect = 2, kProfPartition = 3, kProfRound = 4, kProfKinds = 5 };
void prof_begin(void* prof, int kind, cudaStream_t stream);  // prof: pb_train_state.profile, may be null
void prof_end(void* prof, int kind, cudaStream_t stream);
void count_launch(int n);
void nvtx_push(const char* fmt, long long a);  // PACKBOOST_NVTX=1: NVTX range around a phase
void nvtx_pop();
struct NvtxRange {  // range for the lifetime of the object
    NvtxRange(const char* fmt, long long a) { nvtx_push(fmt, a); }
    ~NvtxRange() { nvtx_pop(); }
    NvtxRange(const NvtxRange&) = delete;
    NvtxRange& operator=(const NvtxRange&) = delete;
};

#define PB_REQUIRE(cond, ...)                               \
    do {                                                    \
        if (!(cond)) return pb::fail_arg(__VA_ARGS__);      \
    } while (0)

// ---- constants --------------------------------------------------------------------------

constexpr int kMaxDepth = PB_MAX_DEPTH;
constexpr int kMaxCtx = 1 << (PB_MAX_DEPTH - 1);        // frontier nodes at the deepest level
constexpr int kMaxTreeNodes = (1 << (PB_MAX_DEPTH + 1)); // 2^(D+1) - 1 rounded up
constexpr int kMaxWinners = (1 << PB_MAX_DEPTH);         // sum over depths of frontier sizes (+1)
constexpr uint16_t kSlotNone = 0xFFFFu;
constexpr int kTileRowsMax = 8160;      // rows one histogram CTA accumulates (255 chunks of 32 rows)
constexpr int kGqBitsMax = 30;          // |gq| <= 2^30 at most; fewer bits when tiles are large

// ---- device-side tables -----------------------------------------------------------------

// Best threshold of one (sampled feature, frontier node) pair.
struct Cand {
    float score;
    int32_t k;            // index into thr_ids, -1: empty entry
    uint32_t left_count;
    uint32_t flags;       // bit 0: a globally valid threshold of this feature scored NaN; bits 8-15: bin id of threshold k
    int64_t left_gq;
};
static_assert(sizeof(Cand) == 24, "Cand layout");

struct FrontierNode {
    int32_t tree_node;
    int32_t count;
    int64_t gq;
};

struct PartEntry {
    int32_t feature;      // global id, -1: node keeps its rows (no split)
    int32_t threshold;
    uint16_t slot_left, slot_right;
    uint16_t leaf_left, leaf_right;
};
static_assert(sizeof(PartEntry) == 16, "PartEntry layout");

struct CtlHead {
    uint32_t max_abs_bits;
    float scale;
    float inv_scale;
    int32_t n_tree_nodes;
    int64_t root_gq;
    int32_t n_ctx[kMaxDepth + 2];
    int32_t any_dir[kMaxDepth + 2];
    uint32_t select_ticket;  // CTAs of the running select launch that have written their node (reset by the last)
    uint32_t debug_flags;    // PB_DEBUG_BOUNDS builds: sticky bits of index violations seen by the kernels
};

// Bits of CtlHead::debug_flags (builds with -DPB_DEBUG_BOUNDS check the indices they are handed and
// record a violation here instead of using the index; other builds never set them).
constexpr uint32_t kDbgSlot = 1u;     // a row's frontier slot is neither "none" nor below the frontier's capacity
constexpr uint32_t kDbgCode = 2u;     // a bin code is >= max_bins
constexpr uint32_t kDbgFeature = 4u;  // a winner's feature id is outside the data set or not held by this device

// Addresses of the sub-tables inside the caller's control block.
struct Ctl {
    CtlHead* head;
    FrontierNode* frontier[2];  // indexed by depth parity
    PartEntry* part;
    pb_round_log_header* log_head;
    pb_winner* winners;
    double* node_value;
    float* delta;
    int32_t* sel_flag;  // per frontier node: bit 0 split, bit 1 left child stays active, bit 2 right child
};

constexpr size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

constexpr size_t kOffHead = 0;
constexpr size_t kOffFrontier0 = align_up(sizeof(CtlHead), 256);
constexpr size_t kOffFrontier1 = kOffFrontier0 + align_up(sizeof(FrontierNode) * kMaxCtx, 256);
constexpr size_t kOffPart = kOffFrontier1 + align_up(sizeof(FrontierNode) * kMaxCtx, 256);
constexpr size_t kOffLog = kOffPart + align_up(sizeof(PartEntry) * kMaxCtx, 256);
constexpr size_t kLogBytes = sizeof(pb_round_log_header) + sizeof(pb_winner) * kMaxWinners;
constexpr size_t kOffNodeValue = kOffLog + align_up(kLogBytes, 256);
constexpr size_t kOffDelta = kOffNodeValue + align_up(sizeof(double) * kMaxTreeNodes, 256);
constexpr size_t kOffSelFlag = kOffDelta + align_up(sizeof(float) * kMaxTreeNodes, 256);
constexpr size_t kCtlBytes = kOffSelFlag + align_up(sizeof(int32_t) * kMaxCtx, 256);

inline __host__ __device__ Ctl ctl_view(void* base) {
    char* p = static_cast<char*>(base);
    Ctl c;
    c.head = reinterpret_cast<CtlHead*>(p + kOffHead);
    c.frontier[0] = reinterpret_cast<FrontierNode*>(p + kOffFrontier0);
    c.frontier[1] = reinterpret_cast<FrontierNode*>(p + kOffFrontier1);
    c.part = reinterpret_cast<PartEntry*>(p + kOffPart);
    c.log_head = reinterpret_cast<pb_round_log_header*>(p + kOffLog);
    c.winners = reinterpret_cast<pb_winner*>(p + kOffLog + sizeof(pb_round_log_header));
    c.node_value = reinterpret_cast<double*>(p + kOffNodeValue);
    c.delta = reinterpret_cast<float*>(p + kOffDelta);
    c.sel_flag = reinterpret_cast<int32_t*>(p + kOffSelFlag);
    return c;
}

inline int64_t rows_padded(int64_t n) { return (n + 255) / 256 * 256; }

// ---- histogram launch (hist.cu) -----------------------------------------------------------

struct HistLaunch {
    const uint8_t* codes;
    int64_t pitch;
    int code_bits;
    const int32_t* feat_rows;  // device: local feature row per histogram feature
    int n_feat;
    const int32_t* gq;
    const uint16_t* slot;
    const int32_t* era_offsets;
    int n_eras;
    int max_bins;
    int max_era_rows;
    const int32_t* n_nodes_ptr;  // device count of frontier nodes, or nullptr
    int n_nodes;                 // upper bound (grid sizing) and value when n_nodes_ptr == nullptr
    int node_stride;
    int count_bits;              // CB: tile rows < 2^CB
    int lo_bits;                 // LB = 32 - 2*CB
    int max_arity;               // largest feature tuple of the lane kernel (1 or 2)
    uint32_t* cnt;
    int64_t* gsum;
    // Fused flush (null: write the histogram as above).  When set and hist_can_fuse(h) holds, the
    // histogram is never stored: the flush turns the cells of each (feature, node) of the CTA's era
    // into the per-threshold (gain, weight) rows and adds the left counts / gradient sums into the
    // era-summed tables, i.e. it does the work of the scorer's gain kernel.
    struct HistFuse* fuse;
    void* prof;                  // pb_train_state.profile
    uint32_t* debug_flags;       // &CtlHead::debug_flags, or nullptr
};
struct HistFuse {
    float2* gw;                  // [n_feat][n_eras][node_stride][n_thr]
    uint32_t* lc_tot;            // lane layout, see tot_index(); zeroed by launch_hist
    int64_t* lg_tot;
    const int32_t* thr_ids;      // device: [n_thr] ascending bin ids
    int n_thr;
    int full_sweep;              // thr_ids[k] == k for all k and n_thr == max_bins - 1
    const float* inv_scale_ptr;
    float lambda_l2, era_alpha;
    int tot_fpl, tot_lanes;      // OUT: layout of the totals tables chosen by launch_hist
};
// True when launch_hist(h) would run the lane kernel with one tile per era, which is what the
// fused flush needs (a CTA then holds the complete cells of its era).
bool hist_can_fuse(const HistLaunch& h);
int launch_hist(const HistLaunch& h, cudaStream_t stream);
int hist_max_arity();  // default tuple-size cap of the lane kernel (PACKBOOST_HIST_MAX_ARITY=1 lowers it)

// ---- scorer launch (score.cu) -------------------------------------------------------------

struct ScoreLaunch {
    const uint32_t* cnt;
    const int64_t* gsum;
    int n_feat;                  // features in this histogram block
    const int32_t* feat_pos;     // device: sampled position of each histogram feature
    int node_stride;
    int n_nodes_max;
    const int32_t* n_nodes_ptr;
    const FrontierNode* frontier;
    const int32_t* any_dir_ptr;
    const float* inv_scale_ptr;
    int n_eras;
    int max_bins;
    int n_thr;
    const int32_t* thr_ids;      // [n_thr] ascending bin ids, or [n_feat][n_thr] with thr_per_feature
    int thr_per_feature;         // 1: every feature of the block has its own threshold list (mass cuts)
    float lambda_l2, lambda_dro, direction_weight, era_alpha;
    int direction_form;          // 0: agreement with the parent's direction, 1: +1 / -1 by comparing the child values
    int min_samples_leaf;
    Cand* cand;                  // [n_sampled][node_stride]
    // scratch of the two-kernel scorer, for the n_feat features of this block
    float2* gw;                  // [n_feat][n_eras][node_stride][n_thr] (gain, validity weight)
    uint32_t* lc_tot;            // [n_feat][node_stride][n_thr] left counts summed over eras
    int64_t* lg_tot;             // [n_feat][node_stride][n_thr] left gradient sums summed over eras
    void* prof;                  // pb_train_state.profile
    int fused;                   // 1: gw and the totals were written by the histogram kernel's fused flush
    int tot_fpl, tot_lanes;      // layout of lc_tot / lg_tot (tot_index(); 0, 0: the classic layout above)
};
int launch_score(const ScoreLaunch& s, cudaStream_t stream);
// Per-feature threshold lists at the count-mass quantiles of the frontier rows (mass K-cuts), from a
// stored histogram: thr_out[f][n_thr].
int launch_mass_thresholds(const uint32_t* cnt, int n_feat, const int32_t* n_nodes_ptr, int n_nodes_max, int node_stride,
                           int n_eras, int max_bins, int n_thr, int32_t* thr_out, cudaStream_t stream);
size_t score_scratch_bytes_per_feature(int node_stride, int n_eras, int n_thr);

}  // namespace pb
