/*
 * packboost_b200 — C ABI of the B200 (sm_100a) backend for PackBoost's training and
 * prediction hot path.
 *
 * The library is loaded with ctypes / dlopen.  Every entry point is `extern "C"`, takes
 * plain device pointers, sizes and a CUDA stream (as an opaque `void*`, i.e. a
 * `cudaStream_t`), allocates nothing on the device (the one exception is stated at its
 * declaration), never synchronises the device unless its comment says so, and returns 0
 * on success or a negative `PB_ERR_*` code; `pb_last_error()` then holds a thread-local
 * message.  Callers own every buffer.
 *
 * Each declaration cites the reference interface it stands in for (paths are relative to
 * the reference project root).
 *
 * Data layout shared by the training entry points
 * -----------------------------------------------
 *  rows        are ordered by (era, original row); `era_offsets[e]..era_offsets[e+1]` is the
 *              row range of era `e` (int32, E+1 entries).
 *  codes       feature-major bin codes, one row of `pitch` bytes per (locally owned)
 *              feature.  `code_bits == 8`: one byte per row.  `code_bits == 4` (max_bins
 *              <= 16): two rows per byte, even row in the low nibble.  `pitch` is a
 *              multiple of 128 and covers `rows_padded = roundup(n_rows, 256)` rows; the
 *              buffer starts on a 32-byte boundary (the histogram kernel reads whole
 *              32-byte sectors with one 256-bit load).
 *  gq          int32 fixed-point gradient per row, `gq = rint(g * scale)` with `scale` a
 *              power of two chosen per round so that `max|gq| <= 2^gq_bits`; gq_bits is 30
 *              when no era tile exceeds 2047 rows, 27 up to 4095 rows and 24 up to 8160 rows
 *              (the histogram kernel accumulates a tile in 32-bit shared-memory words).
 *  slot        uint16 frontier slot of the row at the current depth (index into the list of
 *              active nodes) or 0xFFFF when the row sits in a finished leaf.
 *  leaf        uint16 id of the tree node the row currently sits in (BFS-compact ids: a
 *              split appends `left = n_nodes, right = n_nodes + 1`).
 *  histograms  `cnt` uint32 and `gsum` int64, both `[feature][era][node][bin]`.
 */
#ifndef PACKBOOST_B200_H
#define PACKBOOST_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PB_OK 0
#define PB_ERR_ARG (-1)      /* bad argument (null pointer, size out of range, misalignment) */
#define PB_ERR_CUDA (-2)     /* a CUDA runtime call failed; message starts with "CUDA error" */
#define PB_ERR_WORKSPACE (-3)/* workspace too small */
#define PB_ERR_NO_DEVICE (-4)

#define PB_SLOT_NONE 0xFFFFu
#define PB_MAX_DEPTH 12

/* ---- library / device probes --------------------------------------------------------- */

/* Thread-local message of the last failing call ("" if none). */
const char* pb_last_error(void);

/* ABI version of this header; bumped on any layout or signature change. */
int pb_abi_version(void);

/* Number of visible CUDA devices with compute capability 10.x; 0 when there is none.
 * Stands in for `_cuda_available()` (packboost/backends/cuda/frontier_cuda.cu:1077,
 * probed by packboost/backends/__init__.py:101-119). */
int pb_device_count(void);

/* Instrumentation (the reference times its phases with perf_counter buckets,
 * packboost/booster.py:220-270, and a cudaEvent pair around its kernel,
 * packboost/backends/cuda/frontier_cuda.cu:670-710).  A profile object belongs to one training
 * state (`pb_train_state.profile`, NULL = no timing): while it is set, every launch of a kernel
 * family made through that state is bracketed by two events on its stream (not inside a stream
 * capture).  After synchronising, pb_profile_collect returns per family (0 histogram, 1 scorer,
 * 2 select, 3 partition, 4 round begin/end) the summed milliseconds and the number of bracketed
 * launches; pb_profile_collect_launches returns the launches one by one in issue order (family and
 * milliseconds, at most `cap`; `*n_out` is how many there were).  Both take the launches that have
 * finished, in issue order up to the first unfinished one, and remove them from the record.  States
 * with different profile objects may run concurrently.  pb_launch_count is the number of kernels
 * this library launched since it was loaded.  With PACKBOOST_NVTX=1 in the environment every phase
 * entry point opens an NVTX range ("pb.hist_score d=3", ...) for tools that attach to the process. */
void* pb_profile_create(void);
void pb_profile_destroy(void* profile);
int pb_profile_collect(void* profile, double* ms_by_kind /* [5] */, int64_t* launches_by_kind /* [5] */);
int pb_profile_collect_launches(void* profile, int32_t* kinds, float* ms, int64_t cap, int64_t* n_out);
int64_t pb_launch_count(void);

/* ---- binning and packing (packboost/data.py:45-58, 96-111) ---------------------------- */

/* Bin a row-major float32 chunk `x[n_chunk][n_features]` with per-feature edges
 * `edges[n_edges][n_features]` (code = number of edges < x, NaN -> last bin, clipped to
 * max_bins-1) and write the codes feature-major into `codes` at rows
 * `row_offset..row_offset+n_chunk`.  Replaces the searchsorted loop of quantile_bin /
 * apply_bins (packboost/data.py:51-57, 105-110). `row_offset` must be even in 4-bit mode.
 * `feature_map[j]` gives the destination feature row of input column j, or -1 to drop the
 * column (used by feature sharding); NULL maps column j to row j. */
int pb_bin_pack_f32(const float* x, int64_t n_chunk, int64_t n_features, int64_t row_offset,
                    const float* edges, int64_t n_edges, int64_t max_bins,
                    const int32_t* feature_map, uint8_t* codes, int64_t pitch,
                    int64_t code_bits, void* stream);

/* Same for input that already holds bin ids (uint8/int8 values in [0, max_bins)); the
 * prebinned passthrough of packboost/data.py:78-91. */
int pb_pack_codes_u8(const uint8_t* x, int64_t n_chunk, int64_t n_features, int64_t row_offset,
                     const int32_t* feature_map, uint8_t* codes, int64_t pitch,
                     int64_t code_bits, void* stream);

/* Row-major packing for the predictor: `out[row][pitch_row]`, 4-bit (two features per byte,
 * even feature in the low nibble) or 8-bit.  Float input is binned with `edges` first
 * (`edges == NULL`: input is uint8 bin ids). */
int pb_pack_rows(const void* x, int64_t x_is_f32, int64_t n_rows, int64_t n_features,
                 const float* edges, int64_t n_edges, int64_t max_bins,
                 uint8_t* out, int64_t pitch_row, int64_t code_bits, void* stream);

/* ---- training state ------------------------------------------------------------------ */

/* All fields are 8 bytes wide so that a ctypes.Structure mirrors the layout trivially. */
typedef struct pb_train_state {
    /* problem shape */
    int64_t n_rows;
    int64_t n_features_total;    /* F of the data set (feature ids in trees are global) */
    int64_t n_features_local;    /* feature rows held in `codes` on this device */
    int64_t n_eras;
    int64_t max_bins;
    int64_t code_bits;           /* 4 or 8 */
    int64_t pitch;               /* bytes per feature row of `codes` */
    /* hyper-parameters (packboost/config.py:68-90) */
    int64_t max_depth;
    int64_t pack_size;
    int64_t min_samples_leaf;
    int64_t n_thresholds;        /* K: max_bins-1 for the full sweep, fewer for k_cuts */
    int64_t feature_block_size;  /* resolved block size of the sampled-feature order */
    double lambda_l2;
    double lambda_dro;
    double direction_weight;
    double era_alpha;
    double learning_rate;
    /* device buffers owned by the caller */
    const uint8_t* codes;        /* [n_features_local][pitch], 32-byte aligned */
    const int32_t* era_offsets;  /* [n_eras + 1] */
    const int32_t* thr_ids;      /* [n_thresholds] threshold (bin) ids, ascending */
    const int32_t* feat_local;   /* [n_features_total] local row of a global feature, -1 if not held */
    const float* y;              /* [n_rows], 16-byte aligned */
    float* preds;                /* [n_rows], 16-byte aligned */
    int32_t* gq;                 /* [rows_padded], 16-byte aligned */
    uint16_t* slot;              /* [rows_padded], 16-byte aligned; pb_round_begin sets the entries past n_rows to 0xFFFF */
    uint16_t* leaf;              /* [rows_padded], 16-byte aligned */
    void* ctl;                   /* control block, pb_ctl_bytes() bytes, zero-initialised once */
    void* workspace;             /* histogram + candidate scratch; NULL (with workspace_bytes 0) for a host that
                                    cannot allocate one: see pb_depth_hist_score_static */
    int64_t workspace_bytes;
    /* tiling of the rows computed by pb_train_prepare (host side, read-only afterwards) */
    int64_t max_era_rows;
    int64_t hist_rows_per_tile;
    int64_t gq_bits;             /* |gq| <= 2^gq_bits */
    int64_t count_bits;          /* CB: rows of a histogram tile < 2^CB */
    int64_t lo_bits;             /* LB = 32 - 2*CB: low gradient bits kept beside the count */
    int64_t cut_mass;            /* 1: k_cuts with cut_selection="mass": the n_thresholds thresholds of a feature are
                                    taken per depth at the quantiles of its bin masses over the frontier rows
                                    (packboost/backends/cpu/frontier_cpu.cpp:59-109); thr_ids is then unused */
    void* profile;               /* pb_profile_create() object, or NULL: see "Instrumentation" */
    int64_t direction_form;      /* directional term of the score (direction_weight != 0): 0 = agreement of the two
                                    child directions with the parent's, the torch frontier's form
                                    (packboost/booster.py:1811-1815, 1873-1880); 1 = +1 where the left child value
                                    exceeds the right one, else -1, the form of the reference's helper and native
                                    code (packboost/booster.py:869-907, backends/cpu/frontier_cpu.cpp:395-401) */
} pb_train_state;

/* Index checks for debugging (the reference checks its inputs on the host,
 * packboost/booster.py:349-367, and guards indices in its kernels,
 * packboost/backends/cuda/frontier_cuda.cu:279-303, 451).  A library built with -DPB_DEBUG_BOUNDS
 * (`python -m packboost_b200.build --debug-bounds`) makes the training kernels check the frontier
 * slot and the bin codes of every row they accumulate and the feature id of every split they apply;
 * a violation is recorded in a sticky word of the control block and the offending index is skipped
 * - nothing traps.  pb_debug_flags copies that word to the host (it synchronises the device):
 * bit 0 slot out of range, bit 1 bin code >= max_bins, bit 2 feature id out of range.  In a regular
 * build the checks are compiled out and the word stays 0; pb_debug_bounds_enabled says which build
 * this is. */
int pb_debug_bounds_enabled(void);
int pb_debug_flags(const pb_train_state* st, uint32_t* flags_out);

/* sizeof(pb_train_state), so that a binding can verify its mirror of the struct. */
int64_t pb_train_state_bytes(void);

/* Bytes of the device control block (`ctl`): round scalars, frontier tables, the
 * per-round decision log and the leaf-value tables. */
int64_t pb_ctl_bytes(void);

/* Smallest useful `workspace_bytes` for the shape in `st` (enough for one block of
 * `feature_block_size` features at the deepest level is NOT required: the histogram pass
 * loops over as many features as fit). */
int64_t pb_workspace_min_bytes(const pb_train_state* st);

/* Validate `st`, derive the tiling fields.  `era_offsets_host` is the host copy of the era
 * offsets.  No device work. */
int pb_train_prepare(pb_train_state* st, const int32_t* era_offsets_host);

/* ---- one boosting round, phase by phase ------------------------------------------------
 * Together these replace the per-round body of PackBoost.fit (packboost/booster.py:494-599)
 * and the torch frontier it calls (packboost/booster.py:1598-2133).  The host keeps the
 * control flow: it draws the per-depth feature subset with its own generator
 * (packboost/booster.py:787-792) and launches the phases in order on one stream. */

/* Start of a round (packboost/booster.py:496-513, 582-597 of the PREVIOUS round, and
 * 2149-2154): preds += delta[leaf] when `apply_previous` != 0, then g = preds - y, the
 * per-round power-of-two scale, gq, every row back to slot 0 / tree node 0, and the root
 * entry of the frontier (count, gradient sum, root leaf value). */
int pb_round_begin(const pb_train_state* st, int64_t apply_previous, void* stream);

/* Histograms and DES scores for one depth (packboost/booster.py:933-977, 1759-1908):
 * `feat_rows[i]` is the local feature row of the i-th locally held sampled feature and
 * `feat_pos[i]` its position in the sampled order (both device int32[n_feat]).  For every
 * (sampled position, frontier node) the best threshold under the order (score, left count,
 * threshold) is written to the candidate table, `n_sampled` x nodes entries; positions not
 * listed in `feat_pos` are left untouched (another device fills them). */
int pb_depth_hist_score(const pb_train_state* st, int64_t depth, const int32_t* feat_rows,
                        const int32_t* feat_pos, int64_t n_feat, int64_t n_sampled, void* stream);

/* Device pointer and byte size of the candidate table of `depth` (for the cross-device
 * exchange: entries are disjoint per device, so a SUM all-reduce over int32 words merges
 * them; `pb_depth_clear_candidates` must run first when more than one device takes part). */
int pb_candidates_buffer(const pb_train_state* st, int64_t depth, int64_t n_sampled,
                         void** ptr, int64_t* bytes);
int pb_depth_clear_candidates(const pb_train_state* st, int64_t depth, int64_t n_sampled, void* stream);

/* Same computation as pb_depth_hist_score for callers that cannot provide a workspace because
 * they cannot allocate device memory at all: processes whose device memory is reserved in full
 * by another component's pool at start-up, or deployments that forbid device allocation once
 * they are running.  This entry point has no counterpart in the reference.  The per-block
 * histograms and scorer tables live in a fixed 64 MiB array inside the library image
 * (pb_static_scratch_bytes(); every GPU that loads the library holds it until the process
 * exits); `st->workspace` is not touched and may be NULL (with `workspace_bytes` 0, which
 * pb_train_prepare accepts).  The candidate table is written to the caller's `cand_out`
 * (24-byte records, `n_sampled` x (1 << depth), same layout as pb_candidates_buffer); hand the
 * same buffer to pb_depth_select_cand for the next phase.  pb_round_begin, pb_depth_partition,
 * pb_round_end and pb_apply_leaf_delta never use the workspace, so a whole round runs without one.
 * Nothing is allocated or freed.  A shape whose single-feature scratch at `depth`,
 *   (1 << depth) * (n_eras * (max_bins * 12 + n_thresholds * 8) + n_thresholds * 12) + 1280 bytes
 * (histogram, per-era gain table, era-summed left counts and gradient sums, alignment), exceeds
 * the array is rejected with PB_ERR_ARG.  (Where the histogram kernel computes the gains itself
 * (few bins, one tile per era) the histogram term max_bins * 12 drops out and
 * (1 << depth) * n_thresholds * 3072 bytes of table padding are added.)  The first call on a device looks up the array's device
 * address (cudaGetSymbolAddress) with that device current; make that first call outside any
 * stream capture.  All calls in a process share the one array, which keeps whatever the previous
 * call left in it: the kernels rewrite every cell they later read, but two calls whose kernels
 * overlap on the GPU (different streams) race on it — serialise them. */
int64_t pb_static_scratch_bytes(void);
int pb_depth_hist_score_static(const pb_train_state* st, int64_t depth, const int32_t* feat_rows,
                               const int32_t* feat_pos, int64_t n_feat, int64_t n_sampled,
                               void* cand_out, void* stream);

/* Pick the winner of every frontier node (packboost/booster.py:1912-1981: in-block order
 * score, left count, position; across blocks strictly greater on score, left count,
 * feature id, threshold), assign BFS-compact child ids (packboost/booster.py:181-187),
 * compute child leaf values in float64 (packboost/booster.py:545-546, 2103-2108), decide
 * which children stay on the frontier (packboost/booster.py:794-796) and write the depth's
 * decision log.  `sampled_features` is the device int32[n_sampled] list of global feature
 * ids in sampled order. */
int pb_depth_select(const pb_train_state* st, int64_t depth, const int32_t* sampled_features,
                    int64_t n_sampled, void* stream);
/* The same with the candidate table passed explicitly (`cand`: 24-byte records, `n_sampled` x
 * (1 << depth)) instead of being read from the workspace: the table pb_depth_hist_score_static
 * wrote, or one assembled by the caller from several devices. */
int pb_depth_select_cand(const pb_train_state* st, int64_t depth, const int32_t* sampled_features,
                         int64_t n_sampled, const void* cand, void* stream);

/* Route every frontier row to its child (packboost/booster.py:2172-2188: left when
 * code <= threshold) and update `slot` / `leaf`.  Single-device form. */
int pb_depth_partition(const pb_train_state* st, int64_t depth, void* stream);

/* Feature-sharded form: each device sets the go-left bit of the rows whose winning feature
 * it holds (`bits` is uint32[rows_padded/32], zero elsewhere); after a SUM/OR all-reduce
 * of `bits` every device applies them. */
int pb_depth_goleft_bits(const pb_train_state* st, int64_t depth, uint32_t* bits, void* stream);
int pb_depth_apply_bits(const pb_train_state* st, int64_t depth, const uint32_t* bits, void* stream);

/* ---- cross-device exchange (several devices, features sharded) ----------------------------------
 * The reference is single-device and has nothing to cite here.  With the sampled features of a
 * depth split over several devices, each device fills the candidate entries of its own features
 * (pb_depth_clear_candidates first) and the tables are merged by a SUM all-reduce over their
 * int32 words (entries are disjoint); in the memory-sharded layout the go-left bits are merged the
 * same way (disjoint bits: SUM is OR).  These entry points do that on NCCL, on the caller's stream,
 * for hosts that have no collective library of their own (a framework that already holds a
 * communicator can all-reduce the buffers itself).  NCCL is looked up at run time; without it they
 * return PB_ERR_ARG and say so.  Usage: one rank calls pb_comm_unique_id and hands the
 * PB_COMM_ID_BYTES bytes to the others by whatever means the host has, every rank calls
 * pb_comm_init with its device current, then per depth pb_comm_allreduce_candidates between
 * pb_depth_hist_score and pb_depth_select (and pb_comm_allreduce_mask between pb_depth_goleft_bits
 * and pb_depth_apply_bits).  A failure of an earlier collective (for instance a peer that left) is
 * reported by the next call as an error code.  pb_comm_destroy after the last collective has
 * finished. */
#define PB_COMM_ID_BYTES 128
int pb_comm_unique_id(void* id_out /* PB_COMM_ID_BYTES */);
int pb_comm_init(void** comm_out, const void* unique_id, int64_t n_ranks, int64_t rank);
int pb_comm_allreduce_candidates(void* comm, const pb_train_state* st, int64_t depth, int64_t n_sampled, void* stream);
int pb_comm_allreduce_mask(void* comm, uint32_t* bits, int64_t n_words, void* stream);
int pb_comm_destroy(void* comm);

/* End of a round: finish the leaf-delta table (pack aggregation, packboost/booster.py:
 * 582-598: every one of the B identical trees adds its float32 leaf value, scaled by the
 * float32 learning rate).  The predictions themselves are updated by the next
 * pb_round_begin or by pb_apply_leaf_delta. */
int pb_round_end(const pb_train_state* st, void* stream);
int pb_apply_leaf_delta(const pb_train_state* st, void* stream);

/* Per-era Pearson correlation of `preds` and `y` (device float32[n_rows], rows ordered by era,
 * `era_offsets` device int32[n_eras+1]) into `corr_out` (device float64[n_eras]); replaces the
 * host loop of packboost/booster.py:909-929 (`_era_correlation_np`), which needs both arrays on
 * the host every round.  An era the reference skips (fewer than two rows, a standard deviation
 * <= 1e-12, a non-finite quotient) yields NaN; the metric is the mean of the other entries. */
int pb_era_correlation(const float* y, const float* preds, const int32_t* era_offsets, int64_t n_eras,
                       double* corr_out, void* stream);

/* Device address and size of the round's decision log (copy it to the host after
 * pb_round_end; layout: pb_round_log below). */
int pb_round_log_buffer(const pb_train_state* st, void** ptr, int64_t* bytes);

typedef struct pb_winner {
    int32_t feature;      /* global feature id, -1: node not split */
    int32_t threshold;    /* bin id: rows with code <= threshold go left */
    float score;
    int32_t tree_node;    /* id of the split node */
    int64_t left_count;
    int64_t total_count;
    int64_t left_gq;      /* exact fixed-point sums */
    int64_t total_gq;
    int32_t left_id;      /* child ids (BFS-compact) */
    int32_t right_id;
    double left_value;    /* float64 leaf values of the children */
    double right_value;
    float left_grad;      /* float32 sums as used for the leaf values */
    float total_grad;
} pb_winner;

typedef struct pb_round_log_header {
    double root_value;
    float scale;          /* gq = rint(g * scale) */
    float max_abs_grad;
    int64_t root_gq;
    int32_t n_ctx[PB_MAX_DEPTH + 1]; /* frontier nodes per depth; winners of depth d start at (1<<d)-1 */
    int32_t n_tree_nodes;
    int32_t reserved[2];
} pb_round_log_header;
/* The log is a pb_round_log_header followed by (1 << max_depth) - 1 pb_winner records. */

/* ---- kernel-level entry points (used directly by the parity tests and the benchmark) ---- */

/* Histogram pass alone (packboost/booster.py:933-977, counts and gradient sums; the
 * hessian of the squared loss is 1, so its histogram is the count).  Output layout
 * `[n_feat][n_eras][node_stride][max_bins]`. `n_nodes` frontier slots are accumulated. */
int pb_hist_build(const pb_train_state* st, const int32_t* feat_rows, int64_t n_feat,
                  int64_t n_nodes, int64_t node_stride, uint32_t* cnt, int64_t* gsum, void* stream);

/* Best threshold of every feature for ONE node with general (per-row) hessians: the single-node
 * form of the frontier (`PackBoost._find_best_split`, packboost/booster.py:1010-1290, exercised by
 * the reference's hand-built DES test, tests/test_des.py:9-217).  `cnt` / `gsum` / `hsum` are the
 * node's histograms `[n_feat][n_eras][max_bins]` (two pb_hist_build passes with node_stride 1: the
 * second with the fixed-point hessians in place of the gradients); `inv_scale_g` / `inv_scale_h`
 * turn the integer sums back into float32; `total_count` / `total_gq` are the node's row count and
 * fixed-point gradient sum.  The training loop does not use this entry (the squared loss has unit
 * hessians).  `out[f]` receives the feature's best threshold under (score, left count, index). */
typedef struct pb_split_general {
    float score;
    int32_t k;            /* index into thr_ids, -1: none */
    int32_t threshold;    /* bin id */
    int32_t has_nan;      /* a threshold of this feature scored NaN */
    int64_t left_count;
    int64_t left_gq;      /* fixed-point sums of the left child */
    int64_t left_hq;
} pb_split_general;
int pb_score_node_general(const uint32_t* cnt, const int64_t* gsum, const int64_t* hsum, int64_t n_feat,
                          int64_t n_eras, int64_t max_bins, const int32_t* thr_ids, int64_t n_thresholds,
                          float inv_scale_g, float inv_scale_h, float lambda_l2, float lambda_dro,
                          float direction_weight, float era_alpha, int64_t direction_form,
                          int64_t min_samples_leaf, int64_t total_count, int64_t total_gq,
                          pb_split_general* out, void* stream);

/* ---- prediction ----------------------------------------------------------------------- */

/* Ensemble over row-major packed codes (see pb_pack_rows):
 * out[row] = fold over trees in order of out + weight * leaf(tree, row), in float32 without
 * contraction — the CPU route of PackBoost.predict (packboost/booster.py:709-712) with
 * Tree routing (packboost/booster.py:131-169).  Trees are concatenated node arrays;
 * `tree_offsets[t]` is the first node of tree t, children are tree-relative.
 * `repeat[t]` (may be NULL = 1) adds tree t that many times in a row (identical trees of a
 * pack are stored once).  The accumulation starts from `init[row]` (NULL: from 0), which
 * lets a caller extend earlier predictions by the trees added since; `out` is overwritten
 * and may alias `init`. */
int pb_predict_rows(const uint8_t* codes, int64_t n_rows, int64_t pitch_row, int64_t code_bits,
                    const int32_t* feature, const int32_t* threshold, const int32_t* left,
                    const int32_t* right, const float* value, const uint8_t* is_leaf,
                    const int32_t* tree_offsets, const int32_t* repeat, int64_t n_trees,
                    float weight, float* out, const float* init, void* stream);

/* Same ensemble sum with the trees in the packed form the training loop can produce directly:
 * one 8-byte record per node, word 0 = feature (bits 0-15) | threshold (bits 16-23) | leaf flag
 * (bit 31), word 1 = tree-relative index of the left child (the right child is the next node,
 * as in the BFS-compact numbering of packboost/booster.py:181-187) or the float bits of a leaf
 * value.  Requires feature ids < 65536 and thresholds < 256.  `max_tree_nodes` is the node count
 * of the largest tree: trees of up to 512 nodes are streamed through shared memory in batches,
 * larger ones are read from global memory. */
int pb_predict_rows_packed(const uint8_t* codes, int64_t n_rows, int64_t pitch_row, int64_t code_bits,
                           const void* nodes, const int32_t* tree_offsets, const int32_t* repeat,
                           int64_t n_trees, int64_t max_tree_nodes, float weight, float* out,
                           const float* init, void* stream);

/* Single tree over feature-major uint8 codes `bins[F][N]`: the argument list of
 * predict_bins_cuda (packboost/backends/cuda/frontier_cuda.cu:853-861). */
int pb_predict_bins_fm(const uint8_t* bins, int64_t n_features, int64_t n_rows,
                       const int32_t* feature, const int32_t* threshold, const int32_t* left,
                       const int32_t* right, const float* value, const uint8_t* is_leaf,
                       int64_t n_nodes, float* out, void* stream);

/* One pack over feature-major uint8 codes, out[row] = tree_weight * sum over trees of the
 * leaf value: the argument list of predict_pack_cuda
 * (packboost/backends/cuda/frontier_cuda.cu:989-999); children are absolute node ids. */
int pb_predict_pack_fm(const uint8_t* bins, int64_t n_features, int64_t n_rows,
                       const int32_t* feature, const int32_t* threshold, const int32_t* left_abs,
                       const int32_t* right_abs, const float* value, const uint8_t* is_leaf,
                       const int32_t* offsets, int64_t n_trees, float tree_weight,
                       float* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PACKBOOST_B200_H */
