// Per-(feature, node, era, bin) histograms of counts and fixed-point gradient sums.
//
// Rows are ordered by era, so an era is a contiguous row range.  One CTA owns one row tile of
// one era (at most kTileRowsMax rows) and a contiguous range of the sampled features, accumulates
// them in shared memory and writes (or, when an era is cut into several tiles, atomically adds)
// the result to the global histogram.  Every cell is an integer, so the result does not depend
// on the order of the additions.
//
// Shared-memory cell: two 32-bit words updated with one native 32-bit shared atomic each
// (64-bit shared atomics are an order of magnitude slower on this part):
//   A = (sum of lo) << CB | count        lo = gq & (2^LB - 1)
//   B = sum of hi                        hi = gq >> LB (arithmetic)
// With fewer than 2^CB rows per tile, LB = 32 - 2*CB and |gq| <= 2^(63 - 3*CB) (capped at
// 2^30) neither word can overflow; pb_train_prepare derives CB/LB and the gradient scale from
// the largest tile.
//
// Two kernels share that cell format:
//  * hist_lane_kernel (few cells per feature: nodes * bins^A <= kLaneCellsMax): a lane owns a
//    tuple of A features and a private column of cells (bank == lane, so the shared atomics of a
//    warp never conflict); all lanes of a warp walk the same rows, whose state (cell base, word A,
//    word B) is staged per warp and read with one broadcast load; the codes reach the lanes through
//    a block staged in shared memory by whole-line asynchronous copies.  With A > 1 the cell index is
//    the joint code of the tuple, one pair of atomics serves A features, and the per-feature
//    histograms are the marginals of the joint table, taken when the tile is flushed.
//  * hist_kernel (everything else): a thread owns one 16-byte chunk of codes per feature (32 rows
//    of 4-bit codes, 16 rows of 8-bit codes); the slot and gradient of those rows stay in registers
//    while the thread walks the CTA's features, prefetching the next feature's chunk.  Cells of a
//    feature are shared by the CTA and, when few, replicated ("copies") to thin out conflicts.
//
// Output layout: [feature][era][node_stride][bin] for both arrays.

#include <stdio.h>
#include <stdlib.h>

#include <type_traits>

#include "common.cuh"
#include "des_math.cuh"

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
    int fuse;        // 1: the lane kernel's flush writes gains and era-summed totals instead of the histogram
    HistFuse fz;
    uint32_t* debug_flags;
};

template <int BITS, int THREADS>
__global__ void __launch_bounds__(THREADS) hist_kernel(HistKernelArgs a) {
    constexpr int RPI = (BITS == 4) ? 32 : 16;  // rows per thread (16 bytes of codes)
    extern __shared__ uint32_t cells[];         // word A plane [group][cells_per_feat][copies], then word B plane
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
        const int plane = a.group * cells_per_feat * copies;  // words per plane
        const int total_words = nf * cells_per_feat * copies;
        for (int i = threadIdx.x; i < total_words; i += blockDim.x) {
            cells[i] = 0u;
            cells[plane + i] = 0u;
        }
        __syncthreads();

        for (int fi = 0; fi < nf; ++fi) {
            uint4 nxt = make_uint4(0, 0, 0, 0);
            const int fnext = g0 + fi + 1;
            if (has && fnext < fb)
                nxt = __ldg(reinterpret_cast<const uint4*>(a.codes + (int64_t)s_frow[fnext - fa] * a.pitch) + c);
            if (has) {
                const uint32_t w[4] = {cur.x, cur.y, cur.z, cur.w};
                uint32_t* fc = cells + (size_t)fi * cells_per_feat * copies + lane_copy;
#pragma unroll
                for (int j = 0; j < RPI; ++j) {
                    int code;
                    if (BITS == 4) {
                        code = (w[j >> 3] >> ((j & 7) * 4)) & 0xF;
                    } else {
                        code = (w[j >> 2] >> ((j & 3) * 8)) & 0xFF;
                    }
                    const uint32_t base = (cb2[j >> 1] >> ((j & 1) * 16)) & 0xFFFFu;
#ifdef PB_DEBUG_BOUNDS
                    if (base != 0xFFFFu && code >= nb) {
                        if (a.debug_flags) atomicOr(a.debug_flags, kDbgCode);
                        continue;
                    }
#endif
                    if (base != 0xFFFFu) {
                        uint32_t* cell = fc + (size_t)(base + code) * copies;
                        atomicAdd(cell, (((uint32_t)g[j] & lo_mask) << CB) + 1u);
                        atomicAdd(reinterpret_cast<int*>(cell + plane), g[j] >> LB);
                    }
                }
            }
            cur = nxt;
        }
        __syncthreads();

        // flush: fold the copies, rebuild count and gradient sum, write [feature][era][node][bin]
        const int out_cells = nf * cells_per_feat;
        for (int i = threadIdx.x; i < out_cells; i += blockDim.x) {
            const int fi = i / cells_per_feat;
            const int rem = i - fi * cells_per_feat;
            const int node = node_lo + rem / nb;
            const int bin = rem - (rem / nb) * nb;
            const uint32_t* src = cells + (size_t)i * copies;
            uint32_t count = 0;
            long long lo_sum = 0, hi_sum = 0;
            for (int k = 0; k < copies; ++k) {
                const uint32_t A = src[k];
                count += A & ((1u << CB) - 1u);
                lo_sum += (long long)(A >> CB);
                hi_sum += (long long)(int32_t)src[plane + k];
            }
            const long long gs = hi_sum * (1ll << LB) + lo_sum;
            const size_t o = (((size_t)(g0 + fi) * a.n_eras + era) * a.node_stride + node) * nb + bin;
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


// ---- lane-private kernel for small cell counts ------------------------------------------------

constexpr int kLaneCellBytes = 256;        // word A of lane l at l*4, word B at 128 + l*4: bank == lane
__host__ __device__ constexpr int lane_cell_bytes(int R) { return R == 2 ? 128 : 256; }  // (two row phases share a column)
constexpr int kLaneCellsMax = 100 * 1024;  // bytes of cells of one CTA (two CTAs per SM with the staged codes)
constexpr int kLaneWarps = 8;
constexpr int kLaneRows = 32;              // rows per warp and CTA step
constexpr int kBlockRows = kLaneWarps * kLaneRows;  // 256 rows: one 128-byte line of 4-bit codes per feature
constexpr int kStagePitch = 144;           // bytes per feature of the staged code block (see below)

// The CTA walks its tile in blocks of 256 rows.  The codes of a block are one 128-byte line per
// feature; they are copied to shared memory with 16-byte asynchronous copies in which eight
// consecutive threads fetch one line, so that every memory request is a whole line.  (A warp whose
// lanes each read 32 bytes of a different feature row issues 32 one-sector requests per
// instruction; the memory system serves requests, not bytes, and that pattern measured 1.6 TB/s
// against 6.1 TB/s for whole lines on the same data.)  Warp w then owns rows [32 w, 32 w + 32) of
// the block: a lane reads the 16 bytes of those rows of each of its features from the staged block
// into registers (feature slots 144 bytes apart: consecutive lanes read consecutive slots, which
// spreads a quarter-warp over all banks), and the next block is fetched while the rows are
// accumulated.
//
// All lanes of a warp walk the same rows, so the row state is warp-uniform.  It is staged per
// warp as one 8-byte record per row {word A addend with the index of the node's first cell in its
// unused bits, word B addend}, written once per row by one lane and read by all lanes with a single
// broadcast load.  A row that is not accumulated has an all-zero record: it adds zero to the cells
// of node 0, so the row steps carry no branch.  A lane owns T tuples of A features (T*A consecutive
// sampled features), each tuple with its own set of cells.
//
// With few features per launch (a feature shard of a multi-GPU run) the warp is split into R row
// phases: 32 / R lanes own tuples and phase p of them walks rows [p, p + 1) * 32 / R of the warp's
// rows, so a row step of the warp covers R rows.  The R lanes that own the same tuple keep private
// cell columns as always; the flush adds them up.
constexpr int kLaneBinsMax = 16;  // 4-bit codes

// The nb bins of one (feature, node) are contiguous in both output arrays but start on an odd or
// even element: they are written as pairs (8 bytes of counts, 16 bytes of sums) from the first
// even element on, which takes three stores per array for five bins instead of five.  The lanes
// of a warp write to 32 different features, so every store of a lane is a memory wavefront of its
// own and their number is what the flush costs.
template <int ODD>
__device__ __forceinline__ void store_bins(uint32_t* cnt, int64_t* gsum, const uint32_t (&cb)[kLaneBinsMax],
                                           const long long (&gb)[kLaneBinsMax], int nb) {
    if (ODD) {
        cnt[0] = cb[0];
        gsum[0] = gb[0];
    }
#pragma unroll
    for (int k = ODD; k < kLaneBinsMax; k += 2) {
        if (k + 1 < nb) {
            *reinterpret_cast<uint2*>(cnt + k) = make_uint2(cb[k], cb[(k + 1) % kLaneBinsMax]);
            *reinterpret_cast<longlong2*>(gsum + k) = make_longlong2(gb[k], gb[(k + 1) % kLaneBinsMax]);
        } else if (k < nb) {
            cnt[k] = cb[k];
            gsum[k] = gb[k];
        }
    }
}

// Shared memory of a lane-kernel CTA: cells | row records | staged code block | feature row offsets.
__host__ __device__ constexpr size_t lane_record_bytes(int R) { return (size_t)kLaneWarps * (kLaneRows + R) * sizeof(uint2); }
__host__ __device__ constexpr size_t lane_extra_bytes(int R, int fpl) {
    return lane_record_bytes(R) + (size_t)(32 / R) * fpl * (kStagePitch + sizeof(int64_t));
}

template <int A, int T, int R>
__global__ void __launch_bounds__(kLaneWarps * 32, 2) hist_lane_kernel(HistKernelArgs a) {
    extern __shared__ __align__(16) unsigned char smb[];
    const int n_nodes = a.n_nodes_ptr ? min(*a.n_nodes_ptr, a.n_nodes) : a.n_nodes;
    if (n_nodes <= 0) return;
    const int era = blockIdx.x / a.tiles_per_era;
    const int tile = blockIdx.x - era * a.tiles_per_era;
    const int era_begin = a.era_offsets[era];
    const int era_end = a.era_offsets[era + 1];
    const int r0 = era_begin + tile * a.tile_rows;
    const int r1 = min(era_end, r0 + a.tile_rows);
    if (r0 >= r1 && a.use_atomics) return;

    const int nb = a.max_bins;
    int cpn = nb;  // cells per node = bins^A
#pragma unroll
    for (int i = 1; i < A; ++i) cpn *= nb;
    const int n_cells = a.n_nodes * cpn;  // per tuple, sized for the upper bound of nodes
    // Cell layout.  R != 2: every lane has a private column, word A of lane l at l*4 and word B at
    // 128 + l*4 of a 256-byte cell.  R == 2: the two row phases of a tuple-lane share one column of a
    // 128-byte cell (word A of column c at c*4, word B at 64 + c*4): phase 0 adds the word A of its
    // row while phase 1 adds the word B of its own, then the other way round, so a warp instruction
    // still touches every bank once, and twice as many cells fit.
    constexpr bool SHARED = (R == 2);
    constexpr int CELL_BYTES = lane_cell_bytes(R);
    constexpr int CSH = SHARED ? 7 : 8;          // log2(CELL_BYTES)
    constexpr int CW = CELL_BYTES / 4;           // words per cell
    constexpr int BOFF = CW / 2;                 // word B follows the word-A columns
    constexpr int PHS = SHARED ? 1 : R;          // phase columns the flush adds up
    const uint32_t slot_bytes = (uint32_t)n_cells * CELL_BYTES;
    constexpr int FPL = A * T;
    constexpr int TL = 32 / R;            // tuple-owning lanes per phase
    constexpr int NF = TL * FPL;          // features of the CTA
    constexpr int PR = kLaneRows / R;     // rows of a warp step walked by one phase
    constexpr int WPP = PR / 8;           // 32-bit code words per feature and phase
    uint32_t* cells = reinterpret_cast<uint32_t*>(smb);
    uint2* records = reinterpret_cast<uint2*>(smb + (size_t)T * slot_bytes);
    unsigned char* stage = smb + (size_t)T * slot_bytes + lane_record_bytes(R);
    int64_t* frow_s = reinterpret_cast<int64_t*>(stage + (size_t)NF * kStagePitch);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int CB = a.count_bits, LB = a.lo_bits;
    const uint32_t lo_mask = (1u << LB) - 1u;
    // record word x = (lo << CB) | (first cell of the node << 1) | 1: the addend of word A with the
    // cell index in the bits the count field leaves free (a tile has fewer than 2^CB rows and a
    // tuple fewer than 2^(CB-1) cells: pb_train_prepare keeps CB >= 11)
    const uint32_t off_mask = ((1u << (CB - 1)) - 1u) << CSH;
    const uint32_t a_mask = ~(((1u << CB) - 1u) & ~1u);

    {  // (a cell is 128 or 256 bytes: whole 16-byte stores)
        uint4* z = reinterpret_cast<uint4*>(cells);
        for (int i = threadIdx.x; i < T * n_cells * (CW / 4); i += blockDim.x) z[i] = make_uint4(0u, 0u, 0u, 0u);
    }

    // features of this lane: T tuples of A consecutive sampled features.  Staged slot of feature i
    // of tuple-lane l: i * TL + l.
    const int phase = lane / TL;
    const int col0 = lane - phase * TL;
    const int feat0 = (blockIdx.y * TL + col0) * FPL;
    const int n_mine = max(0, min(FPL, a.n_feat - feat0));
    for (int s = threadIdx.x; s < NF; s += blockDim.x) {
        const int f = (blockIdx.y * TL + (s % TL)) * FPL + s / TL;
        frow_s[s] = (int64_t)__ldg(a.feat_rows + min(f, a.n_feat - 1)) * a.pitch;
    }
    __syncthreads();

    // one block of codes: NF lines of 128 bytes, eight consecutive threads per line
    auto fetch_block = [&](int b) {
        for (int p = threadIdx.x; p < NF * 8; p += blockDim.x) {
            const int s = p >> 3, part = p & 7;
            const unsigned char* src = a.codes + frow_s[s] + (int64_t)b * (kBlockRows / 2) + part * 16;
            const uint32_t dst = (uint32_t)__cvta_generic_to_shared(stage + s * kStagePitch + part * 16);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };

    // first word this lane adds to and the distance to the second one
    unsigned char* lane_base = SHARED ? smb + col0 * 4 + phase * 64 : smb + lane * 4;
    const int second = SHARED ? (phase ? -64 : 64) : 128;
    // (a phase's records start one entry further apart than its rows, which keeps the R broadcast
    // addresses of a row step in different banks)
    uint2* st = records + warp * (kLaneRows + R);
    const uint2* st_mine = st + phase * (PR + 1);
    const int b0 = r0 / kBlockRows, b1 = (r1 + kBlockRows - 1) / kBlockRows;

    int raw_s = 0, raw_g = 0;  // slot and gradient of row (block, warp, lane), loaded one block ahead
    auto load_state = [&](int b, int& rs, int& rg) {
        const int r = b * kBlockRows + warp * kLaneRows + lane;
        rs = a.slot[r];
        rg = a.gq[r];
    };
    if (b0 < b1) {
        fetch_block(b0);
        load_state(b0, raw_s, raw_g);
    }
    for (int b = b0; b < b1; ++b) {
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        __syncthreads();  // the block is complete
        uint32_t w[FPL][WPP];
#pragma unroll
        for (int i = 0; i < FPL; ++i) {
            const unsigned char* p = stage + (i * TL + col0) * kStagePitch + warp * (kLaneRows / 2) + phase * (PR / 2);
            if (R == 1) {
                const uint4 v = *reinterpret_cast<const uint4*>(p);
                w[i][0] = v.x; w[i][1 % WPP] = v.y; w[i][2 % WPP] = v.z; w[i][3 % WPP] = v.w;
            } else if (R == 2) {
                const uint2 v = *reinterpret_cast<const uint2*>(p);
                w[i][0] = v.x; w[i][1 % WPP] = v.y;
            } else {
                w[i][0] = *reinterpret_cast<const uint32_t*>(p);
            }
        }
        __syncthreads();  // every warp holds its codes: the stage is free for the next block
        if (b + 1 < b1) fetch_block(b + 1);

        const int r = b * kBlockRows + warp * kLaneRows + lane;
        const bool ok = (r >= r0) & (r < r1) & (raw_s < n_nodes);
#ifdef PB_DEBUG_BOUNDS
        if ((r >= r0) & (r < r1) & (raw_s != (int)kSlotNone) & (raw_s >= a.n_nodes) && a.debug_flags)
            atomicOr(a.debug_flags, kDbgSlot);
#endif
        {
            uint2 rec;
            rec.x = ok ? ((((uint32_t)raw_g & lo_mask) << CB) | ((uint32_t)(raw_s * cpn) << 1) | 1u) : 0u;
            rec.y = ok ? (uint32_t)(raw_g >> LB) : 0u;
            st[lane + lane / PR] = rec;
        }
        const bool chunk_on = __any_sync(0xFFFFFFFFu, ok);  // (also orders the record stores)
        int nraw_s = 0, nraw_g = 0;
        if (b + 1 < b1) load_state(b + 1, nraw_s, nraw_g);
        if (n_mine > 0 && chunk_on) {
            uint32_t jw[T][2];  // joint codes of eight rows: even rows, odd rows (A == 2)
            uint2 rawn[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) rawn[q] = st_mine[q];
#pragma unroll
            for (int jb = 0; jb < PR; jb += 4) {
                // the records of the next four rows are loaded before the atomics of these four
                uint2 raw[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) raw[q] = rawn[q];
                if (jb + 4 < PR) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) rawn[q] = st_mine[jb + 4 + q];
                }
                uint4 rec[4];  // {cell offset, word A addend, word B addend}
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    rec[q].x = (raw[q].x << (CSH - 1)) & off_mask;
                    const uint32_t wa = raw[q].x & a_mask, wb = raw[q].y;
                    rec[q].y = (SHARED && phase) ? wb : wa;  // added to the first word
                    rec[q].z = (SHARED && phase) ? wa : wb;  // added to the second
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int j = jb + q;
                    const int bit = (j & 7) * 4;
#pragma unroll
                    for (int t = 0; t < T; ++t) {
                        const uint32_t w0 = w[t * A][j >> 3];
#ifdef PB_DEBUG_BOUNDS
                        if (raw[q].x & 1u) {  // an accumulated row: its codes must be bins
                            bool bad = ((w0 >> bit) & 0xFu) >= (uint32_t)nb;
#pragma unroll
                            for (int i = 1; i < A; ++i) bad |= ((w[t * A + i][j >> 3] >> bit) & 0xFu) >= (uint32_t)nb;
                            if (bad && A * t < n_mine) {
                                if (a.debug_flags) atomicOr(a.debug_flags, kDbgCode);
                                continue;
                            }
                        }
#endif
                        uint32_t off;  // joint code of the tuple times the cell pitch
                        if (A == 2) {
                            // Joint codes of eight rows at a time: the even and the odd nibbles of the two
                            // code words as bytes c0 + nb * c1 (at most 240: no carry between bytes); a
                            // row's cell offset is its byte times the cell pitch.
                            if ((j & 7) == 0) {
                                const uint32_t w1 = w[t * A + 1][j >> 3];
                                jw[t][0] = (w1 & 0x0F0F0F0Fu) * (uint32_t)nb + (w0 & 0x0F0F0F0Fu);
                                jw[t][1] = ((w1 >> 4) & 0x0F0F0F0Fu) * (uint32_t)nb + ((w0 >> 4) & 0x0F0F0F0Fu);
                            }
                            off = __byte_perm(jw[t][j & 1], 0u, 0x4440u | (uint32_t)((j & 7) >> 1)) << CSH;
                        } else {
                            off = ((w0 >> bit) & 0xFu) << CSH;
                        }
                        unsigned char* cell = lane_base + (rec[q].x + off + (uint32_t)t * slot_bytes);
                        atomicAdd(reinterpret_cast<uint32_t*>(cell), rec[q].y);
                        atomicAdd(reinterpret_cast<uint32_t*>(cell + second), rec[q].z);
                    }
                }
            }
        }
        __syncwarp();  // the records are rewritten in the next step
        raw_s = nraw_s;
        raw_g = nraw_g;
    }
    __syncthreads();

    // flush: marginals of this lane's joint tables -> [feature][era][node][bin]; the R phases of a
    // warp take different items and add up the columns of the R lanes that own the tuple
    const uint32_t cmask = (1u << CB) - 1u;
    if (a.fuse) {
        // ---- fused flush: per-era gains instead of the histogram -----------------------------------
        // The CTA holds the complete cells of its era (one tile per era), so everything the scorer
        // needs from this era is computed here: the prefix over the bins of every (feature, node), the
        // gain and validity weight of every threshold (one 8-byte entry each), and the era's
        // contribution to the left counts / gradient sums summed over eras (integer atomics: exact and
        // independent of their order).  The histogram itself is never written.
        const HistFuse& z = a.fz;
        __shared__ int s_thr[kLaneBinsMax];
        if (threadIdx.x < kLaneBinsMax) s_thr[threadIdx.x] = (threadIdx.x < z.n_thr) ? z.thr_ids[threadIdx.x] : -1;
        __syncthreads();
        const float inv_scale = *z.inv_scale_ptr;
        const int K = z.n_thr;
        const int lane_global = blockIdx.y * TL + col0;   // == (feat0 + fl) / FPL for every fl
        const int lanes_total = gridDim.y * TL;
        auto fuse_emit = [&](auto nbt_c, int fl, int n, const uint32_t (&aw)[kLaneBinsMax],
                             const uint32_t (&bw)[kLaneBinsMax]) {
            constexpr int NBT = decltype(nbt_c)::value;  // compile-time bound of the bin count
            uint32_t cb[NBT];
            long long gb[NBT];
            uint32_t tc = 0;
            long long tgq = 0;
#pragma unroll
            for (int b = 0; b < NBT; ++b) {
                cb[b] = aw[b] & cmask;
                gb[b] = (long long)(int32_t)bw[b] * (1ll << LB) + (long long)(aw[b] >> CB);
                if (b < nb) {
                    tc += cb[b];
                    tgq += gb[b];
                }
            }
            const EraTotals et = era_totals(tc, tgq, inv_scale, z.lambda_l2, z.era_alpha);
            float2* out = z.gw + (((size_t)(feat0 + fl) * a.n_eras + era) * a.node_stride + n) * K;
            const size_t tot0 = (((size_t)n * K) * FPL + fl) * lanes_total + lane_global;  // threshold 0
            const size_t tot_step = (size_t)FPL * lanes_total;
            uint32_t c = 0;
            long long g = 0;
            if (NBT == 5 && z.full_sweep) {
                float2 gk[4];
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    c += cb[b];
                    g += gb[b];
                    gk[b] = gain_of(c, g, tc, et.tg, et.th, et.parent, inv_scale, z.lambda_l2, et.w_era);
                    if (c) atomicAdd(z.lc_tot + tot0 + b * tot_step, c);
                    if (g) atomicAdd(reinterpret_cast<unsigned long long*>(z.lg_tot + tot0 + b * tot_step), (unsigned long long)g);
                }
reinterpret_cast<float4*>(out)[0] = make_float4(gk[0].x, gk[0].y, gk[1].x, gk[1].y);
                reinterpret_cast<float4*>(out)[1] = make_float4(gk[2].x, gk[2].y, gk[3].x, gk[3].y);
            } else {
                int kk = 0;
                int next = s_thr[0];
#pragma unroll
                for (int b = 0; b < NBT - 1; ++b) {
                    if (b < nb - 1) {
                        c += cb[b];
                        g += gb[b];
                        if (b == next) {
                            out[kk] = gain_of(c, g, tc, et.tg, et.th, et.parent, inv_scale, z.lambda_l2, et.w_era);
                            if (c) atomicAdd(z.lc_tot + tot0 + kk * tot_step, c);
                            if (g) atomicAdd(reinterpret_cast<unsigned long long*>(z.lg_tot + tot0 + kk * tot_step), (unsigned long long)g);
                            ++kk;
                            next = (kk < K) ? s_thr[kk] : -1;
                        }
                    }
                }
            }
        };
        for (int item = warp * R + phase; item < n_nodes * T; item += kLaneWarps * R) {
            const int n = item / T, t = item - n * T;
            if (A * t >= n_mine) continue;
            const uint32_t* tcells = cells + (size_t)t * n_cells * CW;
            if (A == 2 && nb == 5) {
                // every joint cell is read once and added to the row sum of one feature and the column
                // sum of the other
                const uint32_t* tc2 = tcells + (size_t)(n * 25) * CW + col0;
                uint32_t a0[kLaneBinsMax], b0[kLaneBinsMax], a1[kLaneBinsMax], b1[kLaneBinsMax];
#pragma unroll
                for (int b = 0; b < kLaneBinsMax; ++b) a0[b] = b0[b] = a1[b] = b1[b] = 0u;
#pragma unroll
                for (int c1 = 0; c1 < 5; ++c1)
#pragma unroll
                    for (int c0 = 0; c0 < 5; ++c0) {
                        uint32_t aw = 0, bw = 0;
#pragma unroll
                        for (int ph = 0; ph < PHS; ++ph) {
                            aw += tc2[(c1 * 5 + c0) * CW + ph * TL];
                            bw += tc2[(c1 * 5 + c0) * CW + ph * TL + BOFF];
                        }
                        a0[c0] += aw;
                        b0[c0] += bw;
                        a1[c1] += aw;
                        b1[c1] += bw;
                    }
                fuse_emit(std::integral_constant<int, 5>(), 2 * t, n, a0, b0);
                if (2 * t + 1 < n_mine) fuse_emit(std::integral_constant<int, 5>(), 2 * t + 1, n, a1, b1);
            } else {
                int below = 1;  // bins^fi
                for (int fi = 0; fi < A; ++fi, below *= nb) {
                    const int fl = t * A + fi;
                    if (fl >= n_mine) break;
                    const int above = cpn / (below * nb);
                    uint32_t aw[kLaneBinsMax], bw[kLaneBinsMax];
#pragma unroll
                    for (int b = 0; b < kLaneBinsMax; ++b) {
                        aw[b] = 0u;
                        bw[b] = 0u;
                        if (b >= nb) continue;
                        uint32_t a_sum = 0, b_sum = 0;
                        for (int hi = 0; hi < above; ++hi)
                            for (int lo = 0; lo < below; ++lo) {
                                const uint32_t cell = (uint32_t)(n * cpn + (hi * nb + b) * below + lo) * (uint32_t)CW + col0;
#pragma unroll
                                for (int ph = 0; ph < PHS; ++ph) {
                                    a_sum += tcells[cell + ph * TL];
                                    b_sum += tcells[cell + ph * TL + BOFF];
                                }
                            }
                        aw[b] = a_sum;
                        bw[b] = b_sum;
                    }
                    if (nb == 5) fuse_emit(std::integral_constant<int, 5>(), fl, n, aw, bw);
                    else fuse_emit(std::integral_constant<int, kLaneBinsMax>(), fl, n, aw, bw);
                }
            }
        }
        return;
    }

    // decode the packed sums of the bins of one (feature, node) and write them out
    auto emit = [&](int fl, int n, const uint32_t (&aw)[kLaneBinsMax], const uint32_t (&bw)[kLaneBinsMax]) {
        const size_t o0 = (((size_t)(feat0 + fl) * a.n_eras + era) * a.node_stride + n) * nb;
        uint32_t cb[kLaneBinsMax];
        long long gb[kLaneBinsMax];
#pragma unroll
        for (int b = 0; b < kLaneBinsMax; ++b) {
            cb[b] = aw[b] & cmask;
            gb[b] = (long long)(int32_t)bw[b] * (1ll << LB) + (long long)(aw[b] >> CB);
        }
        if (a.use_atomics) {
#pragma unroll
            for (int b = 0; b < kLaneBinsMax; ++b) {
                if (b >= nb) continue;
                if (cb[b]) atomicAdd(a.cnt + o0 + b, cb[b]);
                if (gb[b]) atomicAdd(reinterpret_cast<unsigned long long*>(a.gsum + o0 + b), (unsigned long long)gb[b]);
            }
        } else if (o0 & 1) {
            store_bins<1>(a.cnt + o0, a.gsum + o0, cb, gb, nb);
        } else {
            store_bins<0>(a.cnt + o0, a.gsum + o0, cb, gb, nb);
        }
    };
    if (nb == 5 && !a.use_atomics && ((a.n_nodes | a.node_stride) & 3) == 0 && A <= 2 &&
        ((reinterpret_cast<uintptr_t>(a.cnt) | reinterpret_cast<uintptr_t>(a.gsum)) & 15) == 0) {
        // Five-level codes, four nodes at a time: the 20 bins of a feature in four consecutive nodes
        // are contiguous in both output arrays and start on 16 bytes, so they leave as five 16-byte
        // stores of counts and ten of sums (3.75 store wavefronts per node instead of 6).  Nodes
        // past the live frontier have empty cells and write zeros into rows nobody reads.
        auto emit20 = [&](int fl, int n0, const uint32_t (&aw)[20], const uint32_t (&bw)[20]) {
            const size_t o0 = (((size_t)(feat0 + fl) * a.n_eras + era) * a.node_stride + n0) * 5;
            uint4* pc = reinterpret_cast<uint4*>(a.cnt + o0);
            longlong2* pg = reinterpret_cast<longlong2*>(a.gsum + o0);
#pragma unroll
            for (int i = 0; i < 5; ++i)
                pc[i] = make_uint4(aw[4 * i] & cmask, aw[4 * i + 1] & cmask, aw[4 * i + 2] & cmask, aw[4 * i + 3] & cmask);
#pragma unroll
            for (int i = 0; i < 10; ++i)
                pg[i] = make_longlong2((long long)(int32_t)bw[2 * i] * (1ll << LB) + (long long)(aw[2 * i] >> CB),
                                       (long long)(int32_t)bw[2 * i + 1] * (1ll << LB) + (long long)(aw[2 * i + 1] >> CB));
        };
        const int groups = (n_nodes + 3) >> 2;
        for (int item = warp * R + phase; item < groups * T; item += kLaneWarps * R) {
            const int g = item / T, t = item - g * T;
            if (A * t >= n_mine) continue;
            const int n0 = 4 * g;
            const uint32_t* tc = cells + (size_t)t * n_cells * CW + col0;
            uint32_t a0[20], b0[20], a1[20], b1[20];
#pragma unroll
            for (int i = 0; i < 20; ++i) a0[i] = b0[i] = a1[i] = b1[i] = 0u;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                if (A == 1) {
#pragma unroll
                    for (int c0 = 0; c0 < 5; ++c0) {
#pragma unroll
                        for (int ph = 0; ph < PHS; ++ph) {
                            a0[q * 5 + c0] += tc[((n0 + q) * 5 + c0) * CW + ph * TL];
                            b0[q * 5 + c0] += tc[((n0 + q) * 5 + c0) * CW + ph * TL + BOFF];
                        }
                    }
                } else {
                    // every joint cell is read once and added to the row sum of one feature and the
                    // column sum of the other; the reads are independent
#pragma unroll
                    for (int c1 = 0; c1 < 5; ++c1)
#pragma unroll
                        for (int c0 = 0; c0 < 5; ++c0) {
                            uint32_t aw = 0, bw = 0;
#pragma unroll
                            for (int ph = 0; ph < PHS; ++ph) {
                                aw += tc[((n0 + q) * 25 + c1 * 5 + c0) * CW + ph * TL];
                                bw += tc[((n0 + q) * 25 + c1 * 5 + c0) * CW + ph * TL + BOFF];
                            }
                            a0[q * 5 + c0] += aw;
                            b0[q * 5 + c0] += bw;
                            a1[q * 5 + c1] += aw;
                            b1[q * 5 + c1] += bw;
                        }
                }
            }
            emit20(A * t, n0, a0, b0);
            if (A == 2 && 2 * t + 1 < n_mine) emit20(2 * t + 1, n0, a1, b1);
        }
        return;
    }
    if (A == 2 && nb == 5) {
        // Five-level pairs, the common case: every joint cell is read once and added to the row sum
        // of one feature and the column sum of the other; the 25 reads are independent.
        for (int item = warp * R + phase; item < n_nodes * T; item += kLaneWarps * R) {
            const int n = item / T, t = item - n * T;
            if (2 * t >= n_mine) continue;
            const uint32_t* tc = cells + (size_t)t * n_cells * CW + (size_t)(n * 25) * CW + col0;
            uint32_t a0[kLaneBinsMax], b0[kLaneBinsMax], a1[kLaneBinsMax], b1[kLaneBinsMax];
#pragma unroll
            for (int b = 0; b < kLaneBinsMax; ++b) a0[b] = b0[b] = a1[b] = b1[b] = 0u;
#pragma unroll
            for (int c1 = 0; c1 < 5; ++c1)
#pragma unroll
                for (int c0 = 0; c0 < 5; ++c0) {
                    uint32_t aw = 0, bw = 0;
#pragma unroll
                    for (int ph = 0; ph < PHS; ++ph) {
                        aw += tc[(c1 * 5 + c0) * CW + ph * TL];
                        bw += tc[(c1 * 5 + c0) * CW + ph * TL + BOFF];
                    }
                    a0[c0] += aw;
                    b0[c0] += bw;
                    a1[c1] += aw;
                    b1[c1] += bw;
                }
            emit(2 * t, n, a0, b0);
            if (2 * t + 1 < n_mine) emit(2 * t + 1, n, a1, b1);
        }
        return;
    }
    for (int item = warp * R + phase; item < n_nodes * FPL; item += kLaneWarps * R) {
        const int n = item / FPL, fl = item - n * FPL;  // node, feature of the lane
        if (fl >= n_mine) continue;
        const int t = fl / A, fi = fl - t * A;
        int below = 1;  // bins^fi
        for (int i = 0; i < fi; ++i) below *= nb;
        const int above = cpn / (below * nb);
        const uint32_t* tcells = cells + (size_t)t * n_cells * CW;
        uint32_t aw[kLaneBinsMax], bw[kLaneBinsMax];   // packed sums of the bins of this (feature, node)
#pragma unroll
        for (int b = 0; b < kLaneBinsMax; ++b) {
            aw[b] = 0u;
            bw[b] = 0u;
            if (b >= nb) continue;
            // The packed words of the joint cells are added as they are: the rows behind them are
            // disjoint subsets of the tile, so neither field can overflow; decoded once per bin.
            uint32_t a_sum = 0, b_sum = 0;
            for (int hi = 0; hi < above; ++hi)
                for (int lo = 0; lo < below; ++lo) {
                    const uint32_t cell = (uint32_t)(n * cpn + (hi * nb + b) * below + lo) * (uint32_t)CW + col0;
#pragma unroll
                    for (int ph = 0; ph < PHS; ++ph) {
                        a_sum += tcells[cell + ph * TL];
                        b_sum += tcells[cell + ph * TL + BOFF];
                    }
                }
            aw[b] = a_sum;
            bw[b] = b_sum;
        }
        emit(fl, n, aw, bw);
    }
}

template <int A, int T, int R>
int launch_lane_r(const HistKernelArgs& a, size_t cell_bytes, cudaStream_t stream) {
    const size_t smem = cell_bytes + lane_extra_bytes(R, A * T);
    if (smem > 48 * 1024)
        PB_CUDA_TRY(cudaFuncSetAttribute(hist_lane_kernel<A, T, R>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem));
    const int per_cta = (32 / R) * A * T;
    dim3 grid((unsigned)(a.n_eras * a.tiles_per_era), (unsigned)((a.n_feat + per_cta - 1) / per_cta), 1);
    hist_lane_kernel<A, T, R><<<grid, kLaneWarps * 32, smem, stream>>>(a);
    return PB_OK;
}

template <int A, int T>
int launch_lane(const HistKernelArgs& a, size_t cell_bytes, int phases, cudaStream_t stream) {
    if (phases == 4) return launch_lane_r<A, T, 4>(a, cell_bytes, stream);
    if (phases == 2) return launch_lane_r<A, T, 2>(a, cell_bytes, stream);
    return launch_lane_r<A, T, 1>(a, cell_bytes, stream);
}

}  // namespace

int hist_max_arity() {
    const char* e = getenv("PACKBOOST_HIST_MAX_ARITY");
    if (e && e[0] >= '1' && e[0] <= '2' && e[1] == 0) return e[0] - '0';
    return 2;
}

bool hist_can_fuse(const HistLaunch& h) {
    return h.code_bits == 4 && h.max_era_rows <= kTileRowsMax &&
           (int64_t)h.n_nodes * h.max_bins * kLaneCellBytes <= kLaneCellsMax && h.n_feat > 0 && h.n_nodes > 0;
}

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
    a.fuse = 0;
    memset(&a.fz, 0, sizeof(a.fz));
    a.debug_flags = h.debug_flags;

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

    const size_t out_cells = (size_t)h.n_feat * h.node_stride * h.n_eras * h.max_bins;
    if (a.use_atomics) {
        PB_CUDA_TRY(cudaMemsetAsync(h.cnt, 0, out_cells * sizeof(uint32_t), stream));
        PB_CUDA_TRY(cudaMemsetAsync(h.gsum, 0, out_cells * sizeof(int64_t), stream));
    }

    // lane-private kernel when a lane's cells are few: tuples of A features (joint code) as wide as
    // the cells allow, then T tuples per lane while shared memory lasts (A * T <= 4)
    if (h.code_bits == 4 && (int64_t)h.n_nodes * h.max_bins * kLaneCellBytes <= kLaneCellsMax) {
        // Pick the tuple width A (joint code), the tuples per lane T and the row phases R by a cost
        // model fitted to measured launches (238 features, 574 tiles of 4 700 rows, microseconds per
        // launch).  A pass (the CTAs of one feature range) costs kPass + kPassFeat per feature of a
        // lane (block fetch, code reads, records, barriers) + kTuple * T / R (the row steps: two
        // atomics and the code extraction per tuple) + kCell per KB of cells (zeroing and flush);
        // an SM holds two CTAs (registers) when their shared memory allows, and a single CTA per SM
        // runs about 1.2 times slower than its share of two.  The model reproduces the measured order
        // of every shape at every depth of that workload.
        const int cap = h.max_arity < 2 ? h.max_arity : 2;  // wider joint codes measured slower
        int arity = 1, tuples = 1, phases = 1;
        static const int max_phases = [] {  // PACKBOOST_HIST_PHASES=1|2 lowers the row-phase cap (tuning)
            const char* e = getenv("PACKBOOST_HIST_PHASES");
            return (e && (e[0] == '1' || e[0] == '2') && e[1] == 0) ? e[0] - '0' : 4;
        }();
        // PACKBOOST_HIST_SHAPE="A T R" forces the launch shape where it fits and logs what is launched (tuning)
        static const int* const forced = [] {
            static int v[3];
            const char* e = getenv("PACKBOOST_HIST_SHAPE");
            return (e && sscanf(e, "%d %d %d", &v[0], &v[1], &v[2]) == 3) ? v : (const int*)nullptr;
        }();
        int64_t cpn = h.max_bins;
        double best = 1e30;
        {
            constexpr double kPass = 15.0, kPassFeat = 2.2, kTuple = 33.0, kCell = 0.145;
            const double tile_scale = (double)max_tile / 4700.0;
            int64_t c = h.max_bins;
            for (int a_try = 1; a_try <= cap; ++a_try, c *= h.max_bins) {
                for (int t_try = 1; t_try * a_try <= 8; t_try *= 2) {
                    for (int r_try = 1; r_try <= max_phases; r_try *= 2) {
                        const size_t bytes = (size_t)h.n_nodes * c * lane_cell_bytes(r_try) * t_try;
                        if (bytes > (size_t)kLaneCellsMax) continue;
                        const int per_cta = (32 / r_try) * a_try * t_try;
                        const int blocks = (h.n_feat + per_cta - 1) / per_cta;
                        const size_t smem = bytes + lane_extra_bytes(r_try, a_try * t_try) + 1024;
                        const int per_sm = (2 * smem <= (size_t)228 * 1024) ? 2 : 1;
                        const double ctas = (double)h.n_eras * a.tiles_per_era * blocks;
                        const double slots = 148.0 * per_sm;
                        const double waves = ctas > slots ? ctas / slots : 1.0;
                        // (a few per cent against more phases: equal estimates favour whole-warp tuples)
                        double cost = (r_try == 1 ? 1.0 : r_try == 2 ? 1.04 : 1.08) * waves * per_sm * (per_sm == 1 ? 1.2 : 1.0) *
                                      (tile_scale * (kPass + kPassFeat * a_try * t_try + kTuple * t_try / r_try) +
                                       kCell * (double)bytes / 1024.0);
                        if (forced) cost = (a_try == forced[0] && t_try == forced[1] && r_try == forced[2]) ? 0.0 : cost + 1e9;
                        if (cost < best * (1.0 - 1e-9)) { best = cost; arity = a_try; tuples = t_try; phases = r_try; cpn = c; }
                    }
                }
            }
        }
        if (forced)
            fprintf(stderr, "hist_lane_kernel<%d,%d,%d> nodes=%d features=%d\n", arity, tuples, phases, h.n_nodes, h.n_feat);
        const size_t slot = (size_t)h.n_nodes * cpn * lane_cell_bytes(phases);
        a.nodes_per_chunk = h.n_nodes;
        a.feats_per_cta = (32 / phases) * arity * tuples;
        a.group = arity;
        a.copies = 1;
        const size_t smem = slot * tuples;  // cells; the launcher adds the records and the staged codes
        if (h.fuse && !a.use_atomics) {
            a.fuse = 1;
            h.fuse->tot_fpl = arity * tuples;
            h.fuse->tot_lanes = ((h.n_feat + a.feats_per_cta - 1) / a.feats_per_cta) * (32 / phases);
            a.fz = *h.fuse;
            const size_t tot = (size_t)h.node_stride * a.fz.n_thr * a.fz.tot_fpl * a.fz.tot_lanes;
            PB_CUDA_TRY(cudaMemsetAsync(a.fz.lc_tot, 0, tot * sizeof(uint32_t), stream));
            PB_CUDA_TRY(cudaMemsetAsync(a.fz.lg_tot, 0, tot * sizeof(int64_t), stream));
        } else if (h.fuse) {
            return fail_arg("fused flush requested for a launch that cannot fuse (check hist_can_fuse first)");
        }
        prof_begin(h.prof, kProfHist, stream);
        int rc;
        if (arity == 2) rc = (tuples == 4) ? launch_lane<2, 4>(a, smem, phases, stream)
                             : (tuples == 2) ? launch_lane<2, 2>(a, smem, phases, stream) : launch_lane<2, 1>(a, smem, phases, stream);
        else rc = (tuples == 8) ? launch_lane<1, 8>(a, smem, phases, stream)
                  : (tuples == 4) ? launch_lane<1, 4>(a, smem, phases, stream)
                  : (tuples == 2) ? launch_lane<1, 2>(a, smem, phases, stream) : launch_lane<1, 1>(a, smem, phases, stream);
        prof_end(h.prof, kProfHist, stream);
        if (rc) return rc;
        count_launch(1);
        PB_LAUNCH_CHECK("hist_lane_kernel");
        return PB_OK;
    }

    if (h.fuse) return fail_arg("fused flush requested for a launch that cannot fuse (check hist_can_fuse first)");
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
    while (copies < 32 && per_feat * copies * 2 <= 512) copies *= 2;
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
    dim3 grid((unsigned)n_tiles, (unsigned)((h.n_feat + feats_per_cta - 1) / feats_per_cta), (unsigned)chunks);
    if (grid.y > 65535u || grid.z > 65535u) return fail_arg("histogram grid too large");
    prof_begin(h.prof, kProfHist, stream);
    if (h.code_bits == 4) {
        if (smem > 48 * 1024)
            PB_CUDA_TRY(cudaFuncSetAttribute(hist_kernel<4, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        hist_kernel<4, 256><<<grid, threads, smem, stream>>>(a);
    } else {
        if (smem > 48 * 1024)
            PB_CUDA_TRY(cudaFuncSetAttribute(hist_kernel<8, 512>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        hist_kernel<8, 512><<<grid, threads, smem, stream>>>(a);
    }
    prof_end(h.prof, kProfHist, stream);
    count_launch(1);
    PB_LAUNCH_CHECK("hist_kernel");
    return PB_OK;
}

}  // namespace pb
