// Binning (searchsorted against per-feature edges) and packing of bin codes into the two
// layouts the other kernels read: feature-major (training) and row-major (prediction), each
// with one byte per code or two 4-bit codes per byte.

#include "common.cuh"

namespace pb {

namespace {

constexpr int kTileF = 32;    // features per tile
constexpr int kTileR = 256;   // rows per tile

// code = number of edges strictly below x (np.searchsorted(edges, x, "left")), clipped to
// max_bins-1; NaN compares false to everything and therefore falls through to the last bin,
// as it does when numpy sorts NaN after every edge.
__device__ __forceinline__ int bin_of(float x, const float* edges, int stride, int n_edges, int max_bins) {
    int lo = 0, hi = n_edges;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (edges[mid * stride] < x || x != x) lo = mid + 1; else hi = mid;
    }
    return min(lo, max_bins - 1);
}

struct PackArgs {
    const void* x;
    int x_is_f32;
    int64_t n_chunk;
    int64_t n_features;
    int64_t row_offset;
    const float* edges;
    int n_edges;
    int max_bins;
    const int32_t* feature_map;
    uint8_t* codes;
    int64_t pitch;
};

// Tile of kTileR rows x kTileF features: threads (32, 8); x is read with the feature index
// fastest (coalesced on the row-major input), codes are transposed through shared memory and
// written as 4- or 8-byte words along the feature-major rows.
template <int BITS>
__global__ void __launch_bounds__(256) pack_fm_kernel(PackArgs a) {
    __shared__ uint8_t tile[kTileF][kTileR + 4];
    extern __shared__ float s_edges[];  // [n_edges][kTileF]
    const int fx = threadIdx.x, ry = threadIdx.y;
    const int64_t f = (int64_t)blockIdx.y * kTileF + fx;
    const int64_t rt = (int64_t)blockIdx.x * kTileR;
    const bool f_ok = f < a.n_features;
    if (a.x_is_f32) {
        for (int i = ry; i < a.n_edges; i += 8) s_edges[i * kTileF + fx] = f_ok ? a.edges[(int64_t)i * a.n_features + f] : 0.f;
        __syncthreads();
    }
    for (int rr = ry; rr < kTileR; rr += 8) {
        const int64_t r = rt + rr;
        int code = 0;
        if (f_ok && r < a.n_chunk) {
            if (a.x_is_f32) {
                const float v = static_cast<const float*>(a.x)[r * a.n_features + f];
                code = bin_of(v, s_edges + fx, kTileF, a.n_edges, a.max_bins);
            } else {
                code = static_cast<const uint8_t*>(a.x)[r * a.n_features + f];
            }
        }
        tile[fx][rr] = (uint8_t)code;
    }
    __syncthreads();
    // each warp (ry) writes 4 features; a lane covers 8 consecutive rows
    const int lane = threadIdx.x;
    for (int k = 0; k < kTileF / 8; ++k) {
        const int fl = ry * (kTileF / 8) + k;
        const int64_t fg = (int64_t)blockIdx.y * kTileF + fl;
        if (fg >= a.n_features) continue;
        const int frow = a.feature_map ? a.feature_map[fg] : (int)fg;
        if (frow < 0) continue;
        const uint8_t* src = &tile[fl][lane * 8];
        const int64_t row0 = a.row_offset + rt + lane * 8;
        if (BITS == 4) {
            uint32_t w = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) w |= (uint32_t)(src[j] & 0xF) << (4 * j);
            *reinterpret_cast<uint32_t*>(a.codes + (int64_t)frow * a.pitch + (row0 >> 1)) = w;
        } else {
            uint2 w;
            w.x = src[0] | (src[1] << 8) | (src[2] << 16) | ((uint32_t)src[3] << 24);
            w.y = src[4] | (src[5] << 8) | (src[6] << 16) | ((uint32_t)src[7] << 24);
            *reinterpret_cast<uint2*>(a.codes + (int64_t)frow * a.pitch + row0) = w;
        }
    }
}

struct PackRowsArgs {
    const void* x;
    int x_is_f32;
    int64_t n_rows;
    int64_t n_features;
    const float* edges;
    int n_edges;
    int max_bins;
    uint8_t* out;
    int64_t pitch_row;
};

// Row-major packing: a thread produces one output byte (one or two features of one row).
template <int BITS>
__global__ void __launch_bounds__(256) pack_rows_kernel(PackRowsArgs a) {
    const int64_t bytes_per_row = (BITS == 4) ? (a.n_features + 1) / 2 : a.n_features;
    const int64_t total = a.n_rows * a.pitch_row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / a.pitch_row;
        const int64_t b = i - r * a.pitch_row;
        uint8_t v = 0;
        if (b < bytes_per_row) {
            const int per = (BITS == 4) ? 2 : 1;
            for (int h = 0; h < per; ++h) {
                const int64_t f = b * per + h;
                int code = 0;
                if (f < a.n_features) {
                    if (a.x_is_f32) {
                        const float xv = static_cast<const float*>(a.x)[r * a.n_features + f];
                        code = bin_of(xv, a.edges + f, (int)a.n_features, a.n_edges, a.max_bins);
                    } else {
                        code = static_cast<const uint8_t*>(a.x)[r * a.n_features + f];
                    }
                }
                v |= (uint8_t)((BITS == 4) ? ((code & 0xF) << (4 * h)) : code);
            }
        }
        a.out[i] = v;
    }
}

int pack_fm(const PackArgs& a, int code_bits, cudaStream_t stream) {
    if (a.n_chunk <= 0 || a.n_features <= 0) return PB_OK;
    dim3 grid((unsigned)((a.n_chunk + kTileR - 1) / kTileR), (unsigned)((a.n_features + kTileF - 1) / kTileF));
    dim3 block(32, 8);
    const size_t smem = a.x_is_f32 ? sizeof(float) * (size_t)a.n_edges * kTileF : 0;
    if (code_bits == 4)
        pack_fm_kernel<4><<<grid, block, smem, stream>>>(a);
    else
        pack_fm_kernel<8><<<grid, block, smem, stream>>>(a);
    count_launch(1);
    PB_LAUNCH_CHECK("pack_fm_kernel");
    return PB_OK;
}

}  // namespace
}  // namespace pb

using namespace pb;

static int check_pack(const void* x, int64_t n_chunk, int64_t n_features, int64_t row_offset, const uint8_t* codes,
                      int64_t pitch, int64_t code_bits, int64_t max_bins) {
    PB_REQUIRE(x && codes, "null buffer");
    PB_REQUIRE(n_chunk >= 0 && n_features >= 1, "bad shape");
    PB_REQUIRE(code_bits == 4 || code_bits == 8, "code_bits must be 4 or 8");
    PB_REQUIRE(code_bits == 8 || max_bins <= 16, "4-bit codes need max_bins <= 16");
    PB_REQUIRE(row_offset % 256 == 0, "row_offset must be a multiple of 256");
    PB_REQUIRE(pitch % 128 == 0, "pitch must be a multiple of 128");
    const int64_t rows_cover = pitch * (code_bits == 4 ? 2 : 1);
    PB_REQUIRE(row_offset + (n_chunk + 255) / 256 * 256 <= rows_cover, "chunk exceeds the padded row range");
    return PB_OK;
}

extern "C" int pb_bin_pack_f32(const float* x, int64_t n_chunk, int64_t n_features, int64_t row_offset,
                               const float* edges, int64_t n_edges, int64_t max_bins, const int32_t* feature_map,
                               uint8_t* codes, int64_t pitch, int64_t code_bits, void* stream) {
    int rc = check_pack(x, n_chunk, n_features, row_offset, codes, pitch, code_bits, max_bins);
    if (rc) return rc;
    PB_REQUIRE(edges && n_edges >= 1 && n_edges <= 255 && max_bins >= 2 && max_bins <= 256, "bad edges / max_bins");
    PackArgs a{x, 1, n_chunk, n_features, row_offset, edges, (int)n_edges, (int)max_bins, feature_map, codes, pitch};
    return pack_fm(a, (int)code_bits, (cudaStream_t)stream);
}

extern "C" int pb_pack_codes_u8(const uint8_t* x, int64_t n_chunk, int64_t n_features, int64_t row_offset,
                                const int32_t* feature_map, uint8_t* codes, int64_t pitch, int64_t code_bits,
                                void* stream) {
    int rc = check_pack(x, n_chunk, n_features, row_offset, codes, pitch, code_bits, code_bits == 4 ? 16 : 256);
    if (rc) return rc;
    PackArgs a{x, 0, n_chunk, n_features, row_offset, nullptr, 0, 256, feature_map, codes, pitch};
    return pack_fm(a, (int)code_bits, (cudaStream_t)stream);
}

extern "C" int pb_pack_rows(const void* x, int64_t x_is_f32, int64_t n_rows, int64_t n_features, const float* edges,
                            int64_t n_edges, int64_t max_bins, uint8_t* out, int64_t pitch_row, int64_t code_bits,
                            void* stream) {
    PB_REQUIRE(x && out, "null buffer");
    PB_REQUIRE(code_bits == 4 || code_bits == 8, "code_bits must be 4 or 8");
    PB_REQUIRE(code_bits == 8 || max_bins <= 16, "4-bit codes need max_bins <= 16");
    const int64_t need = (code_bits == 4) ? (n_features + 1) / 2 : n_features;
    PB_REQUIRE(pitch_row >= need && pitch_row % 16 == 0, "pitch_row must cover a row and be a multiple of 16");
    PB_REQUIRE(!x_is_f32 || (edges && n_edges >= 1), "float input needs edges");
    if (n_rows <= 0) return PB_OK;
    PackRowsArgs a{x, (int)(x_is_f32 != 0), n_rows, n_features, edges, (int)n_edges, (int)max_bins, out, pitch_row};
    int64_t blocks = (n_rows * pitch_row + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (code_bits == 4)
        pack_rows_kernel<4><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(a);
    else
        pack_rows_kernel<8><<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(a);
    count_launch(1);
    PB_LAUNCH_CHECK("pack_rows_kernel");
    return PB_OK;
}
