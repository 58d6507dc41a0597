// Tree routing: a row goes left when its code is <= the node's threshold.

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
            int node = 0;
            while (!__ldg(a.is_leaf + base + node)) {
                const int f = __ldg(a.feature + base + node);
                const int thr = __ldg(a.threshold + base + node);
                node = (code_at<BITS>(row, f) <= thr) ? __ldg(a.left + base + node) : __ldg(a.right + base + node);
            }
            const float term = __fmul_rn(a.weight, __ldg(a.value + base + node));
            const int rep = a.repeat ? __ldg(a.repeat + t) : 1;
            for (int k = 0; k < rep; ++k) acc = __fadd_rn(acc, term);
        }
        a.out[row0 + lr] = acc;
    }
}

__global__ void __launch_bounds__(256) predict_bins_fm_kernel(
    const uint8_t* __restrict__ bins, int64_t n_rows, const int32_t* __restrict__ feature,
    const int32_t* __restrict__ threshold, const int32_t* __restrict__ left, const int32_t* __restrict__ right,
    const float* __restrict__ value, const uint8_t* __restrict__ is_leaf, float* __restrict__ out) {
    for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < n_rows; r += (int64_t)gridDim.x * blockDim.x) {
        int node = 0;
        while (!__ldg(is_leaf + node)) {
            const int f = __ldg(feature + node);
            node = ((int)bins[(int64_t)f * n_rows + r] <= __ldg(threshold + node)) ? __ldg(left + node) : __ldg(right + node);
        }
        out[r] = __ldg(value + node);
    }
}

__global__ void __launch_bounds__(256) predict_pack_fm_kernel(
    const uint8_t* __restrict__ bins, int64_t n_rows, const int32_t* __restrict__ feature,
    const int32_t* __restrict__ threshold, const int32_t* __restrict__ left_abs, const int32_t* __restrict__ right_abs,
    const float* __restrict__ value, const uint8_t* __restrict__ is_leaf, const int32_t* __restrict__ offsets,
    int n_trees, float tree_weight, float* __restrict__ out) {
    for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < n_rows; r += (int64_t)gridDim.x * blockDim.x) {
        float sum = 0.f;
        for (int t = 0; t < n_trees; ++t) {
            int node = __ldg(offsets + t);
            const int end = __ldg(offsets + t + 1);
            if (node >= end) continue;
            while (!__ldg(is_leaf + node)) {
                const int f = __ldg(feature + node);
                node = ((int)bins[(int64_t)f * n_rows + r] <= __ldg(threshold + node)) ? __ldg(left_abs + node)
                                                                                       : __ldg(right_abs + node);
            }
            sum = __fadd_rn(sum, __ldg(value + node));
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
                      tree_offsets, repeat, (int)n_trees, weight, out, init, 128, 1};
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
    predict_bins_fm_kernel<<<row_blocks(n_rows), 256, 0, (cudaStream_t)stream>>>(bins, n_rows, feature, threshold, left,
                                                                                right, value, is_leaf, out);
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
    predict_pack_fm_kernel<<<row_blocks(n_rows), 256, 0, (cudaStream_t)stream>>>(
        bins, n_rows, feature, threshold, left_abs, right_abs, value, is_leaf, offsets, (int)n_trees, tree_weight, out);
    count_launch(1);
    PB_LAUNCH_CHECK("predict_pack_fm_kernel");
    return PB_OK;
}
