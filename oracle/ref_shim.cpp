// Shim around the reference's own CPU statements of the Softmax / TopK path (TEST INFRASTRUCTURE).
//
// The three function bodies included below are not part of this repository: oracle/build_ref.py cuts
// them out of the reference checkout at build time (core/function.cpp Function::get_top_k_predictions,
// tests/SoftmaxTest.cpp softmax_nd, tests/TopkTest.cpp get_top_k_predictions) into oracle/_ref/*.inc.
// This file only gives them what they need around them and C entry points for ctypes.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <iostream>
#include <utility>
#include <vector>

namespace vkop {
namespace core {
// core/function.hpp:49 declares the function as a static member of this class.
class Function {
  public:
    static std::vector<std::pair<int, float>> get_top_k_predictions(const std::vector<float> &probs, int k);
};
#include "_ref/function_get_top_k_predictions.inc"
}  // namespace core
}  // namespace vkop

namespace ref_softmax_test {
#include "_ref/softmax_nd.inc"
}

namespace ref_topk_test {
#include "_ref/topk_get_top_k_predictions.inc"
}

extern "C" {

// core/function.cpp Function::get_top_k_predictions on every row of x [rows, cols] (rows in parallel:
// the reference function itself is single-threaded and takes one row).  The rows are scaled by
// inv_temperature first (the reference has no temperature; 1.0f leaves them as they are).
// out_index / out_prob: [rows, k].
int ref_function_top_k_predictions(const float *x, int64_t rows, int64_t cols, int64_t row_stride, float inv_temperature,
                                   int k, int32_t *out_index, float *out_prob) {
    if (!x || rows < 0 || cols < 1 || k < 1 || k > cols)
        return -1;
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t r = 0; r < rows; r++) {
        std::vector<float> row(x + r * row_stride, x + r * row_stride + cols);
        if (inv_temperature != 1.0f)
            for (auto &v : row)
                v *= inv_temperature;
        const auto best = vkop::core::Function::get_top_k_predictions(row, k);
        for (int i = 0; i < k; i++) {
            out_index[r * k + i] = best[i].first;
            out_prob[r * k + i] = best[i].second;
        }
    }
    return 0;
}

// tests/SoftmaxTest.cpp softmax_nd.
int ref_softmax_nd(const float *input, float *output, int N, int C, int H, int W, int axis) {
    if (!input || !output || axis < 0 || axis > 3)
        return -1;
    ref_softmax_test::softmax_nd(input, output, N, C, H, W, axis);
    return 0;
}

// tests/TopkTest.cpp get_top_k_predictions: indices come back flat (row * cols + column).
int ref_topk_rows(const float *x, int rows, int cols, int k, int32_t *out_flat_index, float *out_value) {
    if (!x || rows < 1 || cols < 1 || k < 1 || k > cols)
        return -1;
    std::vector<std::vector<float>> in(rows);
    for (int r = 0; r < rows; r++)
        in[r].assign(x + static_cast<int64_t>(r) * cols, x + static_cast<int64_t>(r + 1) * cols);
    const auto out = ref_topk_test::get_top_k_predictions(in, k);
    for (int r = 0; r < rows; r++)
        for (int i = 0; i < k; i++) {
            out_flat_index[r * k + i] = out[r][i].first;
            out_value[r * k + i] = out[r][i].second;
        }
    return 0;
}

}  // extern "C"
