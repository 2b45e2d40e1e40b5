// Shim around the reference's own NMS expectation (TEST INFRASTRUCTURE).
//
// tests/NmsTest.cpp NmsTest::compute_expected_nms is a member function written on libtorch tensors; its
// body is not part of this repository: oracle/build_ref.py cuts it out of the reference checkout at build
// time into oracle/_ref/nms_compute_expected_nms.inc.  This file supplies the class it is a member of
// (the two thresholds), a stand-in for the reference's Tensor<int> result type, and a C entry point.
#include <torch/torch.h>

#include <iostream>
#include <memory>
#include <sstream>
#include <vector>

namespace {

// What the function needs of core::Tensor<int>: construction from a shape, fillToCPU, print_tensor.
template <typename T>
struct Tensor {
    std::vector<int> shape;
    std::vector<T> data;
    explicit Tensor(const std::vector<int> &s) : shape(s) {}
    void fillToCPU(const std::vector<T> &v) { data = v; }
    void print_tensor() const {}
};

struct RefNms {
    float iou_threshold_;
    float score_threshold_;
#include "_ref/nms_compute_expected_nms.inc"
};

}  // namespace

extern "C" {

// boxes [B, N, 4] corners, scores [B, C, N]; rows_out [cap, 3] receives (batch, class, box) rows in the
// reference's order; returns the number of rows (which may exceed cap: then only cap were written), or -1.
int ref_nms_expected(const float *boxes, const float *scores, int B, int C, int N, float iou_threshold,
                     float score_threshold, int32_t *rows_out, int cap) {
    if (!boxes || !scores || B < 1 || C < 1 || N < 1)
        return -1;
    auto tb = torch::from_blob(const_cast<float *>(boxes), {B, N, 4}, torch::kFloat32).clone();
    auto ts = torch::from_blob(const_cast<float *>(scores), {B, C, N}, torch::kFloat32).clone();
    RefNms ref{iou_threshold, score_threshold};
    // the function prints its inputs and its result: keep that off the test output
    std::ostringstream sink;
    std::streambuf *old = std::cout.rdbuf(sink.rdbuf());
    std::shared_ptr<Tensor<int>> out;
    try {
        out = ref.compute_expected_nms(tb, ts);
    } catch (...) {
        std::cout.rdbuf(old);
        return -1;
    }
    std::cout.rdbuf(old);
    const int n = static_cast<int>(out->data.size() / 3);
    for (int i = 0; i < n && i < cap; i++)
        for (int j = 0; j < 3; j++)
            rows_out[i * 3 + j] = out->data[i * 3 + j];
    return n;
}

}  // extern "C"
