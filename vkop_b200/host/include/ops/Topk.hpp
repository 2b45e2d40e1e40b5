// TopK operator: interface of the reference's ops/Topk.hpp (:31-225).
// Attributes "K" / "k" (default 1), "largest" (1), "sorted" (1), "axis" (-1).
// Outputs: values in the input's element type and indices (int32 as in the
// reference, :121, or int64), shaped like the input with shape[axis] = k;
// outputs that are not empty are used as they are (benchmark/main.cpp:92-94
// passes full-shape tensors: the first rows * k entries are written).
// Differences from the reference, all widenings: k may be up to 4096 (the
// reference asserts k < 256, :103), k is not rounded up to even for fp16
// (:104-106), equal values are ordered by index (the reference's bitonic
// network leaves them in network order), any axis 0 .. 2 of the tensor is
// selected along (the reference's shader always walks the last axis of a 1-D
// or 2-D tensor, shaders/topk.comp:119-175), and sorted = 0 gives the k entries
// in ascending index order (the reference ignores the attribute).
#ifndef VKOP_HOST_OPS_TOPK_HPP_
#define VKOP_HOST_OPS_TOPK_HPP_

#include "ops/Operator.hpp"

namespace vkop {
namespace ops {

class Topk : public Operator {
  public:
    explicit Topk(int fp16 = 0) : Operator(OpType::TOPK, fp16) {}

    void setAttribute(const std::unordered_map<std::string, std::string> &attributes) override {
        if (attributes.count("K"))
            k_ = static_cast<int>(std::stol(attributes.at("K")));
        else if (attributes.count("k"))
            k_ = static_cast<int>(std::stol(attributes.at("k")));
        if (attributes.count("largest"))
            largest_ = static_cast<int>(std::stol(attributes.at("largest")));
        if (attributes.count("sorted"))
            sorted_ = static_cast<int>(std::stol(attributes.at("sorted")));
        if (attributes.count("axis"))
            axis_ = static_cast<int>(std::stol(attributes.at("axis")));
    }
    int k() const { return k_; }

  protected:
    // Shared by the fused operator: describes the selection over the last axis.
    vkop_softmax_topk_desc describe(const std::shared_ptr<core::ITensor> &input, const std::shared_ptr<core::ITensor> &indices,
                                    std::vector<int> *out_shape) const {
        const auto shape = input->getShape();
        const int rank = input->num_dims();
        const int axis = axis_ < 0 ? axis_ + rank : axis_;
        if (axis < 0 || axis > 2 || axis >= rank)
            throw std::invalid_argument("TopK: axis out of range");  // the reference asserts axis <= 2
        if (axis != rank - 1)
            throw std::invalid_argument("TopK: only the last axis is supported");
        vkop_softmax_topk_desc d = {};
        d.rows = 1;
        for (int i = 0; i < axis; i++)
            d.rows *= shape[i];
        d.cols = shape[axis];
        d.row_stride = d.cols;
        d.dtype = value_dtype(input);
        d.k = k_;
        d.index_dtype = indices->dtype() == typeid(int64_t) ? VKOP_I64 : VKOP_I32;
        d.value_kind = VKOP_VALUE_RAW;
        d.inv_temperature = 1.0f;
        d.largest = largest_;
        *out_shape = shape;
        (*out_shape)[axis] = k_;
        return d;
    }

    void execute(const std::vector<std::shared_ptr<core::ITensor>> &inputs,
                 const std::vector<std::shared_ptr<core::ITensor>> &outputs) override {
        if (outputs.size() < 2)
            throw std::invalid_argument("TopK: needs a values and an indices output");
        if (outputs[1]->dtype() != typeid(int) && outputs[1]->dtype() != typeid(int64_t))
            throw std::invalid_argument("TopK: indices must be int or int64_t");
        const auto shape = inputs[0]->getShape();
        const int rank = inputs[0]->num_dims();
        const int axis = axis_ < 0 ? axis_ + rank : axis_;
        if (axis < 0 || axis > 2 || axis >= rank)
            throw std::invalid_argument("TopK: axis out of range");  // the reference asserts axis <= 2
        vkop_topk_axis_desc d = {};
        d.outer = 1;
        d.inner = 1;
        for (int i = 0; i < axis; i++)
            d.outer *= shape[i];
        for (int i = axis + 1; i < rank; i++)
            d.inner *= shape[i];
        d.axis_len = shape[axis];
        d.dtype = value_dtype(inputs[0]);
        d.k = k_;
        d.index_dtype = outputs[1]->dtype() == typeid(int64_t) ? VKOP_I64 : VKOP_I32;
        d.largest = largest_;
        d.sorted = sorted_;
        d.path = VKOP_PATH_AUTO;
        std::vector<int> out_shape = shape;
        out_shape[axis] = k_;
        resize_if_empty(outputs[0], out_shape);
        resize_if_empty(outputs[1], out_shape);
        if (outputs[0]->dtype() != inputs[0]->dtype())
            throw std::invalid_argument("TopK: values must have the input's element type");
        const int64_t produced = d.outer * d.inner * d.k;
        if (outputs[0]->num_elements() < produced || outputs[1]->num_elements() < produced)
            throw std::invalid_argument("TopK: output tensors are too small");
        size_t need = 0;
        check(vkop_cuda_topk_axis_workspace(&d, &need), "vkop_cuda_topk_axis_workspace");
        uint64_t key = 1469598103934665603ull;
        for (uint64_t v : {static_cast<uint64_t>(d.outer), static_cast<uint64_t>(d.axis_len), static_cast<uint64_t>(d.inner),
                           static_cast<uint64_t>(d.dtype), static_cast<uint64_t>(d.k), static_cast<uint64_t>(d.largest)})
            key = (key ^ v) * 1099511628211ull;
        key &= ~1ull;  // the selection descriptors of the fused operator hash to odd keys
        void *ws = workspace(need, key);
        check(vkop_cuda_topk_axis(&d, device_of(inputs[0]), device_of(outputs[0]), device_of(outputs[1]), ws, workspace_bytes(),
                                  stream()),
              "vkop_cuda_topk_axis");
    }

    int k_ = 1, axis_ = -1, largest_ = 1, sorted_ = 1;
};

}  // namespace ops
}  // namespace vkop
#endif  // VKOP_HOST_OPS_TOPK_HPP_
