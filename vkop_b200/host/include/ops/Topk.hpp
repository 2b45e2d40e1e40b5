// TopK operator: interface of the reference's ops/Topk.hpp (:31-225).
// Attributes "K" / "k" (default 1), "largest" (1), "sorted" (1), "axis" (-1).
// Outputs: values in the input's element type and indices (int32 as in the
// reference, :121, or int64), shaped like the input with shape[axis] = k;
// outputs that are not empty are used as they are (benchmark/main.cpp:92-94
// passes full-shape tensors: the first rows * k entries are written).
// Differences from the reference, all widenings: k may be up to 4096 (the
// reference asserts k < 256, :103), k is not rounded up to even for fp16
// (:104-106), equal values are ordered by index (the reference's bitonic
// network leaves them in network order).  The axis must be the last one.
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
        std::vector<int> out_shape;
        vkop_softmax_topk_desc d = describe(inputs[0], outputs[1], &out_shape);
        resize_if_empty(outputs[0], out_shape);
        resize_if_empty(outputs[1], out_shape);
        if (outputs[0]->dtype() != inputs[0]->dtype())
            throw std::invalid_argument("TopK: values must have the input's element type");
        if (outputs[0]->num_elements() < d.rows * d.k || outputs[1]->num_elements() < d.rows * d.k)
            throw std::invalid_argument("TopK: output tensors are too small");
        size_t need = 0;
        check(vkop_cuda_softmax_topk_workspace(&d, &need), "vkop_cuda_softmax_topk_workspace");
        void *ws = workspace(need, shape_key(d));
        check(vkop_cuda_topk(&d, device_of(inputs[0]), device_of(outputs[0]), device_of(outputs[1]), ws, workspace_bytes(), stream()),
              "vkop_cuda_topk");
    }

    int k_ = 1, axis_ = -1, largest_ = 1, sorted_ = 1;
};

}  // namespace ops
}  // namespace vkop
#endif  // VKOP_HOST_OPS_TOPK_HPP_
