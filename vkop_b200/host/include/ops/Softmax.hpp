// Softmax operator: interface of the reference's ops/Softmax.hpp (:26-144).
// Attributes "axis" / "dim" (default -1), "nan_optimization",
// "nan_replacement_value"; every key is parsed independently (the reference's
// else-if chain reads only the first one present, :48-57).  Output is resized
// to the input shape when empty.  Rank 1 is treated as [1, n] (:116-120).
// The use_ssbo flag of the reference selects between its buffer and image
// shaders; here every rank runs on linear memory, the flag is accepted and
// ignored.
#ifndef VKOP_HOST_OPS_SOFTMAX_HPP_
#define VKOP_HOST_OPS_SOFTMAX_HPP_

#include "ops/Operator.hpp"

namespace vkop {
namespace ops {

class Softmax : public Operator {
  public:
    explicit Softmax(bool use_ssbo = false) : Operator(OpType::SOFTMAX) { (void)use_ssbo; }

    void setAttribute(const std::unordered_map<std::string, std::string> &attributes) override {
        auto it = attributes.find("axis");
        if (it == attributes.end())
            it = attributes.find("dim");
        if (it != attributes.end())
            axis_ = static_cast<int>(std::stol(it->second));
        if (attributes.count("nan_optimization"))
            nanwhere_ = 1;
        if (attributes.count("nan_replacement_value"))
            nanvalue_ = std::stof(attributes.at("nan_replacement_value"));
    }
    int axis() const { return axis_; }

  private:
    void execute(const std::vector<std::shared_ptr<core::ITensor>> &inputs,
                 const std::vector<std::shared_ptr<core::ITensor>> &outputs) override {
        const auto shape = inputs[0]->getShape();
        const int rank = inputs[0]->num_dims();
        if (rank < 1 || rank > 4)
            throw std::invalid_argument("Softmax: rank must be 1..4");
        resize_if_empty(outputs[0], shape);
        if (inputs[0]->dtype() != outputs[0]->dtype())
            throw std::invalid_argument("Softmax: input and output element types differ");
        int axis = axis_ < 0 ? axis_ + rank : axis_;
        if (axis < 0 || axis >= rank)
            throw std::invalid_argument("Softmax: axis out of range");
        vkop_softmax_desc d;
        d.outer = 1;
        d.inner = 1;
        for (int i = 0; i < axis; i++)
            d.outer *= shape[i];
        for (int i = axis + 1; i < rank; i++)
            d.inner *= shape[i];
        d.axis_len = shape[axis];
        d.dtype = value_dtype(inputs[0]);
        d.inv_temperature = 1.0f;
        check(vkop_cuda_softmax(&d, device_of(inputs[0]), device_of(outputs[0]), stream()), "vkop_cuda_softmax");
    }

    int axis_ = -1;
    int nanwhere_ = 0;
    float nanvalue_ = 0.0f;
};

}  // namespace ops
}  // namespace vkop
#endif  // VKOP_HOST_OPS_SOFTMAX_HPP_
