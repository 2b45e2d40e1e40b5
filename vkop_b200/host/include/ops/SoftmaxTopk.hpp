// Fused Softmax + TopK operator (OpType::SOFTMAX_TOPK, "SoftmaxTopK"): what
// the reference runs as a Softmax dispatch followed by the multi-pass TopK
// dispatches (benchmark/main.cpp:85-101) as one pass over the logits.
// Attributes: those of TopK ("k"/"K", "axis" = last) plus "temperature"
// (default 1; the softmax is taken of x / temperature).  Outputs: the
// probabilities of the k best logits (input element type) and their indices.
// Selection is on the stored logits, so the result equals Softmax followed by
// TopK wherever distinct logits keep distinct probabilities.
#ifndef VKOP_HOST_OPS_SOFTMAXTOPK_HPP_
#define VKOP_HOST_OPS_SOFTMAXTOPK_HPP_

#include "ops/Topk.hpp"

namespace vkop {
namespace ops {

class SoftmaxTopk : public Topk {
  public:
    explicit SoftmaxTopk(int fp16 = 0) : Topk(fp16) { type_ = OpType::SOFTMAX_TOPK; }

    void setAttribute(const std::unordered_map<std::string, std::string> &attributes) override {
        Topk::setAttribute(attributes);
        if (attributes.count("temperature")) {
            const float t = std::stof(attributes.at("temperature"));
            if (!(t > 0.0f))
                throw std::invalid_argument("SoftmaxTopK: temperature must be positive");
            inv_temperature_ = 1.0f / t;
        }
        if (attributes.count("input_ready"))
            input_ready_ = std::stol(attributes.at("input_ready")) != 0;
    }

  private:
    void execute(const std::vector<std::shared_ptr<core::ITensor>> &inputs,
                 const std::vector<std::shared_ptr<core::ITensor>> &outputs) override {
        if (outputs.size() < 2)
            throw std::invalid_argument("SoftmaxTopK: needs a values and an indices output");
        if (largest_ != 1)
            throw std::invalid_argument("SoftmaxTopK: only the largest probabilities are selected");
        std::vector<int> out_shape;
        vkop_softmax_topk_desc d = describe(inputs[0], outputs[1], &out_shape);
        d.value_kind = VKOP_VALUE_PROBABILITY;
        d.inv_temperature = inv_temperature_;
        d.flags = input_ready_ ? VKOP_FLAG_INPUT_READY : 0;
        resize_if_empty(outputs[0], out_shape);
        resize_if_empty(outputs[1], out_shape);
        if (outputs[0]->dtype() != inputs[0]->dtype())
            throw std::invalid_argument("SoftmaxTopK: values must have the input's element type");
        if (outputs[0]->num_elements() < d.rows * d.k || outputs[1]->num_elements() < d.rows * d.k)
            throw std::invalid_argument("SoftmaxTopK: output tensors are too small");
        size_t need = 0;
        check(vkop_cuda_softmax_topk_workspace(&d, &need), "vkop_cuda_softmax_topk_workspace");
        void *ws = workspace(need, shape_key(d));
        check(vkop_cuda_softmax_topk(&d, device_of(inputs[0]), device_of(outputs[0]), device_of(outputs[1]), ws, workspace_bytes(),
                                     stream()),
              "vkop_cuda_softmax_topk");
    }

    float inv_temperature_ = 1.0f;
    bool input_ready_ = false;
};

}  // namespace ops
}  // namespace vkop
#endif  // VKOP_HOST_OPS_SOFTMAXTOPK_HPP_
