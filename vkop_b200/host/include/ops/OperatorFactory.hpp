// Operator factory: create_from_type of the reference (ops/OperatorFactory.hpp:
// 56-143) for the post-processing operators.  Types that are not on this path
// return nullptr, which is also what the reference returns for a type it does
// not know.
#ifndef VKOP_HOST_OPS_OPERATOR_FACTORY_HPP_
#define VKOP_HOST_OPS_OPERATOR_FACTORY_HPP_

#include <memory>

#include "ops/Nms.hpp"
#include "ops/Operator.hpp"
#include "ops/Softmax.hpp"
#include "ops/SoftmaxTopk.hpp"
#include "ops/Topk.hpp"

namespace vkop {
namespace ops {

static inline std::unique_ptr<Operator> create_from_type(OpType type, bool use_ssbo = false, int fp16 = 0,
                                                         bool use_tensorcore = false) {
    (void)use_tensorcore;
    switch (type) {
    case OpType::TOPK:
        return std::make_unique<Topk>(fp16);
    case OpType::SOFTMAX:
        return std::make_unique<Softmax>(use_ssbo);
    case OpType::NMS:
        return std::make_unique<Nms>();
    case OpType::SOFTMAX_TOPK:
        return std::make_unique<SoftmaxTopk>(fp16);
    default:
        return nullptr;
    }
}

}  // namespace ops
}  // namespace vkop
#endif  // VKOP_HOST_OPS_OPERATOR_FACTORY_HPP_
