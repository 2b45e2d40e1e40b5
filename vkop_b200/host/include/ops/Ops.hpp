// Operator types: the reference's enumeration (ops/Ops.hpp:11-54) with the
// same numeric values, plus SOFTMAX_TOPK for the fused post-processing
// operator, placed after WHERE so that every reference value keeps its number.
// Only the post-processing operators have an implementation here; the names
// of the others are kept so that type <-> string round trips match.
#ifndef VKOP_HOST_OPS_OPS_HPP_
#define VKOP_HOST_OPS_OPS_HPP_

#include <cstdio>
#include <string>

namespace vkop {
namespace ops {

// X(enumerator, primary name, alternative name or nullptr)
#define VKOP_OP_TABLE(X)                                  \
    X(UNKNOWN, "Unknown", nullptr)                        \
    X(ADD, "Add", nullptr)                                \
    X(ATAN, "Atan", nullptr)                              \
    X(AVERAGEPOOL, "AveragePool", nullptr)                \
    X(BATCHNORM, "BatchNorm", "BatchNormalization")       \
    X(COL2IM, "Col2Im", nullptr)                          \
    X(CONCAT, "Concat", nullptr)                          \
    X(CONV2D, "Conv2d", "Conv")                           \
    X(DIV, "Div", nullptr)                                \
    X(ERF, "Erf", nullptr)                                \
    X(FLOOR, "Floor", nullptr)                            \
    X(GEMM, "Gemm", nullptr)                              \
    X(GLOBALAVERAGEPOOL, "GlobalAveragePool", nullptr)    \
    X(GRIDSAMPLE, "GridSample", nullptr)                  \
    X(LAYERNORM, "LayerNorm", "LayerNormalization")       \
    X(MATMUL, "MatMul", nullptr)                          \
    X(MAXPOOL2D, "MaxPool2d", "MaxPool")                  \
    X(MUL, "Mul", nullptr)                                \
    X(POW, "Pow", nullptr)                                \
    X(PRELU, "PRelu", nullptr)                            \
    X(REDUCE, "Reduce", nullptr)                          \
    X(RELU, "Relu", nullptr)                              \
    X(RESHAPE, "Reshape", nullptr)                        \
    X(RESIZE, "Resize", nullptr)                          \
    X(SIGMOID, "Sigmoid", nullptr)                        \
    X(SLICE, "Slice", nullptr)                            \
    X(SOFTMAX, "Softmax", nullptr)                        \
    X(SOFTPLUS, "Softplus", nullptr)                      \
    X(SPLIT, "Split", nullptr)                            \
    X(SUB, "Sub", nullptr)                                \
    X(TOPK, "TopK", nullptr)                              \
    X(TRANSPOSE, "Transpose", nullptr)                    \
    X(NMS, "Nms", "NonMaxSuppression")                              \
    X(GATHER, "Gather", nullptr)                          \
    X(RANGE, "Range", nullptr)                            \
    X(EXPAND, "Expand", nullptr)                          \
    X(SQRT, "Sqrt", nullptr)                              \
    X(SIN, "Sin", nullptr)                                \
    X(COS, "Cos", nullptr)                                \
    X(NEG, "Neg", nullptr)                                \
    X(WHERE, "Where", nullptr)                            \
    X(SOFTMAX_TOPK, "SoftmaxTopK", nullptr)

enum class OpType {
#define VKOP_ENUM(e, n, a) e,
    VKOP_OP_TABLE(VKOP_ENUM)
#undef VKOP_ENUM
        TOTAL_NUM
};

inline std::string convert_optype_to_string(const OpType &type) {
    switch (type) {
#define VKOP_NAME(e, n, a) \
    case OpType::e:        \
        return n;
        VKOP_OP_TABLE(VKOP_NAME)
#undef VKOP_NAME
    default:
        return "Unknown";
    }
}

inline OpType convert_opstring_to_enum(const std::string &name) {
#define VKOP_PARSE(e, n, a)                                                           \
    if (OpType::e != OpType::UNKNOWN && (name == n || (a != nullptr && name == (a ? a : "")))) \
        return OpType::e;
    VKOP_OP_TABLE(VKOP_PARSE)
#undef VKOP_PARSE
    std::printf("Unknown op type: %s\n", name.c_str());  // as the reference: report and carry on
    return OpType::UNKNOWN;
}

}  // namespace ops
}  // namespace vkop
#endif  // VKOP_HOST_OPS_OPS_HPP_
