// Runtime: the post-processing part of the reference's core/runtime.{hpp,cpp}:
// RegisterPostProcess (runtime.cpp:480-520), Run (:404-458), ReadResult
// (:460-478), TraceNode (:522-529), GetInput / GetOutput, and LoadModel
// (runtime.cpp:33-363) for model files whose nodes are all operators of this
// path (Softmax, TopK, NonMaxSuppression): the converted tail of a model.  A
// node of any other type makes LoadModel throw and name it.  Without a model
// file the tensor a model would produce is bound with BindOutput and stands in
// for Runtime::GetOutput()'s model output.
//
// RegisterPostProcess(SOFTMAX) immediately followed by
// RegisterPostProcess(TOPK) on the softmax output -- what benchmark/main.cpp:
// 85-101 does -- is executed as one fused SoftmaxTopK operator.
#ifndef VKOP_HOST_CORE_RUNTIME_HPP_
#define VKOP_HOST_CORE_RUNTIME_HPP_

#include <string>
#include <unordered_map>
#include <vector>

#include "core/Tensor.hpp"
#include "ops/Operator.hpp"

namespace vkop {
namespace core {

class Runtime {
  public:
    Runtime(const std::shared_ptr<VulkanCommandPool> &cmdpool, std::string model_path, int precision,
            std::string cache_dir = "");
    Runtime(const std::shared_ptr<VulkanCommandPool> &cmdpool, std::string model_path, std::string cache_dir = "");
    ~Runtime();

    // Parses model_path (a .vkopbin file), creates the tensors and one operator per node, in the order of
    // the file's concurrent levels.  Throws std::runtime_error for a node type that is not on this path.
    void LoadModel();
    std::shared_ptr<ITensor> GetInput(const std::string &name = "") const;

    // The tensor that plays the role of the model's output (first one bound is the default).
    void BindOutput(const std::string &name, const std::shared_ptr<ITensor> &tensor);
    std::shared_ptr<ITensor> GetOutput(const std::string &name = "") const;

    void RegisterPostProcess(ops::OpType ops, const std::unordered_map<std::string, std::string> &attributes,
                             const std::vector<std::shared_ptr<ITensor>> &inputs,
                             const std::vector<std::shared_ptr<ITensor>> &outputs);
    // Disables the Softmax + TopK pattern fusion (for comparisons).
    void SetFusePostProcess(bool on) { fuse_ = on; }

    double Run();       // executes the registered operators, waits, returns host milliseconds
    void ReadResult();  // copies the outputs of the last registered operator to the host
    void TraceNode(const std::string &name);

    void setPrecision(int precision) { precision_ = precision; }
    int getPrecision() const { return precision_; }
    size_t NumOperators() const { return node_ops_.size(); }

  private:
    void plan();

    int precision_ = 0;  // 0: fp32, 1: fp16
    std::shared_ptr<VulkanCommandPool> m_cmdpool_;
    std::string model_path_, cache_dir_;
    std::unordered_map<std::string, std::shared_ptr<ITensor>> inputs_, outputs_;
    std::string first_input_, first_output_;
    std::unordered_map<std::string, std::shared_ptr<ITensor>> real_outputs_;
    std::vector<std::unique_ptr<ops::Operator>> node_ops_;
    std::vector<std::unordered_map<std::string, std::string>> node_attrs_;
    std::vector<std::vector<std::shared_ptr<ITensor>>> node_input_tensors_;
    std::vector<std::vector<std::shared_ptr<ITensor>>> node_output_tensors_;
    // execution plan: operators actually run, after pattern fusion
    struct Step {
        ops::Operator *op;
        std::vector<std::shared_ptr<ITensor>> inputs, outputs;
    };
    std::vector<Step> steps_;
    std::vector<std::unique_ptr<ops::Operator>> fused_ops_;
    bool planned_ = false;
    bool fuse_ = true;
};

}  // namespace core
}  // namespace vkop
#endif  // VKOP_HOST_CORE_RUNTIME_HPP_
