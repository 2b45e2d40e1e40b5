// Post-processing subset of the reference runtime (core/runtime.cpp:404-529).
#include "core/runtime.hpp"

#include <chrono>

#include "ops/OperatorFactory.hpp"

namespace vkop {
namespace core {

Runtime::Runtime(const std::shared_ptr<VulkanCommandPool> &cmdpool, std::string model_path, int precision, std::string cache_dir)
    : precision_(precision), m_cmdpool_(cmdpool), model_path_(std::move(model_path)), cache_dir_(std::move(cache_dir)) {}

Runtime::Runtime(const std::shared_ptr<VulkanCommandPool> &cmdpool, std::string model_path, std::string cache_dir)
    : m_cmdpool_(cmdpool), model_path_(std::move(model_path)), cache_dir_(std::move(cache_dir)) {}

Runtime::~Runtime() = default;

void Runtime::LoadModel() {
    throw std::runtime_error("Runtime::LoadModel: model graphs are outside the post-processing path; bind the logits with BindOutput");
}

void Runtime::BindOutput(const std::string &name, const std::shared_ptr<ITensor> &tensor) {
    if (outputs_.empty())
        first_output_ = name;
    outputs_[name] = tensor;
}

std::shared_ptr<ITensor> Runtime::GetOutput(const std::string &name) const {
    if (outputs_.empty())
        return nullptr;
    auto it = outputs_.find(name.empty() ? first_output_ : name);
    return it == outputs_.end() ? nullptr : it->second;
}

// core/runtime.cpp:480-520: create the operator, name it post_<Type>, append it after everything
// registered so far and make its outputs the results ReadResult copies back.
void Runtime::RegisterPostProcess(ops::OpType ops, const std::unordered_map<std::string, std::string> &attributes,
                                  const std::vector<std::shared_ptr<ITensor>> &inputs,
                                  const std::vector<std::shared_ptr<ITensor>> &outputs) {
    if (outputs.empty() || inputs.empty())
        throw std::invalid_argument("RegisterPostProcess: needs inputs and outputs");
    auto dev = m_cmdpool_->getVulkanDevice();
    auto op = ops::create_from_type(ops, outputs[0]->num_dims() <= 2, precision_, dev->is_support_nv_tensor_core());
    if (!op)
        throw std::invalid_argument("RegisterPostProcess: operator type is not on the post-processing path: " +
                                    ops::convert_optype_to_string(ops));
    op->set_name("post_" + ops::convert_optype_to_string(ops));
    op->set_runtime_device(dev, m_cmdpool_);
    op->setAttribute(attributes);
    node_ops_.push_back(std::move(op));
    node_attrs_.push_back(attributes);
    node_input_tensors_.push_back(inputs);
    node_output_tensors_.push_back(outputs);
    real_outputs_.clear();
    for (size_t i = 0; i < outputs.size(); ++i)
        real_outputs_["post_" + ops::convert_optype_to_string(ops) + std::to_string(i)] = outputs[i];
    planned_ = false;
}

void Runtime::plan() {
    steps_.clear();
    fused_ops_.clear();
    auto dev = m_cmdpool_->getVulkanDevice();
    for (size_t i = 0; i < node_ops_.size(); i++) {
        const bool softmax_then_topk =
            fuse_ && i + 1 < node_ops_.size() && node_ops_[i]->get_type() == ops::OpType::SOFTMAX &&
            node_ops_[i + 1]->get_type() == ops::OpType::TOPK && node_input_tensors_[i + 1].size() == 1 &&
            node_input_tensors_[i + 1][0] == node_output_tensors_[i][0];
        if (softmax_then_topk) {
            // the softmax must run over the axis TopK selects on (the last one) and TopK must take the largest
            const auto &sm = node_attrs_[i];
            const auto &tk = node_attrs_[i + 1];
            const int rank = node_input_tensors_[i][0]->num_dims();
            auto axis_of = [&](const std::unordered_map<std::string, std::string> &a, const char *k1, const char *k2) {
                auto it = a.find(k1);
                if (it == a.end() && k2)
                    it = a.find(k2);
                int ax = it == a.end() ? -1 : static_cast<int>(std::stol(it->second));
                return ax < 0 ? ax + rank : ax;
            };
            const bool largest = !tk.count("largest") || std::stol(tk.at("largest")) != 0;
            if (axis_of(sm, "axis", "dim") == rank - 1 && axis_of(tk, "axis", nullptr) == rank - 1 && largest) {
                auto fused = ops::create_from_type(ops::OpType::SOFTMAX_TOPK, true, precision_, false);
                fused->set_name("post_SoftmaxTopK");
                fused->set_runtime_device(dev, m_cmdpool_);
                fused->setAttribute(tk);
                steps_.push_back(Step{fused.get(), node_input_tensors_[i], node_output_tensors_[i + 1]});
                fused_ops_.push_back(std::move(fused));
                i++;
                continue;
            }
        }
        steps_.push_back(Step{node_ops_[i].get(), node_input_tensors_[i], node_output_tensors_[i]});
    }
    planned_ = true;
}

// core/runtime.cpp:404-458: execute every operator, wait for the last, return the host time in ms.
double Runtime::Run() {
    if (!planned_)
        plan();
    const auto start = std::chrono::steady_clock::now();
    ops::Operator *last = nullptr;
    for (auto &s : steps_) {
        s.op->onExecute(s.inputs, s.outputs, 0);  // one queue: post-processing operators depend on each other
        last = s.op;
    }
    if (last)
        last->get_record()->wait();
    const std::chrono::duration<double> elapsed = std::chrono::steady_clock::now() - start;
    return elapsed.count() * 1000.0;
}

// core/runtime.cpp:460-478
void Runtime::ReadResult() {
    m_cmdpool_->getVulkanDevice()->wait_all_done();
    for (auto &p : real_outputs_) {
        const std::type_info &ty = p.second->dtype();
        if (ty == typeid(float))
            as_tensor<float>(p.second)->copyToCPU(m_cmdpool_);
        else if (ty == typeid(int))
            as_tensor<int>(p.second)->copyToCPU(m_cmdpool_);
        else if (ty == typeid(uint16_t))
            as_tensor<uint16_t>(p.second)->copyToCPU(m_cmdpool_);
        else if (ty == typeid(int64_t))
            as_tensor<int64_t>(p.second)->copyToCPU(m_cmdpool_);
        else
            throw std::runtime_error("ReadResult: unsupported output type");
    }
}

void Runtime::TraceNode(const std::string &name) {
    for (auto &op : node_ops_) {
        if (op->get_name() == name) {
            op->enable_trace();
            break;
        }
    }
}

}  // namespace core
}  // namespace vkop
