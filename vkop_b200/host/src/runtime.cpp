// Post-processing subset of the reference runtime (core/runtime.cpp:404-529).
#include "core/runtime.hpp"

#include <chrono>

#include <cstring>

#include "model/load.hpp"
#include "ops/OperatorFactory.hpp"

namespace vkop {
namespace core {

Runtime::Runtime(const std::shared_ptr<VulkanCommandPool> &cmdpool, std::string model_path, int precision, std::string cache_dir)
    : precision_(precision), m_cmdpool_(cmdpool), model_path_(std::move(model_path)), cache_dir_(std::move(cache_dir)) {}

Runtime::Runtime(const std::shared_ptr<VulkanCommandPool> &cmdpool, std::string model_path, std::string cache_dir)
    : m_cmdpool_(cmdpool), model_path_(std::move(model_path)), cache_dir_(std::move(cache_dir)) {}

Runtime::~Runtime() = default;

namespace {

// First element of a small integer or float initializer, as the text an attribute holds.
std::string scalar_text(const load::VkModel &model, const load::Initializer &init) {
    const uint8_t *p = model.initializer_data(init.name);
    if (!p || init.byte_size <= 0)
        throw std::runtime_error("LoadModel: empty initializer " + init.name);
    if (init.dtype == "int64" && init.byte_size >= 8) {
        int64_t v;
        std::memcpy(&v, p, 8);
        return std::to_string(v);
    }
    if (init.dtype == "int32" && init.byte_size >= 4) {
        int32_t v;
        std::memcpy(&v, p, 4);
        return std::to_string(v);
    }
    if (init.dtype == "float32" && init.byte_size >= 4) {
        float v;
        std::memcpy(&v, p, 4);
        return std::to_string(v);
    }
    throw std::runtime_error("LoadModel: initializer " + init.name + " of type " + init.dtype + " cannot parameterise an operator");
}

std::vector<int> to_int_dims(const std::vector<uint32_t> &d) { return std::vector<int>(d.begin(), d.end()); }

}  // namespace

// core/runtime.cpp:33-363, for graphs made of this path's operators.  ONNX passes some parameters as
// inputs (TopK's K; NonMaxSuppression's max_output_boxes_per_class, iou_threshold, score_threshold):
// such an input, given as an initializer, becomes the attribute of the same meaning, unless the node
// already carries that attribute.
void Runtime::LoadModel() {
    const load::VkModel model(model_path_);
    auto dev = m_cmdpool_->getVulkanDevice();
    std::unordered_map<std::string, std::shared_ptr<ITensor>> tensor_map;
    auto make_value_tensor = [&](const std::vector<int> &dims) -> std::shared_ptr<ITensor> {
        if (precision_ == 1)
            return dims.empty() ? std::make_shared<Tensor<uint16_t>>(true) : std::make_shared<Tensor<uint16_t>>(dims, true);
        return dims.empty() ? std::make_shared<Tensor<float>>(true) : std::make_shared<Tensor<float>>(dims, true);
    };
    for (const auto &in : model.inputs) {
        auto t = make_value_tensor(to_int_dims(in.dims));
        if (inputs_.empty())
            first_input_ = in.name;
        inputs_[in.name] = t;
        tensor_map[in.name] = t;
    }
    // node order: the file's levels when they name every node exactly once, else the file's order
    std::unordered_map<std::string, const load::Node *> by_name;
    for (const auto &n : model.nodes)
        by_name[n.name] = &n;
    std::vector<const load::Node *> order;
    for (const auto &level : model.concurrent_execution_levels)
        for (const auto &name : level) {
            auto it = by_name.find(name);
            if (it != by_name.end())
                order.push_back(it->second);
        }
    if (order.size() != model.nodes.size()) {
        order.clear();
        for (const auto &n : model.nodes)
            order.push_back(&n);
    }
    for (const load::Node *n : order) {
        const ops::OpType type = ops::convert_opstring_to_enum(n->op_type);
        const int rank = n->inputs.empty() ? 0 : static_cast<int>(n->inputs[0].dims.size());
        auto op = type == ops::OpType::UNKNOWN ? nullptr : ops::create_from_type(type, rank <= 2, precision_, false);
        if (!op)
            throw std::runtime_error("LoadModel: node '" + n->name + "' of type " + n->op_type +
                                     " has no operator on the post-processing path");
        auto attrs = n->attributes;
        // NonMaxSuppression: the initializer inputs are, in order, max_output_boxes_per_class, iou_threshold and
        // score_threshold (ONNX inputs 2-4; they follow the single detection-head input as well)
        static const char *const kNmsParams[] = {"max_output_boxes_per_class", "iou_threshold", "score_threshold"};
        size_t nms_param = 0;
        std::vector<std::shared_ptr<ITensor>> ins, outs;
        for (size_t i = 0; i < n->inputs.size(); i++) {
            const std::string &name = n->inputs[i].name;
            auto tm = tensor_map.find(name);
            if (tm != tensor_map.end()) {
                ins.push_back(tm->second);
                continue;
            }
            auto init = model.initializers.find(name);
            if (init == model.initializers.end())
                throw std::runtime_error("LoadModel: input '" + name + "' of node '" + n->name + "' is produced by nothing");
            const char *as_attr = nullptr;
            if (type == ops::OpType::TOPK && i == 1)
                as_attr = attrs.count("K") ? "K" : "k";
            else if (type == ops::OpType::NMS && nms_param < 3)
                as_attr = kNmsParams[nms_param++];
            if (as_attr) {
                if (!attrs.count(as_attr))
                    attrs[as_attr] = scalar_text(model, init->second);
                continue;
            }
            if (init->second.dtype != "float32")
                throw std::runtime_error("LoadModel: tensor initializer '" + name + "' must be float32");
            auto t = std::make_shared<Tensor<float>>(to_int_dims(init->second.dims), true);
            if (static_cast<int64_t>(t->num_elements()) * 4 != init->second.byte_size)
                throw std::runtime_error("LoadModel: initializer '" + name + "' has the wrong size");
            t->copyToGPU(m_cmdpool_, reinterpret_cast<const float *>(model.initializer_data(name)));
            tensor_map[name] = t;
            ins.push_back(t);
        }
        for (size_t i = 0; i < n->outputs.size(); i++) {
            std::shared_ptr<ITensor> t;
            const bool integer = (type == ops::OpType::TOPK && i == 1) || type == ops::OpType::NMS;
            if (integer)
                t = std::make_shared<Tensor<int>>(true);
            else
                t = make_value_tensor({});
            tensor_map[n->outputs[i].name] = t;
            outs.push_back(t);
        }
        op->set_name(n->name);
        op->set_runtime_device(dev, m_cmdpool_);
        op->setAttribute(attrs);
        node_ops_.push_back(std::move(op));
        node_attrs_.push_back(attrs);
        node_input_tensors_.push_back(ins);
        node_output_tensors_.push_back(outs);
    }
    real_outputs_.clear();
    for (const auto &o : model.outputs) {
        auto tm = tensor_map.find(o.name);
        if (tm == tensor_map.end())
            throw std::runtime_error("LoadModel: output '" + o.name + "' is produced by no node");
        if (outputs_.empty())
            first_output_ = o.name;
        outputs_[o.name] = tm->second;
        real_outputs_[o.name] = tm->second;
    }
    planned_ = false;
}

std::shared_ptr<ITensor> Runtime::GetInput(const std::string &name) const {
    if (inputs_.empty())
        return nullptr;
    auto it = inputs_.find(name.empty() ? first_input_ : name);
    return it == inputs_.end() ? nullptr : it->second;
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
