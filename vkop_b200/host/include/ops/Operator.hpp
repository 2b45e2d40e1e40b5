// Operator base class: the public interface of the reference's ops/Operator.hpp
// (:19-271) -- set_runtime_device, setAttribute, onExecute, get_record,
// get_type, names and tracing -- with the Vulkan pipeline / descriptor / submit
// machinery (:225-238) replaced by calls into the C ABI of include/vkop_cuda.h
// on the stream of the operator's command buffer.
//
// onExecute enqueues the operator's kernels (the reference records a command
// buffer that the caller then submits; here the work is in the stream as soon
// as onExecute returns) and get_record()->wait() blocks until they are done.
// Argument violations that the reference guards with assert() throw
// std::invalid_argument; failures of the device layer throw std::runtime_error,
// as the reference's Vulkan calls do.  One host thread drives an operator at a
// time.
#ifndef VKOP_HOST_OPS_OPERATOR_HPP_
#define VKOP_HOST_OPS_OPERATOR_HPP_

#include <atomic>
#include <cstdio>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "core/Tensor.hpp"
#include "ops/Ops.hpp"
#include "vkop_cuda.h"

namespace vkop {
namespace ops {

class Operator {
  public:
    explicit Operator(OpType type, int fp16 = 0) : type_(type), fp16_(fp16) { instance_count_.fetch_add(1); }
    virtual ~Operator() { instance_count_.fetch_sub(1); }
    Operator(const Operator &) = delete;
    Operator &operator=(const Operator &) = delete;
    Operator(Operator &&) = delete;
    Operator &operator=(Operator &&) = delete;

    virtual void set_runtime_device(const std::shared_ptr<VulkanDevice> &dev, const std::shared_ptr<VulkanCommandPool> &cmdpool) {
        m_dev_ = dev;
        m_cmdpool_ = cmdpool;
    }

    // (The reference's default prints every attribute; the operators of this path all override it.)
    virtual void setAttribute(const std::unordered_map<std::string, std::string> &) {}

    // "[a,b,c]" -> vector (ops/Operator.hpp:87-118)
    template <typename T>
    std::vector<T> parse_attr_list(const std::string &str) {
        std::vector<T> result;
        if (str.size() >= 2 && str.front() == '[' && str.back() == ']') {
            std::stringstream ss(str.substr(1, str.size() - 2));
            std::string item;
            while (std::getline(ss, item, ',')) {
                try {
                    if (std::is_same<T, float>::value)
                        result.emplace_back(static_cast<T>(std::stof(item)));
                    else
                        result.emplace_back(static_cast<T>(std::stol(item)));
                } catch (const std::invalid_argument &) {
                    throw std::runtime_error("Invalid number in attribute list: " + item);
                } catch (const std::out_of_range &) {
                    throw std::runtime_error("Number out of range in attribute list: " + item);
                }
            }
        }
        return result;
    }

    virtual OpType get_type() { return type_; }
    std::shared_ptr<VulkanCommandBuffer> get_record() { return m_cmd_; }

    void onExecute(const std::vector<std::shared_ptr<core::ITensor>> &inputs,
                   const std::vector<std::shared_ptr<core::ITensor>> &outputs, int id) {
        if (!m_dev_ || !m_cmdpool_)
            throw std::runtime_error("operator used before set_runtime_device");
        if (!m_cmd_ || m_id_ != id)
            m_cmd_ = std::make_shared<VulkanCommandBuffer>(m_cmdpool_, id);
        m_id_ = id;
        m_cmd_->begin();
        execute(inputs, outputs);
        m_cmd_->end();
        if (trace_) {
            m_cmd_->wait();
            std::printf("%s: %s\n", convert_optype_to_string(type_).c_str(), name_.c_str());
            for (size_t i = 0; i < outputs.size(); i++) {
                std::printf("output %zu:\n", i);
                dump(outputs[i]);
            }
        }
    }
    void enable_trace() { trace_ = true; }
    void disable_trace() { trace_ = false; }
    void set_name(const std::string &name) { name_ = name; }
    std::string get_name() const { return name_; }

    static std::atomic<int> instance_count_;

  protected:
    virtual void execute(const std::vector<std::shared_ptr<core::ITensor>> &inputs,
                         const std::vector<std::shared_ptr<core::ITensor>> &outputs) = 0;

    cudaStream_t stream() const { return m_cmd_->stream(); }

    static void check(int status, const char *what) {
        if (status == VKOP_OK)
            return;
        const std::string msg = std::string(what) + ": " + vkop_cuda_status_string(status);
        if (status == VKOP_INVALID_ARG || status == VKOP_UNSUPPORTED)
            throw std::invalid_argument(msg);
        throw std::runtime_error(msg);
    }

    // Scratch memory owned by the operator (the role of Topk's temporary tensors, ops/Topk.hpp:46-54).
    // `shape_key` identifies the descriptor the scratch memory serves: the kernels keep counters in it
    // whose layout follows the shape, so it is cleared again whenever the key changes.
    void *workspace(size_t bytes, uint64_t shape_key = 0) {
        if (bytes == 0)
            return nullptr;
        if (!ws_ || ws_->bytes() < bytes) {
            ws_ = std::make_shared<core::DeviceBuffer>(bytes);
            ws_key_ = shape_key + 1;  // force the clear below
        }
        if (ws_key_ != shape_key) {
            check(vkop_cuda_workspace_init(ws_->ptr(), ws_->bytes(), stream()), "workspace_init");
            ws_key_ = shape_key;
        }
        return ws_->ptr();
    }
    size_t workspace_bytes() const { return ws_ ? ws_->bytes() : 0; }
    // One number per distinct selection descriptor (shape, element type, k, path).
    static uint64_t shape_key(const vkop_softmax_topk_desc &d) {
        uint64_t h = 1469598103934665603ull;
        const uint64_t parts[] = {static_cast<uint64_t>(d.rows), static_cast<uint64_t>(d.cols), static_cast<uint64_t>(d.row_stride),
                                  static_cast<uint64_t>(d.dtype), static_cast<uint64_t>(d.k), static_cast<uint64_t>(d.path),
                                  static_cast<uint64_t>(d.splits), static_cast<uint64_t>(d.flags)};
        for (uint64_t v : parts)
            h = (h ^ v) * 1099511628211ull;
        return h | 1ull;
    }

    // Device storage of a tensor of one of the supported element types.
    void *device_of(const std::shared_ptr<core::ITensor> &t) {
        const std::type_info &ty = t->dtype();
        if (ty == typeid(float))
            return core::as_tensor<float>(t)->as_storage_buffer(m_dev_)->ptr();
        if (ty == typeid(uint16_t))
            return core::as_tensor<uint16_t>(t)->as_storage_buffer(m_dev_)->ptr();
        if (ty == typeid(int))
            return core::as_tensor<int>(t)->as_storage_buffer(m_dev_)->ptr();
        if (ty == typeid(int64_t))
            return core::as_tensor<int64_t>(t)->as_storage_buffer(m_dev_)->ptr();
        if (ty == typeid(int8_t))
            return core::as_tensor<int8_t>(t)->as_storage_buffer(m_dev_)->ptr();
        throw std::runtime_error(std::string("Unsupported dtype: ") + ty.name());
    }
    // Sizes an output the caller left empty (size() == 0), as the reference operators do.
    static void resize_if_empty(const std::shared_ptr<core::ITensor> &t, const std::vector<int> &shape) {
        if (t->size() != 0)
            return;
        const std::type_info &ty = t->dtype();
        if (ty == typeid(float))
            core::as_tensor<float>(t)->resize(shape);
        else if (ty == typeid(uint16_t))
            core::as_tensor<uint16_t>(t)->resize(shape);
        else if (ty == typeid(int))
            core::as_tensor<int>(t)->resize(shape);
        else if (ty == typeid(int64_t))
            core::as_tensor<int64_t>(t)->resize(shape);
        else
            throw std::runtime_error(std::string("Unsupported dtype: ") + ty.name());
    }
    static int value_dtype(const std::shared_ptr<core::ITensor> &t) {
        if (t->dtype() == typeid(float))
            return VKOP_F32;
        if (t->dtype() == typeid(uint16_t))
            return t->is_bf16() ? VKOP_BF16 : VKOP_F16;
        throw std::invalid_argument("values must be float or 16-bit float tensors");
    }
    void dump(const std::shared_ptr<core::ITensor> &t) {
        const std::type_info &ty = t->dtype();
        if (ty == typeid(float)) {
            core::as_tensor<float>(t)->copyToCPU(m_cmdpool_);
            core::as_tensor<float>(t)->print_tensor();
        } else if (ty == typeid(uint16_t)) {
            core::as_tensor<uint16_t>(t)->copyToCPU(m_cmdpool_);
            core::as_tensor<uint16_t>(t)->print_tensor();
        } else if (ty == typeid(int)) {
            core::as_tensor<int>(t)->copyToCPU(m_cmdpool_);
            core::as_tensor<int>(t)->print_tensor();
        }
    }

    std::shared_ptr<VulkanDevice> m_dev_;
    std::shared_ptr<VulkanCommandPool> m_cmdpool_;
    std::shared_ptr<VulkanCommandBuffer> m_cmd_;
    int m_id_ = 0;
    OpType type_;
    int fp16_ = 0;  // 0: fp32, 1: fp16
    bool trace_ = false;
    std::string name_;

  private:
    std::shared_ptr<core::DeviceBuffer> ws_;
    uint64_t ws_key_ = 0;
};

inline std::atomic<int> Operator::instance_count_{0};

}  // namespace ops
}  // namespace vkop
#endif  // VKOP_HOST_OPS_OPERATOR_HPP_
