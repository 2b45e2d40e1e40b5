// CUDA-backed stand-ins for the device handles that appear in the reference's
// operator API (vulkan/VulkanDevice.hpp, vulkan/VulkanCommandPool.hpp,
// vulkan/VulkanCommandBuffer.hpp).  They keep the reference's names and the
// members the post-processing path uses, so callers written against the
// reference compile unchanged; behind them there is a CUDA device ordinal, a
// pair of streams (the reference's two in-flight queues) and an event.
#ifndef VKOP_HOST_VULKAN_DEVICE_HPP_
#define VKOP_HOST_VULKAN_DEVICE_HPP_

#include <cuda_runtime.h>

#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace vkop {

constexpr int kInflight = 2;  // vulkan/VulkanDevice.hpp:13

inline void cuda_check(cudaError_t e, const char *what) {
    if (e != cudaSuccess)
        throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

// A compute queue of the reference is a CUDA stream here.
class VulkanQueue {
  public:
    explicit VulkanQueue(cudaStream_t s) : stream_(s) {}
    cudaStream_t stream() const { return stream_; }

  private:
    cudaStream_t stream_;
};

class VulkanDevice {
  public:
    explicit VulkanDevice(int ordinal = 0) : ordinal_(ordinal) {
        cuda_check(cudaSetDevice(ordinal_), "cudaSetDevice");
        cudaDeviceProp prop;
        cuda_check(cudaGetDeviceProperties(&prop, ordinal_), "cudaGetDeviceProperties");
        name_ = prop.name;
        for (int i = 0; i < kInflight; i++) {
            cudaStream_t s;
            cuda_check(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking), "cudaStreamCreate");
            queues_.push_back(std::make_shared<VulkanQueue>(s));
        }
    }
    ~VulkanDevice() {
        for (auto &q : queues_)
            cudaStreamDestroy(q->stream());
    }
    VulkanDevice(const VulkanDevice &) = delete;
    VulkanDevice &operator=(const VulkanDevice &) = delete;

    int ordinal() const { return ordinal_; }
    std::string getDeviceName() const { return name_; }
    bool is_support_nv_tensor_core() const { return false; }  // nothing on this path is a contraction
    std::shared_ptr<VulkanQueue> getComputeQueue(int i = 0) const { return queues_[static_cast<size_t>(i) % queues_.size()]; }
    void wait_all_done() const { cuda_check(cudaDeviceSynchronize(), "cudaDeviceSynchronize"); }

  private:
    int ordinal_;
    std::string name_;
    std::vector<std::shared_ptr<VulkanQueue>> queues_;
};

class VulkanCommandPool {
  public:
    explicit VulkanCommandPool(std::shared_ptr<VulkanDevice> dev) : dev_(std::move(dev)) {}
    std::shared_ptr<VulkanDevice> getVulkanDevice() const { return dev_; }

  private:
    std::shared_ptr<VulkanDevice> dev_;
};

// What the reference submits to a queue; work recorded here is already enqueued, so it carries nothing.
struct VkSubmitInfo {};

// "Recording" enqueues on the stream of queue `id`; wait() blocks until that work is done.
class VulkanCommandBuffer {
  public:
    explicit VulkanCommandBuffer(std::shared_ptr<VulkanCommandPool> pool, int id = 0)
        : pool_(std::move(pool)), queue_(pool_->getVulkanDevice()->getComputeQueue(id)) {
        cuda_check(cudaEventCreateWithFlags(&done_, cudaEventDisableTiming), "cudaEventCreate");
    }
    ~VulkanCommandBuffer() { cudaEventDestroy(done_); }
    VulkanCommandBuffer(const VulkanCommandBuffer &) = delete;
    VulkanCommandBuffer &operator=(const VulkanCommandBuffer &) = delete;

    void begin() {}
    void end() { cuda_check(cudaEventRecord(done_, queue_->stream()), "cudaEventRecord"); }
    void wait() { cuda_check(cudaEventSynchronize(done_), "cudaEventSynchronize"); }
    void reset() {}
    void clearWaits() {}
    VkSubmitInfo buildSubmitInfo() { return VkSubmitInfo{}; }
    static void submit(const std::shared_ptr<VulkanQueue> &, std::vector<VkSubmitInfo> &) {}
    cudaStream_t stream() const { return queue_->stream(); }
    cudaEvent_t done_event() const { return done_; }

  private:
    std::shared_ptr<VulkanCommandPool> pool_;
    std::shared_ptr<VulkanQueue> queue_;
    cudaEvent_t done_;
};

}  // namespace vkop
#endif  // VKOP_HOST_VULKAN_DEVICE_HPP_
