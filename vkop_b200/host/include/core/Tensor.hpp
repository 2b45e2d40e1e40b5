// Tensor storage for the post-processing path: the storage-buffer subset of
// the reference's core/Tensor.hpp (ITensor :35-209, Tensor<T> :211-1057:
// as_storage_buffer :384-394, copyToGPU :540-554, copyToCPU :556-567,
// fillToCPU :569-578) over cudaMalloc instead of VMA buffers.  The RGBA image
// packing of the reference is a Vulkan artefact and is not reproduced:
// tensors of any rank are linear row-major device buffers.
// T is float, uint16_t (fp16 bit patterns, or bf16 with set_bf16()), int,
// int64_t or int8_t, as in the reference.
#ifndef VKOP_HOST_CORE_TENSOR_HPP_
#define VKOP_HOST_CORE_TENSOR_HPP_

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <memory>
#include <typeinfo>
#include <vector>

#include "vulkan/VulkanDevice.hpp"

namespace vkop {
namespace core {

// The device allocation behind a tensor (the role of VulkanBuffer).
class DeviceBuffer {
  public:
    explicit DeviceBuffer(size_t bytes) : bytes_(bytes) { cuda_check(cudaMalloc(&ptr_, bytes ? bytes : 16), "cudaMalloc"); }
    ~DeviceBuffer() { cudaFree(ptr_); }
    DeviceBuffer(const DeviceBuffer &) = delete;
    DeviceBuffer &operator=(const DeviceBuffer &) = delete;
    void *ptr() const { return ptr_; }
    size_t bytes() const { return bytes_; }

  private:
    void *ptr_ = nullptr;
    size_t bytes_;
};

class ITensor {
  public:
    virtual ~ITensor() = default;
    virtual const std::type_info &dtype() const = 0;
    virtual size_t elem_size() const = 0;

    uint8_t num_dims() const { return static_cast<uint8_t>(shape_.size()); }
    int size() const { return static_cast<int>(num_elements() * static_cast<int64_t>(elem_size())); }  // bytes; 0: "the operator may size me"
    int64_t num_elements() const {
        if (shape_.empty())
            return 0;
        int64_t n = 1;
        for (int d : shape_)
            n *= d;
        return n;
    }
    std::vector<int> getShape() const { return shape_; }
    bool is_on_GPU() const { return on_gpu_; }
    void toGPU() { on_gpu_ = true; }
    void toCPU() { on_gpu_ = false; }
    // uint16_t tensors hold fp16 unless marked as bf16 (the reference has no bf16 tensors)
    void set_bf16(bool v = true) { bf16_ = v; }
    bool is_bf16() const { return bf16_; }

    void *device_ptr() const { return buffer_ ? buffer_->ptr() : nullptr; }

    static float fp16_to_fp32(uint16_t h) {
        const uint32_t sign = static_cast<uint32_t>(h & 0x8000u) << 16;
        uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, u;
        if (exp == 0) {
            if (man == 0) {
                u = sign;
            } else {
                int e = -1;
                do {
                    man <<= 1;
                    e++;
                } while ((man & 0x400u) == 0);
                u = sign | (static_cast<uint32_t>(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
            }
        } else if (exp == 31) {
            u = sign | 0x7F800000u | (man << 13);
        } else {
            u = sign | ((exp + 112) << 23) | (man << 13);
        }
        float f;
        std::memcpy(&f, &u, 4);
        return f;
    }

  protected:
    std::vector<int> shape_;
    bool on_gpu_ = false;
    bool bf16_ = false;
    std::shared_ptr<DeviceBuffer> buffer_;
};

template <typename T>
class Tensor : public ITensor {
  public:
    explicit Tensor(bool is_on_GPU = false) { on_gpu_ = is_on_GPU; }
    template <typename U>
    explicit Tensor(const std::vector<U> &dims, bool is_on_GPU = false) {
        on_gpu_ = is_on_GPU;
        resize(dims);
    }
    Tensor(int n, int c, int h, int w, bool is_on_GPU = false) {
        on_gpu_ = is_on_GPU;
        std::vector<int> d;
        for (int v : {n, c, h, w})
            if (v != 0)
                d.push_back(v);
        resize(d);
    }

    const std::type_info &dtype() const override { return typeid(T); }
    size_t elem_size() const override { return sizeof(T); }

    template <typename U>
    void resize(const std::vector<U> &dims) {
        shape_.assign(dims.begin(), dims.end());
        if (!on_gpu_)
            host_.resize(static_cast<size_t>(num_elements()));
        buffer_.reset();
    }

    T *data() { return host_.data(); }
    const std::vector<T> &host() const { return host_; }
    T &operator[](size_t i) { return host_[i]; }

    void fillToCPU(const std::vector<T> &v) {
        host_ = v;
        host_.resize(static_cast<size_t>(num_elements()));
    }

    // Device storage, padded to a multiple of four elements (core/Tensor.hpp:726).
    std::shared_ptr<DeviceBuffer> as_storage_buffer(const std::shared_ptr<VulkanDevice> &dev,
                                                    const std::shared_ptr<VulkanCommandBuffer> & = nullptr) {
        const size_t padded = (static_cast<size_t>(num_elements()) + 3) / 4 * 4 * sizeof(T);
        if (!buffer_ || buffer_->bytes() < padded) {
            cuda_check(cudaSetDevice(dev->ordinal()), "cudaSetDevice");
            buffer_ = std::make_shared<DeviceBuffer>(padded);
        }
        return buffer_;
    }

    void copyToGPU(const std::shared_ptr<VulkanCommandPool> &pool, const T *src = nullptr) {
        as_storage_buffer(pool->getVulkanDevice());
        const T *from = src ? src : host_.data();
        cuda_check(cudaMemcpy(buffer_->ptr(), from, static_cast<size_t>(num_elements()) * sizeof(T), cudaMemcpyHostToDevice),
                   "cudaMemcpy H2D");
        toGPU();
    }
    // Asynchronous upload from pinned host memory on the pool's first queue.
    void copyToGPUAsync(const std::shared_ptr<VulkanCommandPool> &pool, const T *pinned_src, cudaStream_t stream) {
        as_storage_buffer(pool->getVulkanDevice());
        cuda_check(cudaMemcpyAsync(buffer_->ptr(), pinned_src, static_cast<size_t>(num_elements()) * sizeof(T),
                                   cudaMemcpyHostToDevice, stream),
                   "cudaMemcpyAsync H2D");
        toGPU();
    }

    void copyToCPU(const std::shared_ptr<VulkanCommandPool> &) {
        if (!buffer_)
            throw std::runtime_error("copyToCPU: tensor has no device storage");
        host_.resize(static_cast<size_t>(num_elements()));
        cuda_check(cudaMemcpy(host_.data(), buffer_->ptr(), host_.size() * sizeof(T), cudaMemcpyDeviceToHost), "cudaMemcpy D2H");
    }

    void print_tensor() const {
        const size_t n = host_.size() < 64 ? host_.size() : 64;
        for (size_t i = 0; i < n; i++) {
            if constexpr (std::is_same<T, float>::value)
                std::printf("%g ", static_cast<double>(host_[i]));
            else if constexpr (std::is_same<T, uint16_t>::value)
                std::printf("%g ", static_cast<double>(fp16_to_fp32(host_[i])));
            else
                std::printf("%lld ", static_cast<long long>(host_[i]));
        }
        std::printf(host_.size() > n ? "...\n" : "\n");
    }

  private:
    std::vector<T> host_;
};

template <typename T>
std::shared_ptr<Tensor<T>> as_tensor(const std::shared_ptr<ITensor> &t) {
    return std::dynamic_pointer_cast<Tensor<T>>(t);  // core/Tensor.hpp:1059-1063
}

}  // namespace core
}  // namespace vkop
#endif  // VKOP_HOST_CORE_TENSOR_HPP_
