// Flat C entry points over the C++ operator API, for harnesses that cannot
// include C++ headers (the Python benchmark).  A pipeline is what
// benchmark/main.cpp:85-118 builds: a Runtime with Softmax and TopK registered
// as post-processing on a logits tensor, then Run() and ReadResult().
#include <cstring>

#include "core/runtime.hpp"

using namespace vkop;

namespace {
struct Pipeline {
    std::shared_ptr<VulkanDevice> dev;
    std::shared_ptr<VulkanCommandPool> pool;
    std::unique_ptr<core::Runtime> rt;
    std::shared_ptr<core::ITensor> logits, probs, values, indices;
    int rows, cols, k, dtype;
    std::string error;
};
thread_local std::string g_error;

template <typename T>
void build(Pipeline &p, float temperature, bool fuse) {
    auto logits = std::make_shared<core::Tensor<T>>(std::vector<int>{p.rows, p.cols}, true);
    logits->as_storage_buffer(p.dev);
    if (p.dtype == VKOP_BF16)
        logits->set_bf16();
    p.logits = logits;
    p.rt->BindOutput("logits", logits);
    auto cls = core::as_tensor<T>(p.rt->GetOutput());
    auto sf = std::make_shared<core::Tensor<T>>(cls->getShape(), true);
    p.probs = sf;
    p.rt->RegisterPostProcess(ops::OpType::SOFTMAX, {{"axis", "-1"}}, {cls}, {sf});
    auto idx = std::make_shared<core::Tensor<int>>(std::vector<int>{p.rows, p.k}, true);
    auto vals = std::make_shared<core::Tensor<T>>(std::vector<int>{p.rows, p.k}, true);
    if (p.dtype == VKOP_BF16) {
        sf->set_bf16();
        vals->set_bf16();
    }
    std::unordered_map<std::string, std::string> attrs = {{"k", std::to_string(p.k)}};
    if (temperature != 1.0f)
        attrs["temperature"] = std::to_string(temperature);
    p.rt->RegisterPostProcess(ops::OpType::TOPK, attrs, {sf}, {vals, idx});
    p.rt->SetFusePostProcess(fuse);
    p.values = vals;
    p.indices = idx;
}

template <typename T>
void run(Pipeline &p, const void *host_logits, void *host_values, int32_t *host_indices, double *ms) {
    auto in = core::as_tensor<T>(p.logits);
    in->copyToGPU(p.pool, static_cast<const T *>(host_logits));
    const double t = p.rt->Run();
    if (ms)
        *ms = t;
    p.rt->ReadResult();
    auto v = core::as_tensor<T>(p.values);
    auto i = core::as_tensor<int>(p.indices);
    std::memcpy(host_values, v->data(), static_cast<size_t>(p.rows) * p.k * sizeof(T));
    std::memcpy(host_indices, i->data(), static_cast<size_t>(p.rows) * p.k * sizeof(int));
}
}  // namespace

extern "C" {

const char *vkop_host_last_error(void) { return g_error.c_str(); }

// dtype: vkop_dtype.  fuse != 0: the registered Softmax + TopK pair runs as the fused operator.
void *vkop_host_pipeline_create(int device, int rows, int cols, int dtype, int k, float temperature, int fuse) {
    try {
        auto p = std::make_unique<Pipeline>();
        p->dev = std::make_shared<VulkanDevice>(device);
        p->pool = std::make_shared<VulkanCommandPool>(p->dev);
        p->rt = std::make_unique<core::Runtime>(p->pool, "", dtype == VKOP_F32 ? 0 : 1);
        p->rows = rows;
        p->cols = cols;
        p->k = k;
        p->dtype = dtype;
        if (dtype == VKOP_F32)
            build<float>(*p, temperature, fuse != 0);
        else
            build<uint16_t>(*p, temperature, fuse != 0);
        return p.release();
    } catch (const std::exception &e) {
        g_error = e.what();
        return nullptr;
    }
}

// host_logits: rows * cols elements; host_values: rows * k elements; host_indices: rows * k int32.
int vkop_host_pipeline_run(void *handle, const void *host_logits, void *host_values, int32_t *host_indices, double *run_ms) {
    auto *p = static_cast<Pipeline *>(handle);
    if (!p || !host_logits || !host_values || !host_indices)
        return VKOP_INVALID_ARG;
    try {
        if (p->dtype == VKOP_F32)
            run<float>(*p, host_logits, host_values, host_indices, run_ms);
        else
            run<uint16_t>(*p, host_logits, host_values, host_indices, run_ms);
        return VKOP_OK;
    } catch (const std::invalid_argument &e) {
        g_error = e.what();
        return VKOP_INVALID_ARG;
    } catch (const std::exception &e) {
        g_error = e.what();
        return VKOP_CUDA_ERROR;
    }
}

void vkop_host_pipeline_destroy(void *handle) { delete static_cast<Pipeline *>(handle); }

}  // extern "C"
