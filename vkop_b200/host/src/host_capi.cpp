// Flat C entry points over the C++ operator API, for harnesses that cannot
// include C++ headers (the Python benchmark).  A pipeline is what
// benchmark/main.cpp:85-118 builds: a Runtime with Softmax and TopK registered
// as post-processing on a logits tensor, then Run() and ReadResult().
#include <cstring>

#include "core/runtime.hpp"
#include "model/load.hpp"

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
// (for the other translation units of this library)
void vkop_host_set_error(const char *text) { g_error = text ? text : ""; }

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

// Parses a .vkopbin model file (no device needed) and writes its description, one line per input, output,
// node, initializer and level, into buf (NUL-terminated, truncated to cap).  Returns the full length, or
// -1 with vkop_host_last_error() set.
long vkop_host_model_describe(const char *path, char *buf, size_t cap) {
    try {
        const load::VkModel model(path ? path : "");
        const std::string text = model.describe();
        if (buf && cap > 0) {
            const size_t n = text.size() < cap - 1 ? text.size() : cap - 1;
            std::memcpy(buf, text.data(), n);
            buf[n] = 0;
        }
        return static_cast<long>(text.size());
    } catch (const std::exception &e) {
        g_error = e.what();
        return -1;
    }
}

// Loads a .vkopbin model made of this path's operators (Runtime::LoadModel), copies fp32 host data into its
// first input, runs it and copies up to two of its outputs (in the file's order) back: out_bytes[i] is the
// capacity on entry and the bytes written on return.  precision: 0 fp32.
int vkop_host_model_run(int device, const char *path, const float *host_input, size_t input_elements, void *out0,
                        size_t *out0_bytes, void *out1, size_t *out1_bytes, double *run_ms) {
    if (!path || !host_input)
        return VKOP_INVALID_ARG;
    try {
        const load::VkModel model(path);
        auto dev = std::make_shared<VulkanDevice>(device);
        auto pool = std::make_shared<VulkanCommandPool>(dev);
        core::Runtime rt(pool, path, 0);
        rt.LoadModel();
        auto in = core::as_tensor<float>(rt.GetInput());
        if (!in || static_cast<size_t>(in->num_elements()) != input_elements) {
            g_error = "vkop_host_model_run: the first input has another element count";
            return VKOP_INVALID_ARG;
        }
        in->copyToGPU(pool, host_input);
        const double t = rt.Run();
        if (run_ms)
            *run_ms = t;
        rt.ReadResult();
        void *dst[2] = {out0, out1};
        size_t *cap[2] = {out0_bytes, out1_bytes};
        for (size_t i = 0; i < model.outputs.size() && i < 2; i++) {
            if (!dst[i] || !cap[i])
                continue;
            auto t_out = rt.GetOutput(model.outputs[i].name);
            size_t bytes = 0;
            const void *src = nullptr;
            if (t_out->dtype() == typeid(float)) {
                auto tt = core::as_tensor<float>(t_out);
                bytes = static_cast<size_t>(tt->num_elements()) * sizeof(float);
                src = tt->data();
            } else if (t_out->dtype() == typeid(int)) {
                auto tt = core::as_tensor<int>(t_out);
                bytes = static_cast<size_t>(tt->num_elements()) * sizeof(int);
                src = tt->data();
            } else {
                g_error = "vkop_host_model_run: unsupported output type";
                return VKOP_UNSUPPORTED;
            }
            if (bytes > *cap[i]) {
                g_error = "vkop_host_model_run: output buffer too small";
                return VKOP_WORKSPACE_TOO_SMALL;
            }
            std::memcpy(dst[i], src, bytes);
            *cap[i] = bytes;
        }
        return VKOP_OK;
    } catch (const std::invalid_argument &e) {
        g_error = e.what();
        return VKOP_INVALID_ARG;
    } catch (const std::exception &e) {
        g_error = e.what();
        return VKOP_CUDA_ERROR;
    }
}

}  // extern "C"
