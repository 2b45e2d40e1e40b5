// Drives the operators through the C++ API the way the reference's tests do
// (tests/setup.hpp:129-202: create_from_type -> set_runtime_device ->
// setAttribute -> inputs to the GPU -> onExecute -> submit / wait -> copyToCPU
// -> compare), with the CPU oracle supplying the expectations instead of
// libtorch, and the way benchmark/main.cpp:85-118 uses the runtime.
// Exit code 0 = every case passed.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <functional>
#include <memory>

#include "core/runtime.hpp"
#include "ops/OperatorFactory.hpp"
#include "ops/SoftmaxTopkSharded.hpp"

extern "C" {
int oracle_softmax_topk(const void *logits, int dtype, int64_t rows, int64_t cols, int64_t row_stride, int k,
                        float inv_temperature, int value_kind, int sum_mode, int full_sort, float *out_values,
                        int64_t *out_indices);
int oracle_softmax(const void *x, int dtype, int64_t outer, int64_t axis_len, int64_t inner, float inv_temperature,
                   int sum_mode, float *out);
int oracle_topk(const void *x, int dtype, int64_t outer, int64_t axis_len, int64_t inner, int k, int largest, int sorted,
                float *out_values, int64_t *out_indices);
int oracle_nms(const float *boxes, const float *scores, int B, int C, int N, int center_point_box,
               int max_output_boxes_per_class, float iou_threshold, float score_threshold, int pre_topk, int32_t *out_rows,
               int64_t capacity_rows, int64_t *out_count, int32_t *per_problem_count);
}

using namespace vkop;
using core::ITensor;
using core::Tensor;

static int g_failures = 0;
#define EXPECT(cond, ...)                                   \
    do {                                                    \
        if (!(cond)) {                                      \
            std::printf("FAIL %s:%d: ", __FILE__, __LINE__); \
            std::printf(__VA_ARGS__);                       \
            std::printf("\n");                              \
            g_failures++;                                   \
        }                                                   \
    } while (0)

// deterministic N(0,1)-ish data (sum of uniforms), no dependency on a random library
struct Lcg {
    uint64_t s;
    explicit Lcg(uint64_t seed) : s(seed * 2862933555777941757ull + 3037000493ull) {}
    float uniform() {
        s = s * 6364136223846793005ull + 1442695040888963407ull;
        return static_cast<float>((s >> 40) & 0xFFFFFF) / 16777216.0f;
    }
    float normal() {
        float a = 0;
        for (int i = 0; i < 12; i++)
            a += uniform();
        return a - 6.0f;
    }
};

struct Env {
    std::shared_ptr<VulkanDevice> dev = std::make_shared<VulkanDevice>(0);
    std::shared_ptr<VulkanCommandPool> cmdpool = std::make_shared<VulkanCommandPool>(dev);
};

// tests/setup.hpp:129-202
static void run_op(Env &env, const std::string &name, std::vector<std::shared_ptr<ITensor>> inputs,
                   std::vector<std::shared_ptr<ITensor>> outputs,
                   const std::unordered_map<std::string, std::string> &attributes, std::unique_ptr<ops::Operator> *keep = nullptr) {
    auto op = ops::create_from_type(ops::convert_opstring_to_enum(name), inputs[0]->num_dims() <= 2, 0,
                                    env.dev->is_support_nv_tensor_core());
    if (!op) {
        EXPECT(false, "create_from_type(%s) returned null", name.c_str());
        return;
    }
    op->set_runtime_device(env.dev, env.cmdpool);
    op->setAttribute(attributes);
    for (auto &in : inputs) {
        if (in->dtype() == typeid(float)) {
            auto t = core::as_tensor<float>(in);
            t->as_storage_buffer(env.dev);
            t->copyToGPU(env.cmdpool);
        }
    }
    op->onExecute(inputs, outputs, 0);
    auto cmd = op->get_record();
    std::vector<VkSubmitInfo> info;
    info.push_back(cmd->buildSubmitInfo());
    VulkanCommandBuffer::submit(env.dev->getComputeQueue(), info);
    cmd->wait();
    env.dev->wait_all_done();
    if (keep)
        *keep = std::move(op);
}

static void test_topk(Env &env) {
    // tests/TopkTest.cpp:93-99
    const std::vector<std::tuple<std::vector<int>, int>> cases = {
        {{1, 200}, 7}, {{1, 400}, 8}, {{1, 600}, 7}, {{3, 2000}, 7}, {{1, 2000}, 6}};
    for (const auto &[shape, k] : cases) {
        Lcg rng(56);
        auto input = std::make_shared<Tensor<float>>(shape);
        for (int64_t i = 0; i < input->num_elements(); i++)
            (*input)[i] = rng.normal();
        auto values = std::make_shared<Tensor<float>>(true);
        auto indices = std::make_shared<Tensor<int>>(true);
        run_op(env, "TopK", {input}, {values, indices},
               {{"k", std::to_string(k)}, {"axis", "-1"}, {"largest", "1"}, {"sorted", "1"}});
        values->copyToCPU(env.cmdpool);
        indices->copyToCPU(env.cmdpool);
        EXPECT(values->getShape() == (std::vector<int>{shape[0], k}), "TopK output shape");
        std::vector<float> wv(static_cast<size_t>(shape[0]) * k);
        std::vector<int64_t> wi(wv.size());
        oracle_topk(input->data(), 0, shape[0], shape[1], 1, k, 1, 1, wv.data(), wi.data());
        for (size_t i = 0; i < wv.size(); i++) {
            EXPECT((*indices)[i] == static_cast<int>(wi[i]), "TopK index %zu: %d vs %lld", i, (*indices)[i], static_cast<long long>(wi[i]));
            EXPECT((*values)[i] == wv[i], "TopK value %zu", i);
        }
    }
}

static void test_topk_axis_and_order(Env &env) {
    // ops/Topk.hpp:62-79, 98-103: "axis" 0 .. 2 and "sorted"; expectation = the oracle's TopK on the same view
    struct Case {
        std::vector<int> shape;
        int axis, k, largest, sorted;
    };
    const std::vector<Case> cases = {{{3, 2000}, 0, 2, 1, 1},     {{3, 2000}, 0, 3, 0, 0},  {{4, 50, 33}, 1, 7, 1, 1},
                                     {{4, 50, 33}, 1, 7, 1, 0},   {{2, 300, 5}, -2, 9, 0, 1}, {{5, 64, 40}, 0, 3, 1, 0},
                                     {{3, 2000}, -1, 7, 1, 0},    {{2, 6, 1000}, 2, 11, 0, 0}};
    for (const auto &c : cases) {
        Lcg rng(77);
        auto input = std::make_shared<Tensor<float>>(c.shape);
        for (int64_t i = 0; i < input->num_elements(); i++)
            (*input)[i] = std::round(rng.normal() * 8.0f) / 8.0f;  // ties
        auto values = std::make_shared<Tensor<float>>(true);
        auto indices = std::make_shared<Tensor<int>>(true);
        run_op(env, "TopK", {input}, {values, indices},
               {{"k", std::to_string(c.k)}, {"axis", std::to_string(c.axis)}, {"largest", std::to_string(c.largest)},
                {"sorted", std::to_string(c.sorted)}});
        values->copyToCPU(env.cmdpool);
        indices->copyToCPU(env.cmdpool);
        const int rank = static_cast<int>(c.shape.size());
        const int axis = c.axis < 0 ? c.axis + rank : c.axis;
        std::vector<int> want_shape = c.shape;
        want_shape[axis] = c.k;
        EXPECT(values->getShape() == want_shape && indices->getShape() == want_shape, "TopK axis %d output shape", c.axis);
        int64_t outer = 1, inner = 1;
        for (int i = 0; i < axis; i++)
            outer *= c.shape[i];
        for (int i = axis + 1; i < rank; i++)
            inner *= c.shape[i];
        std::vector<float> wv(static_cast<size_t>(outer * inner * c.k));
        std::vector<int64_t> wi(wv.size());
        oracle_topk(input->data(), 0, outer, c.shape[axis], inner, c.k, c.largest, c.sorted, wv.data(), wi.data());
        for (size_t i = 0; i < wv.size(); i++) {
            EXPECT((*indices)[i] == static_cast<int>(wi[i]), "TopK axis %d sorted %d index %zu: %d vs %lld", c.axis, c.sorted, i,
                   (*indices)[i], static_cast<long long>(wi[i]));
            EXPECT((*values)[i] == wv[i], "TopK axis %d value %zu", c.axis, i);
        }
    }
}

static void test_softmax(Env &env) {
    // tests/SoftmaxTest.cpp:195-202
    const std::vector<std::tuple<std::vector<int>, int>> cases = {{{1, 10, 7, 7}, 1}, {{1, 6, 8, 8}, 3}, {{2, 4, 10, 10}, 2},
                                                                  {{1, 8, 6, 6}, 2},  {{1, 16, 5, 5}, 1}, {{4, 1000}, 1}};
    for (const auto &[shape, axis] : cases) {
        Lcg rng(42);
        auto input = std::make_shared<Tensor<float>>(shape);
        for (int64_t i = 0; i < input->num_elements(); i++)
            (*input)[i] = rng.normal();
        auto output = std::make_shared<Tensor<float>>(true);
        run_op(env, "Softmax", {input}, {output}, {{"dim", std::to_string(axis)}});
        output->copyToCPU(env.cmdpool);
        int64_t outer = 1, inner = 1;
        for (int i = 0; i < axis; i++)
            outer *= shape[i];
        for (size_t i = axis + 1; i < shape.size(); i++)
            inner *= shape[i];
        std::vector<float> want(static_cast<size_t>(input->num_elements()));
        oracle_softmax(input->data(), 0, outer, shape[axis], inner, 1.0f, 1, want.data());
        for (size_t i = 0; i < want.size(); i++)
            EXPECT(std::fabs((*output)[i] - want[i]) <= 1e-6f + 1e-5f * std::fabs(want[i]), "Softmax %zu: %g vs %g", i,
                   static_cast<double>((*output)[i]), static_cast<double>(want[i]));
    }
}

static void test_nms(Env &env) {
    // tests/NmsTest.cpp:181-185 (boxes built as in :40-56)
    const std::vector<std::tuple<int, int, int, int, float, float>> cases = {
        {1, 2, 10, 0, 0.5f, 0.5f}, {1, 1, 200, 50, 0.7f, 0.4f}, {1, 7, 50, 0, 0.3f, 0.2f}, {3, 5, 300, 20, 0.45f, 0.25f}};
    for (const auto &[B, C, N, max_per_class, iou_thr, score_thr] : cases) {
        Lcg rng(7);
        auto boxes = std::make_shared<Tensor<float>>(std::vector<int>{B, N, 4});
        auto scores = std::make_shared<Tensor<float>>(std::vector<int>{B, C, N});
        for (int64_t i = 0; i < scores->num_elements(); i++)
            (*scores)[i] = rng.uniform();
        for (int i = 0; i < B * N; i++) {
            const float cx = rng.uniform(), cy = rng.uniform(), w = rng.uniform() * 1.3f, h = rng.uniform() * 1.3f;
            auto clamp01 = [](float v) { return v < 0.0f ? 0.0f : (v > 1.0f ? 1.0f : v); };
            (*boxes)[i * 4 + 0] = clamp01(cx - w / 2);
            (*boxes)[i * 4 + 1] = clamp01(cy - h / 2);
            (*boxes)[i * 4 + 2] = clamp01(cx + w / 2);
            (*boxes)[i * 4 + 3] = clamp01(cy + h / 2);
        }
        auto out = std::make_shared<Tensor<int>>(true);
        std::unique_ptr<ops::Operator> op;
        run_op(env, "Nms", {boxes, scores}, {out},
               {{"max_output_boxes_per_class", std::to_string(max_per_class)},
                {"iou_threshold", std::to_string(iou_thr)},
                {"score_threshold", std::to_string(score_thr)}},
               &op);
        const int count = dynamic_cast<ops::Nms *>(op.get())->last_count();
        out->copyToCPU(env.cmdpool);
        std::vector<int32_t> want(static_cast<size_t>(B) * C * N * 3);
        int64_t total = 0;
        oracle_nms(boxes->data(), scores->data(), B, C, N, 0, max_per_class, iou_thr, score_thr, 0, want.data(), B * C * N, &total,
                   nullptr);
        EXPECT(count == total, "Nms count %d vs %lld", count, static_cast<long long>(total));
        for (int64_t i = 0; i < total * 3 && i < out->num_elements(); i++)
            EXPECT((*out)[i] == want[i], "Nms row value %lld", static_cast<long long>(i));
        if (total * 3 < out->num_elements())
            EXPECT((*out)[total * 3] == -1, "Nms: the row after the result must be (-1,-1,-1)");
        // the same problem as one detection head [B, 4 + C, N]: coordinate planes, then the score planes
        auto head = std::make_shared<Tensor<float>>(std::vector<int>{B, 4 + C, N});
        for (int b = 0; b < B; b++) {
            for (int q = 0; q < 4; q++)
                for (int i = 0; i < N; i++)
                    (*head)[(static_cast<int64_t>(b) * (4 + C) + q) * N + i] = (*boxes)[(static_cast<int64_t>(b) * N + i) * 4 + q];
            for (int c = 0; c < C; c++)
                for (int i = 0; i < N; i++)
                    (*head)[(static_cast<int64_t>(b) * (4 + C) + 4 + c) * N + i] = (*scores)[(static_cast<int64_t>(b) * C + c) * N + i];
        }
        auto out2 = std::make_shared<Tensor<int>>(true);
        std::unique_ptr<ops::Operator> op2;
        run_op(env, "Nms", {head}, {out2},
               {{"max_output_boxes_per_class", std::to_string(max_per_class)},
                {"iou_threshold", std::to_string(iou_thr)},
                {"score_threshold", std::to_string(score_thr)}},
               &op2);
        EXPECT(dynamic_cast<ops::Nms *>(op2.get())->last_count() == total, "Nms on a head: count");
        out2->copyToCPU(env.cmdpool);
        for (int64_t i = 0; i < total * 3 && i < out2->num_elements(); i++)
            EXPECT((*out2)[i] == want[i], "Nms on a head: row value %lld", static_cast<long long>(i));
    }
}

// benchmark/main.cpp:85-118 with a bound logits tensor in place of a model
static void test_runtime_pipeline(Env &env) {
    const int rows = 4, cols = 1000, k = 10;
    Lcg rng(3);
    std::vector<float> logits(static_cast<size_t>(rows) * cols);
    for (auto &v : logits)
        v = rng.normal() * 3.0f;
    std::vector<float> wv(static_cast<size_t>(rows) * k);
    std::vector<int64_t> wi(wv.size());
    oracle_softmax_topk(logits.data(), 0, rows, cols, cols, k, 1.0f, 0, 1, 0, wv.data(), wi.data());
    for (int fuse = 1; fuse >= 0; fuse--) {
        auto rt = std::make_shared<core::Runtime>(env.cmdpool, "", 0);
        auto cls_in = std::make_shared<Tensor<float>>(std::vector<int>{rows, cols});
        cls_in->fillToCPU(logits);
        cls_in->as_storage_buffer(env.dev);
        cls_in->copyToGPU(env.cmdpool);
        rt->BindOutput("logits", cls_in);
        rt->SetFusePostProcess(fuse != 0);
        auto cls = core::as_tensor<float>(rt->GetOutput());
        const auto shape = cls->getShape();
        auto sf = std::make_shared<Tensor<float>>(shape, true);
        rt->RegisterPostProcess(ops::OpType::SOFTMAX, {{"axis", "-1"}}, {cls}, {sf});
        auto indexs = std::make_shared<Tensor<int>>(shape, true);  // full shape, as the reference's caller allocates them
        auto values = std::make_shared<Tensor<float>>(shape, true);
        rt->RegisterPostProcess(ops::OpType::TOPK, {{"k", std::to_string(k)}}, {sf}, {values, indexs});
        double total = 0;
        for (int i = 0; i < 3; i++)
            total += rt->Run();
        rt->ReadResult();
        EXPECT(total > 0, "Run() must report a time");
        for (int r = 0; r < rows; r++) {
            for (int j = 0; j < k; j++) {
                const size_t o = static_cast<size_t>(r) * k + j;
                EXPECT((*indexs)[o] == static_cast<int>(wi[o]), "pipeline(fuse=%d) index row %d rank %d: %d vs %lld", fuse, r, j,
                       (*indexs)[o], static_cast<long long>(wi[o]));
                EXPECT(std::fabs((*values)[o] - wv[o]) <= 1e-6f + 1e-5f * std::fabs(wv[o]), "pipeline(fuse=%d) value row %d rank %d",
                       fuse, r, j);
            }
        }
    }
}

static void test_errors(Env &env) {
    EXPECT(ops::create_from_type(ops::OpType::CONV2D) == nullptr, "operators off the path are not created");
    EXPECT(ops::convert_opstring_to_enum("TopK") == ops::OpType::TOPK, "string -> type");
    EXPECT(ops::convert_optype_to_string(ops::OpType::NMS) == "Nms", "type -> string");
    EXPECT(static_cast<int>(ops::OpType::WHERE) == 40 && static_cast<int>(ops::OpType::SOFTMAX) == 26 &&
               static_cast<int>(ops::OpType::TOPK) == 30 && static_cast<int>(ops::OpType::NMS) == 32,
           "reference enumerator values are kept");
    auto input = std::make_shared<Tensor<float>>(std::vector<int>{2, 50});
    auto values = std::make_shared<Tensor<float>>(true);
    auto indices = std::make_shared<Tensor<int>>(true);
    bool threw = false;
    try {
        run_op(env, "TopK", {input}, {values, indices}, {{"k", "51"}});
    } catch (const std::invalid_argument &) {
        threw = true;
    }
    EXPECT(threw, "k > axis length must be rejected");
}

// The vocabulary-sharded operator, two ranks of this process on one device: each holds half the columns
// of the same logits; both must end with the k best of the whole row (softmax over all columns).
static void test_sharded(Env &) {
    const int rows = 16, cols = 40000, k = 10, world = 2;
    Lcg rng(77);
    std::vector<float> x(static_cast<size_t>(rows) * cols);
    for (auto &v : x)
        v = rng.normal() * 2.0f;
    std::vector<float> wv(static_cast<size_t>(rows) * k);
    std::vector<int64_t> wi(wv.size());
    oracle_softmax_topk(x.data(), 0, rows, cols, cols, k, 1.0f, 0, 0, 0, wv.data(), wi.data());
    const int half = cols / world;
    std::vector<std::unique_ptr<ops::SoftmaxTopkSharded>> ranks;
    std::vector<float *> d_logits(world), d_values(world);
    std::vector<int *> d_indices(world);
    for (int r = 0; r < world; r++) {
        ops::SoftmaxTopkSharded::Config c;
        c.rank = r;
        c.world = world;
        c.rows = rows;
        c.cols_local = half;
        c.col_offset = static_cast<int64_t>(r) * half;
        c.k = k;
        ranks.emplace_back(new ops::SoftmaxTopkSharded(c));
        cudaMalloc(&d_logits[r], sizeof(float) * rows * half);
        cudaMalloc(&d_values[r], sizeof(float) * rows * k);
        cudaMalloc(&d_indices[r], sizeof(int) * rows * k);
        cudaMemcpy2D(d_logits[r], sizeof(float) * half, x.data() + static_cast<size_t>(r) * half, sizeof(float) * cols,
                     sizeof(float) * half, rows, cudaMemcpyHostToDevice);
    }
    std::vector<ops::SoftmaxTopkSharded *> peers;
    for (auto &r : ranks)
        peers.push_back(r.get());
    for (auto &r : ranks)
        r->connect_local(peers.data());
    for (int step = 0; step < 3; step++) {
        for (int r = 0; r < world; r++)
            ranks[r]->begin(d_logits[r], nullptr);
        for (int r = 0; r < world; r++)
            ranks[r]->finish(d_values[r], d_indices[r], nullptr);
    }
    cudaDeviceSynchronize();
    for (int r = 0; r < world; r++) {
        EXPECT(!ranks[r]->timed_out(), "sharded rank %d: a wait gave up", r);
        std::vector<float> v(wv.size());
        std::vector<int> idx(wv.size());
        cudaMemcpy(v.data(), d_values[r], sizeof(float) * v.size(), cudaMemcpyDeviceToHost);
        cudaMemcpy(idx.data(), d_indices[r], sizeof(int) * idx.size(), cudaMemcpyDeviceToHost);
        for (size_t i = 0; i < v.size(); i++) {
            EXPECT(idx[i] == static_cast<int>(wi[i]), "sharded rank %d index %zu: %d vs %lld", r, i, idx[i], static_cast<long long>(wi[i]));
            EXPECT(std::fabs(v[i] - wv[i]) <= 1e-6f + 1e-5f * std::fabs(wv[i]), "sharded rank %d value %zu: %g vs %g", r, i, v[i], wv[i]);
        }
        cudaFree(d_logits[r]);
        cudaFree(d_values[r]);
        cudaFree(d_indices[r]);
    }
    bool threw = false;
    try {
        ops::SoftmaxTopkSharded::Config c;
        c.world = 2;
        c.rank = 2;
        c.rows = 1;
        c.cols_local = 10;
        ops::SoftmaxTopkSharded bad(c);
    } catch (const std::invalid_argument &) {
        threw = true;
    }
    EXPECT(threw, "a rank outside the world must be rejected");
}

int main() {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
        std::printf("no CUDA device\n");
        return 2;
    }
    Env env;
    std::printf("device: %s\n", env.dev->getDeviceName().c_str());
    test_topk(env);
    test_topk_axis_and_order(env);
    test_softmax(env);
    test_nms(env);
    test_runtime_pipeline(env);
    test_errors(env);
    test_sharded(env);
    std::printf(g_failures ? "%d FAILURES\n" : "all operator API cases passed\n", g_failures);
    return g_failures ? 1 : 0;
}
