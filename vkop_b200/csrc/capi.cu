// C ABI: argument validation and dispatch.  Declared in include/vkop_cuda.h.
#include <atomic>
#include <cmath>
#include <mutex>

#include "common.cuh"
#include "launchers.h"

namespace vkop_cuda {

static std::atomic<uint64_t> g_launches{0};
void note_launch(int n) { g_launches.fetch_add(static_cast<uint64_t>(n), std::memory_order_relaxed); }

static int validate_select(const vkop_softmax_topk_desc *d, bool check_ptrs, const void *in, bool need_outputs,
                           const void *ov, const void *oi) {
    if (!d)
        return VKOP_INVALID_ARG;
    if (d->rows < 0 || d->cols < 1 || d->k < 1 || d->k > d->cols || d->k > kMaxK)
        return VKOP_INVALID_ARG;
    if (d->dtype != VKOP_F32 && d->dtype != VKOP_F16 && d->dtype != VKOP_BF16)
        return VKOP_INVALID_ARG;
    if (d->index_dtype != VKOP_I32 && d->index_dtype != VKOP_I64)
        return VKOP_INVALID_ARG;
    if (d->value_kind != VKOP_VALUE_PROBABILITY && d->value_kind != VKOP_VALUE_RAW)
        return VKOP_INVALID_ARG;
    if (!(d->inv_temperature > 0.0f) || !std::isfinite(d->inv_temperature))
        return VKOP_INVALID_ARG;
    if (d->row_stride != 0 && d->row_stride < d->cols)
        return VKOP_INVALID_ARG;
    if (d->path < VKOP_PATH_AUTO || d->path > VKOP_PATH_BULK || d->splits < 0)
        return VKOP_INVALID_ARG;
    if (d->index_offset < 0 || d->index_offset + d->cols > 0xFFFFFFFFll)
        return VKOP_INVALID_ARG;
    if (d->index_dtype == VKOP_I32 && d->index_offset + d->cols > 0x7FFFFFFFll)
        return VKOP_INVALID_ARG;
    if (check_ptrs && d->rows > 0) {
        if (!in || (need_outputs && (!ov || !oi)))
            return VKOP_INVALID_ARG;
        const size_t esz = d->dtype == VKOP_F32 ? 4 : 2;
        if (reinterpret_cast<uintptr_t>(in) % esz != 0)
            return VKOP_INVALID_ARG;
    }
    return VKOP_OK;
}

// Chooses the path and sizes the scratch memory.
// `in` is the logits pointer, or null for a size query (then the larger of the aligned / unaligned plans counts).
static int plan_select(const vkop_softmax_topk_desc &d, const void *in, SelectPlan *plan) {
    int rc = VKOP_UNSUPPORTED;
    const int64_t row_bytes = d.cols * (d.dtype == VKOP_F32 ? 4 : 2);
    // rows longer than one CTA's register tile, and enough of them: the streaming kernel
    // (several hundred rows of 32 KB and more also stream: one light CTA per row fills the GPU in one wave)
    const bool one_wave = d.rows >= 2 * 148 && d.rows <= 4 * 148 && row_bytes >= 32 * 1024;
    const bool prefer_stream = (row_bytes > 64 * 1024 || one_wave) && d.rows * row_bytes >= (2ll << 20);
    if (d.path == VKOP_PATH_STREAM || d.path == VKOP_PATH_BULK || (d.path == VKOP_PATH_AUTO && prefer_stream && d.splits == 0)) {
        // Two implementations serve this kind: the cp.async kernel (any alignment) and the bulk-copy
        // kernels (16-byte aligned long rows).  Both number their calls in one shared head of the
        // workspace, and each has its own part behind it.
        const bool base_aligned = reinterpret_cast<uintptr_t>(in) % 16 == 0;
        // (the bulk-copy kernels are chosen by name only: measured, they do not beat the cp.async kernel yet)
        const bool want_bulk = d.path == VKOP_PATH_BULK, want_stream = d.path != VKOP_PATH_BULK;
        const int rcb = want_bulk ? plan_bulk(d, in ? base_aligned : true, &plan->bulk) : VKOP_UNSUPPORTED;
        size_t stream_bytes = 0;
        rc = want_stream ? plan_stream(d, base_aligned, &plan->stream) : VKOP_UNSUPPORTED;
        if (rc == VKOP_OK) {
            stream_bytes = plan->stream.counters_bytes + plan->stream.lists_bytes;
            StreamPlan other;
            if (plan_stream(d, !base_aligned, &other) == VKOP_OK && other.counters_bytes + other.lists_bytes > stream_bytes)
                stream_bytes = other.counters_bytes + other.lists_bytes;
        }
        if (rc == VKOP_OK || rcb == VKOP_OK) {
            plan->kind = kSelectStream;
            plan->use_bulk = rcb == VKOP_OK;
            const size_t bulk_bytes = rcb == VKOP_OK ? plan->bulk.scratch_bytes : 0;
            plan->bulk_off = stream_common_bytes(d.rows);
            plan->stream_off = plan->bulk_off + bulk_bytes;
            plan->bytes = plan->stream_off + stream_bytes;
            return VKOP_OK;
        }
        if (d.path == VKOP_PATH_STREAM || d.path == VKOP_PATH_BULK)
            return d.path == VKOP_PATH_BULK ? rcb : rc;
    }
    if (d.path != VKOP_PATH_RADIX)
        rc = plan_chunk(d, &plan->chunk);
    if (rc == VKOP_OK) {
        plan->kind = kSelectChunk;
        plan->bytes = plan->chunk.counters_bytes + plan->chunk.packets_bytes;
        return VKOP_OK;
    }
    if (d.path == VKOP_PATH_CHUNK)
        return rc;
    plan->kind = kSelectRadix;
    rc = plan_radix(d, &plan->radix);
    if (rc == VKOP_OK)
        plan->bytes = plan->radix.bytes;
    return rc;
}

static int run_select(const vkop_softmax_topk_desc &d, const void *in, void *ov, void *oi, void *packets_out,
                      void *ws, size_t ws_bytes, int need_sum, void *stream) {
    SelectPlan plan;
    int rc = plan_select(d, in, &plan);
    if (rc != VKOP_OK)
        return rc;
    if (plan.bytes > 0 && (!ws || ws_bytes < plan.bytes))
        return VKOP_WORKSPACE_TOO_SMALL;
    if (plan.bytes > 0 && reinterpret_cast<uintptr_t>(ws) % 16 != 0)
        return VKOP_INVALID_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (plan.kind) {
    case kSelectStream:
        if (plan.use_bulk)
            return launch_bulk(d, plan.bulk, in, ov, oi, packets_out, ws, static_cast<char *>(ws) + plan.bulk_off, need_sum, s);
        return launch_stream(d, plan.stream, in, ov, oi, packets_out, ws, static_cast<char *>(ws) + plan.stream_off, need_sum, s);
    case kSelectRadix: return launch_radix(d, plan.radix, in, ov, oi, packets_out, ws, need_sum, s);
    default: return launch_chunk(d, plan.chunk, in, ov, oi, packets_out, ws, need_sum, s);
    }
}

}  // namespace vkop_cuda

using namespace vkop_cuda;

// see vkop_cuda_workspace_init
static __global__ void workspace_ready_kernel() {}

extern "C" {

int vkop_cuda_version(void) { return VKOP_CUDA_VERSION; }

const char *vkop_cuda_status_string(int status) {
    switch (status) {
    case VKOP_OK: return "VKOP_OK";
    case VKOP_INVALID_ARG: return "VKOP_INVALID_ARG";
    case VKOP_UNSUPPORTED: return "VKOP_UNSUPPORTED";
    case VKOP_WORKSPACE_TOO_SMALL: return "VKOP_WORKSPACE_TOO_SMALL";
    case VKOP_CUDA_ERROR: return "VKOP_CUDA_ERROR";
    case VKOP_TIMEOUT: return "VKOP_TIMEOUT";
    default: return "VKOP_UNKNOWN_STATUS";
    }
}

uint64_t vkop_cuda_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int vkop_cuda_workspace_init(void *workspace, size_t bytes, void *stream) {
    if (bytes == 0)
        return VKOP_OK;
    if (!workspace)
        return VKOP_INVALID_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (cudaMemsetAsync(workspace, 0, bytes, s) != cudaSuccess)
        return VKOP_CUDA_ERROR;
    // A kernel launched with programmatic stream serialization that does not wait for its predecessor
    // (a call with VKOP_FLAG_INPUT_READY) may start as soon as that predecessor's blocks have ended,
    // before its writes are flushed.  With this empty kernel behind the clearing, such a call's
    // predecessor is a kernel that wrote nothing and that itself started after the cleared bytes were
    // visible: the call reads zeros, not what the memory held before.
    workspace_ready_kernel<<<1, 32, 0, s>>>();
    return cudaGetLastError() == cudaSuccess ? VKOP_OK : VKOP_CUDA_ERROR;
}

int vkop_cuda_softmax_topk_workspace(const vkop_softmax_topk_desc *desc, size_t *bytes) {
    if (!bytes)
        return VKOP_INVALID_ARG;
    int rc = validate_select(desc, false, nullptr, false, nullptr, nullptr);
    if (rc != VKOP_OK)
        return rc;
    SelectPlan plan;
    rc = plan_select(*desc, nullptr, &plan);
    if (rc != VKOP_OK)
        return rc;
    *bytes = plan.bytes;
    return VKOP_OK;
}

int vkop_cuda_softmax_topk(const vkop_softmax_topk_desc *desc, const void *logits, void *out_values,
                           void *out_indices, void *workspace, size_t workspace_bytes, void *stream) {
    int rc = validate_select(desc, true, logits, true, out_values, out_indices);
    if (rc != VKOP_OK)
        return rc;
    if (!desc->largest && desc->value_kind != VKOP_VALUE_RAW)
        return VKOP_UNSUPPORTED;  // "smallest" is a TopK attribute; softmax of the smallest is not a reference path
    return run_select(*desc, logits, out_values, out_indices, nullptr, workspace, workspace_bytes,
                      desc->value_kind == VKOP_VALUE_PROBABILITY, stream);
}

int vkop_cuda_topk(const vkop_softmax_topk_desc *desc, const void *input, void *out_values, void *out_indices,
                   void *workspace, size_t workspace_bytes, void *stream) {
    int rc = validate_select(desc, true, input, true, out_values, out_indices);
    if (rc != VKOP_OK)
        return rc;
    vkop_softmax_topk_desc d = *desc;
    d.value_kind = VKOP_VALUE_RAW;
    return run_select(d, input, out_values, out_indices, nullptr, workspace, workspace_bytes, 0, stream);
}

// The last-axis selection behind vkop_cuda_topk_axis: rows = outer * inner, raw values, 32-bit indices.
static int topk_axis_select_desc(const vkop_topk_axis_desc *a, vkop_softmax_topk_desc *d) {
    if (!a)
        return VKOP_INVALID_ARG;
    if (a->outer < 0 || a->inner < 0 || a->axis_len < 1 || a->axis_len > 0x7FFFFFFFll)
        return VKOP_INVALID_ARG;
    if (a->outer > 0 && a->inner > 0x7FFFFFFFll / a->outer)
        return VKOP_UNSUPPORTED;
    *d = vkop_softmax_topk_desc{};
    d->rows = a->outer * a->inner;
    d->cols = a->axis_len;
    d->dtype = a->dtype;
    d->k = a->k;
    d->index_dtype = VKOP_I32;
    d->value_kind = VKOP_VALUE_RAW;
    d->inv_temperature = 1.0f;
    d->largest = a->largest ? 1 : 0;
    d->path = a->path;
    if (a->index_dtype != VKOP_I32 && a->index_dtype != VKOP_I64)
        return VKOP_INVALID_ARG;
    return validate_select(d, false, nullptr, false, nullptr, nullptr);
}

int vkop_cuda_topk_axis_workspace(const vkop_topk_axis_desc *desc, size_t *bytes) {
    if (!bytes)
        return VKOP_INVALID_ARG;
    vkop_softmax_topk_desc d;
    int rc = topk_axis_select_desc(desc, &d);
    if (rc != VKOP_OK)
        return rc;
    SelectPlan plan;
    rc = plan_select(d, nullptr, &plan);
    if (rc != VKOP_OK)
        return rc;
    *bytes = topk_axis_transposed_bytes(*desc) + topk_axis_values_bytes(*desc) + topk_axis_indices_bytes(*desc) +
             (plan.bytes + 255) / 256 * 256;
    return VKOP_OK;
}

int vkop_cuda_topk_axis(const vkop_topk_axis_desc *desc, const void *input, void *out_values, void *out_indices,
                        void *workspace, size_t workspace_bytes, void *stream) {
    vkop_softmax_topk_desc d;
    int rc = topk_axis_select_desc(desc, &d);
    if (rc != VKOP_OK)
        return rc;
    if (d.rows == 0)
        return VKOP_OK;
    if (!input || !out_values || !out_indices)
        return VKOP_INVALID_ARG;
    const size_t esz = d.dtype == VKOP_F32 ? 4 : 2;
    if (reinterpret_cast<uintptr_t>(input) % esz != 0 || reinterpret_cast<uintptr_t>(out_values) % esz != 0 ||
        reinterpret_cast<uintptr_t>(out_indices) % (desc->index_dtype == VKOP_I64 ? 8 : 4) != 0)
        return VKOP_INVALID_ARG;
    size_t need = 0;
    rc = vkop_cuda_topk_axis_workspace(desc, &need);
    if (rc != VKOP_OK)
        return rc;
    if (!workspace || workspace_bytes < need)
        return VKOP_WORKSPACE_TOO_SMALL;
    if (reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
        return VKOP_INVALID_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    char *turned = static_cast<char *>(workspace);
    char *vals = turned + topk_axis_transposed_bytes(*desc);
    char *idx = vals + topk_axis_values_bytes(*desc);
    char *select_ws = idx + topk_axis_indices_bytes(*desc);
    const size_t select_bytes = need - static_cast<size_t>(select_ws - turned);
    const void *rows_in = input;
    if (desc->inner > 1) {
        rc = launch_transpose_axis(*desc, input, turned, s);
        if (rc != VKOP_OK)
            return rc;
        rows_in = turned;
    }
    // the scratch sizes were planned for an aligned input; the turned copy is, the caller's tensor may not be
    SelectPlan plan;
    rc = plan_select(d, rows_in, &plan);
    if (rc != VKOP_OK)
        return rc;
    if (plan.bytes > select_bytes)
        return VKOP_WORKSPACE_TOO_SMALL;
    rc = run_select(d, rows_in, vals, idx, nullptr, select_ws, select_bytes, 0, stream);
    if (rc != VKOP_OK)
        return rc;
    return launch_place_results(*desc, vals, idx, out_values, out_indices, s);
}

size_t vkop_cuda_packet_bytes(int32_t k) { return k > 0 ? static_cast<size_t>(packet_words(k)) * 4 : 0; }

int vkop_cuda_softmax_topk_partial(const vkop_softmax_topk_desc *desc, const void *logits_shard, void *packets_out,
                                   void *workspace, size_t workspace_bytes, void *stream) {
    int rc = validate_select(desc, true, logits_shard, false, nullptr, nullptr);
    if (rc != VKOP_OK)
        return rc;
    if (desc->rows > 0 && !packets_out)
        return VKOP_INVALID_ARG;
    if (!desc->largest)
        return VKOP_UNSUPPORTED;
    vkop_softmax_topk_desc d = *desc;
    d.value_kind = VKOP_VALUE_PROBABILITY;
    return run_select(d, logits_shard, nullptr, nullptr, packets_out, workspace, workspace_bytes, 1, stream);
}

int vkop_cuda_softmax_topk_merge(const vkop_softmax_topk_desc *desc, const void *packets, int32_t shards,
                                 void *out_values, void *out_indices, void *stream) {
    if (!desc || shards < 1)
        return VKOP_INVALID_ARG;
    if (desc->rows < 0 || desc->k < 1 || desc->k > kMaxK)
        return VKOP_INVALID_ARG;
    if (desc->dtype != VKOP_F32 && desc->dtype != VKOP_F16 && desc->dtype != VKOP_BF16)
        return VKOP_INVALID_ARG;
    if (desc->index_dtype != VKOP_I32 && desc->index_dtype != VKOP_I64)
        return VKOP_INVALID_ARG;
    if (!(desc->inv_temperature > 0.0f) || !std::isfinite(desc->inv_temperature))
        return VKOP_INVALID_ARG;
    if (desc->rows > 0 && (!packets || !out_values || !out_indices))
        return VKOP_INVALID_ARG;
    return launch_merge(*desc, packets, shards, out_values, out_indices, static_cast<cudaStream_t>(stream));
}

int vkop_cuda_softmax(const vkop_softmax_desc *desc, const void *input, void *output, void *stream) {
    if (!desc || desc->outer < 0 || desc->axis_len < 1 || desc->inner < 1)
        return VKOP_INVALID_ARG;
    if (desc->dtype != VKOP_F32 && desc->dtype != VKOP_F16 && desc->dtype != VKOP_BF16)
        return VKOP_INVALID_ARG;
    if (!(desc->inv_temperature > 0.0f) || !std::isfinite(desc->inv_temperature))
        return VKOP_INVALID_ARG;
    if (desc->outer > 0 && (!input || !output))
        return VKOP_INVALID_ARG;
    return launch_softmax(*desc, input, output, static_cast<cudaStream_t>(stream));
}

int vkop_cuda_nms_workspace(const vkop_nms_desc *desc, size_t *bytes) {
    if (!desc || !bytes)
        return VKOP_INVALID_ARG;
    return plan_nms(*desc, bytes);
}

int vkop_cuda_nms(const vkop_nms_desc *desc, const void *boxes, const void *scores, int32_t *out_rows,
                  int32_t *out_count, void *workspace, size_t workspace_bytes, void *stream) {
    if (!desc || !out_count)
        return VKOP_INVALID_ARG;
    size_t need = 0;
    int rc = plan_nms(*desc, &need);
    if (rc != VKOP_OK)
        return rc;
    const int64_t problems = static_cast<int64_t>(desc->num_batch) * desc->num_class;
    if (problems > 0 && desc->num_boxes > 0 && (!boxes || !scores))
        return VKOP_INVALID_ARG;
    if (desc->capacity_rows > 0 && !out_rows)
        return VKOP_INVALID_ARG;
    if (need > 0 && (!workspace || workspace_bytes < need))
        return VKOP_WORKSPACE_TOO_SMALL;
    return launch_nms(*desc, boxes, scores, out_rows, out_count, workspace, static_cast<cudaStream_t>(stream));
}

int vkop_cuda_yolo_nms(const vkop_nms_desc *desc, const void *head, int32_t *out_rows, int32_t *out_count,
                       void *workspace, size_t workspace_bytes, void *stream) {
    if (!desc || !out_count)
        return VKOP_INVALID_ARG;
    size_t need = 0;
    int rc = plan_nms(*desc, &need);
    if (rc != VKOP_OK)
        return rc;
    const int64_t problems = static_cast<int64_t>(desc->num_batch) * desc->num_class;
    if (problems > 0 && desc->num_boxes > 0 && !head)
        return VKOP_INVALID_ARG;
    if (desc->capacity_rows > 0 && !out_rows)
        return VKOP_INVALID_ARG;
    if (need > 0 && (!workspace || workspace_bytes < need))
        return VKOP_WORKSPACE_TOO_SMALL;
    // head [B, 4 + C, N]: four coordinate planes, then one score plane per class
    const int64_t n = desc->num_boxes, plane = (4 + static_cast<int64_t>(desc->num_class)) * n;
    const float *h = static_cast<const float *>(head);
    return launch_nms(*desc, h, h + 4 * n, out_rows, out_count, workspace, static_cast<cudaStream_t>(stream), plane, plane, n);
}

int vkop_cuda_sample_topk(const void *values, int32_t dtype, const void *indices, int32_t index_dtype, int64_t rows,
                          int32_t k, float top_p, const float *u, int32_t *out_choice, void *out_token, void *stream) {
    if (rows < 0 || k < 1 || k > 4096 || !(top_p > 0.0f) || (index_dtype != VKOP_I32 && index_dtype != VKOP_I64))
        return VKOP_INVALID_ARG;
    if (rows > 0 && (!values || !indices || !u || !out_choice || !out_token))
        return VKOP_INVALID_ARG;
    return launch_sample_topk(values, dtype, indices, index_dtype, rows, k, top_p, u, out_choice, out_token,
                              static_cast<cudaStream_t>(stream));
}

int vkop_cuda_packets_push(const void *packets, size_t packets_bytes, void *const *peer_slots, void *const *peer_flags,
                           int32_t rank, int32_t world, uint32_t seq, void *tickets, void *stream) {
    if (!packets || !peer_slots || !peer_flags || !tickets || world < 1 || world > 1024 || rank < 0 || rank >= world ||
        seq == 0 || packets_bytes % 4 != 0)
        return VKOP_INVALID_ARG;
    return launch_packets_push(packets, packets_bytes, peer_slots, peer_flags, rank, world, seq, tickets,
                               static_cast<cudaStream_t>(stream));
}

int vkop_cuda_packets_wait(const void *flags, int32_t world, uint32_t seq, uint32_t max_polls, int32_t *status,
                           void *stream) {
    if (!flags || !status || world < 1 || world > 1024 || seq == 0 || max_polls == 0)
        return VKOP_INVALID_ARG;
    return launch_packets_wait(flags, world, seq, max_polls, status, static_cast<cudaStream_t>(stream));
}

int vkop_cuda_packets_exchange_all_ranks(const void *const *packets_of, size_t packets_bytes, void *const *peer_slots,
                                         void *const *peer_flags, int32_t world, uint32_t seq, void *const *tickets_of,
                                         uint32_t max_polls, int32_t *status, void *stream) {
    if (!packets_of || !peer_slots || !peer_flags || !tickets_of || !status || world < 1 || world > 32 || seq == 0 ||
        max_polls == 0 || packets_bytes % 4 != 0)
        return VKOP_INVALID_ARG;
    return launch_packets_exchange_all_ranks(packets_of, packets_bytes, peer_slots, peer_flags, world, seq, tickets_of, max_polls,
                                             status, static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------
// Fused Softmax + TopK without a caller workspace.
//
// Some callers cannot hand over scratch memory.  An operator plugged into
// somebody else's runtime is typically given its input and output tensors and
// a stream and nothing else, and has no hook to ask the host application for
// a buffer; and code on a latency-critical or memory-budgeted path must not
// call the allocator when it runs, because cudaMalloc synchronises the whole
// device and can fail once memory is fragmented or used up.  For them the
// chunk kernel of this library can work in a fixed array that is part of the
// loaded module: kStaticScratchBytes of device memory per device that uses
// this entry point, present from module load to unload.
//
// What follows from that, for the caller:
//   - nothing is allocated or freed, on the host or on the device, ever;
//   - only descriptors whose scratch need fits the array are served
//     (VKOP_WORKSPACE_TOO_SMALL otherwise; vkop_cuda_static_scratch_bytes()
//     tells the size), and only on the chunk path (path AUTO or CHUNK);
//   - the first call on a device looks the array's device address up
//     (cudaGetSymbolAddress, with that device current) and should therefore
//     come before any stream capture on that device;
//   - all calls on a device share the one array and it keeps what the last
//     call left there: every call first clears the few hundred bytes of
//     counters its launch shape uses, on the call's stream (no allocation),
//     whatever ran before.  Calls that overlap on the GPU
//     (different streams without an ordering between them) race on the array:
//     give them an order, or use the workspace entry point.
namespace {
constexpr size_t kStaticScratchBytes = 4u << 20;
constexpr int kStaticMaxDevices = 64;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// device address of g_static_scratch per device (not the host-side symbol), looked up once
void *g_static_ptr[kStaticMaxDevices] = {};
std::mutex g_static_mutex;
}  // namespace

size_t vkop_cuda_static_scratch_bytes(void) { return kStaticScratchBytes; }

int vkop_cuda_softmax_topk_static(const vkop_softmax_topk_desc *desc, const void *logits, void *out_values,
                                  void *out_indices, void *stream) {
    if (!desc)
        return VKOP_INVALID_ARG;
    if (desc->path != VKOP_PATH_AUTO && desc->path != VKOP_PATH_CHUNK)
        return VKOP_UNSUPPORTED;
    vkop_softmax_topk_desc d = *desc;
    d.path = VKOP_PATH_CHUNK;
    size_t need = 0;
    int rc = vkop_cuda_softmax_topk_workspace(&d, &need);
    if (rc != VKOP_OK)
        return rc;
    if (need > kStaticScratchBytes)
        return VKOP_WORKSPACE_TOO_SMALL;  // this shape needs more scratch than the built-in array holds
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess)
        return VKOP_CUDA_ERROR;
    if (dev < 0 || dev >= kStaticMaxDevices)
        return VKOP_UNSUPPORTED;
    void *ptr = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_static_mutex);
        if (!g_static_ptr[dev]) {
            // once per device, with that device current: the symbol's address on THIS device
            void *p = nullptr;
            if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || !p) {
                cudaGetLastError();
                return VKOP_CUDA_ERROR;
            }
            g_static_ptr[dev] = p;
        }
        ptr = g_static_ptr[dev];
    }
    // The counters of this launch shape must start at zero and the array holds whatever the last
    // call (of any shape, finished or failed) left: clear them every time.  The lists behind them
    // are written before they are read.
    SelectPlan plan;
    rc = plan_select(d, logits, &plan);
    if (rc != VKOP_OK)
        return rc;
    if (plan.kind != kSelectChunk)
        return VKOP_UNSUPPORTED;
    if (plan.chunk.counters_bytes > 0 &&
        cudaMemsetAsync(ptr, 0, plan.chunk.counters_bytes, static_cast<cudaStream_t>(stream)) != cudaSuccess) {
        cudaGetLastError();
        return VKOP_CUDA_ERROR;
    }
    return vkop_cuda_softmax_topk(&d, logits, out_values, out_indices, ptr, kStaticScratchBytes, stream);
}

}  // extern "C"
