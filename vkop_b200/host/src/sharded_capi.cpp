// Flat C entry points over ops::SoftmaxTopkSharded (the vocabulary-sharded fused
// Softmax + TopK of one rank), for callers that cannot include C++ headers: the
// Python harness passes the 64-byte IPC handles through its process group and
// calls these.  Every function returns 0 or a negative vkop_status (the text
// of the failure through vkop_host_last_error); nothing throws across the
// boundary.  No counterpart in the reference, which runs on one device
// (benchmark/main.cpp:49-50).
#include <exception>
#include <string>

#include "ops/SoftmaxTopkSharded.hpp"

using vkop::ops::SoftmaxTopkSharded;

extern "C" void vkop_host_set_error(const char *text);  // host_capi.cpp

namespace {
template <typename F>
int guarded(F &&f) {
    try {
        f();
        return VKOP_OK;
    } catch (const std::invalid_argument &e) {
        vkop_host_set_error(e.what());
        return VKOP_INVALID_ARG;
    } catch (const std::exception &e) {
        vkop_host_set_error(e.what());
        return VKOP_CUDA_ERROR;
    }
}
}  // namespace

extern "C" {

// One rank of a vocabulary-sharded step on `device`.  dtype / index_dtype: vkop_dtype / vkop_index_dtype.
void *vkop_host_sharded_create(int device, int rank, int world, int64_t rows, int64_t cols_local, int64_t col_offset, int k, int dtype,
                               int index_dtype, float inv_temperature, unsigned max_polls) {
    SoftmaxTopkSharded *h = nullptr;
    guarded([&] {
        SoftmaxTopkSharded::Config c;
        c.device = device;
        c.rank = rank;
        c.world = world;
        c.rows = rows;
        c.cols_local = cols_local;
        c.col_offset = col_offset;
        c.k = k;
        c.dtype = dtype;
        c.index_dtype = index_dtype;
        c.inv_temperature = inv_temperature;
        if (max_polls)
            c.max_polls = max_polls;
        h = new SoftmaxTopkSharded(c);
    });
    return h;
}

void vkop_host_sharded_destroy(void *h) { delete static_cast<SoftmaxTopkSharded *>(h); }

// out64: the 64-byte CUDA IPC handle of this rank's receive buffer.
int vkop_host_sharded_ipc_handle(void *h, void *out64) {
    return guarded([&] { static_cast<SoftmaxTopkSharded *>(h)->ipc_handle(out64); });
}

// handles: world x 64 bytes in rank order, as gathered from all ranks.
int vkop_host_sharded_connect(void *h, const void *handles) {
    return guarded([&] { static_cast<SoftmaxTopkSharded *>(h)->connect(handles); });
}

// peers: `world` objects of this process in rank order (ranks of one process).
int vkop_host_sharded_connect_local(void *h, void *const *peers) {
    return guarded([&] { static_cast<SoftmaxTopkSharded *>(h)->connect_local(reinterpret_cast<SoftmaxTopkSharded *const *>(peers)); });
}

// partial + push on `stream` (a cudaStream_t).
int vkop_host_sharded_begin(void *h, const void *logits_local, void *stream) {
    return guarded([&] { static_cast<SoftmaxTopkSharded *>(h)->begin(logits_local, static_cast<cudaStream_t>(stream)); });
}

// bounded wait + merge on `stream`.
int vkop_host_sharded_finish(void *h, void *out_values, void *out_indices, void *stream) {
    return guarded([&] { static_cast<SoftmaxTopkSharded *>(h)->finish(out_values, out_indices, static_cast<cudaStream_t>(stream)); });
}

int vkop_host_sharded_run(void *h, const void *logits_local, void *out_values, void *out_indices, void *stream) {
    return guarded([&] { static_cast<SoftmaxTopkSharded *>(h)->run(logits_local, out_values, out_indices, static_cast<cudaStream_t>(stream)); });
}

// After a synchronisation: *timed_out = 1 when a bounded wait ever gave up.
int vkop_host_sharded_timed_out(void *h, int *timed_out) {
    return guarded([&] { *timed_out = static_cast<SoftmaxTopkSharded *>(h)->timed_out() ? 1 : 0; });
}

}  // extern "C"
