// Internal interface between the C ABI (capi.cu) and the kernel files.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "vkop_cuda.h"

namespace vkop_cuda {

constexpr int kMaxK = 4096;  // largest k any path serves

// ---- chunk path (softmax_topk.cu) ----
struct ChunkPlan {
    int cfg;
    int splits;
    int64_t vps;
    int list_cap;  // candidates one chunk may publish when a row has several chunks
    size_t counters_bytes, packets_bytes, smem_bytes;
};
int plan_chunk(const vkop_softmax_topk_desc &d, ChunkPlan *plan);
int launch_chunk(const vkop_softmax_topk_desc &d, const ChunkPlan &plan, const void *logits, void *out_values,
                 void *out_indices, void *packets_out, void *workspace, int need_sum, cudaStream_t stream);
int launch_merge(const vkop_softmax_topk_desc &d, const void *packets, int shards, void *out_values,
                 void *out_indices, cudaStream_t stream);

// ---- streaming path (softmax_topk_stream.cu) ----
struct StreamPlan {
    int grid;
    int64_t per_cta, nvv, vstride;
    int maxparts, list_cap, parts_per_row, aligned, cluster, threads;
    int deep;  // whole rows of overlapping calls: smaller tiles, more of them in flight
    size_t counters_bytes, lists_bytes, smem_bytes;
};
// base_aligned: the logits pointer is a multiple of 16 (rows then are too when the row stride is)
int plan_stream(const vkop_softmax_topk_desc &d, bool base_aligned, StreamPlan *plan);
// common_ws: the shared head of the workspace (stream_common_bytes); workspace: this kernel's own part
int launch_stream(const vkop_softmax_topk_desc &d, const StreamPlan &plan, const void *logits, void *out_values,
                  void *out_indices, void *packets_out, void *common_ws, void *workspace, int need_sum, cudaStream_t stream);

// ---- bulk-copy streaming path (softmax_topk_bulk.cu): long, 16-byte aligned rows ----
struct BulkPlan {
    int grid;      // CTAs of the streaming kernel: rows * parts
    int parts;     // parts (CTAs) per row
    int64_t nvv, vstride;
    size_t scratch_bytes, smem_bytes;
};
// Head of a workspace of the streaming kernels, shared by all of them: call counters, arrival counters
// and status word (256 bytes), then one counter of finished calls per row.
size_t stream_common_bytes(int64_t rows);
int plan_bulk(const vkop_softmax_topk_desc &d, bool base_aligned, BulkPlan *plan);
int launch_bulk(const vkop_softmax_topk_desc &d, const BulkPlan &plan, const void *logits, void *out_values, void *out_indices,
                void *packets_out, void *common_ws, void *bulk_ws, int need_sum, cudaStream_t stream);

// ---- radix path (radix_select.cu) ----
struct RadixPlan {
    size_t bytes;
    int ctas_per_row;
};
int plan_radix(const vkop_softmax_topk_desc &d, RadixPlan *plan);
int launch_radix(const vkop_softmax_topk_desc &d, const RadixPlan &plan, const void *logits, void *out_values,
                 void *out_indices, void *packets_out, void *workspace, int need_sum, cudaStream_t stream);

enum SelectKind { kSelectChunk = 0, kSelectStream = 1, kSelectRadix = 2 };
struct SelectPlan {
    int kind;
    ChunkPlan chunk;
    StreamPlan stream;
    BulkPlan bulk;
    int use_bulk;             // streaming kind: this call runs the bulk-copy kernel
    size_t bulk_off, stream_off;  // streaming kind: where the two kernels' own parts of the workspace start
    RadixPlan radix;
    size_t bytes;
};

// ---- unfused softmax (softmax.cu) ----
int launch_softmax(const vkop_softmax_desc &d, const void *input, void *output, cudaStream_t stream);

// ---- NMS (nms.cu) ----
// TopK along any axis: scratch sizes (256-byte multiples), the axis-to-last transpose and the kernel that
// puts the selected rows into the [outer, k, inner] output (in ascending index order when sorted == 0).
size_t topk_axis_transposed_bytes(const vkop_topk_axis_desc &d);
size_t topk_axis_values_bytes(const vkop_topk_axis_desc &d);
size_t topk_axis_indices_bytes(const vkop_topk_axis_desc &d);
int launch_transpose_axis(const vkop_topk_axis_desc &d, const void *in, void *out, cudaStream_t stream);
int launch_place_results(const vkop_topk_axis_desc &d, const void *vals, const void *idx, void *out_values, void *out_indices,
                         cudaStream_t stream);

int plan_nms(const vkop_nms_desc &d, size_t *bytes);
// Strides 0: dense [B, N, 4] boxes and [B, C, N] scores.  Otherwise: elements between the score blocks /
// the boxes of consecutive batches, and between the four coordinate planes of a box.
int launch_nms(const vkop_nms_desc &d, const void *boxes, const void *scores, int32_t *out_rows, int32_t *out_count,
               void *workspace, cudaStream_t stream, int64_t score_bstride = 0, int64_t box_bstride = 0,
               int64_t box_cstride = 0);

// ---- sampling tail (sample.cu) ----
int launch_sample_topk(const void *values, int dtype, const void *indices, int index_dtype, int64_t rows, int k, float top_p,
                       const float *u, int32_t *out_choice, void *out_token, cudaStream_t stream);

// ---- packet exchange over peer memory (peer_exchange.cu) ----
int launch_packets_push(const void *packets, size_t bytes, void *const *peer_slots, void *const *peer_flags, int rank,
                        int world, uint32_t seq, void *tickets, cudaStream_t stream);
int launch_packets_wait(const void *flags, int world, uint32_t seq, uint32_t max_polls, int *status, cudaStream_t stream);
// every rank's push and wait of one step in a single cooperative launch (ranks emulated on one GPU)
int launch_packets_exchange_all_ranks(const void *const *srcs, size_t bytes, void *const *peer_slots, void *const *peer_flags,
                                      int world, uint32_t seq, void *const *tickets, uint32_t max_polls, int *status,
                                      cudaStream_t stream);

}  // namespace vkop_cuda
