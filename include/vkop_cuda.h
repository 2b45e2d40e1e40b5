/*
 * vkop_cuda.h - C ABI of the CUDA (sm_100a) launcher for vkop's GPU
 * post-processing operators: Softmax + TopK (fused and unfused) and NMS.
 *
 * This is the boundary a vkop build binds instead of its Vulkan dispatch for
 * these operators.  In the reference an operator's execute() ends in
 * Operator::submit (ops/Operator.hpp:225-238: descriptor update, pipeline
 * bind, push constants, vkCmdDispatch) on buffers allocated through VMA
 * (core/Tensor.hpp:384-394); here execute() ends in one of the calls below on
 * plain device pointers.
 *
 * Conventions for every entry point:
 *   - all tensor pointers are DEVICE pointers owned by the caller; tensors are
 *     the logical row-major arrays ([rows, cols] logits, boxes [B,N,4],
 *     scores [B,C,N]), not the RGBA image packing the shaders read;
 *   - the call enqueues work on `stream` (a cudaStream_t passed as void*; NULL
 *     is the default stream) and returns without synchronising;
 *   - nothing is allocated; scratch memory comes from the caller
 *     (`*_workspace` tells how much).  A workspace must be cleared once with
 *     vkop_cuda_workspace_init after it is allocated; kernels leave it ready
 *     for the next call with the same descriptor (clear it again before it
 *     serves a different descriptor: the kernels keep counters in it whose
 *     layout follows the shape).  Calls that share a workspace must be
 *     enqueued on one stream, in order; they may then overlap on the device;
 *   - the return value is VKOP_OK (0) or a negative vkop_status; the library
 *     never throws and never aborts.
 */
#ifndef VKOP_CUDA_H_
#define VKOP_CUDA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VKOP_CUDA_VERSION 100

typedef enum vkop_status {
    VKOP_OK = 0,
    VKOP_INVALID_ARG = -1,
    VKOP_UNSUPPORTED = -2,
    VKOP_WORKSPACE_TOO_SMALL = -3,
    VKOP_CUDA_ERROR = -4,
    VKOP_TIMEOUT = -5
} vkop_status;

typedef enum vkop_dtype { VKOP_F32 = 0, VKOP_F16 = 1, VKOP_BF16 = 2 } vkop_dtype;
typedef enum vkop_index_dtype { VKOP_I32 = 0, VKOP_I64 = 1 } vkop_index_dtype;
typedef enum vkop_value_kind { VKOP_VALUE_PROBABILITY = 0, VKOP_VALUE_RAW = 1 } vkop_value_kind;
typedef enum vkop_select_path {
    VKOP_PATH_AUTO = 0,
    VKOP_PATH_CHUNK = 1,  /* one CTA per chunk of a row, the chunk held in registers */
    VKOP_PATH_RADIX = 2,  /* multi-pass radix select (large k, very long rows) */
    VKOP_PATH_STREAM = 3, /* persistent CTAs streaming cp.async tiles with a running threshold (any alignment) */
    VKOP_PATH_BULK = 4    /* streaming CTAs fed by bulk copies (cp.async.bulk + mbarrier) into a shared-memory ring,
                             selection in a second small kernel: long rows that start on 16-byte boundaries.
                             Chosen by name only: AUTO does not pick it */
} vkop_select_path;

/* The logits are complete and visible before the call is enqueued: no earlier
 * operation of the same stream still writes them.  The kernel may then start
 * reading them while the previous kernel of the stream is still draining
 * (programmatic dependent launch); its own writes still wait for that kernel.
 * Leave it clear when the logits come from the kernel just before.
 * Calls with the flag number themselves in their workspace and order their
 * result rows by that number: between two of them that share a workspace or an
 * output buffer, enqueue no other kernel that writes those outputs, and let
 * every output buffer written by overlapping calls belong to one workspace.
 * Results reach the outputs in call order, and the kernel of a call completes
 * only after the kernel before it in the stream has, so a kernel enqueued
 * behind a call in the usual way sees the results of that call and of all
 * earlier ones.  (What may sit between two such calls: calls of this library,
 * with or without the flag, on this or another workspace, and any kernel
 * launched in the usual way.  Not a foreign kernel launched with programmatic
 * stream serialization that neither waits for its predecessor nor ends after
 * it: the chain of completions would break there.) */
#define VKOP_FLAG_INPUT_READY 1

/* Library version (VKOP_CUDA_VERSION of the build). */
int vkop_cuda_version(void);
/* Static, human-readable name of a status code. */
const char *vkop_cuda_status_string(int status);
/* Kernels launched by this library in the calling process so far. */
uint64_t vkop_cuda_launch_count(void);

/* Clears a freshly allocated workspace (asynchronous on `stream`). */
int vkop_cuda_workspace_init(void *workspace, size_t bytes, void *stream);

/* ------------------------------------------------------------------------ */
/* Fused Softmax + TopK over the last axis of a [rows, cols] tensor.
 *
 * Replaces the Softmax dispatch followed by the multi-pass TopK dispatches of
 * the reference (ops/Softmax.hpp:61-141 with shaders/softmax2.comp:50-117;
 * ops/Topk.hpp:95-217 with shaders/topk.comp:110-175) as registered by
 * benchmark/main.cpp:85-101 through Runtime::RegisterPostProcess
 * (core/runtime.cpp:480-520).
 *
 * Selection is on the stored logit: value descending, lower index first among
 * equal values (-0 equals +0; NaN is the largest value: first among the largest,
 * last among the smallest).  Output values are the
 * softmax probabilities of x * inv_temperature (or the raw logits), in the
 * logits' dtype; indices are int32 (as the reference) or int64 (ONNX).
 * Outputs are [rows, k], row-major, sorted best first. */
typedef struct vkop_softmax_topk_desc {
    int64_t rows;
    int64_t cols;
    int64_t row_stride;    /* elements between rows of the logits; 0 means cols */
    int32_t dtype;         /* vkop_dtype of logits and of the output values */
    int32_t k;             /* 1 <= k <= min(cols, 4096) */
    int32_t index_dtype;   /* vkop_index_dtype */
    int32_t value_kind;    /* vkop_value_kind */
    float inv_temperature; /* > 0; 1.0f for a plain softmax */
    int32_t largest;       /* 1 = largest (default semantic); 0 = smallest, raw values only */
    int32_t path;          /* vkop_select_path; AUTO picks by k and row length */
    int32_t splits;        /* CTAs per row on the chunk path; 0 = automatic */
    int64_t index_offset;  /* added to every emitted index (offset of a vocabulary shard) */
    int32_t flags;         /* VKOP_FLAG_* */
    int32_t reserved;      /* 0 */
} vkop_softmax_topk_desc;

int vkop_cuda_softmax_topk_workspace(const vkop_softmax_topk_desc *desc, size_t *bytes);
int vkop_cuda_softmax_topk(const vkop_softmax_topk_desc *desc, const void *logits, void *out_values,
                           void *out_indices, void *workspace, size_t workspace_bytes, void *stream);

/* Standalone TopK (no softmax): same selection, values are copies of the
 * input.  Replaces ops/Topk.hpp:95-217 + shaders/topk.comp when TopK is used
 * on its own (tests/TopkTest.cpp:91-125).  desc->value_kind is ignored. */
int vkop_cuda_topk(const vkop_softmax_topk_desc *desc, const void *input, void *out_values, void *out_indices,
                   void *workspace, size_t workspace_bytes, void *stream);

/* TopK along any axis, and the unsorted output order.  The input is viewed
 * row-major as [outer, axis_len, inner] and the k best along the middle axis
 * go to out_values / out_indices viewed as [outer, k, inner] (the input's
 * shape with shape[axis] = k, as ops/Topk.hpp:108-109 sizes the outputs).
 * Replaces ops/Topk.hpp:62-79 (attributes "axis", "sorted") and :98-103;
 * the reference's shader only ever selects along the last axis of a 1-D or
 * 2-D tensor (shaders/topk.comp:119-175) and ignores "sorted".
 * sorted != 0: best first, as vkop_cuda_topk.  sorted == 0: the same k
 * entries in ascending index order.  Indices run from 0 to axis_len - 1. */
typedef struct vkop_topk_axis_desc {
    int64_t outer;
    int64_t axis_len;
    int64_t inner;
    int32_t dtype;       /* vkop_dtype of the input and of the output values */
    int32_t k;           /* 1 <= k <= min(axis_len, 4096) */
    int32_t index_dtype; /* vkop_index_dtype */
    int32_t largest;     /* 1 = largest, 0 = smallest */
    int32_t sorted;      /* 0 = ascending index order */
    int32_t path;        /* vkop_select_path for the selection itself */
} vkop_topk_axis_desc;

int vkop_cuda_topk_axis_workspace(const vkop_topk_axis_desc *desc, size_t *bytes);
int vkop_cuda_topk_axis(const vkop_topk_axis_desc *desc, const void *input, void *out_values, void *out_indices,
                        void *workspace, size_t workspace_bytes, void *stream);

/* ------------------------------------------------------------------------ */
/* Unfused Softmax with the full probability tensor as output, along the
 * middle axis of a row-major [outer, axis_len, inner] view (inner = 1 for the
 * 2-D post-processing case).  Replaces ops/Softmax.hpp:61-141 with
 * shaders/softmax2.comp (rank <= 2) and shaders/softmax.comp (rank 3/4, whose
 * image packing is not reproduced: the tensor stays linear NCHW). */
typedef struct vkop_softmax_desc {
    int64_t outer;
    int64_t axis_len;
    int64_t inner;
    int32_t dtype; /* input and output dtype */
    float inv_temperature;
} vkop_softmax_desc;

int vkop_cuda_softmax(const vkop_softmax_desc *desc, const void *input, void *output, void *stream);

/* ------------------------------------------------------------------------ */
/* Vocabulary-sharded Softmax + TopK.  Each GPU holds [rows, cols] = one
 * contiguous column slice of the logits (desc->index_offset = first global
 * column).  `partial` writes one packet per row: the shard's softmax maximum
 * and exp-sum and its k best (key, global index) pairs.  The packets of all
 * shards are exchanged by the caller (an all-gather), and `merge` reduces
 * `shards` packets per row to the final [rows, k] outputs.  The reference has
 * no multi-device path; this extends the operator above. */
size_t vkop_cuda_packet_bytes(int32_t k);
int vkop_cuda_softmax_topk_partial(const vkop_softmax_topk_desc *desc, const void *logits_shard, void *packets_out,
                                   void *workspace, size_t workspace_bytes, void *stream);
/* packets: [shards, rows, packet] as an all-gather of packets_out delivers them. */
int vkop_cuda_softmax_topk_merge(const vkop_softmax_topk_desc *desc, const void *packets, int32_t shards,
                                 void *out_values, void *out_indices, void *stream);

/* Sampling tail over the k survivors of vkop_cuda_softmax_topk (no counterpart
 * in the reference: the step that follows top-k in a vocabulary-selection
 * path).  values [rows, k] are the probabilities as the operator wrote them
 * (best first), indices [rows, k] their columns, u [rows] uniform numbers in
 * [0, 1) from the caller.  Per row, all sums sequential in fp32: the nucleus
 * is the shortest prefix whose sum reaches top_p times the sum of all k
 * (top_p >= 1 keeps all k); the choice is the first entry whose prefix sum
 * exceeds u times the nucleus' sum.  out_choice [rows] receives the position
 * (0 .. k-1), out_token [rows] (same type as indices) the column. */
int vkop_cuda_sample_topk(const void *values, int32_t dtype, const void *indices, int32_t index_dtype, int64_t rows,
                          int32_t k, float top_p, const float *u, int32_t *out_choice, void *out_token, void *stream);

/* Packet exchange over peer memory instead of an all-gather (no counterpart in
 * the reference, which is single-device).  Every rank owns a receive buffer
 * `slots` of 2 * world * packets_bytes bytes and `flags` of 2 * world uint32,
 * both zeroed once and mapped into every peer's address space (CUDA IPC or
 * symmetric memory; peer access enabled).  Step `seq` (1, 2, 3, ... on every
 * rank alike) uses half seq & 1 of both.  seq is never 0 (the cleared flags read
 * as 0) and differs from the previous step's in its lowest bit: a 32-bit counter
 * that wraps must skip 0 and keep alternating.
 *
 * vkop_cuda_packets_push stores this rank's packets (the output of `partial`)
 * into slot [seq & 1][rank] of every rank's buffer -- peer_slots / peer_flags
 * are DEVICE arrays of `world` device pointers, entry p being rank p's buffer --
 * and then sets flag [seq & 1][rank] there to seq.  `tickets`: world uint32
 * in local device memory, zeroed once.
 *
 * vkop_cuda_packets_wait makes the stream wait until the flags of all ranks
 * in the LOCAL buffer show seq; `merge` on slots + (seq & 1) * world *
 * packets_bytes follows it on the same stream.  The wait is bounded: after
 * max_polls looks (about a microsecond each) it writes VKOP_TIMEOUT to
 * *status (device memory, set to VKOP_OK by the caller beforehand) and lets
 * the stream go on; read the status after synchronising. */
int vkop_cuda_packets_push(const void *packets, size_t packets_bytes, void *const *peer_slots, void *const *peer_flags,
                           int32_t rank, int32_t world, uint32_t seq, void *tickets, void *stream);
int vkop_cuda_packets_wait(const void *flags, int32_t world, uint32_t seq, uint32_t max_polls, int32_t *status,
                           void *stream);
/* One exchange step of ALL ranks in a single cooperative launch, for a machine with fewer GPUs than
 * ranks (tests, bring-up): kernels that wait for one another must not be separate launches on one GPU,
 * so rank r's push and rank r's bounded wait are block groups of one kernel whose blocks are all
 * resident.  packets_of / tickets_of: DEVICE arrays of `world` device pointers (rank r's packets and
 * tickets); peer_slots / peer_flags as above; status: `world` words, status[r] receives VKOP_TIMEOUT
 * if rank r's wait runs out.  VKOP_UNSUPPORTED when the blocks would not all fit the GPU at once.
 * No counterpart in the reference. */
int vkop_cuda_packets_exchange_all_ranks(const void *const *packets_of, size_t packets_bytes, void *const *peer_slots,
                                         void *const *peer_flags, int32_t world, uint32_t seq, void *const *tickets_of,
                                         uint32_t max_polls, int32_t *status, void *stream);

/* ------------------------------------------------------------------------ */
/* NMS (ONNX NonMaxSuppression) per (batch, class).
 *
 * Replaces ops/Nms.hpp:66-112 with shaders/nms.comp:70-203.  boxes [B,N,4]
 * fp32, scores [B,C,N] fp32.  Candidates are boxes with score >
 * score_threshold, ordered by score descending then index ascending; with
 * pre_topk > 0 only the best pre_topk of them enter the sweep.  IoU is
 * computed in fp32 in the shader's operand order (nms.comp:57-68).  Output
 * rows are (batch, class, box) int32 triples in (batch, class, rank) order;
 * *out_count receives the number of rows produced (rows beyond
 * capacity_rows are counted but not written). */
typedef struct vkop_nms_desc {
    int32_t num_batch;
    int32_t num_class;
    int32_t num_boxes;
    int32_t center_point_box;           /* 0: (x1,y1,x2,y2); 1: (cx,cy,w,h) */
    int32_t max_output_boxes_per_class; /* 0 = unlimited */
    int32_t pre_topk;                   /* 0 = every candidate enters the sweep */
    float iou_threshold;
    float score_threshold;
    int64_t capacity_rows;              /* rows out_rows can hold */
} vkop_nms_desc;

int vkop_cuda_nms_workspace(const vkop_nms_desc *desc, size_t *bytes);
int vkop_cuda_nms(const vkop_nms_desc *desc, const void *boxes, const void *scores, int32_t *out_rows,
                  int32_t *out_count, void *workspace, size_t workspace_bytes, void *stream);

/* The same NMS straight on a detection head as a YOLO-style model emits it:
 * head [B, 4 + C, N] fp32, planes 0-3 the box coordinates (cx, cy, w, h with
 * center_point_box = 1), planes 4.. the class scores.  Nothing is transposed
 * or copied: the score planes are scanned where they lie and the boxes of the
 * surviving candidates are gathered from the four coordinate planes.  Stands
 * in for the CPU post-processing of example/yolo/main.cpp:60-179 (which reads
 * the head back and runs argmax + NMS on the host) in its per-class form.
 * Same descriptor, workspace and outputs as vkop_cuda_nms. */
int vkop_cuda_yolo_nms(const vkop_nms_desc *desc, const void *head, int32_t *out_rows, int32_t *out_count,
                       void *workspace, size_t workspace_bytes, void *stream);

/* ------------------------------------------------------------------------ */
/* Fused Softmax + TopK that needs no workspace from the caller and allocates
 * nothing: the chunk kernel works in a fixed array inside the loaded module
 * (vkop_cuda_static_scratch_bytes() bytes of device memory per device).
 *
 * This entry point has no counterpart in the reference: there every operator
 * allocates its temporaries itself (ops/Topk.hpp:134-152).  It is for callers
 * that are given tensors and a stream and nothing else, or that must not call
 * the allocator when they run (cudaMalloc synchronises the device and can
 * fail under memory pressure).
 *
 * Same arguments and results as vkop_cuda_softmax_topk, without the
 * workspace.  Limits: desc->path AUTO or CHUNK (the chunk kernel is used);
 * VKOP_WORKSPACE_TOO_SMALL when the shape needs more scratch than the array
 * holds.  The first call on a device looks up the array's device address and
 * should come before any stream capture on that device.  All calls on a
 * device share the array, which keeps what the last call left: every call
 * first clears the counters it uses, on its stream.  Calls that overlap on
 * the GPU race on the array, so order them (one stream, or events), or use
 * the workspace entry point. */
size_t vkop_cuda_static_scratch_bytes(void);
int vkop_cuda_softmax_topk_static(const vkop_softmax_topk_desc *desc, const void *logits, void *out_values,
                                  void *out_indices, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* VKOP_CUDA_H_ */
