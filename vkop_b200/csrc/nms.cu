// NMS (ONNX NonMaxSuppression) per (batch, class).
//
// Kernel 1, one CTA per (batch, class):
//   scan    the class's score row is read once with 16-byte loads; boxes with
//           score > threshold become 64-bit candidates (key << 32 | ~index)
//           compacted into shared memory;
//   order   the candidates are sorted (score descending, index ascending) with
//           a bitonic network sized to the next power of two of their number;
//           with pre_topk only the best pre_topk stay (if more candidates pass
//           than shared memory holds, an 8-bit radix select over the 64-bit
//           value picks exactly those pre_topk first);
//   boxes   corner coordinates and areas of the ordered candidates are staged
//           in shared memory;
//   mask    (small problems) a tiled IoU bit mask: bit j of row i is set when
//           box j > i overlaps box i by more than the threshold;
//   sweep   one warp walks the candidates in order: each lane owns one 32-bit
//           word of the "removed" set, a kept box ORs its mask row into it;
//           the per-candidate decision is one ballot-free shared-memory read.
//           Larger problems use an iterative sweep instead (a kept box is
//           tested by all threads against the boxes after it).
// Kernel 2 turns the per-problem kept lists into (batch, class, box) rows in
// (batch, class, rank) order and writes the total.
#include "common.cuh"
#include "launchers.h"

namespace vkop_cuda {

constexpr int kNmsThreads = 256;
constexpr int kNmsMaxSorted = 4096;  // candidates one problem can order in shared memory
constexpr int kNmsMaskMax = 512;     // problems up to this many ordered boxes use the bit-mask sweep

struct NmsParams {
    const float *boxes;   // [B, N, 4], or one component plane per coordinate (box_cstride > 0)
    const float *scores;  // [B, C, N]
    int64_t score_bstride;  // elements between the score blocks of consecutive batches (C * N when dense)
    int64_t box_bstride;    // elements between the boxes of consecutive batches
    int64_t box_cstride;    // 0: a box is 4 consecutive floats; else the distance between its coordinates
    int B, C, N;
    int center_point_box, max_out, pre_topk;
    float iou_thr, score_thr;
    int cap;       // candidate slots in shared memory (power of two)
    int mbound;    // upper bound of ordered candidates per problem
    int kept_cap;  // kept slots per problem in the workspace
    int use_mask;
    int32_t *kept;    // [B*C][kept_cap]
    int32_t *counts;  // [B*C]
    int32_t *out_rows;
    int32_t *out_count;
    int64_t capacity_rows;
};

struct BoxA {
    float x1, y1, x2, y2;
};

// shaders/nms.comp:47-55
__device__ __forceinline__ BoxA to_corners(float4 b, int center_point_box) {
    BoxA r;
    if (!center_point_box) {
        r.x1 = b.x; r.y1 = b.y; r.x2 = b.z; r.y2 = b.w;
    } else {
        const float hw = __fmul_rn(b.z, 0.5f), hh = __fmul_rn(b.w, 0.5f);
        r.x1 = __fsub_rn(b.x, hw);
        r.y1 = __fsub_rn(b.y, hh);
        r.x2 = __fadd_rn(b.x, hw);
        r.y2 = __fadd_rn(b.y, hh);
    }
    return r;
}

__device__ __forceinline__ float box_area(const BoxA &a) {
    return __fmul_rn(__fsub_rn(a.x2, a.x1), __fsub_rn(a.y2, a.y1));
}

// shaders/nms.comp:57-68 with a = the later box, b = the kept box; every
// operation separately rounded, true division.
__device__ __forceinline__ float iou_of(const BoxA &a, float area_a, const BoxA &b, float area_b) {
    const float x1 = fmaxf(a.x1, b.x1), y1 = fmaxf(a.y1, b.y1);
    const float x2 = fminf(a.x2, b.x2), y2 = fminf(a.y2, b.y2);
    if (x2 <= x1 || y2 <= y1)
        return 0.0f;
    const float inter = __fmul_rn(__fsub_rn(x2, x1), __fsub_rn(y2, y1));
    const float uni = __fsub_rn(__fadd_rn(area_a, area_b), inter);
    return uni > 0.0f ? __fdiv_rn(inter, uni) : 0.0f;
}

// Radix select of the `need` best candidates among scores > threshold,
// re-reading the score row; leaves them in s_c[0..need).
__device__ __noinline__ void nms_select_overflow(const float *srow, int N, float thr, int need, uint64_t *s_c,
                                                 int *s_count, int *s_hist, int *s_pick) {
    const int tid = threadIdx.x;
    uint64_t prefix = 0, mask = 0;
    for (int pass = 7; pass >= 0; --pass) {
        const int shift = pass * 8;
        for (int i = tid; i < 256; i += kNmsThreads)
            s_hist[i] = 0;
        __syncthreads();
        for (int i = tid; i < N; i += kNmsThreads) {
            const float s = srow[i];
            if (s > thr) {
                const uint64_t c = make_cand(order_key(s), static_cast<uint32_t>(i));
                if ((c & mask) == prefix)
                    atomicAdd(&s_hist[static_cast<int>(c >> shift) & 255], 1);
            }
        }
        __syncthreads();
        if (tid == 0) {
            int cum = 0, d = 255;
            for (; d > 0; --d) {
                const int c = s_hist[d];
                if (cum + c >= need)
                    break;
                cum += c;
            }
            s_pick[0] = d;
            s_pick[1] = need - cum;
            s_pick[2] = s_hist[d];
        }
        __syncthreads();
        prefix |= static_cast<uint64_t>(s_pick[0]) << shift;
        mask |= 0xFFull << shift;
        need = s_pick[1];
        if (s_pick[2] == need)
            break;
    }
    if (tid == 0)
        *s_count = 0;
    __syncthreads();
    for (int i = tid; i < N; i += kNmsThreads) {
        const float s = srow[i];
        if (s > thr) {
            const uint64_t c = make_cand(order_key(s), static_cast<uint32_t>(i));
            if (c >= prefix) {
                const int pos = atomicAdd(s_count, 1);
                s_c[pos] = c;
            }
        }
    }
    __syncthreads();
}

__global__ void __launch_bounds__(kNmsThreads) nms_problem_kernel(const NmsParams p) {
    extern __shared__ __align__(16) unsigned char s_raw[];
    // layout: candidates [cap] u64 | boxes [mbound] BoxA | areas [mbound] f32 | alive/mask words
    uint64_t *s_c = reinterpret_cast<uint64_t *>(s_raw);
    BoxA *s_box = reinterpret_cast<BoxA *>(s_c + p.cap);
    float *s_area = reinterpret_cast<float *>(s_box + p.mbound);
    uint32_t *s_bits = reinterpret_cast<uint32_t *>(s_area + p.mbound);
    __shared__ int s_count;
    __shared__ int s_hist[256];
    __shared__ int s_pick[4];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int prob = blockIdx.x;
    const int b = prob / p.C;
    const float *srow = p.scores + static_cast<int64_t>(b) * p.score_bstride + static_cast<int64_t>(prob - b * p.C) * p.N;
    const float *brow = p.boxes + static_cast<int64_t>(b) * p.box_bstride;

    if (tid == 0)
        s_count = 0;
    __syncthreads();

    // ---- scan: one read of the score row, 16-byte vectors with a ragged head / tail ----
    {
        const uintptr_t addr = reinterpret_cast<uintptr_t>(srow);
        const int head = static_cast<int>((addr & 15) / 4);
        const uint4 *vb = reinterpret_cast<const uint4 *>(addr & ~static_cast<uintptr_t>(15));
        const int nv = (head + p.N + 3) / 4;
        for (int v = tid; v < nv; v += kNmsThreads) {
            const uint4 d = load_stream(vb + v);
            const float f[4] = {__uint_as_float(d.x), __uint_as_float(d.y), __uint_as_float(d.z), __uint_as_float(d.w)};
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int i = v * 4 + e - head;
                if (i >= 0 && i < p.N && f[e] > p.score_thr) {
                    const int pos = atomicAdd(&s_count, 1);
                    if (pos < p.cap)
                        s_c[pos] = make_cand(order_key(f[e]), static_cast<uint32_t>(i));
                }
            }
        }
    }
    __syncthreads();
    int nc = s_count;
    if (nc > p.cap) {
        // only reachable with pre_topk > 0 (otherwise cap covers every box)
        nms_select_overflow(srow, p.N, p.score_thr, p.pre_topk, s_c, &s_count, s_hist, s_pick);
        nc = s_count;
    }

    // ---- order: bitonic sort, descending ----
    int npow2 = 1;
    while (npow2 < nc)
        npow2 <<= 1;
    for (int i = nc + tid; i < npow2; i += kNmsThreads)
        s_c[i] = 0ull;
    __syncthreads();
    for (int size = 2; size <= npow2; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int t = tid; t < npow2 / 2; t += kNmsThreads) {
                const int lo = 2 * t - (t & (stride - 1));
                const int hi = lo + stride;
                const bool desc = (lo & size) == 0;
                const uint64_t a = s_c[lo], c = s_c[hi];
                if (desc ? (a < c) : (a > c)) {
                    s_c[lo] = c;
                    s_c[hi] = a;
                }
            }
            __syncthreads();
        }
    }
    int M = nc;
    if (p.pre_topk > 0 && M > p.pre_topk)
        M = p.pre_topk;
    int max_out = M;
    if (p.max_out > 0 && p.max_out < M)
        max_out = p.max_out;

    // ---- boxes of the ordered candidates ----
    for (int i = tid; i < M; i += kNmsThreads) {
        const uint32_t idx = cand_idx(s_c[i]);
        float4 raw;
        if (p.box_cstride == 0)
            raw = *reinterpret_cast<const float4 *>(brow + static_cast<int64_t>(idx) * 4);
        else
            raw = make_float4(brow[idx], brow[p.box_cstride + idx], brow[2 * p.box_cstride + idx], brow[3 * p.box_cstride + idx]);
        const BoxA bx = to_corners(raw, p.center_point_box);
        s_box[i] = bx;
        s_area[i] = box_area(bx);
    }
    __syncthreads();

    int32_t *kept = p.kept + static_cast<int64_t>(prob) * p.kept_cap;
    int nkept = 0;
    if (p.use_mask) {
        // ---- IoU bit mask: row i, word w covers boxes 32w .. 32w+31 (only j > i) ----
        const int words = (M + 31) / 32;
        for (int t = tid; t < M * words; t += kNmsThreads) {
            const int i = t / words, w = t - i * words;
            uint32_t bits = 0;
            if (w * 32 + 31 > i) {
                const BoxA bi = s_box[i];
                const float ai = s_area[i];
                const int j0 = w * 32;
#pragma unroll 4
                for (int jj = 0; jj < 32; jj++) {
                    const int j = j0 + jj;
                    if (j > i && j < M && iou_of(s_box[j], s_area[j], bi, ai) > p.iou_thr)
                        bits |= 1u << jj;
                }
            }
            s_bits[t] = bits;
        }
        __syncthreads();
        // ---- sweep: warp 0; lane w holds removed word w (words <= 16 here) ----
        if (warp == 0) {
            uint32_t removed = 0;  // lane w: boxes 32w..32w+31 already suppressed
            for (int i = 0; i < M && nkept < max_out; i++) {
                const uint32_t word = __shfl_sync(kFullMask, removed, i >> 5);
                if ((word >> (i & 31)) & 1u)
                    continue;
                if (lane == 0)
                    kept[nkept] = static_cast<int32_t>(cand_idx(s_c[i]));
                nkept++;
                if (lane < words)
                    removed |= s_bits[i * words + lane];
            }
            if (lane == 0)
                p.counts[prob] = nkept;
        }
    } else {
        // ---- iterative sweep: a kept box is tested against every later live box ----
        uint8_t *s_dead = reinterpret_cast<uint8_t *>(s_bits);
        for (int i = tid; i < M; i += kNmsThreads)
            s_dead[i] = 0;
        __syncthreads();
        for (int i = 0; i < M && nkept < max_out; i++) {
            if (s_dead[i])
                continue;  // uniform: every thread reads the same flag after the last barrier
            if (tid == 0)
                kept[nkept] = static_cast<int32_t>(cand_idx(s_c[i]));
            nkept++;
            const BoxA bi = s_box[i];
            const float ai = s_area[i];
            for (int j = i + 1 + tid; j < M; j += kNmsThreads)
                if (!s_dead[j] && iou_of(s_box[j], s_area[j], bi, ai) > p.iou_thr)
                    s_dead[j] = 1;
            __syncthreads();
        }
        if (tid == 0)
            p.counts[prob] = nkept;
    }
}

// Rows in (batch, class, rank) order: problem p writes at the sum of the counts before it.
__global__ void __launch_bounds__(128) nms_emit_kernel(const NmsParams p) {
    __shared__ int s_part[4];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int prob = blockIdx.x;
    const int problems = p.B * p.C;
    int64_t sum = 0;
    for (int q = tid; q < prob; q += 128)
        sum += p.counts[q];
    int s32 = static_cast<int>(sum);
    s32 = __reduce_add_sync(kFullMask, s32);
    if (lane == 0)
        s_part[warp] = s32;
    __syncthreads();
    const int64_t off = static_cast<int64_t>(s_part[0]) + s_part[1] + s_part[2] + s_part[3];
    const int cnt = p.counts[prob];
    const int c = prob % p.C, b = prob / p.C;
    const int32_t *kept = p.kept + static_cast<int64_t>(prob) * p.kept_cap;
    for (int j = tid; j < cnt; j += 128) {
        const int64_t r = off + j;
        if (r < p.capacity_rows) {
            p.out_rows[r * 3 + 0] = b;
            p.out_rows[r * 3 + 1] = c;
            p.out_rows[r * 3 + 2] = kept[j];
        }
    }
    if (prob == problems - 1 && tid == 0) {
        const int64_t total = off + cnt;
        *p.out_count = total > 0x7FFFFFFFll ? 0x7FFFFFFF : static_cast<int32_t>(total);
    }
}

__global__ void nms_zero_count_kernel(int32_t *out_count) { *out_count = 0; }

// ---------------------------------------------------------------------------

struct NmsPlan {
    int cap, mbound, kept_cap, use_mask;
    size_t smem, kept_bytes, counts_bytes, total;
};

static int make_plan(const vkop_nms_desc &d, NmsPlan *pl) {
    if (d.num_batch < 0 || d.num_class < 0 || d.num_boxes < 0 || d.max_output_boxes_per_class < 0 || d.pre_topk < 0 ||
        d.capacity_rows < 0)
        return VKOP_INVALID_ARG;
    if (d.center_point_box != 0 && d.center_point_box != 1)
        return VKOP_INVALID_ARG;
    if (!(d.iou_threshold == d.iou_threshold) || !(d.score_threshold == d.score_threshold))
        return VKOP_INVALID_ARG;
    const int N = d.num_boxes;
    // with a pre-selection an overflowing candidate list is cut down by a radix select first,
    // so the sort buffer only needs room for the common case
    int cap_limit = kNmsMaxSorted;
    if (d.pre_topk > 0) {
        cap_limit = 1024;
        while (cap_limit < 2 * d.pre_topk)
            cap_limit <<= 1;
        if (cap_limit > kNmsMaxSorted)
            cap_limit = kNmsMaxSorted;
    }
    int cap = 32;
    while (cap < N && cap < cap_limit)
        cap <<= 1;
    if (d.pre_topk == 0 && N > kNmsMaxSorted)
        return VKOP_UNSUPPORTED;  // every candidate enters the sweep: they must all fit the shared-memory sort
    if (d.pre_topk > kNmsMaxSorted)
        return VKOP_UNSUPPORTED;
    int mbound = d.pre_topk > 0 ? (d.pre_topk < N ? d.pre_topk : N) : N;
    if (mbound < 1)
        mbound = 1;
    pl->cap = cap;
    pl->mbound = mbound;
    pl->use_mask = mbound <= kNmsMaskMax ? 1 : 0;
    int kept_cap = mbound;
    if (d.max_output_boxes_per_class > 0 && d.max_output_boxes_per_class < kept_cap)
        kept_cap = d.max_output_boxes_per_class;
    pl->kept_cap = kept_cap;
    const size_t words = static_cast<size_t>((mbound + 31) / 32);
    const size_t bits_bytes = pl->use_mask ? static_cast<size_t>(mbound) * words * 4 : static_cast<size_t>(mbound + 3) / 4 * 4;
    pl->smem = static_cast<size_t>(cap) * 8 + static_cast<size_t>(mbound) * (16 + 4) + bits_bytes;
    if (pl->smem > 200 * 1024)
        return VKOP_UNSUPPORTED;
    const size_t problems = static_cast<size_t>(d.num_batch) * d.num_class;
    pl->counts_bytes = (problems * 4 + 255) / 256 * 256;
    pl->kept_bytes = problems * kept_cap * 4;
    pl->total = pl->counts_bytes + pl->kept_bytes;
    return VKOP_OK;
}

int plan_nms(const vkop_nms_desc &d, size_t *bytes) {
    NmsPlan pl;
    const int rc = make_plan(d, &pl);
    if (rc != VKOP_OK)
        return rc;
    *bytes = pl.total;
    return VKOP_OK;
}

int launch_nms(const vkop_nms_desc &d, const void *boxes, const void *scores, int32_t *out_rows, int32_t *out_count,
               void *workspace, cudaStream_t stream, int64_t score_bstride, int64_t box_bstride, int64_t box_cstride) {
    NmsPlan pl;
    const int rc = make_plan(d, &pl);
    if (rc != VKOP_OK)
        return rc;
    if (reinterpret_cast<uintptr_t>(boxes) % (box_cstride == 0 ? 16 : 4) != 0 || reinterpret_cast<uintptr_t>(scores) % 4 != 0)
        return VKOP_INVALID_ARG;
    const int64_t problems = static_cast<int64_t>(d.num_batch) * d.num_class;
    if (problems == 0 || d.num_boxes == 0) {
        nms_zero_count_kernel<<<1, 1, 0, stream>>>(out_count);
        note_launch();
        return check_launch();
    }
    if (problems > 0x7FFFFFFFll)
        return VKOP_UNSUPPORTED;
    NmsParams p;
    p.boxes = reinterpret_cast<const float *>(boxes);
    p.scores = reinterpret_cast<const float *>(scores);
    p.score_bstride = score_bstride > 0 ? score_bstride : static_cast<int64_t>(d.num_class) * d.num_boxes;
    p.box_bstride = box_bstride > 0 ? box_bstride : static_cast<int64_t>(d.num_boxes) * 4;
    p.box_cstride = box_cstride;
    p.B = d.num_batch;
    p.C = d.num_class;
    p.N = d.num_boxes;
    p.center_point_box = d.center_point_box;
    p.max_out = d.max_output_boxes_per_class;
    p.pre_topk = d.pre_topk;
    p.iou_thr = d.iou_threshold;
    p.score_thr = d.score_threshold;
    p.cap = pl.cap;
    p.mbound = pl.mbound;
    p.kept_cap = pl.kept_cap;
    p.use_mask = pl.use_mask;
    p.counts = reinterpret_cast<int32_t *>(workspace);
    p.kept = reinterpret_cast<int32_t *>(static_cast<char *>(workspace) + pl.counts_bytes);
    p.out_rows = out_rows;
    p.out_count = out_count;
    p.capacity_rows = d.capacity_rows;
    if (pl.smem > 32 * 1024 &&
        cudaFuncSetAttribute(nms_problem_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(pl.smem)) !=
            cudaSuccess)
        return VKOP_CUDA_ERROR;
    nms_problem_kernel<<<static_cast<unsigned>(problems), kNmsThreads, pl.smem, stream>>>(p);
    nms_emit_kernel<<<static_cast<unsigned>(problems), 128, 0, stream>>>(p);
    note_launch(2);
    return check_launch();
}

}  // namespace vkop_cuda
