// NMS (ONNX NonMaxSuppression) per (batch, class).
//
// Kernel 1, one 128-thread CTA per (batch, class); the detection-sized problem (8400 boxes, per-class top-300)
// leaves room for nine CTAs on an SM, so that its 1280 problems are resident together:
//   scan    the class's score row is read once with 16-byte loads, four in flight; boxes with score >
//           threshold become 64-bit candidates (key << 32 | ~index); a warp takes its slots in shared
//           memory with one atomic per round;
//   trim    with pre_topk, a list longer than the sort buffer is cut by a radix select over the 64-bit
//           values (eight bits a pass from the top) that stops as soon as the entries at or above the
//           chosen prefix fit the buffer; if more candidates pass than the scan has slots for, the same
//           select re-reads the score row and picks exactly pre_topk;
//   order   bitonic sort, score descending and index ascending: up to 512 candidates in registers (four
//           per thread; partners in the thread, then by shuffle, three steps through shared memory),
//           longer lists in shared memory;
//   boxes   corner coordinates and areas of the ordered candidates are staged in shared memory;
//   mask    (up to 512 ordered boxes) an IoU bit mask: bit j of row i is set when box j > i overlaps box i
//           by more than the threshold.  A warp takes two rows at a time, one column box per lane, each
//           32-bit word is a ballot.  The test avoids the division where the quotient is not next to the
//           threshold and repeats a row with the exact test otherwise (iou_exceeds_quick);
//   sweep   one warp walks the candidates 32 at a time: lane v owns word v of the "removed" set; the 32
//           boxes of a word are resolved in order from the diagonal words held in registers, then the
//           rows of the kept ones are ORed into the later words.
//           Larger problems use an iterative sweep instead (a kept box is tested by all threads against
//           the boxes after it).
// Kernel 2 turns the per-problem kept lists into (batch, class, box) rows in
// (batch, class, rank) order and writes the total.
#include "common.cuh"
#include "launchers.h"

namespace vkop_cuda {

constexpr int kNmsThreads = 128;
constexpr int kNmsCtasPerSm = 9;  // registers and shared memory of the detection-sized problem leave room for nine
constexpr int kNmsMaxSorted = 4096;  // candidates one problem can order in shared memory
constexpr int kNmsRegSorted = 4 * kNmsThreads;  // lists up to this length are sorted in registers
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
    int cap;       // candidate slots the scan may fill (power of two)
    int sortcap;   // slots of the sort buffer: cap, or cap / 2 when longer lists are cut down first
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

// "IoU > threshold" without the division wherever the answer is not close: the quotient is formed with the
// approximate reciprocal (relative error below 2^-22); when it is further than 2^-20 (relative) from the
// threshold, the correctly rounded quotient lies on the same side.  `doubt` collects the cases where it is not
// (a quotient next to the threshold, or not a number): the caller then repeats the row with the exact test
// (iou_of).  Only used when the threshold lies in [1e-6, 1e6] (so that "no overlap" means "not above") and
// every box of positive extent has an area in [1e-28, 1e28]: two boxes that overlap both have positive
// extents, their intersection is no larger than either (rounding is monotonic), so the union is at least the
// larger area and the reciprocal is safe.
struct IouTest {
    float thr, lo, hi;
    bool quick;
};

__device__ __forceinline__ IouTest make_iou_test(float thr, bool areas_in_range) {
    IouTest t;
    t.thr = thr;
    t.lo = thr * (1.0f - 9.5367431640625e-07f);
    t.hi = thr * (1.0f + 9.5367431640625e-07f);
    t.quick = areas_in_range && thr >= 1e-6f && thr <= 1e6f;
    return t;
}

__device__ __forceinline__ bool iou_exceeds_quick(const BoxA &a, float area_a, const BoxA &b, float area_b, const IouTest &t,
                                                  bool &doubt) {
    const float x1 = fmaxf(a.x1, b.x1), y1 = fmaxf(a.y1, b.y1);
    const float x2 = fminf(a.x2, b.x2), y2 = fminf(a.y2, b.y2);
    const bool overlap = x2 > x1 && y2 > y1;  // otherwise (NaN included) the IoU is 0
    const float inter = __fmul_rn(__fsub_rn(x2, x1), __fsub_rn(y2, y1));
    const float uni = __fsub_rn(__fadd_rn(area_a, area_b), inter);
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(uni));
    const float q = __fmul_rn(inter, r);
    const bool above = q > t.hi;
    doubt = doubt || (overlap && !above && !(q < t.lo));  // the last two hold for NaN as well
    return overlap && above;
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

// Cuts the candidate list s_in[0..nc) down to at most `limit` entries that still contain the `need` best ones
// (need <= limit < nc) and packs them into s_c: a radix select over the 64-bit values, eight bits a pass from
// the top, that stops as soon as the entries at or above the chosen prefix number `limit` or fewer.  Returns
// their number.
__device__ __noinline__ int nms_trim_candidates(const uint64_t *s_in, uint64_t *s_c, int nc, int need, int limit,
                                                int *s_count, int *s_hist, int *s_pick) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint64_t prefix = 0, mask = 0;
    int above = 0;  // entries above every value that carries the current prefix
    for (int pass = 7; pass >= 0; --pass) {
        const int shift = pass * 8;
        for (int i = tid; i < 256; i += kNmsThreads)
            s_hist[i] = 0;
        __syncthreads();
        for (int i = tid; i < nc; i += kNmsThreads) {
            const uint64_t c = s_in[i];
            if ((c & mask) == prefix)
                atomicAdd(&s_hist[static_cast<int>(c >> shift) & 255], 1);
        }
        __syncthreads();
        if (warp == 0) {
            // lane l owns digits 8l .. 8l+7; the digit wanted is the highest d with (entries above d) + hist[d] >= need
            int h[8], tot = 0;
#pragma unroll
            for (int e = 0; e < 8; e++) {
                h[e] = s_hist[lane * 8 + e];
                tot += h[e];
            }
            int suf = tot;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int n = __shfl_down_sync(kFullMask, suf, o);
                if (lane + o < 32)
                    suf += n;
            }
            int cum = above + suf - tot, found = -1, cum_d = 0, h_d = 0;
#pragma unroll
            for (int e = 7; e >= 0; --e)
                if (found < 0) {
                    if (cum + h[e] >= need) {
                        found = lane * 8 + e;
                        cum_d = cum;
                        h_d = h[e];
                    } else {
                        cum += h[e];
                    }
                }
            const uint32_t have = __ballot_sync(kFullMask, found >= 0);
            const int src = have ? 31 - __clz(have) : 0;
            found = __shfl_sync(kFullMask, found, src);
            cum_d = __shfl_sync(kFullMask, cum_d, src);
            h_d = __shfl_sync(kFullMask, h_d, src);
            if (lane == 0) {
                s_pick[0] = found < 0 ? 0 : found;
                s_pick[1] = cum_d;
                s_pick[2] = cum_d + h_d;
            }
        }
        __syncthreads();
        prefix |= static_cast<uint64_t>(s_pick[0]) << shift;
        mask |= 0xFFull << shift;
        above = s_pick[1];
        if (s_pick[2] <= limit)
            break;
    }
    if (tid == 0)
        *s_count = 0;
    __syncthreads();
    for (int i0 = 0; i0 < nc; i0 += kNmsThreads) {
        const int i = i0 + tid;
        const uint64_t c = i < nc ? s_in[i] : 0ull;
        const bool sel = i < nc && c >= prefix;
        const uint32_t who = __ballot_sync(kFullMask, sel);
        if (who == 0)
            continue;
        int base = 0;
        if (lane == 0)
            base = atomicAdd(s_count, __popc(who));
        base = __shfl_sync(kFullMask, base, 0);
        if (sel)
            s_c[base + __popc(who & ((1u << lane) - 1u))] = c;
    }
    __syncthreads();
    return *s_count;
}

// Bitonic sort (descending) of s_c[0..nc), nc <= kNmsRegSorted = 4 * kNmsThreads, padded with zeros: thread t
// holds elements 4t .. 4t+3 in registers; partners at distance 1 and 2 are in the same thread, at distance
// 4 .. 64 in the same warp (shuffles), and only the three steps at distance 128 and 256 go through shared
// memory.  Every thread of the CTA must call it; the sorted list is complete on return.
__device__ __forceinline__ void sort_in_registers(uint64_t *s_c, int nc) {
    const int tid = threadIdx.x, g0 = 4 * tid;
    uint64_t v[4];
#pragma unroll
    for (int e = 0; e < 4; e++)
        v[e] = g0 + e < nc ? s_c[g0 + e] : 0ull;
    // keep the larger of (mine, other) where `larger` is set, else the smaller
    auto keep = [](uint64_t mine, uint64_t other, bool larger) { return (mine < other) == larger ? other : mine; };
    for (int size = 2; size <= kNmsRegSorted; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            if (stride == 1) {
#pragma unroll
                for (int e = 0; e < 4; e += 2) {
                    const bool desc = ((g0 + e) & size) == 0;
                    const uint64_t a = v[e], c = v[e + 1];
                    v[e] = keep(a, c, desc);
                    v[e + 1] = keep(c, a, !desc);
                }
            } else if (stride == 2) {
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const bool desc = ((g0 + e) & size) == 0;
                    const uint64_t a = v[e], c = v[e + 2];
                    v[e] = keep(a, c, desc);
                    v[e + 2] = keep(c, a, !desc);
                }
            } else {
                const int d = stride >> 2;  // distance of the partner thread
                const bool lower = (tid & d) == 0;
                const bool desc = (g0 & size) == 0;  // size >= 8 here: the same for the four elements
                uint64_t o[4];
                if (d < 32) {
#pragma unroll
                    for (int e = 0; e < 4; e++)
                        o[e] = __shfl_xor_sync(kFullMask, v[e], d);
                } else {
                    __syncthreads();
#pragma unroll
                    for (int e = 0; e < 4; e++)
                        s_c[g0 + e] = v[e];
                    __syncthreads();
#pragma unroll
                    for (int e = 0; e < 4; e++)
                        o[e] = s_c[4 * (tid ^ d) + e];
                }
#pragma unroll
                for (int e = 0; e < 4; e++)
                    v[e] = keep(v[e], o[e], lower == desc);
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int e = 0; e < 4; e++)
        s_c[g0 + e] = v[e];
    __syncthreads();
}

__global__ void __launch_bounds__(kNmsThreads, kNmsCtasPerSm) nms_problem_kernel(const NmsParams p) {
    extern __shared__ __align__(16) unsigned char s_raw[];
    // layout: sort buffer [sortcap] u64 | boxes [mbound up to 32] BoxA | areas [same] f32 | alive/mask words;
    // when longer lists are cut down before the sort (sortcap < cap) the scan fills the mask region first
    uint64_t *s_c = reinterpret_cast<uint64_t *>(s_raw);
    const int mpad = (p.mbound + 31) & ~31;  // whole words of boxes: the mask reads the padding
    BoxA *s_box = reinterpret_cast<BoxA *>(s_c + p.sortcap);
    float *s_area = reinterpret_cast<float *>(s_box + mpad);
    uint32_t *s_bits = reinterpret_cast<uint32_t *>(s_area + mpad);
    const bool trims = p.sortcap < p.cap;
    uint64_t *s_in = trims ? reinterpret_cast<uint64_t *>(s_bits) : s_c;
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
        constexpr int kInFlight = 4;  // loads issued before the first is used
        for (int v0 = 0; v0 < nv; v0 += kInFlight * kNmsThreads) {
            uint4 d[kInFlight];
#pragma unroll
            for (int u = 0; u < kInFlight; u++) {
                const int v = v0 + u * kNmsThreads + tid;
                d[u] = make_uint4(0, 0, 0, 0);
                if (v < nv)
                    d[u] = load_stream(vb + v);
            }
#pragma unroll
            for (int u = 0; u < kInFlight; u++) {
                const int v = v0 + u * kNmsThreads + tid;
                const float f[4] = {__uint_as_float(d[u].x), __uint_as_float(d[u].y), __uint_as_float(d[u].z),
                                    __uint_as_float(d[u].w)};
                const int first = v * 4 - head;  // index of f[0] in the row
                bool ok[4];
                int cnt = 0;
                if (v < nv && first >= 0 && first + 4 <= p.N) {
#pragma unroll
                    for (int e = 0; e < 4; e++)
                        ok[e] = f[e] > p.score_thr;
                } else {
#pragma unroll
                    for (int e = 0; e < 4; e++)
                        ok[e] = v < nv && first + e >= 0 && first + e < p.N && f[e] > p.score_thr;
                }
#pragma unroll
                for (int e = 0; e < 4; e++)
                    cnt += ok[e] ? 1 : 0;
                // one shared-memory atomic per warp and round: the lanes take consecutive slots
                int incl = cnt;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int n = __shfl_up_sync(kFullMask, incl, o);
                    if (lane >= o)
                        incl += n;
                }
                const int total = __shfl_sync(kFullMask, incl, 31);
                if (total != 0) {
                    int base = 0;
                    if (lane == 0)
                        base = atomicAdd(&s_count, total);
                    int pos = __shfl_sync(kFullMask, base, 0) + incl - cnt;
#pragma unroll
                    for (int e = 0; e < 4; e++)
                        if (ok[e]) {
                            if (pos < p.cap)
                                s_in[pos] = make_cand(order_key(f[e]), static_cast<uint32_t>(first + e));
                            pos++;
                        }
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
    } else if (trims) {
        // a list longer than the sort buffer is first cut to the part that matters
        if (nc > p.sortcap) {
            nc = nms_trim_candidates(s_in, s_c, nc, p.pre_topk, p.sortcap, &s_count, s_hist, s_pick);
        } else {
            for (int i = tid; i < nc; i += kNmsThreads)
                s_c[i] = s_in[i];
            __syncthreads();
        }
    }

    // ---- order: bitonic sort, descending ----
    if (nc <= kNmsRegSorted) {
        sort_in_registers(s_c, nc);
    } else {
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
    }
    int M = nc;
    if (p.pre_topk > 0 && M > p.pre_topk)
        M = p.pre_topk;
    int max_out = M;
    if (p.max_out > 0 && p.max_out < M)
        max_out = p.max_out;

    // ---- boxes of the ordered candidates ----
    bool odd_area = false;  // a box of positive extent whose area is outside [1e-28, 1e28] (or not a number)
    for (int i = tid; i < M; i += kNmsThreads) {
        const uint32_t idx = cand_idx(s_c[i]);
        float4 raw;
        if (p.box_cstride == 0)
            raw = *reinterpret_cast<const float4 *>(brow + static_cast<int64_t>(idx) * 4);
        else
            raw = make_float4(brow[idx], brow[p.box_cstride + idx], brow[2 * p.box_cstride + idx], brow[3 * p.box_cstride + idx]);
        const BoxA bx = to_corners(raw, p.center_point_box);
        const float area = box_area(bx);
        s_box[i] = bx;
        s_area[i] = area;
        if (bx.x2 > bx.x1 && bx.y2 > bx.y1 && !(area >= 1e-28f && area <= 1e28f))
            odd_area = true;
    }
    const bool areas_in_range = __syncthreads_or(odd_area ? 1 : 0) == 0;
    int32_t *kept = p.kept + static_cast<int64_t>(prob) * p.kept_cap;
    int nkept = 0;
    if (p.use_mask) {
        // ---- IoU bit mask: row i, word w covers boxes 32w .. 32w+31 (only j > i) ----
        // A warp takes one row at a time with box i in registers; for each word from the diagonal one on, lane l
        // tests box 32w + l (one conflict-free 16-byte read each) and the ballot is the word; lane w keeps it,
        // and the row is stored with one write.  Boxes past M are read from the padding and masked away.
        const int words = (M + 31) / 32;
        constexpr int kWarps = kNmsThreads / 32;
        const uint32_t last_valid = (M & 31) ? ((1u << (M & 31)) - 1u) : 0xFFFFFFFFu;
        const IouTest test = make_iou_test(p.iou_thr, areas_in_range);
        // words before the diagonal one are never read; bits of boxes up to i in the diagonal word and of the
        // padding past M are left as they come: the sweep masks both
        auto exact_row = [&](int i) {
            const BoxA bi = s_box[i];
            const float ai = s_area[i];
            for (int w = i >> 5; w < words; w++) {
                const bool over = iou_of(s_box[w * 32 + lane], s_area[w * 32 + lane], bi, ai) > p.iou_thr;
                const uint32_t bits = __ballot_sync(kFullMask, over);
                if (lane == 0)
                    s_bits[i * words + w] = bits;
            }
        };
        if (test.quick) {
            // two rows (an even one and its successor share the diagonal word) against each column box read
            for (int i = 2 * warp; i < M; i += 2 * kWarps) {
                const bool two = i + 1 < M;
                const BoxA b0 = s_box[i], b1 = s_box[i + 1];
                const float a0 = s_area[i], a1 = s_area[i + 1];
                bool doubt = false;
                for (int w = i >> 5; w < words; w++) {
                    const BoxA bj = s_box[w * 32 + lane];
                    const float aj = s_area[w * 32 + lane];
                    const uint32_t m0 = __ballot_sync(kFullMask, iou_exceeds_quick(bj, aj, b0, a0, test, doubt));
                    const uint32_t m1 = __ballot_sync(kFullMask, iou_exceeds_quick(bj, aj, b1, a1, test, doubt));
                    if (lane == 0) {
                        s_bits[i * words + w] = m0;
                        if (two)
                            s_bits[(i + 1) * words + w] = m1;
                    }
                }
                if (__any_sync(kFullMask, doubt)) {
                    exact_row(i);
                    if (two)
                        exact_row(i + 1);
                }
            }
        } else {
            for (int i = warp; i < M; i += kWarps)
                exact_row(i);
        }
        __syncthreads();
        // ---- sweep: warp 0, 32 boxes at a time; lane v holds the removed word v (words <= 16 here) ----
        if (warp == 0) {
            uint32_t removed = 0;
            for (int w = 0; w < words && nkept < max_out; w++) {
                const int base = w * 32, i_l = base + lane;
                uint32_t cur = __shfl_sync(kFullMask, removed, w);
                if (w == words - 1)
                    cur |= ~last_valid;
                const uint32_t diag = i_l < M ? s_bits[i_l * words + w] & ~((2u << lane) - 1u) : 0u;  // boxes after i_l only
                // the 32 boxes of the word in order: a box still alive when its turn comes removes its later ones
#pragma unroll
                for (int b = 0; b < 32; b++) {
                    const uint32_t d = __shfl_sync(kFullMask, diag, b);
                    if (!((cur >> b) & 1u))
                        cur |= d;
                }
                const uint32_t kb = ~cur;  // the kept boxes of this word
                const int r = nkept + __popc(kb & ((1u << lane) - 1u));
                if (((kb >> lane) & 1u) && r < max_out)
                    kept[r] = static_cast<int32_t>(cand_idx(s_c[i_l]));
                nkept += __popc(kb);
                if (nkept >= max_out) {
                    nkept = max_out;
                    break;
                }
                uint32_t acc = 0;
                const bool later = lane > w && lane < words;
#pragma unroll
                for (int b = 0; b < 32; b++)
                    if (((kb >> b) & 1u) && later)
                        acc |= s_bits[(base + b) * words + lane];
                removed |= acc;
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
    int cap, sortcap, mbound, kept_cap, use_mask;
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
    // with a pre-selection that fits half the candidate slots, the sort buffer is half as long and the scan
    // writes into the (then larger) mask region
    pl->sortcap = (d.pre_topk > 0 && d.pre_topk <= cap / 2) ? cap / 2 : cap;
    if (pl->sortcap < kNmsRegSorted)
        pl->sortcap = kNmsRegSorted;  // the register sort exchanges through all of it
    size_t region = bits_bytes;
    if (pl->sortcap < cap && region < static_cast<size_t>(cap) * 8)
        region = static_cast<size_t>(cap) * 8;
    pl->smem = static_cast<size_t>(pl->sortcap) * 8 + static_cast<size_t>((mbound + 31) / 32 * 32) * (16 + 4) + region;
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
    p.sortcap = pl.sortcap;
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
