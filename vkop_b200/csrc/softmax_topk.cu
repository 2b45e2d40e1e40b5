// Fused Softmax + TopK, chunk path.
//
// Each CTA owns one chunk of one row and reads it exactly once with coalesced
// 16-byte loads into registers.  From the registers it derives
//   (1) the chunk maximum and a selection threshold T: every thread takes the
//       maximum of its own elements; the r-th largest thread maximum of each
//       warp, minimised over the warps, has at least k elements at or above
//       it, so the chunk's k best are all >= T while only a hundred or two
//       elements pass;
//   (2) sum exp(z - max) with ex2.approx (statistics only);
//   (3) the candidates >= T, compacted into shared memory as 64-bit
//       (key, ~index) values.
// With one chunk per row the CTA then selects: the candidate list is narrowed
// once more with the same group-maximum argument, the survivors are sorted in
// groups of 32 with a warp bitonic network and every survivor finds its final
// rank by binary search in the other groups.  With several chunks per row a
// CTA only publishes its (unsorted) candidates and statistics; the last CTA
// of the row to arrive gathers them and runs that selection once per row.
// Probabilities are evaluated with expf and a true division for the k
// survivors only.
//
// Exactness does not depend on the threshold heuristic: if more candidates
// pass than shared memory holds, if the row holds NaN, or if the chunk is too
// small for a threshold, the chunk is selected with an 8-bit radix select on
// the 64-bit candidate value (re-reading the chunk, which is in L2 by then).
#include "common.cuh"
#include "launchers.h"
#include "select.cuh"

namespace vkop_cuda {

template <typename T, int THREADS, int VECS>
__global__ void __launch_bounds__(THREADS, 1024 / THREADS) softmax_topk_chunk_kernel(const ChunkParams p) {
    constexpr int EPV = Elem<T>::kPerVec;
    constexpr int NW = THREADS / 32;
    extern __shared__ __align__(16) uint64_t s_cand[];  // chunk filter: kCandCap; row selection: 2 * gathered
    __shared__ uint32_t s_wr[NW], s_wm[NW];
    __shared__ float s_red[NW];
    __shared__ int s_int[8 + 1024];
    __shared__ int s_hist[256];
    __shared__ int s_pick[4];
    __shared__ int s_tmp[2];
    __shared__ int s_count;
    __shared__ int s_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t row = blockIdx.x / p.splits;
    const int sp = static_cast<int>(blockIdx.x - row * p.splits);

    const uintptr_t addr = reinterpret_cast<uintptr_t>(p.logits) + static_cast<uintptr_t>(row * p.row_stride) * sizeof(T);
    const int head = static_cast<int>((addr & 15) / sizeof(T));
    const uint4 *vbase = reinterpret_cast<const uint4 *>(addr & ~static_cast<uintptr_t>(15));
    const int64_t nv = (head + p.cols + EPV - 1) / EPV;
    const int64_t v0 = static_cast<int64_t>(sp) * p.vps;
    const int64_t v1 = (v0 + p.vps < nv) ? v0 + p.vps : nv;
    const int nvc = v1 > v0 ? static_cast<int>(v1 - v0) : 0;  // vectors of this chunk
    const uint4 *cbase = vbase + v0;

    if (tid == 0)
        s_count = 0;

    // ---- one pass over memory: the chunk lands in registers ----
    uint4 d[VECS];
#pragma unroll
    for (int j = 0; j < VECS; j++) {
        const int lv = j * THREADS + tid;
        if (lv < nvc)
            d[j] = load_stream(cbase + lv);
        else
            d[j] = make_uint4(Elem<T>::kNegInfWord, Elem<T>::kNegInfWord, Elem<T>::kNegInfWord, Elem<T>::kNegInfWord);
    }
    if (p.negate) {
        const uint32_t x = sizeof(T) == 4 ? 0x80000000u : 0x80008000u;
#pragma unroll
        for (int j = 0; j < VECS; j++) {
            if (j * THREADS + tid < nvc) {
                d[j].x ^= x; d[j].y ^= x; d[j].z ^= x; d[j].w ^= x;
            }
        }
    }
    {
        // ragged first / last vector of the row: elements outside the row become -inf
        const int lv_first = v0 == 0 ? 0 : -1;
        const int lv_last = (v1 == nv) ? nvc - 1 : -1;
#pragma unroll
        for (int j = 0; j < VECS; j++) {
            const int lv = j * THREADS + tid;
            if (lv < nvc && (lv == lv_first || lv == lv_last)) {
                const int lo = lv == lv_first ? head : 0;
                const int64_t end = head + p.cols - (v0 + lv) * EPV;
                const int hi = end < EPV ? static_cast<int>(end) : EPV;
                mask_vector<T>(d[j], lo, hi);
            }
        }
    }

    // ---- thread maximum ----
    float mt = -INFINITY;
#pragma unroll
    for (int j = 0; j < VECS; j++) {
        float f[EPV];
        Elem<T>::unpack(d[j], f);
#pragma unroll
        for (int e = 0; e < EPV; e++)
            mt = fmaxf(mt, f[e]);
    }

    // ---- threshold: r-th largest thread maximum per full warp, min over warps ----
    const int nfullw = nvc >= THREADS ? NW : nvc / 32;
    const int r = nfullw > 0 ? (p.k + nfullw - 1) / nfullw : 33;
    {
        uint32_t cur = order_key(mt);
        const uint32_t wmax = __reduce_max_sync(kFullMask, cur);
        uint32_t rth = 0;
        if (r <= 32 && warp < nfullw) {
            for (int i = 0; i < r; i++) {
                rth = __reduce_max_sync(kFullMask, cur);
                const unsigned b = __ballot_sync(kFullMask, cur == rth);
                if (lane == __ffs(b) - 1)
                    cur = 0;
            }
        } else if (r <= 32) {
            rth = 0xFFFFFFFFu;  // a partly filled warp does not constrain the threshold
        }
        if (lane == 0) {
            s_wr[warp] = rth;
            s_wm[warp] = wmax;
        }
    }
    __syncthreads();
    const uint32_t tkey = __reduce_min_sync(kFullMask, lane < NW ? s_wr[lane] : 0xFFFFFFFFu);
    const uint32_t mkey = __reduce_max_sync(kFullMask, lane < NW ? s_wm[lane] : 0u);
    const float T_thr = key_to_float(tkey);
    const float mx = key_to_float(mkey);           // chunk maximum of the stored logits
    const float mz = __fmul_rn(mx, p.inv_t);        // chunk maximum of z = x * inv_t
    const float c1 = p.inv_t * kLog2e;
    const float mref = (mx == -INFINITY) ? 0.0f : mx;  // reference of the exp-sum: 2^((x - mx) * c1) = exp(z - mz)
    // No usable threshold (tiny chunk, or only -inf maxima): every valid element is a candidate.
    const bool allpass = tkey == 0u || T_thr == -INFINITY;
    const uint32_t ebase = static_cast<uint32_t>(v0 * EPV - head);  // row index of the chunk's first slot

    // ---- exp-sum (statistics) and candidate compaction ----
    float st = 0.0f;
    if (p.need_sum) {
#pragma unroll
        for (int j = 0; j < VECS; j++) {
            float f[EPV];
            Elem<T>::unpack(d[j], f);
#pragma unroll
            for (int e = 0; e < EPV; e++)
                st += ex2_approx((f[e] - mref) * c1);
        }
    } else {
        // no sum to carry a NaN (the maxima pass it over): look for it, and poison the sum that nobody reads
        bool has_nan = false;
#pragma unroll
        for (int j = 0; j < VECS; j++)
            has_nan |= Elem<T>::vector_has_nan(d[j]);
        if (has_nan)
            st = __int_as_float(0x7FC00000);
    }
    if (!allpass) {
        // padding is -inf and T is above -inf: whatever passes is a valid element
        if (!(mt < T_thr)) {
#pragma unroll
            for (int j = 0; j < VECS; j++) {
                float f[EPV];
                Elem<T>::unpack(d[j], f);
#pragma unroll
                for (int e = 0; e < EPV; e++) {
                    if (!(f[e] < T_thr)) {
                        const int pos = atomicAdd(&s_count, 1);
                        if (pos < kCandCap)
                            s_cand[pos] = make_cand(order_key(f[e]), ebase + static_cast<uint32_t>((j * THREADS + tid) * EPV + e));
                    }
                }
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < VECS; j++) {
            float f[EPV];
            Elem<T>::unpack(d[j], f);
            const int lv = j * THREADS + tid;
#pragma unroll
            for (int e = 0; e < EPV; e++) {
                const int64_t i = (v0 + lv) * EPV + e - head;
                if (lv < nvc && i >= 0 && i < p.cols) {
                    const int pos = atomicAdd(&s_count, 1);
                    if (pos < kCandCap)
                        s_cand[pos] = make_cand(order_key(f[e]), static_cast<uint32_t>(i));
                }
            }
        }
    }
    st = warp_sum(st);
    if (lane == 0)
        s_red[warp] = st;
    __syncthreads();
    const float S = warp_sum(lane < NW ? s_red[lane] : 0.0f);
    int C = s_count;

    // valid elements of this chunk, and how many of them the chunk must deliver
    int64_t e0 = v0 * EPV - head, e1 = v1 * EPV - head;
    if (e0 < 0) e0 = 0;
    if (e1 > p.cols) e1 = p.cols;
    const int64_t nvalid = e1 > e0 ? e1 - e0 : 0;
    const int kk = nvalid < p.k ? static_cast<int>(nvalid) : p.k;

    // A NaN in the chunk poisons the sum; NaN elements rank first but are
    // invisible to the thread maxima, so the threshold filter cannot be trusted.
    if (C > kCandCap || S != S) {
        __syncthreads();
        select_fallback<T, THREADS>(vbase, v0, v1, head, p.cols, p.negate, kk, s_cand, &s_count, s_hist, s_pick);
        C = s_count;
    }

    if (p.splits == 1) {
        if (p.packets_out && tid == 0) {
            uint32_t *pk = p.packets_out + row * packet_words(p.k);
            pk[0] = __float_as_uint(mz);
            pk[1] = __float_as_uint(S);
            pk[2] = static_cast<uint32_t>(kk);
            pk[3] = 0;
        }
        select_and_emit<T, THREADS>(p, row, s_cand, C, s_cand + kCandCap, mz, S, nullptr, s_tmp);
        return;
    }

    // ---- several chunks per row: publish the candidates; the last CTA of the row selects ----
    const int64_t lstride = 2 + p.list_cap;
    unsigned long long *mylist = p.lists + (row * p.splits + sp) * lstride;
    if (C > p.list_cap) {
        // more candidates than a chunk may publish: cut them down to the chunk's own k best
        select_and_emit<T, THREADS>(p, row, s_cand, C, s_cand + kCandCap, 0.0f, 0.0f, mylist + 2, s_tmp);
        C = kk;
    } else {
        for (int i = tid; i < C; i += THREADS)
            mylist[2 + i] = s_cand[i];
    }
    if (tid == 0) {
        mylist[0] = (static_cast<unsigned long long>(__float_as_uint(S)) << 32) | __float_as_uint(mz);
        mylist[1] = static_cast<unsigned long long>(C);
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned int t = atomicAdd(&p.counters[row], 1u);
        s_last = (t == static_cast<unsigned int>(p.splits) - 1u);
    }
    __syncthreads();
    if (!s_last)
        return;
    __threadfence();
    if (tid == 0)
        p.counters[row] = 0;  // ready for the next launch
    merge_lists<T, THREADS>(p, row, p.lists + row * p.splits * lstride, lstride, p.splits, s_cand, nullptr, s_red, s_int, s_tmp);
    __syncthreads();
}

// Merge of packets gathered from several GPUs: [shards][rows][packet].
// A packet lists its shard's candidates best first, so the lists are sorted: the rank of a candidate in
// the row is its place in its own list plus, for every other list, the number of entries there that beat
// it, found by binary search (candidates are distinct 64-bit values, key then lower index, so the order
// is total).  One thread per candidate, no sort, no compaction, one barrier.  A full packet's last entry
// is reached by k candidates of its shard alone, so candidates below the largest of those last entries
// cannot be among the row's k best and are not ranked at all.
template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS) merge_packets_kernel(const ChunkParams p, const uint32_t *packets, int shards) {
    extern __shared__ __align__(16) uint64_t s_buf[];  // [shards][k], padding entries 0 (below every candidate)
    __shared__ float s_red[2];
    __shared__ uint32_t s_bound;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t row = blockIdx.x;
    const int k = p.k, pw = packet_words(p.k);
    const int64_t gstride = p.rows * pw;
    const uint32_t *base = packets + row * pw;
    const int slots = shards * k;
    for (int sl = tid; sl < slots; sl += THREADS) {
        const int g = sl / k, j = sl - g * k;
        const uint32_t *pk = base + g * gstride;
        const int cnt = static_cast<int>(__ldg(pk + 2));
        const uint32_t key = __ldg(pk + 4 + j), idx = __ldg(pk + 4 + k + j);
        s_buf[sl] = j < cnt ? make_cand(key, idx) : 0ull;
    }
    if (warp == 0) {
        float m = -INFINITY;
        uint32_t bound = 0u;
        for (int g = lane; g < shards; g += 32) {
            const uint32_t *pk = base + g * gstride;
            m = fmaxf(m, __uint_as_float(__ldg(pk)));
            if (static_cast<int>(__ldg(pk + 2)) >= k) {
                const uint32_t last = __ldg(pk + 4 + k - 1);
                bound = last > bound ? last : bound;
            }
        }
        m = warp_max(m);
        bound = __reduce_max_sync(kFullMask, bound);
        float s = 0.0f;
        for (int g = lane; g < shards; g += 32) {
            const float mg = __uint_as_float(__ldg(base + g * gstride)), sg = __uint_as_float(__ldg(base + g * gstride + 1));
            if (sg != 0.0f)
                s += sg * expf(mg - m);
        }
        s = warp_sum(s);
        if (lane == 0) {
            s_red[0] = m;
            s_red[1] = s;
            s_bound = bound;
        }
    }
    __syncthreads();
    const float M = s_red[0], S = s_red[1];
    const uint32_t bound = s_bound;
    for (int sl = tid; sl < slots; sl += THREADS) {
        const uint64_t c = s_buf[sl];
        if (c == 0ull || cand_key(c) < bound)
            continue;
        const int g = sl / k;
        int rank = sl - g * k;
        for (int g2 = 0; g2 < shards && rank < k; g2++) {
            if (g2 == g)
                continue;
            const uint64_t *a = s_buf + g2 * k;  // sorted descending: how many of its entries beat c
            int lo = 0, hi = k;
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (a[mid] > c)
                    lo = mid + 1;
                else
                    hi = mid;
            }
            rank += lo;
        }
        if (rank < k)
            emit<T>(p, row, rank, c, M, S, nullptr);
    }
}

// ---------------------------------------------------------------------------
// host side

struct ChunkConfig {
    int threads, vecs;
};
static const ChunkConfig kConfigs[] = {{128, 1}, {128, 2}, {256, 4}, {512, 4}, {512, 8}};
constexpr int kNumConfigs = sizeof(kConfigs) / sizeof(kConfigs[0]);

static inline int elem_size(int dtype) { return dtype == VKOP_F32 ? 4 : 2; }

// Picks the CTA shape and the number of chunks per row.
int plan_chunk(const vkop_softmax_topk_desc &d, ChunkPlan *plan) {
    const int epv = 16 / elem_size(d.dtype);
    const int64_t nv_max = (d.cols + 2 * (epv - 1)) / epv;  // allows for an unaligned row start
    if (d.k > kChunkMaxK)
        return VKOP_UNSUPPORTED;
    int cfg = -1, splits = 0;
    if (d.splits > 0) {
        splits = d.splits;
        int64_t vps = (nv_max + splits - 1) / splits;
        for (int c = 0; c < kNumConfigs; c++)
            if (static_cast<int64_t>(kConfigs[c].threads) * kConfigs[c].vecs >= vps) {
                cfg = c;
                break;
            }
        if (cfg < 0)
            return VKOP_UNSUPPORTED;
    } else {
        const int64_t target_ctas = 2 * 148;
        const int64_t cap_max = static_cast<int64_t>(kConfigs[kNumConfigs - 1].threads) * kConfigs[kNumConfigs - 1].vecs;
        if (d.rows >= target_ctas / 2 || nv_max <= 256) {
            // enough rows to fill the machine: one CTA shape that covers the row, or the largest
            cfg = kNumConfigs - 1;
            for (int c = 0; c < kNumConfigs; c++)
                if (static_cast<int64_t>(kConfigs[c].threads) * kConfigs[c].vecs >= nv_max) {
                    cfg = c;
                    break;
                }
            splits = static_cast<int>((nv_max + cap_max - 1) / cap_max);
            if (cfg != kNumConfigs - 1)
                splits = 1;
        } else {
            // few rows: more, smaller chunks so that every SM has work
            for (int c = kNumConfigs - 1; c >= 1; c--) {
                int64_t cap = static_cast<int64_t>(kConfigs[c].threads) * kConfigs[c].vecs;
                int64_t s = (nv_max + cap - 1) / cap;
                if (s * d.k > kMergeMaxSlots || s > 1024)
                    break;  // the row selection could not hold that many candidate lists
                cfg = c;
                splits = static_cast<int>(s);
                if (d.rows * s >= target_ctas)
                    break;
            }
        }
    }
    if (cfg < 0)
        return VKOP_UNSUPPORTED;
    if (splits < 1)
        splits = 1;
    if (static_cast<int64_t>(splits) * d.k > kMergeMaxSlots || splits > 1024)
        return VKOP_UNSUPPORTED;
    plan->cfg = cfg;
    plan->splits = splits;
    plan->vps = (nv_max + splits - 1) / splits;
    if (plan->vps > static_cast<int64_t>(kConfigs[cfg].threads) * kConfigs[cfg].vecs)
        return VKOP_UNSUPPORTED;
    int list_cap = kMergeMaxSlots / splits;
    if (list_cap > kListCapMax)
        list_cap = kListCapMax;
    plan->list_cap = list_cap;  // >= k by the check above
    plan->counters_bytes = splits > 1 ? ((static_cast<size_t>(d.rows) * 4 + 255) / 256) * 256 : 0;
    plan->packets_bytes = splits > 1 ? static_cast<size_t>(d.rows) * splits * (2 + list_cap) * 8 : 0;
    size_t slots = splits > 1 ? 2 * (static_cast<size_t>(splits) * list_cap + 32) : 0;
    if (slots < 2 * static_cast<size_t>(kCandCap))
        slots = 2 * kCandCap;
    plan->smem_bytes = slots * 8;
    return VKOP_OK;
}

template <typename T, int THREADS, int VECS>
static int launch_cfg(const ChunkParams &p, const ChunkPlan &plan, cudaStream_t stream) {
    auto kern = softmax_topk_chunk_kernel<T, THREADS, VECS>;
    if (plan.smem_bytes > 32 * 1024) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(plan.smem_bytes)) !=
            cudaSuccess)
            return VKOP_CUDA_ERROR;
    }
    const unsigned grid = static_cast<unsigned>(p.rows * p.splits);
    kern<<<grid, THREADS, plan.smem_bytes, stream>>>(p);
    note_launch();
    return check_launch();
}

template <typename T>
static int launch_dtype(const ChunkParams &p, const ChunkPlan &plan, cudaStream_t stream) {
    switch (plan.cfg) {
    case 0: return launch_cfg<T, 128, 1>(p, plan, stream);
    case 1: return launch_cfg<T, 128, 2>(p, plan, stream);
    case 2: return launch_cfg<T, 256, 4>(p, plan, stream);
    case 3: return launch_cfg<T, 512, 4>(p, plan, stream);
    default: return launch_cfg<T, 512, 8>(p, plan, stream);
    }
}

// Launches the chunk path.  packets_out != nullptr selects packet emission.
int launch_chunk(const vkop_softmax_topk_desc &d, const ChunkPlan &plan, const void *logits, void *out_values,
                 void *out_indices, void *packets_out, void *workspace, int need_sum, cudaStream_t stream) {
    if (d.rows == 0)
        return VKOP_OK;
    if (d.rows * plan.splits > 0x7FFFFFFFll)
        return VKOP_UNSUPPORTED;
    ChunkParams p;
    p.logits = logits;
    p.rows = d.rows;
    p.cols = d.cols;
    p.row_stride = d.row_stride ? d.row_stride : d.cols;
    p.k = d.k;
    p.splits = plan.splits;
    p.vps = static_cast<int>(plan.vps);
    p.list_cap = plan.list_cap;
    p.inv_t = d.inv_temperature;
    p.value_kind = d.value_kind;
    p.index_dtype = d.index_dtype;
    p.negate = d.largest ? 0 : 1;
    p.need_sum = need_sum;
    p.index_offset = d.index_offset;
    p.out_values = out_values;
    p.out_indices = out_indices;
    p.counters = reinterpret_cast<unsigned int *>(workspace);
    p.lists = reinterpret_cast<unsigned long long *>(static_cast<char *>(workspace) + plan.counters_bytes);
    p.packets_out = reinterpret_cast<uint32_t *>(packets_out);
    switch (d.dtype) {
    case VKOP_F32: return launch_dtype<float>(p, plan, stream);
    case VKOP_F16: return launch_dtype<__half>(p, plan, stream);
    case VKOP_BF16: return launch_dtype<__nv_bfloat16>(p, plan, stream);
    default: return VKOP_INVALID_ARG;
    }
}

int launch_merge(const vkop_softmax_topk_desc &d, const void *packets, int shards, void *out_values,
                 void *out_indices, cudaStream_t stream) {
    if (d.rows == 0)
        return VKOP_OK;
    if (static_cast<int64_t>(shards) * d.k > kMergeMaxSlots || d.k > kChunkMaxK)
        return VKOP_UNSUPPORTED;
    ChunkParams p = {};
    p.logits = nullptr;
    p.rows = d.rows;
    p.cols = d.cols;
    p.row_stride = d.row_stride ? d.row_stride : d.cols;
    p.k = d.k;
    p.splits = shards;
    p.inv_t = d.inv_temperature;
    p.value_kind = VKOP_VALUE_PROBABILITY;
    p.index_dtype = d.index_dtype;
    p.index_offset = 0;  // packets carry global indices
    p.out_values = out_values;
    p.out_indices = out_indices;
    const size_t smem = 2 * (static_cast<size_t>(shards) * d.k + 32) * 8;
    constexpr int THREADS = 256;
    const unsigned grid = static_cast<unsigned>(d.rows);
    const uint32_t *pk = reinterpret_cast<const uint32_t *>(packets);
#define VKOP_MERGE(T)                                                                                       \
    do {                                                                                                    \
        auto kern = merge_packets_kernel<T, THREADS>;                                                       \
        if (smem > 32 * 1024 &&                                                                             \
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != \
                cudaSuccess)                                                                                \
            return VKOP_CUDA_ERROR;                                                                         \
        kern<<<grid, THREADS, smem, stream>>>(p, pk, shards);                                               \
    } while (0)
    switch (d.dtype) {
    case VKOP_F32: VKOP_MERGE(float); break;
    case VKOP_F16: VKOP_MERGE(__half); break;
    case VKOP_BF16: VKOP_MERGE(__nv_bfloat16); break;
    default: return VKOP_INVALID_ARG;
    }
#undef VKOP_MERGE
    note_launch();
    return check_launch();
}

}  // namespace vkop_cuda

