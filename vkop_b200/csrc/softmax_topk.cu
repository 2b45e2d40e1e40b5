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

namespace vkop_cuda {

constexpr int kCandCap = 1024;        // candidate slots of the chunk filter
constexpr int kChunkMaxK = 128;       // largest k served by the chunk path
constexpr int kMergeMaxSlots = 4096;  // candidates one row may gather for its selection
constexpr int kListCapMax = 512;      // most candidates one chunk publishes

struct ChunkParams {
    const void *logits;
    int64_t rows, cols, row_stride;
    int k, splits;
    int vps;        // 16-byte vectors per split
    int list_cap;   // candidates a chunk may publish (splits > 1)
    float inv_t;
    int value_kind, index_dtype, negate, need_sum;
    int64_t index_offset;
    void *out_values, *out_indices;
    unsigned long long *lists;  // [rows][splits][2 + list_cap]: header (m, s, count, -) then candidates
    unsigned int *counters;     // [rows] arrival counters, zero between launches
    uint32_t *packets_out;      // non-null: emit one packet per row instead of values/indices
};

#ifdef VKOP_PHASE_PROF
// Development aid, compiled only on request: per-CTA timestamps of the kernel's phases.
__device__ unsigned long long g_phase_prof[16384 * 16];
__device__ __forceinline__ void prof_mark(int slot) {
    if (threadIdx.x == 0 && blockIdx.x < 16384) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        g_phase_prof[blockIdx.x * 16 + slot] = t;
    }
}
#define PROF_MARK(s) prof_mark(s)
#else
#define PROF_MARK(s)
#endif

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Where a ranked survivor goes: the final outputs, a packet, or a candidate list.
template <typename T>
__device__ __forceinline__ void emit(const ChunkParams &p, int64_t row, int rank, uint64_t comp, float m, float s,
                                     unsigned long long *list_out) {
    if (list_out) {
        list_out[rank] = comp;
        return;
    }
    const uint32_t idx = cand_idx(comp);
    if (p.packets_out) {
        uint32_t *pk = p.packets_out + row * packet_words(p.k);
        pk[4 + rank] = cand_key(comp);
        pk[4 + p.k + rank] = idx + static_cast<uint32_t>(p.index_offset);
        return;
    }
    const int64_t o = row * p.k + rank;
    if (p.value_kind == VKOP_VALUE_RAW) {
        reinterpret_cast<T *>(p.out_values)[o] = reinterpret_cast<const T *>(p.logits)[row * p.row_stride + idx];
    } else {
        store_value<T>(p.out_values, o, softmax_prob(key_to_float(cand_key(comp)), p.inv_t, m, s));
    }
    store_index(p.out_indices, p.index_dtype, o, static_cast<int64_t>(idx) + p.index_offset);
}

// Warp bitonic sort of one 64-bit value per lane, descending by lane.
__device__ __forceinline__ uint64_t warp_sort_desc(uint64_t v, int lane) {
#pragma unroll
    for (int size = 2; size <= 32; size <<= 1) {
#pragma unroll
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            const uint64_t other = __shfl_xor_sync(kFullMask, v, stride);
            const bool desc_block = (lane & size) == 0;
            const bool low_lane = (lane & stride) == 0;
            const uint64_t hi = v > other ? v : other, lo = v > other ? other : v;
            v = (desc_block == low_lane) ? hi : lo;
        }
    }
    return v;
}

// Exact selection of the best min(k, n) of n distinct candidates held in shared
// memory (list[0..n)); `work` is a second region of at least n slots.  The
// survivors are emitted at their rank.  Executed by the whole CTA; list and
// work are clobbered.
template <typename T, int THREADS>
__device__ void select_and_emit(const ChunkParams &p, int64_t row, uint64_t *list, int n, uint64_t *work, float M,
                                float S, unsigned long long *list_out, int *s_tmp) {
    constexpr int NW = THREADS / 32;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int k = p.k;
    // ---- narrow: r-th largest key of every full group of 32, minimised over the groups ----
    const int nfull = n / 32;
    const int r = nfull > 0 ? (k + nfull - 1) / nfull : 99;
    uint64_t *src = list;
    int n2 = n;
    if (n > 2 * k + 32 && r <= 8) {
        if (tid == 0) {
            s_tmp[0] = 0x7FFFFFFF;  // threshold key >> 1 (kept positive for atomicMin on int)
            s_tmp[1] = 0;
        }
        __syncthreads();
        for (int g = warp; g < nfull; g += NW) {
            uint32_t cur = cand_key(list[g * 32 + lane]);
            uint32_t rth = 0;
            for (int i = 0; i < r; i++) {
                rth = __reduce_max_sync(kFullMask, cur);
                const unsigned b = __ballot_sync(kFullMask, cur == rth);
                if (lane == __ffs(b) - 1)
                    cur = 0;
            }
            if (lane == 0)
                atomicMin(&s_tmp[0], static_cast<int>(rth >> 1));
        }
        __syncthreads();
        const uint32_t tkey = static_cast<uint32_t>(s_tmp[0]) << 1;  // rounded down: keeps the bound valid
        for (int i = tid; i < n; i += THREADS) {
            const uint64_t c = list[i];
            if (cand_key(c) >= tkey) {
                const int pos = atomicAdd(&s_tmp[1], 1);
                work[pos] = c;
            }
        }
        __syncthreads();
        n2 = s_tmp[1];
        src = work;
        work = list;
    }
    // ---- sort groups of 32, then rank every survivor against the other groups ----
    PROF_MARK(10);
    const int ng = (n2 + 31) / 32;
    for (int g = warp; g < ng; g += NW) {
        const int i = g * 32 + lane;
        uint64_t v = i < n2 ? src[i] : 0ull;
        v = warp_sort_desc(v, lane);
        work[i] = v;
    }
    __syncthreads();
    PROF_MARK(11);
    for (int g = warp; g < ng; g += NW) {
        const uint64_t me = work[g * 32 + lane];
        int rank = lane;
        if (me != 0ull) {
            for (int o = 0; o < ng && rank < k; o++) {
                if (o == g)
                    continue;
                const uint64_t *a = work + o * 32;
                int lo = 0, hi = 32;
#pragma unroll
                for (int step = 0; step < 6; step++) {
                    if (lo < hi) {
                        const int mid = (lo + hi) >> 1;
                        if (a[mid] > me)
                            lo = mid + 1;
                        else
                            hi = mid;
                    }
                }
                rank += lo;
            }
            if (rank < k)
                emit<T>(p, row, rank, me, M, S, list_out);
        }
    }
}

// Exact selection of the kk best (key, ~index) values of a chunk by an 8-bit
// most-significant-digit radix select over the 64-bit candidate value.  The
// chunk is re-read from memory.  Leaves exactly kk candidates in s_cand.
template <typename T, int THREADS>
__device__ __noinline__ void select_fallback(const uint4 *vbase, int64_t v0, int64_t v1, int head, int64_t cols,
                                             int negate, int kk, uint64_t *s_cand, int *s_count, int *s_hist,
                                             int *s_pick) {
    constexpr int EPV = Elem<T>::kPerVec;
    const int tid = threadIdx.x;
    uint64_t prefix = 0, mask = 0;
    int need = kk;
    for (int pass = 7; pass >= 0; --pass) {
        const int shift = pass * 8;
        for (int i = tid; i < 256; i += THREADS)
            s_hist[i] = 0;
        __syncthreads();
        for (int64_t v = v0 + tid; v < v1; v += THREADS) {
            uint4 d = vbase[v];
            if (negate) {
                const uint32_t x = sizeof(T) == 4 ? 0x80000000u : 0x80008000u;
                d.x ^= x; d.y ^= x; d.z ^= x; d.w ^= x;
            }
            float f[EPV];
            Elem<T>::unpack(d, f);
#pragma unroll
            for (int e = 0; e < EPV; e++) {
                int64_t i = v * EPV + e - head;
                if (i >= 0 && i < cols) {
                    uint64_t c = make_cand(order_key(f[e]), static_cast<uint32_t>(i));
                    if ((c & mask) == prefix)
                        atomicAdd(&s_hist[static_cast<int>(c >> shift) & 255], 1);
                }
            }
        }
        __syncthreads();
        if (tid == 0) {
            int cum = 0, d = 255;
            for (; d > 0; --d) {
                int c = s_hist[d];
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
            break;  // the whole bin is taken: threshold = prefix
    }
    if (tid == 0)
        *s_count = 0;
    __syncthreads();
    for (int64_t v = v0 + tid; v < v1; v += THREADS) {
        uint4 d = vbase[v];
        if (negate) {
            const uint32_t x = sizeof(T) == 4 ? 0x80000000u : 0x80008000u;
            d.x ^= x; d.y ^= x; d.z ^= x; d.w ^= x;
        }
        float f[EPV];
        Elem<T>::unpack(d, f);
#pragma unroll
        for (int e = 0; e < EPV; e++) {
            int64_t i = v * EPV + e - head;
            if (i >= 0 && i < cols) {
                uint64_t c = make_cand(order_key(f[e]), static_cast<uint32_t>(i));
                if (c >= prefix) {
                    int pos = atomicAdd(s_count, 1);
                    if (pos < kCandCap)
                        s_cand[pos] = c;
                }
            }
        }
    }
    __syncthreads();
}

// Gathers the candidate lists of the G parts of one row into shared memory,
// merges their statistics and selects.  Executed by one whole CTA.
// lists: G blocks of `stride` 64-bit words: header word 0 = (m, s) as float
// bits, header word 1 = count; then the candidates.
template <typename T, int THREADS>
__device__ void merge_lists(const ChunkParams &p, int64_t row, const unsigned long long *lists, int64_t stride, int G,
                            uint64_t *s_buf, float *s_red, int *s_int, int *s_tmp) {
    constexpr int NW = THREADS / 32;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // statistics and list offsets (one warp walks the headers)
    if (warp == 0) {
        float m = -INFINITY;
        for (int g = lane; g < G; g += 32)
            m = fmaxf(m, __uint_as_float(static_cast<uint32_t>(__ldcg(lists + g * stride))));
        m = warp_max(m);
        float s = 0.0f;
        int base = 0;
        for (int g0 = 0; g0 < G; g0 += 32) {
            const int g = g0 + lane;
            int cnt = 0;
            if (g < G) {
                const unsigned long long h = __ldcg(lists + g * stride);
                const float mg = __uint_as_float(static_cast<uint32_t>(h));
                const float sg = __uint_as_float(static_cast<uint32_t>(h >> 32));
                if (sg != 0.0f)  // an all -inf part has sum 0 and no defined maximum
                    s += sg * expf(mg - m);
                cnt = static_cast<int>(__ldcg(lists + g * stride + 1));
            }
            int incl = cnt;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(kFullMask, incl, o);
                if (lane >= o)
                    incl += v;
            }
            if (g < G)
                s_int[8 + g] = base + incl - cnt;  // offset of list g
            base += __shfl_sync(kFullMask, incl, 31);
        }
        s = warp_sum(s);
        if (lane == 0) {
            s_red[0] = m;
            s_red[1] = s;
            s_int[0] = base;
        }
    }
    __syncthreads();
    PROF_MARK(8);
    const float M = s_red[0], S = s_red[1];
    const int n = s_int[0];
    // gather: warp per list
    for (int g = warp; g < G; g += NW) {
        const int off = s_int[8 + g];
        const int end = (g + 1 < G) ? s_int[8 + g + 1] : n;
        const unsigned long long *src = lists + g * stride + 2;
        for (int i = lane; i < end - off; i += 32)
            s_buf[off + i] = __ldcg(src + i);
    }
    __syncthreads();
    PROF_MARK(9);
    const int nsel = n < p.k ? n : p.k;
    if (p.packets_out && tid == 0) {
        uint32_t *pk = p.packets_out + row * packet_words(p.k);
        pk[0] = __float_as_uint(M);
        pk[1] = __float_as_uint(S);
        pk[2] = static_cast<uint32_t>(nsel);
        pk[3] = 0;
    }
    select_and_emit<T, THREADS>(p, row, s_buf, n, s_buf + ((n + 31) & ~31), M, S, nullptr, s_tmp);
}

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
    PROF_MARK(0);

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

    PROF_MARK(1);
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
    const float c2 = (mx == -INFINITY) ? 0.0f : mz * kLog2e;
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
                st += ex2_approx(fmaf(f[e], c1, -c2));
        }
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
    PROF_MARK(2);

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
    PROF_MARK(3);
    __threadfence();
    __syncthreads();
    PROF_MARK(4);
    if (tid == 0) {
        const unsigned int t = atomicAdd(&p.counters[row], 1u);
        s_last = (t == static_cast<unsigned int>(p.splits) - 1u);
    }
    __syncthreads();
    PROF_MARK(5);
    if (!s_last)
        return;
    __threadfence();
    if (tid == 0)
        p.counters[row] = 0;  // ready for the next launch
    merge_lists<T, THREADS>(p, row, p.lists + row * p.splits * lstride, lstride, p.splits, s_cand, s_red, s_int, s_tmp);
    __syncthreads();
    PROF_MARK(6);
}

// Merge of packets gathered from several GPUs: [shards][rows][packet].
template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS) merge_packets_kernel(const ChunkParams p, const uint32_t *packets, int shards) {
    extern __shared__ __align__(16) uint64_t s_buf[];
    __shared__ float s_red[THREADS / 32];
    __shared__ int s_tmp[2];
    constexpr int NW = THREADS / 32;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t row = blockIdx.x;
    const int k = p.k, pw = packet_words(p.k);
    const int64_t gstride = p.rows * pw;
    const uint32_t *base = packets + row * pw;
    if (warp == 0) {
        float m = -INFINITY;
        for (int g = lane; g < shards; g += 32)
            m = fmaxf(m, __uint_as_float(__ldg(base + g * gstride)));
        m = warp_max(m);
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
        }
    }
    const int slots = shards * k;
    for (int sl = tid; sl < slots; sl += THREADS) {
        const int g = sl / k, j = sl - g * k;
        const uint32_t *pk = base + g * gstride;
        const int cnt = static_cast<int>(__ldg(pk + 2));
        // entries past a part's count are padding: key 0 never beats a valid candidate and is never emitted
        s_buf[sl] = j < cnt ? make_cand(__ldg(pk + 4 + j), __ldg(pk + 4 + k + j)) : 0ull;
    }
    __syncthreads();
    (void)NW;
    select_and_emit<T, THREADS>(p, row, s_buf, slots, s_buf + ((slots + 31) & ~31), s_red[0], s_red[1], nullptr, s_tmp);
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

#ifdef VKOP_PHASE_PROF
extern "C" int vkop_debug_read_phase_prof(unsigned long long *host, size_t count) {
    return cudaMemcpyFromSymbol(host, vkop_cuda::g_phase_prof, count * sizeof(unsigned long long)) == cudaSuccess ? 0 : -4;
}
#endif
