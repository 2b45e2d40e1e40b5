// Fused Softmax + TopK, chunk path.
//
// Each CTA owns one chunk of one row and reads it exactly once with coalesced
// 16-byte loads into registers.  From the registers it derives
//   (1) the chunk maximum and a selection threshold T: every thread takes the
//       maximum of its own elements; the r-th largest thread maximum of each
//       warp, minimised over the warps, has at least k elements at or above
//       it, so the chunk's k best are all >= T while only a few hundred
//       elements pass;
//   (2) sum exp(z - max) with ex2.approx (statistics only);
//   (3) the candidates >= T, compacted into shared memory and ranked exactly
//       by (key descending, index ascending).
// A chunk emits a packet (max, sum, k best).  With several chunks per row the
// last CTA to finish a row merges the packets; the merge ranks each candidate
// by binary search in the other (sorted) lists.  Probabilities are evaluated
// with expf and a true division for the k survivors only.
//
// Exactness does not depend on the threshold heuristic: if more candidates
// pass than shared memory holds, or the row holds NaN, the chunk is re-read
// and selected with an 8-bit radix select on the 64-bit (key, ~index) value.
#include "common.cuh"
#include "launchers.h"

namespace vkop_cuda {

constexpr int kCandCap = 1024;     // candidate slots of the chunk filter
constexpr int kChunkMaxK = 128;    // largest k served by the chunk path
constexpr int kMergeMaxSlots = 8192;  // splits * k limit of the in-kernel merge

struct ChunkParams {
    const void *logits;
    int64_t rows, cols, row_stride;
    int k, splits;
    int64_t vps;  // 16-byte vectors per split
    float inv_t;
    int value_kind, index_dtype, negate, need_sum;
    int64_t index_offset;
    void *out_values, *out_indices;
    uint32_t *packets;       // [rows][splits][packet_words] scratch (splits > 1)
    unsigned int *counters;  // [rows] arrival counters, zero between launches
    uint32_t *packets_out;   // non-null: emit one packet per row instead of values/indices
};

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Final emission of one ranked survivor.
template <typename T>
__device__ __forceinline__ void emit(const ChunkParams &p, int64_t row, int rank, uint64_t comp, float m, float s) {
    uint32_t idx = cand_idx(comp);
    if (p.packets_out) {
        uint32_t *pk = p.packets_out + row * packet_words(p.k);
        pk[4 + rank] = cand_key(comp);
        pk[4 + p.k + rank] = idx + static_cast<uint32_t>(p.index_offset);
        return;
    }
    int64_t o = row * p.k + rank;
    if (p.value_kind == VKOP_VALUE_RAW) {
        reinterpret_cast<T *>(p.out_values)[o] = reinterpret_cast<const T *>(p.logits)[row * p.row_stride + idx];
    } else {
        store_value<T>(p.out_values, o, softmax_prob(key_to_float(cand_key(comp)), p.inv_t, m, s));
    }
    store_index(p.out_indices, p.index_dtype, o, static_cast<int64_t>(idx) + p.index_offset);
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

// Merge of G packets of one row (executed by one whole CTA).
template <typename T, int THREADS>
__device__ void merge_row(const ChunkParams &p, int64_t row, const uint32_t *pk_base, int64_t pk_stride, int G,
                          uint64_t *s_cand, float *s_red, int *s_int) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int NW = THREADS / 32;
    const int k = p.k;
    // statistics
    float m = -INFINITY;
    int total = 0;
    for (int g = tid; g < G; g += THREADS) {
        const uint32_t *pk = pk_base + g * pk_stride;
        m = fmaxf(m, __uint_as_float(__ldcg(pk)));
        total += static_cast<int>(__ldcg(pk + 2));
    }
    m = warp_max(m);
    total = __reduce_add_sync(kFullMask, total);
    if (lane == 0) {
        s_red[warp] = m;
        s_int[warp] = total;
    }
    __syncthreads();
    float M = -INFINITY;
    total = 0;
#pragma unroll
    for (int w = 0; w < NW; w++) {
        M = fmaxf(M, s_red[w]);
        total += s_int[w];
    }
    __syncthreads();
    float s = 0.0f;
    for (int g = tid; g < G; g += THREADS) {
        const uint32_t *pk = pk_base + g * pk_stride;
        float mg = __uint_as_float(__ldcg(pk)), sg = __uint_as_float(__ldcg(pk + 1));
        if (sg != 0.0f)  // an all -inf part has sum 0 and no defined maximum
            s += sg * expf(mg - M);
    }
    s = warp_sum(s);
    if (lane == 0)
        s_red[warp] = s;
    // candidates (own list position = rank inside the own sorted list)
    const int slots = G * k;
    for (int sl = tid; sl < slots; sl += THREADS) {
        int g = sl / k, j = sl - g * k;
        const uint32_t *pk = pk_base + g * pk_stride;
        int cnt = static_cast<int>(__ldcg(pk + 2));
        s_cand[sl] = j < cnt ? make_cand(__ldcg(pk + 4 + j), __ldcg(pk + 4 + k + j)) : 0ull;
    }
    __syncthreads();
    float S = 0.0f;
#pragma unroll
    for (int w = 0; w < NW; w++)
        S += s_red[w];
    const int nsel = total < k ? total : k;
    if (p.packets_out && tid == 0) {
        uint32_t *pk = p.packets_out + row * packet_words(k);
        pk[0] = __float_as_uint(M);
        pk[1] = __float_as_uint(S);
        pk[2] = static_cast<uint32_t>(nsel);
        pk[3] = 0;
    }
    for (int sl = tid; sl < slots; sl += THREADS) {
        uint64_t me = s_cand[sl];
        if (me == 0ull)
            continue;
        int g = sl / k;
        int rank = sl - g * k;
        for (int o = 0; o < G && rank < k; o++) {
            if (o == g)
                continue;
            const uint64_t *a = s_cand + o * k;
            int lo = 0, hi = k;
            while (lo < hi) {
                int mid = (lo + hi) >> 1;
                if (a[mid] > me)
                    lo = mid + 1;
                else
                    hi = mid;
            }
            rank += lo;
        }
        if (rank < k)
            emit<T>(p, row, rank, me, M, S);
    }
}

template <typename T, int THREADS, int VECS>
__global__ void __launch_bounds__(THREADS, 1024 / THREADS) softmax_topk_chunk_kernel(const ChunkParams p) {
    constexpr int EPV = Elem<T>::kPerVec;
    constexpr int NW = THREADS / 32;
    extern __shared__ __align__(16) uint64_t s_cand[];
    __shared__ uint32_t s_wr[NW], s_wm[NW];
    __shared__ float s_red[NW];
    __shared__ int s_int[NW];
    __shared__ int s_hist[256];
    __shared__ int s_pick[4];
    __shared__ int s_count;
    __shared__ int s_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t row = blockIdx.x / p.splits;
    const int sp = static_cast<int>(blockIdx.x - row * p.splits);

    const uintptr_t addr = reinterpret_cast<uintptr_t>(p.logits) + static_cast<uintptr_t>(row * p.row_stride) * sizeof(T);
    const int head = static_cast<int>((addr & 15) / sizeof(T));
    const uint4 *vbase = reinterpret_cast<const uint4 *>(addr & ~static_cast<uintptr_t>(15));
    const int64_t nv = (head + p.cols + EPV - 1) / EPV;
    const int64_t v0 = sp * p.vps;
    const int64_t v1 = (v0 + p.vps < nv) ? v0 + p.vps : nv;
    const int64_t nvc = v1 > v0 ? v1 - v0 : 0;

    if (tid == 0)
        s_count = 0;

    // ---- one pass over memory: the chunk lands in registers ----
    uint4 d[VECS];
#pragma unroll
    for (int j = 0; j < VECS; j++) {
        int64_t v = v0 + j * THREADS + tid;
        if (v < v1)
            d[j] = load_stream(vbase + v);
        else
            d[j] = make_uint4(Elem<T>::kNegInfWord, Elem<T>::kNegInfWord, Elem<T>::kNegInfWord, Elem<T>::kNegInfWord);
    }
    if (p.negate) {
        const uint32_t x = sizeof(T) == 4 ? 0x80000000u : 0x80008000u;
#pragma unroll
        for (int j = 0; j < VECS; j++) {
            int64_t v = v0 + j * THREADS + tid;
            if (v < v1) {
                d[j].x ^= x; d[j].y ^= x; d[j].z ^= x; d[j].w ^= x;
            }
        }
    }
#pragma unroll
    for (int j = 0; j < VECS; j++) {
        int64_t v = v0 + j * THREADS + tid;
        if (v < v1 && (v == 0 || v == nv - 1)) {  // ragged first / last vector of the row
            int lo = v == 0 ? head : 0;
            int64_t end = head + p.cols - v * EPV;
            int hi = end < EPV ? static_cast<int>(end) : EPV;
            mask_vector<T>(d[j], lo, hi);
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
    const int nfullw = nvc >= THREADS ? NW : static_cast<int>(nvc / 32);
    const int r = nfullw > 0 ? (p.k + nfullw - 1) / nfullw : 33;
    {
        uint32_t cur = order_key(mt);
        uint32_t wmax = __reduce_max_sync(kFullMask, cur);
        uint32_t rth = 0;
        if (r <= 32 && warp < nfullw) {
            for (int i = 0; i < r; i++) {
                rth = __reduce_max_sync(kFullMask, cur);
                unsigned b = __ballot_sync(kFullMask, cur == rth);
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
    uint32_t tkey = 0xFFFFFFFFu, mkey = 0;
#pragma unroll
    for (int w = 0; w < NW; w++) {
        tkey = min(tkey, s_wr[w]);
        mkey = max(mkey, s_wm[w]);
    }
    // tkey == 0 ("everything passes") maps to NaN, for which !(x < T) holds for every x
    const float T_thr = key_to_float(tkey);
    const float mx = key_to_float(mkey);           // chunk maximum of the stored logits
    const float mz = __fmul_rn(mx, p.inv_t);        // chunk maximum of z = x * inv_t
    const float c1 = p.inv_t * kLog2e;
    const float c2 = (mx == -INFINITY) ? 0.0f : mz * kLog2e;

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
    if (!(mt < T_thr)) {
#pragma unroll
        for (int j = 0; j < VECS; j++) {
            float f[EPV];
            Elem<T>::unpack(d[j], f);
            const int64_t ibase = (v0 + j * THREADS + tid) * EPV - head;
#pragma unroll
            for (int e = 0; e < EPV; e++) {
                if (!(f[e] < T_thr)) {
                    int64_t i = ibase + e;
                    if (i >= 0 && i < p.cols && (v0 + j * THREADS + tid) < v1) {
                        int pos = atomicAdd(&s_count, 1);
                        if (pos < kCandCap)
                            s_cand[pos] = make_cand(order_key(f[e]), static_cast<uint32_t>(i));
                    }
                }
            }
        }
    }
    st = warp_sum(st);
    if (lane == 0)
        s_red[warp] = st;
    __syncthreads();
    float S = 0.0f;
#pragma unroll
    for (int w = 0; w < NW; w++)
        S += s_red[w];
    int C = s_count;

    // valid elements of this chunk, and how many of them the chunk must emit
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
        for (int c = tid; c < C; c += THREADS) {
            const uint64_t me = s_cand[c];
            int rank = 0;
            for (int j = 0; j < C; j++)
                rank += s_cand[j] > me;
            if (rank < p.k)
                emit<T>(p, row, rank, me, mz, S);
        }
        return;
    }

    // ---- several chunks per row: packet to scratch, last CTA of the row merges ----
    const int pw = packet_words(p.k);
    uint32_t *pk = p.packets + (row * p.splits + sp) * pw;
    if (tid == 0) {
        pk[0] = __float_as_uint(mz);
        pk[1] = __float_as_uint(S);
        pk[2] = static_cast<uint32_t>(kk);
        pk[3] = 0;
    }
    for (int c = tid; c < C; c += THREADS) {
        const uint64_t me = s_cand[c];
        int rank = 0;
        for (int j = 0; j < C; j++)
            rank += s_cand[j] > me;
        if (rank < p.k) {
            pk[4 + rank] = cand_key(me);
            pk[4 + p.k + rank] = cand_idx(me);
        }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        unsigned int t = atomicAdd(&p.counters[row], 1u);
        s_last = (t == static_cast<unsigned int>(p.splits) - 1u);
    }
    __syncthreads();
    if (!s_last)
        return;
    __threadfence();
    if (tid == 0)
        p.counters[row] = 0;  // ready for the next launch
    merge_row<T, THREADS>(p, row, p.packets + row * p.splits * pw, pw, p.splits, s_cand, s_red, s_int);
}

// Merge of packets gathered from several GPUs: [shards][rows][packet].
template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS) merge_packets_kernel(const ChunkParams p, const uint32_t *packets, int shards) {
    extern __shared__ __align__(16) uint64_t s_cand[];
    __shared__ float s_red[THREADS / 32];
    __shared__ int s_int[THREADS / 32];
    const int64_t row = blockIdx.x;
    const int pw = packet_words(p.k);
    merge_row<T, THREADS>(p, row, packets + row * pw, p.rows * pw, shards, s_cand, s_red, s_int);
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
                cfg = c;
                splits = static_cast<int>(s);
                if (d.rows * s >= target_ctas)
                    break;
            }
        }
    }
    if (splits < 1)
        splits = 1;
    if (static_cast<int64_t>(splits) * d.k > kMergeMaxSlots)
        return VKOP_UNSUPPORTED;
    plan->cfg = cfg;
    plan->splits = splits;
    plan->vps = (nv_max + splits - 1) / splits;
    if (plan->vps > static_cast<int64_t>(kConfigs[cfg].threads) * kConfigs[cfg].vecs)
        return VKOP_UNSUPPORTED;
    plan->counters_bytes = splits > 1 ? ((static_cast<size_t>(d.rows) * 4 + 255) / 256) * 256 : 0;
    plan->packets_bytes = splits > 1 ? static_cast<size_t>(d.rows) * splits * packet_words(d.k) * 4 : 0;
    size_t slots = static_cast<size_t>(splits) * d.k;
    if (slots < static_cast<size_t>(kCandCap))
        slots = kCandCap;
    plan->smem_bytes = slots * 8;
    return VKOP_OK;
}

template <typename T, int THREADS, int VECS>
static int launch_cfg(const ChunkParams &p, const ChunkPlan &plan, cudaStream_t stream) {
    auto kern = softmax_topk_chunk_kernel<T, THREADS, VECS>;
    if (plan.smem_bytes > 40 * 1024) {
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
    p.vps = plan.vps;
    p.inv_t = d.inv_temperature;
    p.value_kind = d.value_kind;
    p.index_dtype = d.index_dtype;
    p.negate = d.largest ? 0 : 1;
    p.need_sum = need_sum;
    p.index_offset = d.index_offset;
    p.out_values = out_values;
    p.out_indices = out_indices;
    p.counters = reinterpret_cast<unsigned int *>(workspace);
    p.packets = reinterpret_cast<uint32_t *>(static_cast<char *>(workspace) + plan.counters_bytes);
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
    const size_t smem = static_cast<size_t>(shards) * d.k * 8;
    constexpr int THREADS = 256;
    const unsigned grid = static_cast<unsigned>(d.rows);
    const uint32_t *pk = reinterpret_cast<const uint32_t *>(packets);
#define VKOP_MERGE(T)                                                                                       \
    do {                                                                                                    \
        auto kern = merge_packets_kernel<T, THREADS>;                                                       \
        if (smem > 40 * 1024 &&                                                                             \
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
