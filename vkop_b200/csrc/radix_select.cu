// Fused Softmax + TopK, radix path: large k or rows too long for the chunk
// path (for example one row of 16 Mi elements, k = 1024).
//
// Every CTA owns a contiguous segment of one row.  The k-th best candidate is
// found by a most-significant-digit radix select on the 64-bit value
// (order-preserving key << 32 | ~index): digits of 11, 11 and 10 bits cover the
// key; if equal keys straddle the k-th place the same digits continue over the
// index, which makes the lower index win.  Each pass builds a histogram of the
// current digit in shared memory, adds it to a per-row histogram in global
// memory, and the last CTA of the row to arrive picks the digit and publishes
// the new prefix.  Passes that follow a decided row return at once.  The first
// pass also accumulates the softmax statistics; only it has to come from HBM,
// the later sweeps of a row that fits the L2 are served from there.  A collect
// sweep gathers the k candidates at or above the final threshold and a last
// kernel sorts them and writes probabilities and indices.
#include "common.cuh"
#include "launchers.h"

namespace vkop_cuda {

constexpr int kRadixThreads = 512;
constexpr int kRadixBins = 2048;
constexpr int kRadixPasses = 6;
// digit position (shift, bits) of each pass within the 64-bit candidate value
__constant__ int c_shift[kRadixPasses] = {53, 42, 32, 21, 10, 0};
__constant__ int c_bits[kRadixPasses] = {11, 11, 10, 11, 11, 10};

struct RadixState {
    unsigned long long prefix, mask;
    int need, done, pad0, pad1;
};

struct RadixParams {
    const void *logits;
    int64_t rows, cols, row_stride;
    int k, cpr;       // CTAs per row
    int64_t vpc;      // vectors per CTA segment
    float inv_t;
    int value_kind, index_dtype, negate, need_sum;
    int64_t index_offset;
    void *out_values, *out_indices;
    RadixState *state;          // [rows]
    int *hist;                  // [rows][kRadixBins], zero between passes
    unsigned int *tickets;      // [rows]
    int *cand_count;            // [rows], zero between calls
    float2 *stats;              // [rows][cpr] (max z, sum)
    unsigned long long *cand;   // [rows][k]
};

__device__ __forceinline__ float ex2f(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct Segment {
    const uint4 *vbase;
    int64_t v0, v1;
    int head;
};

template <typename T>
__device__ __forceinline__ Segment segment_of(const RadixParams &p, int64_t row, int part) {
    constexpr int EPV = Elem<T>::kPerVec;
    const uintptr_t addr = reinterpret_cast<uintptr_t>(p.logits) + static_cast<uintptr_t>(row * p.row_stride) * sizeof(T);
    Segment s;
    s.head = static_cast<int>((addr & 15) / sizeof(T));
    s.vbase = reinterpret_cast<const uint4 *>(addr & ~static_cast<uintptr_t>(15));
    const int64_t nv = (s.head + p.cols + EPV - 1) / EPV;
    s.v0 = part * p.vpc;
    s.v1 = s.v0 + p.vpc < nv ? s.v0 + p.vpc : nv;
    return s;
}

// Finds, from the top bin down, the bin holding the need-th element.  One warp.
// Returns the bin, the number of elements above it and its own count.
__device__ void find_bin(const int *s_hist, int nbins, int need, int *bin, int *above, int *count) {
    const int lane = threadIdx.x & 31;
    const int per = nbins / 32;
    const int hi = nbins - 1 - lane * per;  // lane 0 owns the top bins
    int sum = 0;
    for (int i = 0; i < per; i++)
        sum += s_hist[hi - i];
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int v = __shfl_up_sync(kFullMask, incl, o);
        if (lane >= o)
            incl += v;
    }
    const int excl = incl - sum;
    const bool mine = excl < need && need <= incl;
    unsigned who = __ballot_sync(kFullMask, mine);
    int b = 0, a = 0, c = 0;
    if (who == 0) {  // fewer than `need` elements in total: take the lowest bin
        b = 0;
        a = __shfl_sync(kFullMask, incl, 31) - s_hist[0];
        c = s_hist[0];
    } else {
        if (mine) {
            int cum = excl;
            for (int i = 0; i < per; i++) {
                int h = s_hist[hi - i];
                if (cum + h >= need) {
                    b = hi - i;
                    a = cum;
                    c = h;
                    break;
                }
                cum += h;
            }
        }
        const int src = __ffs(who) - 1;
        b = __shfl_sync(kFullMask, b, src);
        a = __shfl_sync(kFullMask, a, src);
        c = __shfl_sync(kFullMask, c, src);
    }
    *bin = b;
    *above = a;
    *count = c;
}

template <typename T>
__global__ void __launch_bounds__(kRadixThreads) radix_hist_kernel(const RadixParams p, int pass) {
    constexpr int EPV = Elem<T>::kPerVec;
    __shared__ int s_hist[kRadixBins];
    __shared__ float s_m[kRadixThreads / 32], s_s[kRadixThreads / 32];
    __shared__ int s_last;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t row = blockIdx.x / p.cpr;
    const int part = static_cast<int>(blockIdx.x - row * p.cpr);

    unsigned long long prefix = 0, mask = 0;
    int need = p.k;
    if (pass > 0) {
        const RadixState st = p.state[row];
        if (st.done)
            return;
        prefix = st.prefix;
        mask = st.mask;
        need = st.need;
    }
    const int shift = c_shift[pass];
    const int nbins = 1 << c_bits[pass];
    for (int i = tid; i < kRadixBins; i += kRadixThreads)
        s_hist[i] = 0;
    __syncthreads();

    const Segment sg = segment_of<T>(p, row, part);
    const float c1 = p.inv_t * kLog2e;
    float m = -INFINITY, s = 0.0f;  // running max of x and sum of exp2((x - m) * c1)
    const bool stats = pass == 0 && p.need_sum;
#pragma unroll 2
    for (int64_t v = sg.v0 + tid; v < sg.v1; v += kRadixThreads) {
        uint4 d = load_stream(sg.vbase + v);
        if (p.negate) {
            const uint32_t x = sizeof(T) == 4 ? 0x80000000u : 0x80008000u;
            d.x ^= x; d.y ^= x; d.z ^= x; d.w ^= x;
        }
        float f[EPV];
        Elem<T>::unpack(d, f);
        const int64_t ibase = v * EPV - sg.head;
        const bool ragged = ibase < 0 || ibase + EPV > p.cols;
        if (stats) {
            float vm = -INFINITY;
#pragma unroll
            for (int e = 0; e < EPV; e++)
                if (!ragged || (ibase + e >= 0 && ibase + e < p.cols))
                    vm = fmaxf(vm, f[e]);
            if (vm > m) {
                s *= ex2f((m - vm) * c1);
                m = vm;
            }
            if (m != -INFINITY) {
#pragma unroll
                for (int e = 0; e < EPV; e++)
                    if (!ragged || (ibase + e >= 0 && ibase + e < p.cols))
                        s += ex2f((f[e] - m) * c1);
            }
        }
#pragma unroll
        for (int e = 0; e < EPV; e++) {
            const int64_t i = ibase + e;
            if (!ragged || (i >= 0 && i < p.cols)) {
                const unsigned long long c = make_cand(order_key_sel(f[e], p.negate), static_cast<uint32_t>(i));
                if ((c & mask) == prefix)
                    atomicAdd(&s_hist[static_cast<unsigned>(c >> shift) & (nbins - 1)], 1);
            }
        }
    }
    __syncthreads();
    int *gh = p.hist + row * kRadixBins;
    for (int i = tid; i < nbins; i += kRadixThreads) {
        const int h = s_hist[i];
        if (h)
            atomicAdd(&gh[i], h);
    }
    if (stats) {
        // merge (m, s) pairs: warp, then CTA
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float m2 = __shfl_xor_sync(kFullMask, m, o), s2 = __shfl_xor_sync(kFullMask, s, o);
            const float mm = fmaxf(m, m2);
            const float a = (m == -INFINITY) ? 0.0f : s * ex2f((m - mm) * c1);
            const float b = (m2 == -INFINITY) ? 0.0f : s2 * ex2f((m2 - mm) * c1);
            m = mm;
            s = a + b;
        }
        if (lane == 0) {
            s_m[warp] = m;
            s_s[warp] = s;
        }
    }
    __threadfence();
    __syncthreads();
    if (stats && tid == 0) {
        float mm = -INFINITY;
        for (int w = 0; w < kRadixThreads / 32; w++)
            mm = fmaxf(mm, s_m[w]);
        float ss = 0.0f;
        for (int w = 0; w < kRadixThreads / 32; w++)
            if (s_m[w] != -INFINITY)
                ss += s_s[w] * ex2f((s_m[w] - mm) * c1);
        // the statistic is kept relative to max z = fl(max x * inv_t)
        p.stats[row * p.cpr + part] = make_float2(__fmul_rn(mm, p.inv_t), ss);
        __threadfence();
    }
    if (tid == 0) {
        const unsigned t = atomicAdd(&p.tickets[row], 1u);
        s_last = (t == static_cast<unsigned>(p.cpr) - 1u);
    }
    __syncthreads();
    if (!s_last)
        return;
    // ---- last CTA of the row: pick the digit, publish the state, clear the histogram ----
    __threadfence();
    for (int i = tid; i < kRadixBins; i += kRadixThreads) {
        s_hist[i] = i < nbins ? __ldcg(&gh[i]) : 0;
        gh[i] = 0;
    }
    __syncthreads();
    if (warp == 0) {
        int bin, above, count;
        find_bin(s_hist, nbins, need, &bin, &above, &count);
        if (lane == 0) {
            RadixState st;
            st.prefix = prefix | (static_cast<unsigned long long>(bin) << shift);
            st.mask = mask | (static_cast<unsigned long long>(nbins - 1) << shift);
            st.need = need - above;
            // decided when the whole bin is taken (always true after the last pass: candidates are distinct)
            st.done = (count <= st.need || pass == kRadixPasses - 1) ? 1 : 0;
            st.pad0 = st.pad1 = 0;
            p.state[row] = st;
            p.tickets[row] = 0;
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(kRadixThreads) radix_collect_kernel(const RadixParams p) {
    constexpr int EPV = Elem<T>::kPerVec;
    const int tid = threadIdx.x;
    const int64_t row = blockIdx.x / p.cpr;
    const int part = static_cast<int>(blockIdx.x - row * p.cpr);
    const unsigned long long thr = p.state[row].prefix;
    const Segment sg = segment_of<T>(p, row, part);
#pragma unroll 2
    for (int64_t v = sg.v0 + tid; v < sg.v1; v += kRadixThreads) {
        uint4 d = load_stream(sg.vbase + v);
        if (p.negate) {
            const uint32_t x = sizeof(T) == 4 ? 0x80000000u : 0x80008000u;
            d.x ^= x; d.y ^= x; d.z ^= x; d.w ^= x;
        }
        float f[EPV];
        Elem<T>::unpack(d, f);
        const int64_t ibase = v * EPV - sg.head;
#pragma unroll
        for (int e = 0; e < EPV; e++) {
            const int64_t i = ibase + e;
            if (i >= 0 && i < p.cols) {
                const unsigned long long c = make_cand(order_key_sel(f[e], p.negate), static_cast<uint32_t>(i));
                if (c >= thr) {
                    const int pos = atomicAdd(&p.cand_count[row], 1);
                    if (pos < p.k)
                        p.cand[row * p.k + pos] = c;
                }
            }
        }
    }
}

// Sorts the k candidates of a row (bitonic, shared memory) and writes the outputs.
template <typename T>
__global__ void __launch_bounds__(kRadixThreads) radix_final_kernel(const RadixParams p, int npow2) {
    extern __shared__ __align__(16) unsigned long long s_c[];
    __shared__ float s_m[kRadixThreads / 32], s_s[kRadixThreads / 32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t row = blockIdx.x;
    int cnt = p.cand_count[row];
    if (cnt > p.k)
        cnt = p.k;
    for (int i = tid; i < npow2; i += kRadixThreads)
        s_c[i] = i < cnt ? __ldcg(&p.cand[row * p.k + i]) : 0ull;
    // statistics of the row
    float m = -INFINITY;
    if (p.need_sum)
        for (int g = tid; g < p.cpr; g += kRadixThreads)
            m = fmaxf(m, __ldcg(&p.stats[row * p.cpr + g].x));
    m = warp_max(m);
    if (lane == 0)
        s_m[warp] = m;
    __syncthreads();
    float M = -INFINITY;
    for (int w = 0; w < kRadixThreads / 32; w++)
        M = fmaxf(M, s_m[w]);
    float s = 0.0f;
    if (p.need_sum)
        for (int g = tid; g < p.cpr; g += kRadixThreads) {
            const float mg = __ldcg(&p.stats[row * p.cpr + g].x), sgm = __ldcg(&p.stats[row * p.cpr + g].y);
            if (sgm != 0.0f)
                s += sgm * expf(mg - M);
        }
    s = warp_sum(s);
    if (lane == 0)
        s_s[warp] = s;
    __syncthreads();
    float S = 0.0f;
    for (int w = 0; w < kRadixThreads / 32; w++)
        S += s_s[w];
    // bitonic sort, descending
    for (int size = 2; size <= npow2; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int t = tid; t < npow2 / 2; t += kRadixThreads) {
                const int lo = 2 * t - (t & (stride - 1));
                const int hi = lo + stride;
                const bool desc = (lo & size) == 0;
                const unsigned long long a = s_c[lo], b = s_c[hi];
                if (desc ? (a < b) : (a > b)) {
                    s_c[lo] = b;
                    s_c[hi] = a;
                }
            }
            __syncthreads();
        }
    }
    if (tid == 0)
        p.cand_count[row] = 0;  // ready for the next call
    for (int r = tid; r < cnt; r += kRadixThreads) {
        const unsigned long long c = s_c[r];
        const uint32_t idx = cand_idx(c);
        const int64_t o = row * p.k + r;
        if (p.value_kind == VKOP_VALUE_RAW)
            reinterpret_cast<T *>(p.out_values)[o] = reinterpret_cast<const T *>(p.logits)[row * p.row_stride + idx];
        else
            store_value<T>(p.out_values, o, softmax_prob(key_to_float(cand_key(c)), p.inv_t, M, S));
        store_index(p.out_indices, p.index_dtype, o, static_cast<int64_t>(idx) + p.index_offset);
    }
}

// ---------------------------------------------------------------------------

static inline size_t align256(size_t n) { return (n + 255) / 256 * 256; }

struct RadixLayout {
    size_t state, hist, tickets, cand_count, stats, cand, total;
};

static RadixLayout radix_layout(const vkop_softmax_topk_desc &d, int cpr) {
    RadixLayout l;
    size_t off = 0;
    l.state = off;      off += align256(static_cast<size_t>(d.rows) * sizeof(RadixState));
    l.hist = off;       off += align256(static_cast<size_t>(d.rows) * kRadixBins * sizeof(int));
    l.tickets = off;    off += align256(static_cast<size_t>(d.rows) * 4);
    l.cand_count = off; off += align256(static_cast<size_t>(d.rows) * 4);
    l.stats = off;      off += align256(static_cast<size_t>(d.rows) * cpr * sizeof(float2));
    l.cand = off;       off += align256(static_cast<size_t>(d.rows) * d.k * 8);
    l.total = off;
    return l;
}

int plan_radix(const vkop_softmax_topk_desc &d, RadixPlan *plan) {
    if (d.k > kMaxK)
        return VKOP_UNSUPPORTED;
    const int epv = d.dtype == VKOP_F32 ? 4 : 8;
    const int64_t nv_max = (d.cols + 2 * (epv - 1)) / epv;
    // about four CTAs per SM in total, at least 4 vectors per thread and CTA
    int64_t cpr = (4 * 148 + (d.rows > 0 ? d.rows : 1) - 1) / (d.rows > 0 ? d.rows : 1);
    const int64_t max_cpr = (nv_max + 4 * kRadixThreads - 1) / (4 * kRadixThreads);
    if (cpr > max_cpr)
        cpr = max_cpr;
    if (cpr < 1)
        cpr = 1;
    if (d.rows * cpr > 0x7FFFFFFFll)
        return VKOP_UNSUPPORTED;
    plan->ctas_per_row = static_cast<int>(cpr);
    plan->bytes = radix_layout(d, plan->ctas_per_row).total;
    return VKOP_OK;
}

template <typename T>
static int launch_radix_t(const RadixParams &p, cudaStream_t stream) {
    const unsigned grid = static_cast<unsigned>(p.rows * p.cpr);
    for (int pass = 0; pass < kRadixPasses; pass++)
        radix_hist_kernel<T><<<grid, kRadixThreads, 0, stream>>>(p, pass);
    radix_collect_kernel<T><<<grid, kRadixThreads, 0, stream>>>(p);
    int npow2 = 2;
    while (npow2 < p.k)
        npow2 <<= 1;
    radix_final_kernel<T><<<static_cast<unsigned>(p.rows), kRadixThreads, static_cast<size_t>(npow2) * 8, stream>>>(p, npow2);
    note_launch(kRadixPasses + 2);
    return check_launch();
}

int launch_radix(const vkop_softmax_topk_desc &d, const RadixPlan &plan, const void *logits, void *out_values,
                 void *out_indices, void *packets_out, void *workspace, int need_sum, cudaStream_t stream) {
    if (packets_out)
        return VKOP_UNSUPPORTED;  // packets are produced by the chunk path only (k <= 128)
    if (d.rows == 0)
        return VKOP_OK;
    const int epv = d.dtype == VKOP_F32 ? 4 : 8;
    const int64_t nv_max = (d.cols + 2 * (epv - 1)) / epv;
    const RadixLayout l = radix_layout(d, plan.ctas_per_row);
    char *ws = static_cast<char *>(workspace);
    RadixParams p;
    p.logits = logits;
    p.rows = d.rows;
    p.cols = d.cols;
    p.row_stride = d.row_stride ? d.row_stride : d.cols;
    p.k = d.k;
    p.cpr = plan.ctas_per_row;
    p.vpc = (nv_max + p.cpr - 1) / p.cpr;
    p.inv_t = d.inv_temperature;
    p.value_kind = d.value_kind;
    p.index_dtype = d.index_dtype;
    p.negate = d.largest ? 0 : 1;
    p.need_sum = need_sum;
    p.index_offset = d.index_offset;
    p.out_values = out_values;
    p.out_indices = out_indices;
    p.state = reinterpret_cast<RadixState *>(ws + l.state);
    p.hist = reinterpret_cast<int *>(ws + l.hist);
    p.tickets = reinterpret_cast<unsigned int *>(ws + l.tickets);
    p.cand_count = reinterpret_cast<int *>(ws + l.cand_count);
    p.stats = reinterpret_cast<float2 *>(ws + l.stats);
    p.cand = reinterpret_cast<unsigned long long *>(ws + l.cand);
    switch (d.dtype) {
    case VKOP_F32: return launch_radix_t<float>(p, stream);
    case VKOP_F16: return launch_radix_t<__half>(p, stream);
    case VKOP_BF16: return launch_radix_t<__nv_bfloat16>(p, stream);
    default: return VKOP_INVALID_ARG;
    }
}

}  // namespace vkop_cuda
