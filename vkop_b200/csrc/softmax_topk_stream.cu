// Fused Softmax + TopK, streaming path: the kernel for large batches.
//
// A fixed grid of CTAs (all resident at once, two per SM) splits the whole
// [rows, cols] tensor by bytes.  Every CTA owns one contiguous range of
// 16-byte vector slots; range boundaries are snapped to multiples of 256
// vectors inside a row, so that a CTA never holds a sliver of a row, and with
// few rows every row is cut into the same number of CTAs and no CTA crosses a
// row.  A CTA walks its range in tiles; the loads of the next tile are issued
// before the current tile is processed, so the memory system always has a
// tile per thread in flight while the arithmetic runs (software pipelining in
// registers; no spin-wait anywhere).
//
// Per tile and thread: the maximum of its elements updates a running maximum
// m_t and rescales a running exp-sum s_t (online softmax); the r-th largest
// running thread maximum of each warp, minimised over the warps, refreshes the
// selection threshold T (one barrier per tile), which only rises while the CTA
// stays in one row; elements >= T are appended to a candidate list in shared
// memory.  Early tiles pass a hundred candidates, later ones a handful.
//
// When a CTA leaves a row (or its range ends) it publishes that row part:
// statistics and candidates go to global scratch, then one thread adds the
// part's length to the row's progress counter while the CTA already streams on;
// the part that completes a row gathers all parts of the row and selects the k
// best (select.cuh) at the next tile boundary.
//
// The kernel is launched with programmatic stream serialization: it lets the
// next kernel of the stream start while it drains (griddepcontrol.launch_dependents
// on entry) and itself waits for the previous kernel (griddepcontrol.wait)
// before it reads the logits -- or, when the caller states that the logits
// were complete before the launch, only before its first write to scratch
// memory or outputs, so that back-to-back calls overlap launch latency and the
// selection tail with streaming.
#include "common.cuh"
#include "launchers.h"
#include "select.cuh"

namespace vkop_cuda {

constexpr int kStreamThreads = 512;
constexpr int kStreamVecs = 4;
constexpr int kStreamCtasPerSm = 2;
constexpr int kNumSms = 148;
constexpr int kUnit = 256;  // range boundaries inside a row are multiples of this many vectors

// Snaps a slot offset inside a row to the nearest allowed boundary.
__host__ __device__ inline uint32_t snap_in_row(uint32_t v, uint32_t nvv) {
    const uint32_t units = nvv / kUnit > 0 ? nvv / kUnit : 1;
    const uint32_t u = (v + kUnit / 2) / kUnit;
    return u >= units ? nvv : u * kUnit;
}

// First slot of CTA c (all arithmetic in 32 bits: rows * nvv < 2^32).
// parts > 0: CTA c serves part c % parts of row c / parts.
__host__ __device__ inline uint32_t stream_boundary(uint32_t c, uint32_t grid, uint32_t per, uint32_t nvv, uint32_t total,
                                                    uint32_t parts) {
    if (c >= grid)
        return total;
    if (parts > 0) {
        const uint32_t r = c / parts, j = c - r * parts;
        return r * nvv + snap_in_row(static_cast<uint32_t>(static_cast<uint64_t>(j) * nvv / parts), nvv);
    }
    const uint64_t v64 = static_cast<uint64_t>(c) * per;
    if (v64 >= total)
        return total;
    const uint32_t V = static_cast<uint32_t>(v64);
    const uint32_t r = V / nvv;
    return r * nvv + snap_in_row(V - r * nvv, nvv);
}

// Largest CTA index whose range starts at or before slot V (V < total).
__device__ inline uint32_t stream_owner(uint32_t V, uint32_t grid, uint32_t per, uint32_t nvv, uint32_t total, uint32_t parts) {
    uint32_t c;
    if (parts > 0) {
        const uint32_t r = V / nvv;
        c = r * parts + static_cast<uint32_t>(static_cast<uint64_t>(V - r * nvv) * parts / nvv);
    } else {
        c = V / per;
    }
    if (c >= grid)
        c = grid - 1;
    while (c + 1 < grid && stream_boundary(c + 1, grid, per, nvv, total, parts) <= V)
        c++;
    while (c > 0 && stream_boundary(c, grid, per, nvv, total, parts) > V)
        c--;
    return c;
}

template <typename T, int THREADS, int VECS, bool ALIGNED>
__global__ void __launch_bounds__(THREADS, 1024 / THREADS) softmax_topk_stream_kernel(const ChunkParams p) {
    constexpr int EPV = Elem<T>::kPerVec;
    constexpr int NW = THREADS / 32;
    constexpr int TV = THREADS * VECS;  // vectors per tile
    extern __shared__ __align__(16) uint64_t s_dyn[];
    uint64_t *s_cand = s_dyn;                   // candidates of the current row part: kCandCap slots
    uint64_t *s_work = s_dyn + kCandCap;        // second region for the in-CTA selection: kCandCap slots
    uint64_t *s_merge = s_dyn + 2 * kCandCap;   // gather buffer of a row selection
    __shared__ uint32_t s_wr[2][NW], s_wm[2][NW];
    __shared__ float s_red[NW];
    __shared__ int s_int[8 + 1024];
    __shared__ int s_hist[256];
    __shared__ int s_pick[4];
    __shared__ int s_tmp[2];
    __shared__ int s_count;
    __shared__ int s_merge_row;  // row this CTA has to select for, or -1

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    asm volatile("griddepcontrol.launch_dependents;");
    const uint32_t grid = gridDim.x;
    const uint32_t nvv = static_cast<uint32_t>(p.nvv);
    const uint32_t total = static_cast<uint32_t>(p.rows) * nvv;
    const uint32_t per = static_cast<uint32_t>(p.per_cta);
    const uint32_t parts = static_cast<uint32_t>(p.parts_per_row);
    const uint32_t Vs = stream_boundary(blockIdx.x, grid, per, nvv, total, parts);
    const uint32_t Ve = stream_boundary(blockIdx.x + 1, grid, per, nvv, total, parts);
    if (Ve <= Vs)
        return;
    int remaining = static_cast<int>(Ve - Vs);
    bool waited = false;
    if (!p.input_ready) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        waited = true;
    }
    const uint32_t filler = Elem<T>::kNegInfWord;
    const float c1 = p.inv_t * kLog2e;
    const int64_t lstride = 2 + p.list_cap;
    const int cols = static_cast<int>(p.cols);

    // Geometry of a row: element offset of the row start inside its first vector, vectors that hold
    // data, and the 16-byte aligned base.  With aligned rows the first two are constants.
    auto row_geom = [&](int r, int &head, int &nvr, const uint4 *&vbase) {
        if (ALIGNED) {
            head = 0;
            nvr = static_cast<int>(nvv);
            vbase = reinterpret_cast<const uint4 *>(p.logits) + static_cast<int64_t>(r) * p.vstride;
        } else {
            const uintptr_t addr = reinterpret_cast<uintptr_t>(p.logits) + static_cast<uintptr_t>(r) * p.row_stride * sizeof(T);
            head = static_cast<int>((addr & 15) / sizeof(T));
            nvr = (head + cols + EPV - 1) / EPV;
            vbase = reinterpret_cast<const uint4 *>(addr & ~static_cast<uintptr_t>(15));
        }
    };

    // ---- tile iterator: (row, first vector slot, slots in the tile, last tile of the row part) ----
    int row = static_cast<int>(Vs / nvv);
    int v0 = static_cast<int>(Vs - static_cast<uint32_t>(row) * nvv);
    int nvt = TV < static_cast<int>(nvv) - v0 ? TV : static_cast<int>(nvv) - v0;
    if (nvt > remaining)
        nvt = remaining;
    bool part_last = (v0 + nvt == static_cast<int>(nvv)) || (nvt == remaining);

    PROF_MARK(0);

    // ---- state of the current row part ----
    float m_t = -INFINITY, s_t = 0.0f;
    uint32_t tkey = 0;       // running threshold key (0 = none yet)
    int part_v0 = v0;        // first slot of the part
    int nfullw = (nvt < THREADS ? nvt : THREADS) / 32;  // warps whose threads all own data in this part
    int r_sel = nfullw > 0 ? (p.k + nfullw - 1) / nfullw : 33;
    int parity = 0;
    if (tid == 0) {
        s_count = 0;
        s_merge_row = -1;
    }
    __syncthreads();

    for (;;) {
        const int c_row = row;
        const int c_v0 = v0, c_nvt = nvt;
        const bool c_last = part_last;
        int head, nvr;
        const uint4 *vbase;
        row_geom(c_row, head, nvr, vbase);
        // The tile: VECS independent 16-byte loads per thread.  With 32 resident warps per SM the loads of
        // the other warps and of the other CTA cover the latency; no register double buffering is needed.
        uint4 d[VECS];
        {
            const int lim = c_nvt < nvr - c_v0 ? c_nvt : nvr - c_v0;
            const uint4 *src = vbase + c_v0;
#pragma unroll
            for (int j = 0; j < VECS; j++) {
                const int lv = j * THREADS + tid;
                if (lv < lim)
                    d[j] = load_stream(src + lv);
                else
                    d[j] = make_uint4(filler, filler, filler, filler);
            }
        }
        // advance the iterator
        remaining -= nvt;
        const bool has_next = remaining > 0;
        if (has_next) {
            v0 += nvt;
            if (v0 >= static_cast<int>(nvv)) {
                row++;
                v0 = 0;
            }
            nvt = TV < static_cast<int>(nvv) - v0 ? TV : static_cast<int>(nvv) - v0;
            if (nvt > remaining)
                nvt = remaining;
            part_last = (v0 + nvt == static_cast<int>(nvv)) || (nvt == remaining);
        }

        if (p.negate) {
            const uint32_t x = sizeof(T) == 4 ? 0x80000000u : 0x80008000u;
#pragma unroll
            for (int j = 0; j < VECS; j++) {
                if (c_v0 + j * THREADS + tid < nvr && j * THREADS + tid < c_nvt) {
                    d[j].x ^= x; d[j].y ^= x; d[j].z ^= x; d[j].w ^= x;
                }
            }
        }
        // ragged ends of the row: elements outside the row become -inf
        if ((!ALIGNED && c_v0 == 0) || (c_v0 + c_nvt >= nvr && (ALIGNED ? (cols % EPV != 0) : true))) {
#pragma unroll
            for (int j = 0; j < VECS; j++) {
                const int v = c_v0 + j * THREADS + tid;
                if (j * THREADS + tid < c_nvt && ((!ALIGNED && v == 0) || v == nvr - 1)) {
                    const int lo = v == 0 ? head : 0;
                    const int end = head + cols - v * EPV;
                    const int hi = end < EPV ? end : EPV;
                    mask_vector<T>(d[j], lo, hi);
                }
            }
        }

        // ---- tile maximum of this thread; online softmax statistics ----
        float vm = -INFINITY;
#pragma unroll
        for (int j = 0; j < VECS; j++) {
            float f[EPV];
            Elem<T>::unpack(d[j], f);
#pragma unroll
            for (int e = 0; e < EPV; e++)
                vm = fmaxf(vm, f[e]);
        }
        if (vm > m_t) {
            s_t *= ex2_approx((m_t - vm) * c1);
            m_t = vm;
        }
        if (p.need_sum && m_t != -INFINITY) {
            // (x - m) first: the difference is exact for nearby values whatever their magnitude
#pragma unroll
            for (int j = 0; j < VECS; j++) {
                float f[EPV];
                Elem<T>::unpack(d[j], f);
#pragma unroll
                for (int e = 0; e < EPV; e++)
                    s_t += ex2_approx((f[e] - m_t) * c1);
            }
        }

        // ---- threshold refresh from the running thread maxima (and the part maximum) ----
        {
            uint32_t cur = order_key(m_t);
            const uint32_t wmax = __reduce_max_sync(kFullMask, cur);
            uint32_t rth = 0;
            if (r_sel <= 32) {
                if (warp < nfullw) {
                    for (int i = 0; i < r_sel; i++) {
                        rth = __reduce_max_sync(kFullMask, cur);
                        const unsigned b = __ballot_sync(kFullMask, cur == rth);
                        if (lane == __ffs(b) - 1)
                            cur = 0;
                    }
                } else {
                    rth = 0xFFFFFFFFu;
                }
            }
            if (lane == 0) {
                s_wr[parity][warp] = rth;
                s_wm[parity][warp] = wmax;
            }
        }
        __syncthreads();
        const uint32_t t_new = __reduce_min_sync(kFullMask, lane < NW ? s_wr[parity][lane] : 0xFFFFFFFFu);
        tkey = t_new > tkey ? t_new : tkey;
        const float T_thr = key_to_float(tkey);
        const bool allpass = tkey == 0u || T_thr == -INFINITY;

        // a row selection handed to this CTA by an earlier part's completion (published before the barrier above)
        if (s_merge_row >= 0) {
            const int mrow = s_merge_row;
            const uint32_t cf = stream_owner(static_cast<uint32_t>(mrow) * nvv, grid, per, nvv, total, parts);
            const uint32_t cl = stream_owner(static_cast<uint32_t>(mrow + 1) * nvv - 1, grid, per, nvv, total, parts);
            merge_lists<T, THREADS>(p, mrow, p.lists + static_cast<int64_t>(mrow) * p.splits * lstride, lstride,
                                    static_cast<int>(cl - cf + 1), s_merge, s_red, s_int, s_tmp);
            __syncthreads();
            if (tid == 0)
                s_merge_row = -1;
        }

        // ---- candidates of this tile ----
        if (!allpass) {
            if (!(vm < T_thr)) {
#pragma unroll
                for (int j = 0; j < VECS; j++) {
                    float f[EPV];
                    Elem<T>::unpack(d[j], f);
#pragma unroll
                    for (int e = 0; e < EPV; e++) {
                        if (!(f[e] < T_thr)) {
                            const int pos = atomicAdd(&s_count, 1);
                            if (pos < kCandCap)
                                s_cand[pos] = make_cand(order_key(f[e]),
                                                        static_cast<uint32_t>((c_v0 + j * THREADS + tid) * EPV + e - head));
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
                    const int i = (c_v0 + lv) * EPV + e - head;
                    if (lv < c_nvt && i >= 0 && i < cols) {
                        const int pos = atomicAdd(&s_count, 1);
                        if (pos < kCandCap)
                            s_cand[pos] = make_cand(order_key(f[e]), static_cast<uint32_t>(i));
                    }
                }
            }
        }

        if (c_last) {
            PROF_MARK(4);
            // ================= end of a row part: statistics, publish =================
            const uint32_t mkey = __reduce_max_sync(kFullMask, lane < NW ? s_wm[parity][lane] : 0u);
            const float mx = key_to_float(mkey);  // part maximum of the stored logits
            float s = (m_t == -INFINITY) ? 0.0f : s_t * ex2_approx((m_t - mx) * c1);
            s = warp_sum(s);
            if (lane == 0)
                s_red[warp] = s;
            __syncthreads();
            const float S = warp_sum(lane < NW ? s_red[lane] : 0.0f);
            const float mz = __fmul_rn(mx, p.inv_t);
            int C = s_count;

            const int part_v1 = c_v0 + c_nvt;
            int e0 = part_v0 * EPV - head, e1 = part_v1 * EPV - head;
            if (e0 < 0) e0 = 0;
            if (e1 > cols) e1 = cols;
            const int nvalid = e1 > e0 ? e1 - e0 : 0;
            const int kk = nvalid < p.k ? nvalid : p.k;

            if (C > kCandCap || (p.need_sum && S != S)) {
                __syncthreads();
                const int fv1 = part_v1 < nvr ? part_v1 : nvr;
                select_fallback<T, THREADS>(vbase, part_v0, fv1, head, p.cols, p.negate, kk, s_cand, &s_count, s_hist, s_pick);
                C = s_count;
            }
            // Candidates pushed under the weaker thresholds of the early tiles are dropped now: at least
            // k elements of this part reach the final threshold.
            uint64_t *s_list = s_cand, *s_other = s_work;
            if (tkey != 0u && C > p.k) {
                if (tid == 0)
                    s_tmp[0] = 0;
                __syncthreads();
                for (int i = tid; i < C; i += THREADS) {
                    const uint64_t c = s_cand[i];
                    if (cand_key(c) >= tkey)
                        s_work[atomicAdd(&s_tmp[0], 1)] = c;
                }
                __syncthreads();
                C = s_tmp[0];
                s_list = s_work;
                s_other = s_cand;
                __syncthreads();
            }
            PROF_MARK(5);

            if (!waited) {  // first write to memory another launch may still be using
                asm volatile("griddepcontrol.wait;" ::: "memory");
                waited = true;
            }
            const bool whole_row = part_v0 == 0 && part_v1 == static_cast<int>(nvv);
            if (whole_row) {
                if (p.packets_out && tid == 0) {
                    uint32_t *pk = p.packets_out + static_cast<int64_t>(c_row) * packet_words(p.k);
                    pk[0] = __float_as_uint(mz);
                    pk[1] = __float_as_uint(S);
                    pk[2] = static_cast<uint32_t>(kk);
                    pk[3] = 0;
                }
                select_and_emit<T, THREADS>(p, c_row, s_list, C, s_other, mz, S, nullptr, s_tmp);
            } else {
                const uint32_t c_first = stream_owner(static_cast<uint32_t>(c_row) * nvv, grid, per, nvv, total, parts);
                const int pidx = static_cast<int>(blockIdx.x - c_first);
                unsigned long long *mylist = p.lists + (static_cast<int64_t>(c_row) * p.splits + pidx) * lstride;
                if (C > p.list_cap) {
                    select_and_emit<T, THREADS>(p, c_row, s_list, C, s_other, 0.0f, 0.0f, mylist + 2, s_tmp);
                    C = kk;
                } else {
                    for (int i = tid; i < C; i += THREADS)
                        mylist[2 + i] = s_list[i];
                }
                if (tid == 0) {
                    mylist[0] = (static_cast<unsigned long long>(__float_as_uint(S)) << 32) | __float_as_uint(mz);
                    mylist[1] = static_cast<unsigned long long>(C);
                }
                __syncthreads();
                // One thread orders the CTA's writes (made visible to it by the barrier) before the row's
                // progress counter; the others stream on.  The part that completes the row selects.
                if (tid == 0) {
                    __threadfence();
                    const unsigned int len = static_cast<unsigned int>(part_v1 - part_v0);
                    const unsigned int done = atomicAdd(&p.counters[c_row], len) + len;
                    PROF_MARK(6);
                    if (done == nvv) {
                        p.counters[c_row] = 0;  // ready for the next launch
                        __threadfence();
                        s_merge_row = c_row;
                    }
                }
            }
            if (has_next) {
                // ---- reset for the next row part ----
                // (every read of the candidate list and its count lies before a barrier above; the next
                // pushes come after the next tile's barrier)
                m_t = -INFINITY;
                s_t = 0.0f;
                tkey = 0;
                part_v0 = v0;
                nfullw = (nvt < THREADS ? nvt : THREADS) / 32;
                r_sel = nfullw > 0 ? (p.k + nfullw - 1) / nfullw : 33;
                if (tid == THREADS - 1)
                    s_count = 0;
            }
        }
        parity ^= 1;
        if (!has_next)
            break;
    }
    // a selection triggered by the CTA's last part
    __syncthreads();
    PROF_MARK(7);
    if (s_merge_row >= 0) {
        const int mrow = s_merge_row;
        const uint32_t cf = stream_owner(static_cast<uint32_t>(mrow) * nvv, grid, per, nvv, total, parts);
        const uint32_t cl = stream_owner(static_cast<uint32_t>(mrow + 1) * nvv - 1, grid, per, nvv, total, parts);
        merge_lists<T, THREADS>(p, mrow, p.lists + static_cast<int64_t>(mrow) * p.splits * lstride, lstride,
                                static_cast<int>(cl - cf + 1), s_merge, s_red, s_int, s_tmp);
        __syncthreads();
        PROF_MARK(12);
    }
}

// ---------------------------------------------------------------------------

int plan_stream(const vkop_softmax_topk_desc &d, bool base_aligned, StreamPlan *plan) {
    if (d.k > kChunkMaxK)
        return VKOP_UNSUPPORTED;
    const int esz = d.dtype == VKOP_F32 ? 4 : 2;
    const int epv = 16 / esz;
    const int64_t stride = d.row_stride ? d.row_stride : d.cols;
    // rows that all start on a 16-byte boundary (given an aligned base, checked at launch): exact slot count
    const bool aligned = base_aligned && (stride * esz) % 16 == 0;
    const int64_t nvv = aligned ? (d.cols + epv - 1) / epv : (d.cols + 2 * (epv - 1)) / epv;
    if (d.rows <= 0 || d.cols >= (1ll << 30) || d.rows * nvv >= (1ll << 32) - (1ll << 20))
        return VKOP_UNSUPPORTED;
    const int64_t total = d.rows * nvv;
    const int64_t slots = kNumSms * kStreamCtasPerSm;
    const int64_t tile = static_cast<int64_t>(kStreamThreads) * kStreamVecs;
    const int64_t tiles = (total + tile - 1) / tile;
    int64_t grid = slots < tiles ? slots : tiles;
    int parts_per_row = 0;
    if (d.rows <= slots / 2) {
        const int64_t s = slots / d.rows;
        if (nvv / s >= 2 * kUnit && d.rows * s <= tiles) {
            parts_per_row = static_cast<int>(s);  // the same number of CTAs for every row: no CTA crosses a row
            grid = d.rows * s;
        }
    }
    const int64_t per = (total + grid - 1) / grid;
    // parts a row can be cut into: its share of the CTAs, plus one at either end
    const int64_t maxparts = parts_per_row > 0 ? parts_per_row : (nvv + per - 1) / per + 2;
    if (maxparts * d.k > kMergeMaxSlots || maxparts > 1024)
        return VKOP_UNSUPPORTED;
    int list_cap = static_cast<int>(kMergeMaxSlots / maxparts);
    if (list_cap > kListCapMax)
        list_cap = kListCapMax;
    plan->grid = static_cast<int>(grid);
    plan->per_cta = per;
    plan->nvv = nvv;
    plan->vstride = aligned ? stride * esz / 16 : 0;
    plan->aligned = aligned ? 1 : 0;
    plan->parts_per_row = parts_per_row;
    plan->maxparts = static_cast<int>(maxparts);
    plan->list_cap = list_cap;
    plan->counters_bytes = ((static_cast<size_t>(d.rows) * 4 + 255) / 256) * 256;
    plan->lists_bytes = static_cast<size_t>(d.rows) * maxparts * (2 + list_cap) * 8;
    plan->smem_bytes = (2 * static_cast<size_t>(kCandCap) + 2 * (static_cast<size_t>(maxparts) * list_cap + 32)) * 8;
    return VKOP_OK;
}

template <typename T, bool ALIGNED>
static int launch_stream_t(const ChunkParams &p, const StreamPlan &plan, cudaStream_t stream) {
    auto kern = softmax_topk_stream_kernel<T, kStreamThreads, kStreamVecs, ALIGNED>;
    if (plan.smem_bytes > 32 * 1024 &&
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(plan.smem_bytes)) !=
            cudaSuccess)
        return VKOP_CUDA_ERROR;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(plan.grid));
    cfg.blockDim = dim3(kStreamThreads);
    cfg.dynamicSmemBytes = plan.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kern, p) != cudaSuccess)
        return VKOP_CUDA_ERROR;
    note_launch();
    return check_launch();
}

int launch_stream(const vkop_softmax_topk_desc &d, const StreamPlan &plan, const void *logits, void *out_values,
                  void *out_indices, void *packets_out, void *workspace, int need_sum, cudaStream_t stream) {
    if (d.rows == 0)
        return VKOP_OK;
    ChunkParams p = {};
    p.logits = logits;
    p.rows = d.rows;
    p.cols = d.cols;
    p.row_stride = d.row_stride ? d.row_stride : d.cols;
    p.k = d.k;
    p.splits = plan.maxparts;
    p.vps = 0;
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
    p.nvv = plan.nvv;
    p.per_cta = plan.per_cta;
    p.vstride = plan.vstride;
    p.parts_per_row = plan.parts_per_row;
    p.input_ready = (d.flags & VKOP_FLAG_INPUT_READY) ? 1 : 0;
    if (plan.aligned && reinterpret_cast<uintptr_t>(logits) % 16 != 0)
        return VKOP_INVALID_ARG;  // planned for an aligned base
#define VKOP_STREAM(T) (plan.aligned ? launch_stream_t<T, true>(p, plan, stream) : launch_stream_t<T, false>(p, plan, stream))
    switch (d.dtype) {
    case VKOP_F32: return VKOP_STREAM(float);
    case VKOP_F16: return VKOP_STREAM(__half);
    case VKOP_BF16: return VKOP_STREAM(__nv_bfloat16);
    default: return VKOP_INVALID_ARG;
    }
#undef VKOP_STREAM
}

}  // namespace vkop_cuda

#ifdef VKOP_PHASE_PROF
extern "C" int vkop_debug_read_phase_prof(unsigned long long *host, size_t count) {
    return cudaMemcpyFromSymbol(host, vkop_cuda::g_phase_prof, count * sizeof(unsigned long long)) == cudaSuccess ? 0 : -4;
}
#endif
