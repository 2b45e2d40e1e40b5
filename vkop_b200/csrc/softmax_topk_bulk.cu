// Fused Softmax + TopK, bulk-copy streaming path: the kernel for long, 16-byte aligned rows.
//
// Data movement.  Every CTA owns one contiguous range of 16-byte vector slots of the [rows, cols]
// tensor (byte-balanced over the grid, one CTA per SM, ranges may run across rows).  One elected
// thread of a producer warp walks the range in tiles of kTileVecs vectors and hands every tile to
// the copy engine with a single bulk copy (cp.async.bulk.shared::cluster.global, plain form: no
// multicast, the source is this GPU's own memory) into a ring of shared-memory stages; every stage
// has a "full" mbarrier that the copy completes (expect-tx / complete-tx bytes) and an "empty"
// mbarrier that the consumer warps arrive at once they hold the tile in registers.  The consumer
// threads issue no copy, compute no address and wait only on the full barrier.
//
// Per tile and consumer thread: four 16-byte shared-memory loads, the maximum of the 16 (or 32)
// elements, and the exp-sum against a per-thread offset o = -(m * c1): one FFMA, one ex2 and one add
// per element (the offset moves, and the sum is rescaled, only when the thread's maximum rises).
//
// Selection.  Any value that at least k thread maxima reach bounds the k-th largest element of the
// row part from below.  The thread maxima live in shared memory as order-preserving keys; the
// bound T is found by a warp-level bisection over them: once after the first tile of a part (all
// consumers wait for it), then on tiles 1, 3, 7, ... by one consumer warp in turn while the others
// keep streaming.  In the loop a thread only tests the maximum of its 16 elements against T; when
// it reaches T the thread records where it is (one predicated 32-bit shared-memory store, no
// branch).  At the end of the part the recorded groups (a few hundred) are read again from L2,
// filtered by the final bound and ranked.
//
// Rows cut across CTAs: every part publishes (max, sum, bound, candidates) to scratch memory; the
// last part of a row to arrive (ticket counter) merges the row and writes its result.  Launches use
// programmatic stream serialization as the other streaming kernel does: with
// VKOP_FLAG_INPUT_READY consecutive calls overlap, scratch lists alternate between two sets by call
// parity and a per-row counter of finished calls orders results and list reuse.
//
// Every wait on an mbarrier is bounded (about a second); a wait that runs out sets an abort flag and
// VKOP_TIMEOUT in the workspace status word, the CTA stops issuing copies, waits (bounded) for the
// copies in flight and returns.
#include <cstdlib>

#include "common.cuh"
#include "launchers.h"
#include "select.cuh"
#include "stream_ranges.cuh"

namespace vkop_cuda {

constexpr int kBulkConsumers = 256;                 // consumer threads (8 warps)
constexpr int kBulkThreads = kBulkConsumers + 32;   // plus the producer warp
constexpr int kBulkTileVecs = 1024;                 // 16 KB per tile
constexpr int kBulkStages = 5;                      // 80 KB ring
constexpr int kBulkJ = kBulkTileVecs / kBulkConsumers;  // vectors per consumer thread and tile
constexpr int kBulkSlots = 4;                       // private record slots per consumer thread
constexpr int kBulkOverflow = 256;                  // shared overflow records
constexpr int kBulkRegion = 1024;                   // 64-bit slots of each of the two work regions
constexpr int kBulkMaxParts = 56;                   // most CTAs one row may be cut across
constexpr int kBar = 1;                             // named barrier of the consumer threads
constexpr unsigned long long kWaitLimitNs = 1000000000ull;

// ---- mbarrier / bulk copy wrappers (shared-memory addresses as 32-bit) ----
__device__ __forceinline__ uint32_t smem_addr(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Waits for the phase with the given parity; false when the limit ran out (then *abort is set).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort) {
    if (mbar_test(bar, parity))
        return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 256; i++) {
            if (mbar_test(bar, parity))
                return true;
        }
        if (*abort)
            return false;
        if (global_ns() - t0 > kWaitLimitNs) {
            *abort = 1;
            return false;
        }
    }
}
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}

// Maximum of three floats (NaN operands are passed over, as fmaxf does).
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

struct BulkParams {
    ChunkParams c;            // shared with the selection helpers (logits, shape, outputs, lists, counters)
    int *status;              // workspace: VKOP_OK or VKOP_TIMEOUT
    int trigger_tile;         // tile after which the CTA lets the next call of the stream in
    int debug;                // TEMPORARY: experiment switches
};

// Walks the tiles of a CTA's range: tiles never cross a row and never exceed kBulkTileVecs vectors.
struct TileWalk {
    uint32_t nvv;
    int row, v0, nv, remaining;
    bool part_first, part_last;
    __device__ __forceinline__ void start(uint32_t Vs, uint32_t Ve, uint32_t nvv_) {
        nvv = nvv_;
        row = static_cast<int>(Vs / nvv);
        v0 = static_cast<int>(Vs - static_cast<uint32_t>(row) * nvv);
        remaining = static_cast<int>(Ve - Vs);
        part_first = true;
        shape();
    }
    __device__ __forceinline__ void shape() {
        const int left = static_cast<int>(nvv) - v0;
        nv = kBulkTileVecs < left ? kBulkTileVecs : left;
        if (nv > remaining)
            nv = remaining;
        part_last = (v0 + nv == static_cast<int>(nvv)) || (nv == remaining);
    }
    // moves to the next tile; false when the range is exhausted
    __device__ __forceinline__ bool next() {
        remaining -= nv;
        if (remaining <= 0)
            return false;
        part_first = part_last;
        v0 += nv;
        if (v0 >= static_cast<int>(nvv)) {
            row++;
            v0 = 0;
        }
        shape();
        return true;
    }
};

// Largest key v such that at least k of the 256 keys reach it (0: fewer than k keys are set), by
// bisection between `lo` (0, or a key already known to be reached by k keys) and the largest key.
// Executed by one warp; the keys only grow while it runs, which keeps any answer valid.
__device__ __noinline__ uint32_t bulk_bisect(const volatile uint32_t *keys, int k, uint32_t lo, int iters) {
    const int lane = threadIdx.x & 31;
    uint32_t kv[kBulkConsumers / 32];
    uint32_t hi = 0;
    int set = 0;
#pragma unroll
    for (int i = 0; i < kBulkConsumers / 32; i++) {
        kv[i] = keys[lane + 32 * i];
        hi = kv[i] > hi ? kv[i] : hi;
        set += kv[i] != 0u ? 1 : 0;
    }
    hi = __reduce_max_sync(kFullMask, hi);
    set = __reduce_add_sync(kFullMask, set);
    if (set < k)
        return 0u;
    if (lo == 0u)
        lo = 1u;
    for (int it = 0; it < iters && hi > lo; it++) {
        const uint32_t mid = lo + ((hi - lo + 1u) >> 1);
        int c = 0;
#pragma unroll
        for (int i = 0; i < kBulkConsumers / 32; i++)
            c += kv[i] >= mid ? 1 : 0;
        c = __reduce_add_sync(kFullMask, c);
        if (c >= k)
            lo = mid;
        else
            hi = mid - 1u;
    }
    return lo;
}

// Pointers into the CTA's shared memory.
struct BulkShared {
    uint4 *tiles;               // kBulkStages stages of kBulkTileVecs vectors
    uint64_t *ra, *rb;          // two work regions of kBulkRegion 64-bit slots, contiguous
    uint32_t *rec;              // (kBulkSlots + 1) x kBulkConsumers private records (the last row is a dummy)
    uint32_t *ovf;              // shared overflow records
    volatile uint32_t *keys;    // running thread maxima of the current part as order keys (0: none)
    int *hist, *sint, *tmp, *pick, *count, *flag;
    float *red;
    int *nrec, *novf, *ncand;   // compacted records, overflow records, candidates
    uint32_t *tkey;             // bound of the current part as a key (0: none)
    volatile int *abort;
};

// What the end of a row part needs from the streaming loop.
struct BulkPartEnd {
    float m_t, o_t, s_t;   // this thread's maximum, exponent offset and exp-sum against that offset
    int cnt;               // groups this thread recorded
    bool nan_seen;         // (selection without a sum) the thread met a NaN
    int row, part_v0, part_v1;
    uint32_t epoch;
    bool waited;
};

// End of a row part, executed by the consumer threads: statistics, expansion of the recorded groups
// into candidates, then selection (the part is a whole row) or publication and, for the last part
// of the row to arrive, the merge of the row.  Returns whether the CTA has waited for the previous
// call by now.
template <typename T>
__device__ __noinline__ bool bulk_finish_part(const BulkParams &bp, const BulkShared &sh, const BulkPartEnd e) {
    constexpr int EPV = Elem<T>::kPerVec;
    constexpr int NC = kBulkConsumers;
    constexpr int NW = NC / 32;
    const ChunkParams &p = bp.c;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t grid = gridDim.x;
    const uint32_t nvv = static_cast<uint32_t>(p.nvv);
    const uint32_t total = static_cast<uint32_t>(p.rows) * nvv;
    const uint32_t per = static_cast<uint32_t>(p.per_cta);
    const int cols = static_cast<int>(p.cols);
    const float c1 = p.inv_t * kLog2e;
    const int64_t lstride = 2 + p.list_cap;
    const int row = e.row;
    const uint32_t epoch = e.epoch;
    const int64_t set = epoch & 1u;
    const uint4 *const vbase = reinterpret_cast<const uint4 *>(p.logits) + static_cast<int64_t>(row) * p.vstride;
    const bool whole = e.part_v0 == 0 && e.part_v1 == static_cast<int>(nvv);
    bool waited = e.waited;

    // Has the call before the previous one finished with this row (its lists are about to be
    // overwritten), has the previous call written the row's result?  Asked early, used later.
    unsigned int done_calls = 0;
    if (tid == 0) {
        if (!waited)
            asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(done_calls) : "l"(p.row_done + row) : "memory");
        sh.flag[0] = whole ? done_calls == epoch : static_cast<int>(done_calls - epoch + 1u) >= 0;
    }
    if (e.nan_seen)
        sh.flag[2] = 1;
    cta_sync<kBar, NC>();  // #1: keys, records and the overflow count are final

    // ---- statistics (every warp reduces the 256 keys itself: no second barrier for the maximum) ----
    uint32_t mkey = 0;
#pragma unroll
    for (int i = 0; i < NC / 32; i++) {
        const uint32_t kv = sh.keys[lane + 32 * i];
        mkey = kv > mkey ? kv : mkey;
    }
    mkey = __reduce_max_sync(kFullMask, mkey);
    const float M = mkey ? key_to_float(mkey) : -INFINITY;  // part maximum of the stored logits
    const float O = -__fmul_rn(M, c1);
    {
        const float contrib = (e.m_t == -INFINITY && e.s_t == e.s_t) ? 0.0f : e.s_t * ex2_approx(O - e.o_t);
        const float ws = warp_sum(contrib);
        if (lane == 0)
            sh.red[warp] = ws;
    }
    // ---- the recorded groups go to one dense list (region B as 32-bit words) ----
    uint32_t *const list = reinterpret_cast<uint32_t *>(sh.rb);
    {
        const int mine = e.cnt < kBulkSlots ? e.cnt : kBulkSlots;
        int incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(kFullMask, incl, o);
            if (lane >= o)
                incl += v;
        }
        int base = 0;
        if (lane == 31)
            base = atomicAdd(sh.nrec, incl);
        base = __shfl_sync(kFullMask, base, 31) + incl - mine;
        for (int q = 0; q < mine; q++)
            list[base + q] = sh.rec[q * NC + tid];
    }
    if (warp == 0) {
        // the final bound: exact (the bisection runs until it closes)
        const uint32_t t = bulk_bisect(sh.keys, p.k, *sh.tkey, 32);
        if (lane == 0 && t > *sh.tkey)
            *sh.tkey = t;
    }
    cta_sync<kBar, NC>();  // #2
    float S = 0.0f;
#pragma unroll
    for (int w = 0; w < NW; w++)
        S += sh.red[w];
    // S is relative to the offset O = -rn(M * c1); the published sum is relative to M exactly
    if (M != -INFINITY)
        S *= ex2_approx(-__fmaf_rn(M, c1, O));
    const float mz = __fmul_rn(M, p.inv_t);
    uint32_t tpub = *sh.tkey;
    const float Tf = tpub ? key_to_float(tpub) : -INFINITY;
    const int n_rec = *sh.nrec;
    const int novf = *sh.novf;
    const int nvalid = (e.part_v1 * EPV < cols ? e.part_v1 * EPV : cols) - e.part_v0 * EPV;
    const int kk = nvalid < p.k ? nvalid : p.k;
    const bool bad = sh.flag[2] != 0 || novf > kBulkOverflow || (p.need_sum && S != S);
    const uint32_t xmask = p.negate ? (sizeof(T) == 4 ? 0x80000000u : 0x80008000u) : 0u;

    int C = kBulkRegion + 1;
    if (!bad) {
        // ---- expansion: every recorded group is kBulkJ vectors, re-read from L2 ----
        const int ngroups = n_rec + novf;
        const int nvec = ngroups * kBulkJ;
        for (int base = 0; base < nvec; base += NC * 4) {
            uint4 d[4];
            int vv[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int i = base + u * NC + tid;
                vv[u] = -1;
                if (i < nvec) {
                    const int g = i / kBulkJ;
                    const uint32_t r = g < n_rec ? list[g] : sh.ovf[g - n_rec];
                    const int v = static_cast<int>(r) + (i - g * kBulkJ) * NC;
                    if (v < e.part_v1) {
                        vv[u] = v;
                        d[u] = __ldcg(vbase + v);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                if (vv[u] < 0)
                    continue;
                d[u].x ^= xmask; d[u].y ^= xmask; d[u].z ^= xmask; d[u].w ^= xmask;
                float f[EPV];
                Elem<T>::unpack(d[u], f);
#pragma unroll
                for (int q = 0; q < EPV; q++) {
                    const int idx = vv[u] * EPV + q;
                    if (idx < cols && f[q] >= Tf) {
                        const int pos = atomicAdd(sh.ncand, 1);
                        if (pos < kBulkRegion)
                            sh.ra[pos] = make_cand(order_key(f[q]), static_cast<uint32_t>(idx));
                    }
                }
            }
        }
        cta_sync<kBar, NC>();  // #3
        C = *sh.ncand;
    }
    if (C > kBulkRegion) {
        // Rare: NaN in the part, threads that ran out of record slots, or more candidates than the
        // region holds (massive ties).  Exact radix select over the part, re-read from L2; it works
        // in both regions as one list.
        cta_sync<kBar, NC>();
        select_fallback<T, NC, kBar>(vbase, e.part_v0, e.part_v1, 0, p.cols, p.negate, kk, sh.ra, sh.count, sh.hist, sh.pick);
        C = *sh.count;
        tpub = 0;
    }

    if (whole) {
        // ---- the part is the row: select and write.  Results of one row are written in call order. ----
        if (!waited && !sh.flag[0]) {
            if (tid == 0) {  // look once more before giving up
                unsigned int dn;
                asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(dn) : "l"(p.row_done + row) : "memory");
                sh.flag[1] = dn == epoch;
            }
            cta_sync<kBar, NC>();
            if (!sh.flag[1]) {
                asm volatile("griddepcontrol.wait;" ::: "memory");
                waited = true;
            }
        }
        if (p.packets_out && tid == 0) {
            uint32_t *pk = p.packets_out + static_cast<int64_t>(row) * packet_words(p.k);
            pk[0] = __float_as_uint(mz);
            pk[1] = __float_as_uint(S);
            pk[2] = static_cast<uint32_t>(C < p.k ? C : p.k);
            pk[3] = 0;
        }
        select_and_emit<T, NC, kBar>(p, row, sh.ra, C, sh.rb, mz, S, nullptr, sh.tmp);
        cta_sync<kBar, NC>();
        if (tid == 0) {
            const unsigned int d = epoch + 1u;
            asm volatile("st.release.gpu.u32 [%0], %1;" ::"l"(p.row_done + row), "r"(d) : "memory");
        }
        return waited;
    }

    // ---- publish the part; the last part of the row to arrive merges the row ----
    const uint32_t c_first = stream_owner(static_cast<uint32_t>(row) * nvv, grid, per, nvv, total, 0u);
    const int pidx = static_cast<int>(blockIdx.x - c_first);
    unsigned long long *const rowlists = p.lists + (set * p.rows + row) * p.splits * lstride;
    unsigned long long *const mylist = rowlists + pidx * lstride;
    if (!waited && !sh.flag[0]) {  // rare: the row's lists may still be in use by the call before the previous one
        asm volatile("griddepcontrol.wait;" ::: "memory");
        waited = true;
    }
    if (C > p.list_cap) {
        // more than a part may publish: its own best kk, ranked, go out instead
        select_and_emit<T, NC, kBar>(p, row, sh.ra, C, sh.rb, 0.0f, 0.0f, mylist + 2, sh.tmp);
        C = kk;
        tpub = 0;
    } else {
        for (int i = tid; i < C; i += NC)
            mylist[2 + i] = sh.ra[i];
    }
    cta_sync<kBar, NC>();
    if (tid == 0) {
        mylist[0] = (static_cast<unsigned long long>(__float_as_uint(S)) << 32) | __float_as_uint(mz);
        mylist[1] = (static_cast<unsigned long long>(tpub) << 16) | static_cast<unsigned long long>(C);
        const uint32_t c_end = stream_owner(static_cast<uint32_t>(row + 1) * nvv - 1u, grid, per, nvv, total, 0u);
        const int nparts = static_cast<int>(c_end - c_first + 1u);
        unsigned int arrived;
        unsigned int *ticket = p.counters + set * p.rows + row;
        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(arrived) : "l"(ticket) : "memory");
        const bool last = arrived == static_cast<unsigned int>(nparts - 1);
        int in_order = 1;
        if (last) {
            *ticket = 0;  // ready for the next call that uses this set
            unsigned int d;
            asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(d) : "l"(p.row_done + row) : "memory");
            in_order = d == epoch;
        }
        sh.flag[1] = last ? nparts : 0;
        sh.flag[0] = in_order;
    }
    cta_sync<kBar, NC>();
    const int nparts = sh.flag[1];
    if (nparts > 0) {
        if (!waited && !sh.flag[0]) {  // rare: the previous call has not written this row yet
            asm volatile("griddepcontrol.wait;" ::: "memory");
            waited = true;
        }
        merge_lists<T, NC, false, kBar>(p, row, rowlists, lstride, nparts, sh.ra, sh.rb, sh.red, sh.sint, sh.tmp);
        cta_sync<kBar, NC>();
        if (tid == 0) {
            const unsigned int d = epoch + 1u;
            asm volatile("st.release.gpu.u32 [%0], %1;" ::"l"(p.row_done + row), "r"(d) : "memory");
        }
    }
    return waited;
}

template <typename T>
__global__ void __launch_bounds__(kBulkThreads, 2) softmax_topk_bulk_kernel(const BulkParams bp) {
    constexpr int EPV = Elem<T>::kPerVec;
    constexpr int NC = kBulkConsumers;
    constexpr int TV = kBulkTileVecs;
    constexpr int J = kBulkJ;
    constexpr int S = kBulkStages;
    const ChunkParams &p = bp.c;
    extern __shared__ __align__(128) unsigned char s_dyn[];
    __shared__ __align__(8) uint64_t s_full[S], s_empty[S];
    __shared__ int s_hist[256];
    __shared__ int s_int[8 + 64];
    __shared__ float s_red[NC / 32];
    __shared__ int s_tmp[2], s_pick[4], s_count, s_flag[4];
    __shared__ int s_nrec, s_novf, s_ncand;
    __shared__ uint32_t s_tkey, s_epoch;
    __shared__ int s_abort;

    uint4 *const s_tiles = reinterpret_cast<uint4 *>(s_dyn);
    uint64_t *const s_ra = reinterpret_cast<uint64_t *>(s_dyn + static_cast<size_t>(S) * TV * 16);
    uint64_t *const s_rb = s_ra + kBulkRegion;
    uint32_t *const s_rec = reinterpret_cast<uint32_t *>(s_rb + kBulkRegion);
    uint32_t *const s_ovf = s_rec + (kBulkSlots + 1) * NC;
    volatile uint32_t *const s_keys = s_ovf + kBulkOverflow;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t grid = gridDim.x;
    const uint32_t nvv = static_cast<uint32_t>(p.nvv);
    const uint32_t total = static_cast<uint32_t>(p.rows) * nvv;
    const uint32_t per = static_cast<uint32_t>(p.per_cta);
    const uint32_t Vs = stream_boundary(blockIdx.x, grid, per, nvv, total, 0u);
    const uint32_t Ve = stream_boundary(blockIdx.x + 1, grid, per, nvv, total, 0u);

    if (tid == 0) {
        for (int s = 0; s < S; s++) {
            mbar_init(smem_addr(&s_full[s]), 1u);
            mbar_init(smem_addr(&s_empty[s]), NC / 32);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        s_nrec = 0;
        s_novf = 0;
        s_ncand = 0;
        s_tkey = 0;
        s_abort = 0;
        s_flag[2] = 0;
    }
    if (tid < NC)
        s_keys[tid] = 0u;
    bool waited = false;
    if (!p.input_ready) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        waited = true;
    }
    // The place of this call among the calls on its workspace: every CTA reads the call counter and
    // then draws an arrival ticket; the CTA that draws the last ticket of the call advances the
    // counter.  The next call is let in only after every CTA of this one has done so (the barrier
    // below orders the draw before the signal), so all CTAs of a call read the same number.
    if (tid == 0) {
        unsigned int e, t;
        asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(e) : "l"(p.epoch_word) : "memory");
        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(t) : "l"(p.arrive_word) : "memory");
        if (t == grid - 1u) {
            *p.arrive_word = 0u;
            const unsigned int n = e + 1u;
            asm volatile("st.release.gpu.u32 [%0], %1;" ::"l"(p.epoch_word), "r"(n) : "memory");
        }
        s_epoch = e;
    }
    __syncthreads();
    const uint32_t epoch = s_epoch;
    if (bp.trigger_tile <= 0 || Ve <= Vs)
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the next call of the stream may start
    if (Ve <= Vs)
        return;

    if (warp == NC / 32) {
        // ================= producer: one thread feeds the ring =================
        if (lane == 0) {
            TileWalk w;
            w.start(Vs, Ve, nvv);
            const char *base = static_cast<const char *>(p.logits);
            int t = 0;
            bool triggered = bp.trigger_tile <= 0;
            for (;;) {
                const int stage = t % S;
                if (t >= S && !mbar_wait(smem_addr(&s_empty[stage]), static_cast<uint32_t>((t / S - 1) & 1), &s_abort))
                    break;
                const uint32_t bytes = static_cast<uint32_t>(w.nv) * 16u;
                const char *src = base + (static_cast<int64_t>(w.row) * p.vstride + w.v0) * 16;
                const uint32_t bar = smem_addr(&s_full[stage]);
                mbar_expect_tx(bar, bytes);
                bulk_copy_g2s(smem_addr(s_tiles + stage * TV), src, bytes, bar);
                if (t == bp.trigger_tile && !triggered) {
                    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
                    triggered = true;
                }
                t++;
                if (!w.next())
                    break;
            }
            if (!triggered)
                asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
            if (s_abort) {
                // copies in flight must land before the CTA's shared memory is given up
                if (bp.status)
                    *bp.status = VKOP_TIMEOUT;
                for (int u = (t > S ? t - S : 0); u < t; u++) {
                    volatile int ignore = 0;
                    mbar_wait(smem_addr(&s_full[u % S]), static_cast<uint32_t>((u / S) & 1), &ignore);
                }
            }
        }
        return;
    }

    // ================= consumers =================
    const float c1 = p.inv_t * kLog2e;
    const int cols = static_cast<int>(p.cols);
    const bool ragged = cols % EPV != 0;
    const uint32_t xmask = p.negate ? (sizeof(T) == 4 ? 0x80000000u : 0x80008000u) : 0u;
    uint32_t *const my_rec = s_rec + tid;
    TileWalk w;
    w.start(Vs, Ve, nvv);
    int t = 0, pt = 0;
    float m_t = -INFINITY, o_t = 0.0f;
    float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
    int cnt = 0;
    bool nan_seen = false;
    uint32_t tk_seen = 0u;
    float T_f = -INFINITY;
    int part_v0 = w.v0;
    for (;;) {
        const int stage = t % S;
        if (!mbar_wait(smem_addr(&s_full[stage]), static_cast<uint32_t>((t / S) & 1), &s_abort))
            break;
        uint4 d[J];
        {
            const uint4 *src = s_tiles + stage * TV + tid;
#pragma unroll
            for (int j = 0; j < J; j++)
                d[j] = src[j * NC];
        }
        __syncwarp();
        if (lane == 0)
            mbar_arrive(smem_addr(&s_empty[stage]));
        if (xmask) {  // "smallest": the sign bits are flipped and the largest are selected
#pragma unroll
            for (int j = 0; j < J; j++) {
                d[j].x ^= xmask; d[j].y ^= xmask; d[j].z ^= xmask; d[j].w ^= xmask;
            }
        }
        const bool row_end = w.v0 + w.nv == static_cast<int>(nvv);
        if (w.nv != TV || (ragged && row_end)) {
            // a short tile, or the vector that holds the ragged end of the row: what is not data becomes -inf
#pragma unroll
            for (int j = 0; j < J; j++) {
                const int lv = j * NC + tid;
                if (lv >= w.nv) {
                    const uint32_t f = Elem<T>::kNegInfWord;
                    d[j] = make_uint4(f, f, f, f);
                } else if (ragged && w.v0 + lv == static_cast<int>(nvv) - 1) {
                    mask_vector<T>(d[j], 0, cols - (static_cast<int>(nvv) - 1) * EPV);
                }
            }
        }
        // ---- maximum of the thread's elements of this tile ----
        float vm;
        {
            float a[J];
#pragma unroll
            for (int j = 0; j < J; j++)
                a[j] = Elem<T>::vector_max(d[j]);
            vm = a[0];
#pragma unroll
            for (int j = 1; j < J; j++)
                vm = fmaxf(vm, a[j]);
        }
        if (vm > m_t) {
            // the thread's maximum rises: new offset, the sum so far is rescaled
            const float o_new = -__fmul_rn(vm, c1);
            const float s = (s0 + s1) + (s2 + s3);
            s0 = (m_t == -INFINITY && s == s) ? 0.0f : s * ex2_approx(o_new - o_t);
            s1 = s2 = s3 = 0.0f;
            m_t = vm;
            o_t = o_new;
            s_keys[tid] = order_key(vm);
        }
        if (p.need_sum && !(bp.debug & 4)) {
#pragma unroll
            for (int j = 0; j < J; j++) {
                float f[EPV];
                Elem<T>::unpack(d[j], f);
#pragma unroll
                for (int q = 0; q < EPV; q += 4) {
                    s0 += ex2_approx(__fmaf_rn(f[q], c1, o_t));
                    s1 += ex2_approx(__fmaf_rn(f[q + 1], c1, o_t));
                    s2 += ex2_approx(__fmaf_rn(f[q + 2], c1, o_t));
                    s3 += ex2_approx(__fmaf_rn(f[q + 3], c1, o_t));
                }
            }
        } else {
            // no sum to carry a NaN: look for it (fmaxf passes NaN over)
#pragma unroll
            for (int j = 0; j < J; j++)
                nan_seen |= Elem<T>::vector_has_nan(d[j]);
        }

        // ---- the bound ----
        if (bp.debug & 8) {
        } else if (w.part_first) {
            // first tile of a part: everybody waits for the first bound
            cta_sync<kBar, NC>();
            if (warp == 0) {
                const uint32_t tk = bulk_bisect(s_keys, p.k, 0u, 24);
                if (lane == 0)
                    s_tkey = tk;
            }
            cta_sync<kBar, NC>();
        } else if ((pt & (pt + 1)) == 0 && warp == ((31 - __clz(pt + 1)) & (NC / 32 - 1))) {
            // tiles 1, 3, 7, ...: one warp in turn tightens the bound while the others stream on
            const uint32_t tk = bulk_bisect(s_keys, p.k, *reinterpret_cast<volatile uint32_t *>(&s_tkey), 20);
            if (lane == 0)
                atomicMax(&s_tkey, tk);
        }
        {
            const uint32_t tk = *reinterpret_cast<volatile uint32_t *>(&s_tkey);
            if (tk != tk_seen) {
                tk_seen = tk;
                T_f = key_to_float(tk);
            }
        }
        // ---- a group that reaches the bound is recorded (where it is, not what it holds) ----
        {
            const bool hit = (bp.debug & 2) ? false : vm >= T_f;
            const int slot = cnt < kBulkSlots ? cnt : kBulkSlots;
            if (hit)
                my_rec[slot * NC] = static_cast<uint32_t>(w.v0 + tid);
            if (hit && cnt >= kBulkSlots) {
                const int pos = atomicAdd(&s_novf, 1);
                if (pos < kBulkOverflow)
                    s_ovf[pos] = static_cast<uint32_t>(w.v0 + tid);
            }
            cnt += hit ? 1 : 0;
        }

        const bool part_last = w.part_last;
        const int c_row = w.row, c_v1 = w.v0 + w.nv;
        const bool more = w.next();
        t++;
        pt++;
        if (part_last) {
            BulkPartEnd e;
            e.m_t = m_t;
            e.o_t = o_t;
            e.s_t = (s0 + s1) + (s2 + s3);
            e.cnt = cnt;
            e.nan_seen = nan_seen;
            e.row = c_row;
            e.part_v0 = part_v0;
            e.part_v1 = c_v1;
            e.epoch = epoch;
            e.waited = waited;
            BulkShared sh;
            sh.tiles = s_tiles;
            sh.ra = s_ra;
            sh.rb = s_rb;
            sh.rec = s_rec;
            sh.ovf = s_ovf;
            sh.keys = s_keys;
            sh.hist = s_hist;
            sh.sint = s_int;
            sh.tmp = s_tmp;
            sh.pick = s_pick;
            sh.count = &s_count;
            sh.flag = s_flag;
            sh.red = s_red;
            sh.nrec = &s_nrec;
            sh.novf = &s_novf;
            sh.ncand = &s_ncand;
            sh.tkey = &s_tkey;
            sh.abort = &s_abort;
            if (!(bp.debug & 1))
                waited = bulk_finish_part<T>(bp, sh, e);
            if (more) {
                // ---- reset for the next row part ----
                cta_sync<kBar, NC>();  // everybody is done with the regions, the keys and the counters
                s_keys[tid] = 0u;
                if (tid == 0) {
                    s_nrec = 0;
                    s_novf = 0;
                    s_ncand = 0;
                    s_tkey = 0;
                    s_flag[2] = 0;
                }
                m_t = -INFINITY;
                o_t = 0.0f;
                s0 = s1 = s2 = s3 = 0.0f;
                cnt = 0;
                nan_seen = false;
                tk_seen = 0u;
                T_f = -INFINITY;
                part_v0 = w.v0;
                pt = 0;
                cta_sync<kBar, NC>();
            }
        }
        if (!more)
            break;
    }
    if (s_abort && tid == 0 && bp.status)
        *bp.status = VKOP_TIMEOUT;
}

// ---------------------------------------------------------------------------

size_t stream_common_bytes(int64_t rows) { return 256 + ((static_cast<size_t>(rows) * 4 + 255) / 256) * 256; }

int plan_bulk(const vkop_softmax_topk_desc &d, bool base_aligned, BulkPlan *plan) {
    if (d.k > kChunkMaxK || d.splits > 0)
        return VKOP_UNSUPPORTED;
    const int esz = d.dtype == VKOP_F32 ? 4 : 2;
    const int epv = 16 / esz;
    const int64_t stride = d.row_stride ? d.row_stride : d.cols;
    if (!base_aligned || (stride * esz) % 16 != 0)
        return VKOP_UNSUPPORTED;  // the bulk copies need 16-byte aligned rows
    const int64_t nvv = (d.cols + epv - 1) / epv;
    if (d.rows <= 0 || d.rows >= (1ll << 31) || d.cols >= (1ll << 30) || d.rows * nvv >= (1ll << 32) - (1ll << 20))
        return VKOP_UNSUPPORTED;
    if (nvv < 2 * kBulkTileVecs)
        return VKOP_UNSUPPORTED;  // short rows: a row end per tile or two would dominate
    const int64_t total = d.rows * nvv;
    const int64_t tiles = (total + kBulkTileVecs - 1) / kBulkTileVecs;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess)
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaGetLastError();
    int64_t grid = sms < tiles ? sms : tiles;  // one CTA per SM; a second call may share the SM
    const int64_t need = d.k > 64 ? d.k : 64;  // a part publishes at least its own k best
    // parts a row can be cut into: its share of the CTAs, plus one at either end.  The CTA that merges
    // a row gathers all its parts' lists in one work region: fewer CTAs when that would not fit.
    int64_t per, maxparts;
    for (;;) {
        per = (total + grid - 1) / grid;
        maxparts = (nvv + per - 1) / per + 2;
        if ((maxparts <= kBulkMaxParts && maxparts * need <= kBulkRegion) || grid == 1)
            break;
        grid = grid * 7 / 8 > 0 ? grid * 7 / 8 : 1;
    }
    if (maxparts > kBulkMaxParts || maxparts * need > kBulkRegion)
        return VKOP_UNSUPPORTED;
    int list_cap = static_cast<int>(kBulkRegion / maxparts);
    if (list_cap > 256)
        list_cap = 256;
    plan->grid = static_cast<int>(grid);
    plan->per_cta = per;
    plan->nvv = nvv;
    plan->vstride = stride * esz / 16;
    plan->maxparts = static_cast<int>(maxparts);
    plan->list_cap = list_cap;
    plan->counters_bytes = ((static_cast<size_t>(d.rows) * 2 * 4 + 255) / 256) * 256;
    plan->lists_bytes = 2 * static_cast<size_t>(d.rows) * maxparts * (2 + list_cap) * 8;
    plan->smem_bytes = static_cast<size_t>(kBulkStages) * kBulkTileVecs * 16 + 2 * static_cast<size_t>(kBulkRegion) * 8 +
                       (static_cast<size_t>(kBulkSlots + 1) * kBulkConsumers + kBulkOverflow + kBulkConsumers) * 4;
    return VKOP_OK;
}

template <typename T>
static int launch_bulk_t(const BulkParams &bp, const BulkPlan &plan, cudaStream_t stream) {
    auto kern = softmax_topk_bulk_kernel<T>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(plan.smem_bytes)) != cudaSuccess)
        return VKOP_CUDA_ERROR;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(plan.grid));
    cfg.blockDim = dim3(kBulkThreads);
    cfg.dynamicSmemBytes = plan.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kern, bp) != cudaSuccess)
        return VKOP_CUDA_ERROR;
    note_launch(1);
    return check_launch();
}

int launch_bulk(const vkop_softmax_topk_desc &d, const BulkPlan &plan, const void *logits, void *out_values, void *out_indices,
                void *packets_out, void *common_ws, void *bulk_ws, int need_sum, cudaStream_t stream) {
    if (d.rows == 0)
        return VKOP_OK;
    if (reinterpret_cast<uintptr_t>(logits) % 16 != 0)
        return VKOP_INVALID_ARG;  // planned for an aligned base
    BulkParams bp = {};
    ChunkParams &p = bp.c;
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
    p.packets_out = reinterpret_cast<uint32_t *>(packets_out);
    p.nvv = plan.nvv;
    p.per_cta = plan.per_cta;
    p.vstride = plan.vstride;
    p.parts_per_row = 0;
    p.input_ready = (d.flags & VKOP_FLAG_INPUT_READY) ? 1 : 0;
    char *cw = static_cast<char *>(common_ws);
    p.arrive_word = reinterpret_cast<unsigned int *>(cw);
    p.epoch_word = reinterpret_cast<unsigned int *>(cw + 4);
    bp.status = reinterpret_cast<int *>(cw + 8);
    p.row_done = reinterpret_cast<unsigned int *>(cw + 256);
    p.counters = reinterpret_cast<unsigned int *>(bulk_ws);
    p.lists = reinterpret_cast<unsigned long long *>(static_cast<char *>(bulk_ws) + plan.counters_bytes);
    bp.trigger_tile = getenv("VKOP_BULK_TRIGGER") ? atoi(getenv("VKOP_BULK_TRIGGER")) : 0;
    bp.debug = getenv("VKOP_BULK_DEBUG") ? atoi(getenv("VKOP_BULK_DEBUG")) : 0;
    switch (d.dtype) {
    case VKOP_F32: return launch_bulk_t<float>(bp, plan, stream);
    case VKOP_F16: return launch_bulk_t<__half>(bp, plan, stream);
    case VKOP_BF16: return launch_bulk_t<__nv_bfloat16>(bp, plan, stream);
    default: return VKOP_INVALID_ARG;
    }
}

}  // namespace vkop_cuda
