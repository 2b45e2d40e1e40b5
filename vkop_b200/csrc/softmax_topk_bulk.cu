// Fused Softmax + TopK, bulk-copy streaming path: two kernels for long, 16-byte aligned rows.
//
// Kernel 1, bulk_stream_kernel, reads every logit once.  Every row is cut into P equal parts, one
// CTA each (P chosen so that the parts of one call fill the GPU about twice).  Inside a CTA every
// consumer warp has its own ring of shared-memory stages and takes tiles warp, warp + W, ... of the
// part (a tile is 2 KB: four 16-byte vectors per lane).  A producer warp hands the tiles to the copy
// engine, lane w feeding the ring of consumer warp w with one bulk copy per tile
// (cp.async.bulk.shared::cluster.global, plain form: no multicast, the source is this GPU's own
// memory); every stage has a "full" mbarrier that the copy completes (expect-tx / complete-tx bytes)
// and an "empty" mbarrier at which the consumer warp arrives once it holds the tile in registers.
// Consumer warps issue no copy, compute no address, and never wait for one another inside a part
// except once, after their first tile.
//
// Per tile and consumer lane: four 16-byte shared-memory loads, the maximum of the 16 (or 32)
// elements, and the exp-sum against a per-thread offset o = -(m * c1): one FFMA, one ex2 and one add
// per element (the offset moves, and the sum is rescaled, only when the thread's maximum rises).
//
// Selection.  Any value that at least k thread maxima reach bounds the k-th largest element of the
// part from below.  Every warp takes the r-th largest of its 32 running thread maxima
// (r = ceil(k / warps)); the smallest of those over the warps is such a value.  The warps post theirs
// after their first tile of the part (one barrier: the first bound) and again after their tiles 1,
// 3, 7, ... (no barrier: whoever posts recomputes the minimum and raises the shared bound).  In the
// loop a lane only tests the maximum of its elements of the tile against the bound; a vector that
// reaches it goes to a pool in shared memory as it is, with its place in the row.  At the end of the
// part the CTA writes the pool (a few hundred vectors), the part's maximum, exp-sum and bound to
// scratch memory and is gone: the streaming CTAs do nothing that is not streaming.
//
// Kernel 2, bulk_select_kernel, one small CTA per row, launched behind kernel 1 with programmatic
// stream serialization: it lets the next call's kernel 1 in at once, waits for its own kernel 1,
// reads the row's pools (from L2), keeps the elements that reach the largest of the parts' bounds,
// tightens the bound once more on the candidates themselves, ranks the survivors by counting and
// writes the k results.  It runs beside the next call's streaming CTAs.
//
// Order between calls.  Neither kernel touches global memory before it lets its successor in.  With
// VKOP_FLAG_INPUT_READY the streaming CTAs of a call read their logits beside the previous call; what
// they WRITE (the part's pool and header) they write after griddepcontrol.wait at the end of the
// part, that is, after the selection of the previous call has completed.  That selection has read
// the one set of scratch pools there is, and, since it waited for its own streaming kernel, which
// waited for the selection before it, the completed kernels form an unbroken chain: selections run
// one after the other and results reach the outputs in call order.  No call numbers, no counters.
// Without the flag the streaming kernel waits before its first read instead.
//
// Every wait in these kernels is bounded (about a second): a wait that runs out sets an abort flag
// and VKOP_TIMEOUT in the workspace status word; the CTA stops issuing copies, walks on without
// data so that its warps still meet at their barriers, waits (bounded) for the copies in flight and
// returns.

#include "common.cuh"
#include "launchers.h"
#include "select.cuh"
#include "stream_ranges.cuh"

namespace vkop_cuda {

#ifndef VKOP_BULK_STAGES
#define VKOP_BULK_STAGES 3
#endif
#ifndef VKOP_BULK_TILE_VECS
#define VKOP_BULK_TILE_VECS 1024
#endif
#ifndef VKOP_BULK_CTAS_PER_SM
#define VKOP_BULK_CTAS_PER_SM 2
#endif
constexpr int kBulkConsumers = 256;                 // consumer threads of a streaming CTA (8 warps)
constexpr int kBulkWarps = kBulkConsumers / 32;
constexpr int kBulkThreads = kBulkConsumers + 32;   // plus the producer warp
constexpr int kBulkTileVecs = VKOP_BULK_TILE_VECS;  // a tile: 16 KB, one bulk copy, consumed by all consumer warps
constexpr int kBulkStages = VKOP_BULK_STAGES;       // tiles in the ring (48 KB)
constexpr int kBulkJ = kBulkTileVecs / kBulkConsumers;  // vectors per consumer thread and tile
constexpr int kBulkPool = 1024;                     // vectors the pool of a part holds
constexpr int kBulkMaxParts = 8;                    // most parts a row is cut into
constexpr int kBulkMinPartVecs = 2048;              // a part is at least 32 KB
constexpr int kSelThreads = 256;                    // threads of a selecting CTA
constexpr int kSelCap = 1024;                       // candidates a row may gather before the exact fallback takes over
constexpr int kBar = 1;                             // named barrier of the consumer threads
static_assert(kBulkJ >= 1 && kBulkJ <= 8 && kBulkJ * kBulkConsumers == kBulkTileVecs, "every consumer thread takes the same share of a tile");

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
// may suspend the thread for a while when the phase is not complete
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
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
// never suspends
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Waits for the phase with the given parity; false when the limit ran out (then *abort is set) or
// somebody else has given up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort) {
    if (mbar_try(bar, parity))
        return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 256; i++) {
            if (mbar_try(bar, parity))
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

// What a part leaves in scratch memory for the selecting kernel: a header, then the pooled vectors,
// then the place of each in its row (vector index).
struct PartHeader {
    float mz;        // part maximum of z = x * inv_t
    float sum;       // exp-sum of the part relative to mz
    uint32_t tkey;   // bound: at least k elements of the part reach it (0: none)
    int32_t count;   // pooled vectors, or -1: the pool is no use (NaN, or more vectors than it holds)
    uint32_t pad[4];
};
constexpr size_t kPartStride = sizeof(PartHeader) + static_cast<size_t>(kBulkPool) * 20;
static_assert(sizeof(PartHeader) == 32 && kPartStride % 16 == 0, "pooled vectors are stored as 16-byte words");

struct BulkParams {
    ChunkParams c;            // logits, shape, outputs; nvv, vstride, per_cta; parts_per_row = P
    int *status;              // workspace: VKOP_OK or VKOP_TIMEOUT
    unsigned char *scratch;   // [rows * P] parts of kPartStride bytes
};

// Control block of a streaming CTA, behind the arrays in dynamic shared memory.
struct BulkCtl {
    uint64_t full[kBulkStages], empty[kBulkStages];
    float red[kBulkWarps];
    uint32_t wr[kBulkWarps];  // per warp: the r-th largest of its running thread maxima, as a key
    uint32_t wm[kBulkWarps];  // per warp: its largest thread maximum (end of the part)
    int nrec;                 // vectors in the pool (may count past its capacity)
    int nan_seen;
    uint32_t tkey;            // bound of the part as a key (0: none)
    int abort;
    int pad[4];
};

// Dynamic shared memory of the streaming kernel: tile rings | pool of recorded vectors | their places | control.
extern __shared__ __align__(128) unsigned char s_bulk[];
constexpr size_t kOffPool = static_cast<size_t>(kBulkStages) * kBulkTileVecs * 16;
constexpr size_t kOffPoolV = kOffPool + static_cast<size_t>(kBulkPool) * 16;
constexpr size_t kOffCtl = kOffPoolV + static_cast<size_t>(kBulkPool) * 4;
constexpr size_t kBulkSmemBytes = kOffCtl + sizeof(BulkCtl);
static_assert(kOffCtl % 16 == 0, "the control block holds 64-bit barriers");

// The r-th largest of the warp's 32 keys (0 when fewer than r keys are set).
__device__ __forceinline__ uint32_t warp_rth_largest(uint32_t key, int r) {
    const int lane = threadIdx.x & 31;
    uint32_t cur = key, rth = 0;
    for (int i = 0; i < r; i++) {
        rth = __reduce_max_sync(kFullMask, cur);
        const unsigned b = __ballot_sync(kFullMask, cur == rth);
        if (lane == __ffs(b) - 1)
            cur = 0;
    }
    return rth;
}

// The smallest of the warps' posted keys (0: some warp has posted none yet).
template <int NW>
__device__ __forceinline__ uint32_t posted_bound(const uint32_t *posted) {
    const volatile uint32_t *wr = posted;
    uint32_t t = 0xFFFFFFFFu;
#pragma unroll
    for (int q = 0; q < NW; q++) {
        const uint32_t v = wr[q];
        t = v < t ? v : t;
    }
    return t;
}

// ---------------------------------------------------------------------------
// Kernel 1: CTA c streams part c % P of row c / P.
template <typename T>
__global__ void __launch_bounds__(kBulkThreads, VKOP_BULK_CTAS_PER_SM) bulk_stream_kernel(const __grid_constant__ BulkParams bp) {
    constexpr int EPV = Elem<T>::kPerVec;
    constexpr int NC = kBulkConsumers;
    constexpr int NW = kBulkWarps;
    constexpr int TW = kBulkTileVecs;
    constexpr int J = kBulkJ;
    constexpr int R = kBulkStages;
    const ChunkParams &p = bp.c;
    uint4 *const s_tiles = reinterpret_cast<uint4 *>(s_bulk);
    uint4 *const s_pool = reinterpret_cast<uint4 *>(s_bulk + kOffPool);
    uint32_t *const s_pool_v = reinterpret_cast<uint32_t *>(s_bulk + kOffPoolV);
    BulkCtl *const ctl = reinterpret_cast<BulkCtl *>(s_bulk + kOffCtl);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t grid = gridDim.x;
    const uint32_t nvv = static_cast<uint32_t>(p.nvv);
    const uint32_t total = static_cast<uint32_t>(p.rows) * nvv;
    const uint32_t P = static_cast<uint32_t>(p.parts_per_row);
    const uint32_t Vs = stream_boundary(blockIdx.x, grid, 0u, nvv, total, P);
    const uint32_t Ve = stream_boundary(blockIdx.x + 1, grid, 0u, nvv, total, P);
    const int row = static_cast<int>(blockIdx.x / P);
    const int part_v0 = static_cast<int>(Vs - static_cast<uint32_t>(row) * nvv);
    const int part_len = static_cast<int>(Ve - Vs);  // (the planner leaves no part empty)
    const int part_v1 = part_v0 + part_len;
    const int ntiles = (part_len + TW - 1) / TW;

    if (tid < R) {
        mbar_init(smem_addr(&ctl->full[tid]), 1u);
        mbar_init(smem_addr(&ctl->empty[tid]), NW);
    }
    if (tid < NW)
        ctl->wr[tid] = 0u;
    if (tid == 0) {
        ctl->nrec = 0;
        ctl->nan_seen = 0;
        ctl->tkey = 0;
        ctl->abort = 0;
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    bool waited = false;
    if (!p.input_ready) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        waited = true;
    }
    __syncthreads();
    // The next kernel of the stream is let in when EVERY thread of every CTA has said so (or has
    // exited): all threads say so at once.  Nothing in global memory is touched before this.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == NW) {
        // ================= producer warp =================
        // One thread hands the tiles of the part to the copy engine, one bulk copy each, at most R in the ring.
        if (lane == 0) {
            const char *src0 = static_cast<const char *>(p.logits) + (static_cast<int64_t>(row) * p.vstride + part_v0) * 16;
            int t = 0;
            for (; t < ntiles; t++) {
                const int stage = t % R;
                if (t >= R && !mbar_wait(smem_addr(&ctl->empty[stage]), static_cast<uint32_t>((t / R - 1) & 1), &ctl->abort))
                    break;
                const int nv = part_len - t * TW < TW ? part_len - t * TW : TW;
                const uint32_t bytes = static_cast<uint32_t>(nv) * 16u, bar = smem_addr(&ctl->full[stage]);
                mbar_expect_tx(bar, bytes);
                bulk_copy_g2s(smem_addr(s_tiles + stage * TW), src0 + static_cast<int64_t>(t) * TW * 16, bytes, bar);
            }
            if (ctl->abort) {
                // copies in flight must land before the CTA's shared memory is given up
                if (bp.status)
                    *bp.status = VKOP_TIMEOUT;
                for (int u = (t > R ? t - R : 0); u < t; u++) {
                    volatile int ignore = 0;
                    mbar_wait(smem_addr(&ctl->full[u % R]), static_cast<uint32_t>((u / R) & 1), &ignore);
                }
            }
        }
        return;
    }
    // ================= consumer warps =================
    const float c1 = p.inv_t * kLog2e;
    const int cols = static_cast<int>(p.cols);
    const bool ragged = cols % EPV != 0;
    const uint32_t xmask = p.negate ? (sizeof(T) == 4 ? 0x80000000u : 0x80008000u) : 0u;
    const int need_sum = p.need_sum;
    const int rth = (p.k + NW - 1) / NW;  // NW times the rth-largest maximum of a warp: at least k maxima reach the smallest
    const uint4 *const ring = s_tiles + tid;
    float m_t = -INFINITY, o_t = 0.0f;
    float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
    int nan_seen = 0;
    uint32_t tk_seen = 0u;
    float T_f = -INFINITY;
    bool alive = true;
    for (int c = 0, lt = 0;; c++, lt++) {
        const bool have = c < ntiles;
        uint4 d[J];
        float a[J];
        float vm = -INFINITY;
        const int tv0 = part_v0 + c * TW;  // first vector of the tile in the row
        if (have) {
            const int stage = c % R;
            // (a wait that runs out sets the abort flag; the warp then walks on without data, so that it
            // still meets the others at every barrier, and the call reports VKOP_TIMEOUT)
            alive = alive && mbar_wait(smem_addr(&ctl->full[stage]), static_cast<uint32_t>((c / R) & 1), &ctl->abort);
            {
                const uint4 *src = ring + stage * TW;
#pragma unroll
                for (int j = 0; j < J; j++)
                    d[j] = src[j * NC];
            }
            __syncwarp();
            if (lane == 0)
                mbar_arrive(smem_addr(&ctl->empty[stage]));
            if (!alive) {  // (no data came: the tile counts as padding)
                const uint32_t f = Elem<T>::kNegInfWord;
#pragma unroll
                for (int j = 0; j < J; j++)
                    d[j] = make_uint4(f, f, f, f);
            }
            if (xmask) {  // "smallest": the sign bits are flipped and the largest are selected
#pragma unroll
                for (int j = 0; j < J; j++) {
                    d[j].x ^= xmask; d[j].y ^= xmask; d[j].z ^= xmask; d[j].w ^= xmask;
                }
            }
            const int nv = part_v1 - tv0 < TW ? part_v1 - tv0 : TW;
            if (nv != TW || (ragged && tv0 + nv == static_cast<int>(nvv))) {
                // a short tile, or the vector that holds the ragged end of the row: what is not data becomes -inf
#pragma unroll
                for (int j = 0; j < J; j++) {
                    const int lv = j * NC + tid;
                    if (lv >= nv) {
                        const uint32_t f = Elem<T>::kNegInfWord;
                        d[j] = make_uint4(f, f, f, f);
                    } else if (ragged && tv0 + lv == static_cast<int>(nvv) - 1) {
                        mask_vector<T>(d[j], 0, cols - (static_cast<int>(nvv) - 1) * EPV);
                    }
                }
            }
            // ---- maxima of the lane's vectors ----
#pragma unroll
            for (int j = 0; j < J; j++) {
                a[j] = Elem<T>::vector_max(d[j]);
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
            }
            if (need_sum) {
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
                    nan_seen |= Elem<T>::vector_has_nan(d[j]) ? 1 : 0;
            }
        }
        // ---- the bound: after its tiles 0, 1, 3, 7, ... of the part the warp posts the rth largest of
        // its running thread maxima; the smallest posted key is reached by at least k maxima ----
        if ((lt & (lt + 1)) == 0 && (have || lt == 0)) {
            const uint32_t wr = have ? warp_rth_largest(m_t == -INFINITY ? 0u : order_key(m_t), rth) : 0u;
            if (lane == 0)
                *const_cast<volatile uint32_t *>(&ctl->wr[warp]) = wr;
            if (lt == 0) {
                // first tile of the part: everybody waits for the first bound (a warp without a tile
                // posts "none", which leaves a tiny part without a bound)
                cta_sync<kBar, NC>();
                const uint32_t t0 = posted_bound<NW>(ctl->wr);
                if (t0 != 0u) {
                    tk_seen = t0;
                    T_f = key_to_float(t0);
                    if (tid == 0)
                        atomicMax(&ctl->tkey, t0);
                }
            } else {
                // later: no barrier; whoever posts takes the minimum of what is posted (keys only grow)
                __syncwarp();
                const uint32_t tn = posted_bound<NW>(ctl->wr);
                if (lane == 0 && tn > tk_seen)
                    atomicMax(&ctl->tkey, tn);
            }
        }
        if (!have)
            break;
        {
            const uint32_t tk = *reinterpret_cast<volatile uint32_t *>(&ctl->tkey);
            if (tk > tk_seen) {
                tk_seen = tk;
                T_f = key_to_float(tk);
            }
        }
        // ---- a vector that reaches the bound goes to the pool as it is, with its place in the row ----
        if (vm >= T_f) {
            int cnt = 0;
#pragma unroll
            for (int j = 0; j < J; j++)
                cnt += (a[j] >= T_f && tv0 + j * NC + tid < part_v1) ? 1 : 0;
            int pos = atomicAdd(&ctl->nrec, cnt);
#pragma unroll
            for (int j = 0; j < J; j++) {
                const int v = tv0 + j * NC + tid;
                if (a[j] >= T_f && v < part_v1) {
                    if (pos < kBulkPool) {
                        s_pool[pos] = d[j];
                        s_pool_v[pos] = static_cast<uint32_t>(v);
                    }
                    pos++;
                }
            }
        }
    }

    // ================= end of the part: statistics and the pool go to scratch memory =================
    {
        const uint32_t key = m_t == -INFINITY ? 0u : order_key(m_t);
        const uint32_t wm = __reduce_max_sync(kFullMask, key);
        if (lane == 0)
            ctl->wm[warp] = wm;
        if (nan_seen)
            ctl->nan_seen = 1;
    }
    // Everything this CTA writes to global memory comes after the kernel before it in the stream
    // (the selection of the previous call) has completed: that kernel has read the scratch pools this
    // CTA is about to overwrite, and, having itself waited for its predecessor, it stands for every
    // earlier kernel of the stream too.  The streaming above needed no such order.
    if (!waited)
        asm volatile("griddepcontrol.wait;" ::: "memory");
    cta_sync<kBar, NC>();  // maxima, pool and bound are final
    unsigned char *const part = bp.scratch + static_cast<size_t>(blockIdx.x) * kPartStride;
    uint32_t mkey = 0;
#pragma unroll
    for (int q = 0; q < NW; q++)
        mkey = ctl->wm[q] > mkey ? ctl->wm[q] : mkey;
    const float M = mkey ? key_to_float(mkey) : -INFINITY;  // part maximum of the stored logits
    const float O = -__fmul_rn(M, c1);
    {
        const float s_t = (s0 + s1) + (s2 + s3);
        const float contrib = (m_t == -INFINITY && s_t == s_t) ? 0.0f : s_t * ex2_approx(O - o_t);
        const float ws = warp_sum(contrib);
        if (lane == 0)
            ctl->red[warp] = ws;
    }
    const int n_rec = ctl->nrec;
    const bool pool_bad = ctl->nan_seen != 0 || n_rec > kBulkPool || ctl->abort != 0;
    if (!pool_bad) {
        uint4 *const gpool = reinterpret_cast<uint4 *>(part + sizeof(PartHeader));
        uint32_t *const gpos = reinterpret_cast<uint32_t *>(part + sizeof(PartHeader) + static_cast<size_t>(kBulkPool) * 16);
        for (int i = tid; i < n_rec; i += NC) {
            gpool[i] = s_pool[i];
            gpos[i] = s_pool_v[i];
        }
    }
    cta_sync<kBar, NC>();
    if (tid == 0) {
        float S = 0.0f;
#pragma unroll
        for (int w = 0; w < NW; w++)
            S += ctl->red[w];
        // S is relative to the offset O = -rn(M * c1); the published sum is relative to M exactly
        if (M != -INFINITY)
            S *= ex2_approx(-__fmaf_rn(M, c1, O));
        PartHeader h;
        h.mz = __fmul_rn(M, p.inv_t);
        h.sum = S;
        h.tkey = ctl->tkey;
        h.count = (pool_bad || (need_sum && S != S)) ? -1 : n_rec;
        h.pad[0] = h.pad[1] = h.pad[2] = h.pad[3] = 0u;
        *reinterpret_cast<uint4 *>(part) = *reinterpret_cast<const uint4 *>(&h);
        *reinterpret_cast<uint4 *>(part + 16) = *(reinterpret_cast<const uint4 *>(&h) + 1);
        if (ctl->abort && bp.status)
            *bp.status = VKOP_TIMEOUT;
    }
}

// ---------------------------------------------------------------------------
// Kernel 2: one CTA per row gathers what the parts of the row left, selects and writes the result.

// Ranks n distinct candidates held in shared memory by counting (the rank of a candidate is the
// number of candidates that beat it) and emits those of rank < k at their rank.  PER threads share
// one candidate's count.  No barrier; buf is only read.
template <typename T>
__device__ __forceinline__ void rank_emit(const ChunkParams &p, int64_t row, const uint64_t *buf, int n, float M, float S) {
    constexpr int NT = kSelThreads;
    const int tid = threadIdx.x;
    int per = 1;
    while (per < 8 && n * per * 2 <= NT)
        per *= 2;
    const int sub = tid & (per - 1);
    for (int c0 = 0; c0 < n; c0 += NT / per) {
        const int c = c0 + tid / per;
        const uint64_t me = c < n ? buf[c] : ~0ull;
        // (independent counts, several loads in flight: a plain loop would pay the shared-memory
        // latency once per candidate)
        int b0 = 0, b1 = 0, b2 = 0, b3 = 0;
        int i = sub;
        for (; i + 7 * per < n; i += 8 * per) {
            uint64_t x[8];
#pragma unroll
            for (int u = 0; u < 8; u++)
                x[u] = buf[i + u * per];
            b0 += (x[0] > me ? 1 : 0) + (x[4] > me ? 1 : 0);
            b1 += (x[1] > me ? 1 : 0) + (x[5] > me ? 1 : 0);
            b2 += (x[2] > me ? 1 : 0) + (x[6] > me ? 1 : 0);
            b3 += (x[3] > me ? 1 : 0) + (x[7] > me ? 1 : 0);
        }
        for (; i < n; i += per)
            b0 += buf[i] > me ? 1 : 0;
        int beat = (b0 + b1) + (b2 + b3);
        for (int o = 1; o < per; o <<= 1)
            beat += __shfl_xor_sync(kFullMask, beat, o);
        if (c < n && sub == 0 && beat < p.k)
            emit<T>(p, row, beat, me, M, S, nullptr);
    }
}

template <typename T>
__global__ void __launch_bounds__(kSelThreads) bulk_select_kernel(const __grid_constant__ BulkParams bp) {
    constexpr int EPV = Elem<T>::kPerVec;
    constexpr int NT = kSelThreads;
    constexpr int NW = NT / 32;
    const ChunkParams &p = bp.c;
    __shared__ __align__(16) uint64_t s_a[kSelCap], s_b[kCandCap];  // candidates; tightened candidates / exact fallback
    __shared__ PartHeader s_hdr[kBulkMaxParts];
    __shared__ uint32_t s_wr[NW];
    __shared__ int s_hist[256], s_pick[4], s_count, s_n[2];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row = blockIdx.x;
    const int P = p.parts_per_row;
    const int cols = static_cast<int>(p.cols);
    const uint32_t nvv = static_cast<uint32_t>(p.nvv);
    // the next call's streaming kernel may start at once: this kernel is small and runs beside it
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (tid == 0) {
        s_n[0] = 0;
        s_n[1] = 0;
    }
    // Everything the streaming kernel of this call wrote is visible after this; and since that kernel
    // waited for the selection of the previous call before it wrote, the selections of consecutive
    // calls run one after the other: results reach the outputs in call order.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __syncthreads();
    const unsigned char *const set = bp.scratch;
    if (tid < P)
        s_hdr[tid] = *reinterpret_cast<const PartHeader *>(set + (static_cast<size_t>(row) * P + tid) * kPartStride);
    __syncthreads();
    uint32_t trow = 0;
    float M = -INFINITY;
    bool any_bad = false;
    int total = 0;
    for (int j = 0; j < P; j++) {
        trow = s_hdr[j].tkey > trow ? s_hdr[j].tkey : trow;
        M = fmaxf(M, s_hdr[j].mz);
        any_bad |= s_hdr[j].count < 0;
        total += s_hdr[j].count > 0 ? s_hdr[j].count : 0;
    }
    float S = 0.0f;
    for (int j = 0; j < P; j++) {
        const float sj = s_hdr[j].sum;
        if (sj != 0.0f)  // an all -inf part has sum 0 and no defined maximum
            S += sj * expf(s_hdr[j].mz - M);
    }
    // A part whose pool is no use (NaN, massive ties) makes its bound no use either.
    if (any_bad)
        trow = 0;
    const float Tf = trow ? key_to_float(trow) : -INFINITY;

    // ---- the pooled vectors of all parts: the elements that reach the row's bound become candidates ----
    for (int f0 = 0; f0 < total; f0 += 4 * NT) {
        // four pooled vectors in flight per thread: one round trip to L2 for the usual row
        uint4 dd[4];
        int vv[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int f = f0 + u * NT + tid;
            vv[u] = -1;
            if (f < total) {
                int j = 0, i = f;
                while (i >= (s_hdr[j].count > 0 ? s_hdr[j].count : 0)) {
                    i -= s_hdr[j].count > 0 ? s_hdr[j].count : 0;
                    j++;
                }
                const unsigned char *part = set + (static_cast<size_t>(row) * P + j) * kPartStride;
                dd[u] = __ldcg(reinterpret_cast<const uint4 *>(part + sizeof(PartHeader)) + i);
                vv[u] = static_cast<int>(__ldcg(reinterpret_cast<const uint32_t *>(part + sizeof(PartHeader) + static_cast<size_t>(kBulkPool) * 16) + i));
            }
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            float x[EPV];
            Elem<T>::unpack(dd[u], x);
            const int v = vv[u];
            unsigned mine = 0;
            if (v >= 0) {
#pragma unroll
                for (int q = 0; q < EPV; q++)
                    mine |= (v * EPV + q < cols && x[q] >= Tf) ? 1u << q : 0u;
            }
            const int cnt = __popc(mine);
            int incl = cnt;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int y = __shfl_up_sync(kFullMask, incl, o);
                if (lane >= o)
                    incl += y;
            }
            const int wtotal = __shfl_sync(kFullMask, incl, 31);
            if (wtotal == 0)
                continue;
            int base = 0;
            if (lane == 31)
                base = atomicAdd(&s_n[0], wtotal);
            int pos = __shfl_sync(kFullMask, base, 31) + incl - cnt;
#pragma unroll
            for (int q = 0; q < EPV; q++) {
                if (mine & (1u << q)) {
                    if (pos < kSelCap)
                        s_a[pos] = make_cand(order_key(x[q]), static_cast<uint32_t>(v * EPV + q));
                    pos++;
                }
            }
        }
    }
    __syncthreads();
    int n = s_n[0];
    const uint64_t *best = s_a;
    if (any_bad || n > kSelCap) {
        // Rare: exact radix select over the whole row, re-read from L2 (the pooled vectors were sign-
        // flipped where the smallest are wanted; the fallback flips for itself).
        const uint4 *vbase = reinterpret_cast<const uint4 *>(p.logits) + static_cast<int64_t>(row) * p.vstride;
        const int kk = cols < p.k ? cols : p.k;
        select_fallback<T, NT>(vbase, 0, static_cast<int64_t>(nvv), 0, p.cols, p.negate, kk, s_b, &s_count, s_hist, s_pick);
        n = s_count;
        best = s_b;
    } else if (n > 2 * p.k && n > 96) {
        // Many candidates for a ranking by counting: a closer bound first.  Every thread takes the
        // largest key of its share of the candidates, every warp the rth largest of those (NW * rth >=
        // k); at least k candidates reach the smallest of the warps' values.
        uint32_t key = 0;
        for (int c = tid; c < n; c += NT) {
            const uint32_t kc = cand_key(s_a[c]);
            key = kc > key ? kc : key;
        }
        const uint32_t wr = warp_rth_largest(key, (p.k + NW - 1) / NW);
        if (lane == 0)
            s_wr[warp] = wr;
        __syncthreads();
        const uint32_t bound = posted_bound<NW>(s_wr);
        for (int c0 = 0; c0 < n; c0 += NT) {
            const int c = c0 + tid;
            const uint64_t cd = c < n ? s_a[c] : 0ull;
            const bool pass = c < n && cand_key(cd) >= bound;
            const unsigned bal = __ballot_sync(kFullMask, pass);
            if (bal != 0u) {
                int base = 0;
                if (lane == 0)
                    base = atomicAdd(&s_n[1], __popc(bal));
                base = __shfl_sync(kFullMask, base, 0);
                if (pass)
                    s_b[base + __popc(bal & ((1u << lane) - 1u))] = cd;
            }
        }
        __syncthreads();
        n = s_n[1];
        best = s_b;
    }
    if (p.packets_out && tid == 0) {
        uint32_t *pk = p.packets_out + static_cast<int64_t>(row) * packet_words(p.k);
        pk[0] = __float_as_uint(M);
        pk[1] = __float_as_uint(S);
        pk[2] = static_cast<uint32_t>(n < p.k ? n : p.k);
        pk[3] = 0;
    }
    rank_emit<T>(p, row, best, n, M, S);
}

// ---------------------------------------------------------------------------

// head (call counters, status) | per row: order word / calls finished | per row: calls started
size_t stream_common_bytes(int64_t rows) { return 256 + 2 * ((static_cast<size_t>(rows) * 4 + 255) / 256) * 256; }

int plan_bulk(const vkop_softmax_topk_desc &d, bool base_aligned, BulkPlan *plan) {
    if (d.k > kChunkMaxK)
        return VKOP_UNSUPPORTED;
    const int esz = d.dtype == VKOP_F32 ? 4 : 2;
    const int epv = 16 / esz;
    const int64_t stride = d.row_stride ? d.row_stride : d.cols;
    if (!base_aligned || (stride * esz) % 16 != 0)
        return VKOP_UNSUPPORTED;  // the bulk copies need 16-byte aligned rows
    const int64_t nvv = (d.cols + epv - 1) / epv;
    if (d.rows <= 0 || d.rows >= (1ll << 28) || d.cols >= (1ll << 30) || d.rows * nvv >= (1ll << 32) - (1ll << 20))
        return VKOP_UNSUPPORTED;
    if (nvv < kBulkMinPartVecs)
        return VKOP_UNSUPPORTED;  // short rows: the end of a part every few tiles would dominate
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess)
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaGetLastError();
    // Parts per row: the smallest power of two that fills most of the CTA slots of the GPU (two per
    // SM) with one call, every part at least kBulkMinPartVecs vectors (the caller may name it in
    // desc.splits).
    int P = 1;
    if (d.splits > 0) {
        P = d.splits;
        if (P > kBulkMaxParts || nvv / P < kBulkMinPartVecs)
            return VKOP_UNSUPPORTED;
    } else {
        while (P < kBulkMaxParts && d.rows * P * 5 < static_cast<int64_t>(sms) * VKOP_BULK_CTAS_PER_SM * 4 &&
               nvv / (2 * P) >= kBulkMinPartVecs)
            P *= 2;
    }
    plan->nvv = nvv;
    plan->vstride = stride * esz / 16;
    plan->smem_bytes = kBulkSmemBytes;
    plan->parts = P;
    plan->grid = static_cast<int>(d.rows * P);
    plan->scratch_bytes = static_cast<size_t>(d.rows) * P * kPartStride;
    return VKOP_OK;
}

template <typename Kern>
static int launch_pdl(Kern kern, unsigned grid, unsigned block, size_t smem, cudaStream_t stream, const BulkParams &bp) {
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
        return VKOP_CUDA_ERROR;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = smem;
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

template <typename T>
static int launch_bulk_t(const BulkParams &bp, const BulkPlan &plan, cudaStream_t stream) {
    int rc = launch_pdl(bulk_stream_kernel<T>, static_cast<unsigned>(plan.grid), kBulkThreads, plan.smem_bytes, stream, bp);
    if (rc != VKOP_OK)
        return rc;
    return launch_pdl(bulk_select_kernel<T>, static_cast<unsigned>(bp.c.rows), kSelThreads, 0, stream, bp);
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
    p.vstride = plan.vstride;
    p.parts_per_row = plan.parts;
    p.input_ready = (d.flags & VKOP_FLAG_INPUT_READY) ? 1 : 0;
    char *cw = static_cast<char *>(common_ws);
    bp.status = reinterpret_cast<int *>(cw + 8);
    bp.scratch = static_cast<unsigned char *>(bulk_ws);
    switch (d.dtype) {
    case VKOP_F32: return launch_bulk_t<float>(bp, plan, stream);
    case VKOP_F16: return launch_bulk_t<__half>(bp, plan, stream);
    case VKOP_BF16: return launch_bulk_t<__nv_bfloat16>(bp, plan, stream);
    default: return VKOP_INVALID_ARG;
    }
}

}  // namespace vkop_cuda
