// Fused Softmax + TopK, streaming path: one kernel for large batches.
//
// Streaming.  Every CTA owns one contiguous range of 16-byte vector slots of the [rows, cols]
// tensor: a whole row, one of a few equal parts of a row, or (with more rows than CTA slots) a
// byte-balanced range that may run across rows, its boundaries snapped to multiples of 256 vectors
// inside a row so that no CTA holds a sliver.  A CTA walks its range in tiles that are staged
// through shared memory with cp.async, two stages deep (four stages of half-size tiles for whole rows of
// 16-bit logits in overlapping calls): the copies of the next tiles are in flight while the current one is
// processed, every thread copies into and reads back its own slots only, and the only wait of the
// streaming loop is the hardware wait on the thread's own copy groups.
//
// Per tile and thread: the maximum of its elements updates a running maximum m_t and rescales a
// running exp-sum s_t (online softmax).  The running thread maxima give the selection threshold T
// (stream_refresh_threshold): any value that at least k thread maxima reach is a lower bound of the
// k-th largest element; T is refreshed on tiles 0, 1, 3, 7, ... of a part and only rises inside a
// part.  An element >= T is kept: every thread owns a few private slots in shared memory and appends
// there with a plain store; a thread whose slots are full appends to a shared overflow list.
//
// End of a row part (stream_finish_part): the statistics are reduced over the CTA, candidates below
// the final threshold are dropped, and then, by launch shape:
//   whole rows   the CTA selects the k best of its candidates and writes the result;
//   cluster      the CTAs of a row are a thread-block cluster: cluster barrier, then the first CTA
//                reads the other CTAs' lists through distributed shared memory, merges and writes;
//   otherwise    the part is published to scratch memory; the last part of the row to arrive
//                (ticket counter) gathers the lists of the row, merges and writes.
// A CTA never waits for another CTA of its own launch except at the cluster barrier.
//
// Launches use programmatic stream serialization.  A kernel lets its successor in as soon as all
// its CTAs run (griddepcontrol.launch_dependents) and orders itself against its predecessor only
// where memory demands it.  Without VKOP_FLAG_INPUT_READY that is at once (griddepcontrol.wait before
// the first read).  With the flag the logits need no ordering, back-to-back calls overlap several deep,
// and what remains is the order of the results and of the scratch lists:
//   whole rows   Calls number themselves per row: the CTA of a row draws a ticket from the row's own
//                counter, first thing, one round trip before it lets the successor in.  Results of one
//                row reach the outputs in call order through the row's order word and mailbox (OrderWait
//                in select.cuh): a CTA whose predecessor has not finished the row leaves its ranked result
//                for that CTA to deliver and goes; nobody waits holding a place on an SM.  CTA 0 of every
//                kernel waits for the previous kernel before it ends, so that a kernel has completed only
//                when all earlier ones have.
//   otherwise    Calls number themselves in the workspace (a call counter advanced by the last CTA of a
//                call to arrive, before the successor is let in).  Scratch lists alternate between two sets
//                by call parity, so a call only needs the call before its predecessor to be done with a
//                row's lists; and results of one row are written in call order.  Both are checked with one
//                acquire load of a per-row counter of finished calls; when the check fails the CTA falls
//                back to griddepcontrol.wait for the whole previous call.
// A replayed CUDA graph needs no changing parameter either way.
#include "common.cuh"
#include "launchers.h"
#include "select.cuh"
#include "stream_ranges.cuh"

namespace vkop_cuda {

constexpr int kStreamThreads = 512;      // one call at a time: two CTAs per SM
constexpr int kStreamThreadsSmall = 256; // calls that overlap: four lighter CTAs per SM hide each other's row ends
constexpr int kStreamVecs = 4;
constexpr int kStreamDeepVecs = 2;    // whole rows in overlapping calls: smaller tiles ...
constexpr int kStreamDeepStages = 4;  // ... and more of them in flight
constexpr int kStreamCtasPerSm = 2;
constexpr int kNumSms = 148;
constexpr int kStreamSlots = 4;       // private candidate slots of one thread
constexpr int kStreamListCap = 512;   // most candidates one row part publishes
constexpr int kStreamMaxCluster = 8;  // largest portable thread-block cluster

// A lower bound of the k-th largest element of the part seen so far, from the running thread
// maxima (m_t of every thread of the CTA; 0 = no bound).  Any value that at least k thread maxima
// reach is valid, since they are k different elements.  First a coarse pair: lo, the smallest
// maximum over at least k groups of gs lanes (valid, but several times too many elements reach it),
// and hi, the smallest maximum over a few large groups (usually above the k-th largest).  Then a
// histogram of the thread maxima between lo and hi, 256 bins, picks the highest bin edge that k
// maxima still reach.  Two CTA barriers.  sh_hnext is cleared for the refresh after this one.
// Out of line: it runs on a few tiles only and must not cost the streaming loop registers.
template <int THREADS>
__device__ __noinline__ uint32_t stream_refresh_threshold(float m_t, int k, int gs, int nfullw, int hgroups, uint32_t *sh_wr,
                                                          uint32_t *sh_wm, int *sh_hist, int *sh_hnext, uint32_t *sh_tnew) {
    constexpr int NW = THREADS / 32;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t key = order_key(m_t);
    uint32_t glo = key;
    if (gs > 0 && warp < nfullw) {
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t other = __shfl_xor_sync(kFullMask, glo, o);
            glo = o < gs ? max(glo, other) : min(glo, other);  // maximum inside a group, minimum over groups
        }
    } else {
        glo = gs > 0 ? 0xFFFFFFFFu : 0u;  // a partly filled warp does not constrain the threshold
    }
    const uint32_t wmax = __reduce_max_sync(kFullMask, key);
    if (lane == 0) {
        sh_wr[warp] = glo;
        sh_wm[warp] = wmax;
    }
    __syncthreads();
    if (tid < 256)
        sh_hnext[tid] = 0;  // the histogram of the refresh after this one (everybody is done with it)
    uint32_t lo = lane < NW ? sh_wr[lane] : 0xFFFFFFFFu;
    lo = __reduce_min_sync(kFullMask, lo);
    // hi: warps are paired up into hgroups groups; the smallest group maximum
    uint32_t hi = 0xFFFFFFFFu;
    if (lane < hgroups) {
        hi = 0u;
        for (int w = lane; w < NW; w += hgroups)
            hi = max(hi, sh_wm[w]);
    }
    hi = __reduce_min_sync(kFullMask, hi);
    uint32_t t_new = lo;
    if (lo != 0u && hi > lo) {  // (the same for every thread of the CTA)
        const uint32_t range = hi - lo;
        const int shift = range > 255u ? 24 - __clz(range) : 0;  // range >> shift <= 255
        if (key >= lo) {
            const uint32_t b = (key - lo) >> shift;
            atomicAdd(&sh_hist[b < 255u ? b : 255u], 1);
        }
        __syncthreads();
        if (warp == 0) {
            // lane l owns bins 8l .. 8l+7; suffix counts over the lanes, then inside the lane that crosses k
            const int4 h0 = *reinterpret_cast<const int4 *>(&sh_hist[8 * lane]);
            const int4 h1 = *reinterpret_cast<const int4 *>(&sh_hist[8 * lane + 4]);
            const int own = h0.x + h0.y + h0.z + h0.w + h1.x + h1.y + h1.z + h1.w;
            int suf = own;  // maxima in the bins of this lane and of the lanes above
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_down_sync(kFullMask, suf, o);
                if (lane + o < 32)
                    suf += v;
            }
            const unsigned reach = __ballot_sync(kFullMask, suf >= k);  // lane 0 always does: lo is valid
            if (lane == 31 - __clz(reach)) {
                const int c[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
                int acc = suf - own, bin = 8 * lane;
                bool found = false;
#pragma unroll
                for (int q = 7; q >= 0; q--) {
                    acc += c[q];
                    if (!found && acc >= k) {
                        found = true;
                        bin = 8 * lane + q;
                    }
                }
                (*sh_tnew) = lo + (static_cast<uint32_t>(bin) << shift);
            }
        }
        __syncthreads();
        t_new = (*sh_tnew);
    }
    return t_new;
}

// What the end of a row part needs from the streaming loop, by value.
struct PartEnd {
    float m_t, s_t;       // this thread's running maximum and exp-sum
    uint32_t tkey;        // final threshold key of the part
    uint64_t *slot;       // this thread's next private slot (tells how many it filled)
    int c_row, c_v0, c_nvt, part_v0, head, nvr;
    const uint4 *vbase;
    int stage;            // tile stage just consumed (the others may hold copies in flight)
    uint32_t epoch;       // number of this call on its workspace
    bool has_next, waited;
};
// Shared-memory work areas of the streaming kernel (declared there).
struct StreamShared {
    uint32_t *wm0;
    float *red;
    int *hist, *pick, *tmp, *flag, *sint, *count;
};

// End of a row part: statistics, the part's candidate list, and whatever the launch shape asks for
// next (cluster hand-over, direct selection of a whole row, or publication and the row merge by the
// last part to arrive).  Returns whether the CTA has waited for the previous call by now.
// Kept out of line on purpose: inlined, its many live values cost the streaming loop registers
// (the loop spills and runs a third slower).
template <typename T, int THREADS, int VECS, bool ALIGNED, bool CLUSTER, int STAGES>
__device__ __noinline__ bool stream_finish_part(const ChunkParams &p, const PartEnd e, const StreamShared sh, uint64_t *s_dyn) {
    constexpr int EPV = Elem<T>::kPerVec;
    constexpr int NW = THREADS / 32;
    constexpr int TV = THREADS * VECS;
    constexpr int CAP = kStreamSlots * THREADS;
    constexpr int SLOTS = kStreamSlots;
    uint4 *s_tile = reinterpret_cast<uint4 *>(s_dyn);
    uint64_t *s_cand = s_dyn + STAGES * TV * 2;
    uint64_t *s_work = s_cand + CAP;
    uint32_t *s_wm0 = sh.wm0;
    float *s_red = sh.red;
    int *s_hist = sh.hist, *s_pick = sh.pick, *s_tmp = sh.tmp, *s_flag = sh.flag, *s_int = sh.sint;
    int &s_count = *sh.count;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t grid = gridDim.x;
    const uint32_t nvv = static_cast<uint32_t>(p.nvv);
    const uint32_t total = static_cast<uint32_t>(p.rows) * nvv;
    const uint32_t per = static_cast<uint32_t>(p.per_cta);
    const uint32_t parts = static_cast<uint32_t>(p.parts_per_row);
    const float c1 = p.inv_t * kLog2e;
    const int64_t lstride = 2 + p.list_cap;
    const int cols = static_cast<int>(p.cols);
    unsigned int *const row_done = p.row_done;  // per row: calls whose result is written
    const float m_t = e.m_t, s_t = e.s_t;
    const uint32_t tkey = e.tkey;
    uint64_t *const slot = e.slot;
    const int c_row = e.c_row, c_v0 = e.c_v0, c_nvt = e.c_nvt, part_v0 = e.part_v0, head = e.head, nvr = e.nvr;
    const uint4 *const vbase = e.vbase;
    const int stage = e.stage;
    const uint32_t epoch = e.epoch;
    const int64_t set = epoch & 1u;
    const bool has_next = e.has_next;
    (void)has_next;
    bool waited = e.waited;
    // ================= end of a row part: statistics, publish, maybe merge the row =================
    const uint32_t c_first = parts > 0 ? static_cast<uint32_t>(c_row) * parts
                                       : stream_owner(static_cast<uint32_t>(c_row) * nvv, grid, per, nvv, total, parts);
    const int pidx = static_cast<int>(blockIdx.x - c_first);
    // whole: this CTA holds the whole row (one part per row): nothing to publish, it selects itself
    const bool whole = !CLUSTER && parts == 1;
    const bool local = CLUSTER || whole;
    unsigned long long *rowlists = local ? nullptr : p.lists + (set * p.rows + c_row) * p.splits * lstride;
    // where the part is published: scratch memory, or this CTA's second candidate region
    unsigned long long *mylist = local ? reinterpret_cast<unsigned long long *>(s_work) : rowlists + pidx * lstride;
    // This set of lists last served the call before the previous one: is that call's merge of
    // this row finished?  (Asked early, used after the reduction below.)
    unsigned int done_calls = 0;
    if (!CLUSTER && tid == 0 && !waited)
        asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(done_calls) : "l"(row_done + c_row) : "memory");

    // ---- statistics: per warp first, one barrier, then over the warps ----
    uint32_t wkey = order_key(m_t);
#pragma unroll
    for (int o = 1; o < 32; o <<= 1)
        wkey = max(wkey, __shfl_xor_sync(kFullMask, wkey, o));
    {
        const float mw = key_to_float(wkey);
        const float sw = warp_sum((m_t == -INFINITY && s_t == s_t) ? 0.0f : s_t * ex2_approx((m_t - mw) * c1));
        if (lane == 0) {
            s_wm0[warp] = wkey;
            s_red[warp] = sw;
        }
    }
    if (tid == 0) {
        s_tmp[0] = 0;
        // scratch lists: calls 0 .. epoch - 2 are done with them; whole rows: results come in call order
        // (whole rows: the row's order word, calls finished in its low 16 bits; see OrderWait)
        s_flag[0] = whole ? ((done_calls ^ epoch) & 0xFFFFu) == 0u : static_cast<int>(done_calls - epoch + 1u) >= 0;
    }
    __syncthreads();
    uint32_t mkey = lane < NW ? s_wm0[lane] : 0u;
    const float mw = key_to_float(mkey);
    const float sw = lane < NW ? s_red[lane] : 0.0f;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1)
        mkey = max(mkey, __shfl_xor_sync(kFullMask, mkey, o));
    const float mx = key_to_float(mkey);  // part maximum of the stored logits
    const float S = warp_sum(sw != 0.0f ? sw * ex2_approx((mw - mx) * c1) : sw);  // (a NaN sum stays NaN)
    const float mz = __fmul_rn(mx, p.inv_t);
    const int novf = s_count;  // entries of the overflow list

    const int part_v1 = c_v0 + c_nvt;
    int e0 = part_v0 * EPV - head, e1 = part_v1 * EPV - head;
    if (e0 < 0) e0 = 0;
    if (e1 > cols) e1 = cols;
    const int nvalid = e1 > e0 ? e1 - e0 : 0;
    const int kk = nvalid < p.k ? nvalid : p.k;

    // Rare: the row's lists may still be in use.  Waiting for the whole previous call is always
    // enough (it has merged this row only after the call before it had).
    if (!local && !waited && !s_flag[0]) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        waited = true;
    }

    // ---- candidates: private slots -> the part's list in scratch memory ----
    // Entries kept under the weaker thresholds of the early tiles are dropped: at least k elements
    // of this part reach the final threshold.  (No threshold: tkey is 0 and every entry stays.)
    const int held = static_cast<int>((slot - (s_cand + tid)) / THREADS);
    uint32_t tpub = tkey;  // threshold the row merge may rely on
    int C;
    const bool plain = novf == 0 && !(S != S);
    if (plain) {
#pragma unroll
        for (int q = 0; q < SLOTS; q++) {
            uint64_t ent = 0;
            if (q < held)
                ent = s_cand[q * THREADS + tid];
            const uint32_t key = order_key(__uint_as_float(static_cast<uint32_t>(ent >> 32)));
            const bool pass = q < held && key >= tkey;
            const unsigned b = __ballot_sync(kFullMask, pass);
            if (b != 0u) {
                int base = 0;
                if (lane == 0)
                    base = atomicAdd(&s_tmp[0], __popc(b));
                base = __shfl_sync(kFullMask, base, 0);
                const int pos = base + __popc(b & ((1u << lane) - 1u));
                if (pass && pos < p.list_cap)
                    mylist[2 + pos] = make_cand(key, static_cast<uint32_t>(ent));
            }
        }
        __syncthreads();
        C = s_tmp[0];
    } else {
        C = p.list_cap + 1;
    }
    if (C > p.list_cap) {
        // Rare: more candidates than a part may publish, threads that ran out of private slots,
        // or NaN in the part (NaN ranks first but is invisible to the thread maxima).  Everything
        // goes to one dense list in shared memory and the part's own k best are selected.
        __syncthreads();
        uint64_t mine[SLOTS];
#pragma unroll
        for (int q = 0; q < SLOTS; q++)
            mine[q] = q < held ? s_cand[q * THREADS + tid] : 0ull;
        if (tid == 0)
            s_tmp[0] = 0;
        __syncthreads();  // every private slot has been read: the region is free for the list
        auto to_list = [&](uint64_t ent) {
            const uint32_t key = order_key(__uint_as_float(static_cast<uint32_t>(ent >> 32)));
            if (key >= tkey) {
                const int pos = atomicAdd(&s_tmp[0], 1);
                if (pos < CAP)
                    s_cand[pos] = make_cand(key, static_cast<uint32_t>(ent));
            }
        };
#pragma unroll
        for (int q = 0; q < SLOTS; q++) {
            if (q < held)
                to_list(mine[q]);
        }
        for (int i = tid; i < (novf < CAP ? novf : CAP); i += THREADS)
            to_list(s_work[i]);
        __syncthreads();
        C = s_tmp[0];
        if (C > CAP || novf > CAP || S != S) {
            // exact radix select over the part, re-read from L2
            const int fv1 = part_v1 < nvr ? part_v1 : nvr;
            select_fallback<T, THREADS>(vbase, part_v0, fv1, head, p.cols, p.negate, kk, s_cand, sh.count, s_hist, s_pick);
            C = s_count;
        }
        if (C > p.list_cap) {
            // (scratch: the overflow list has been consumed; a part that stays in shared memory is
            // published there, and the tile stages are free: such a CTA does not go on to another row)
            select_and_emit<T, THREADS>(p, c_row, s_cand, C, local ? s_dyn : s_work, 0.0f, 0.0f, mylist + 2, s_tmp);
            C = kk;
        } else {
            for (int i = tid; i < C; i += THREADS)
                mylist[2 + i] = s_cand[i];
        }
        tpub = 0;  // the list holds the part's best, not everything above a threshold
        __syncthreads();
    }

    if (CLUSTER) {
        // ---- the parts of the row meet at the cluster barrier; the first CTA of the row merges
        // them straight from the other CTAs' shared memory ----
        if (tid == 0) {
            mylist[0] = (static_cast<unsigned long long>(__float_as_uint(S)) << 32) | __float_as_uint(mz);
            mylist[1] = (static_cast<unsigned long long>(tpub) << 16) | static_cast<unsigned long long>(C);
        }
        cooperative_groups::cluster_group cluster = cooperative_groups::this_cluster();
        cluster.sync();
        if (cluster.block_rank() == 0) {
            // (the tile stages are free: no CTA of a cluster goes on to another row)
            static_assert(!CLUSTER || STAGES == 2, "the cluster merge splits two tile stages");
            merge_lists<T, THREADS, true>(p, c_row, mylist, 0, static_cast<int>(parts), s_dyn, s_dyn + 2 * TV, s_red, s_int,
                                          s_tmp);
        }
        cluster.sync();  // the other CTAs keep their shared memory until it has been read
    } else if (whole) {
        // ---- the part is the row: select among its candidates and write the result.  Results of one
        // row reach the outputs in call order, without this CTA waiting for the previous call's CTA of
        // the row: when that one has not finished, the result is left in the row's mailbox for it to
        // deliver (OrderWait, row_order_finish). ----
        OrderWait ow;
        ow.word = row_done + c_row;
        ow.epoch = epoch;
        ow.flag = &s_flag[1];
        {
            const uint32_t vb = (static_cast<uint32_t>(p.k) * sizeof(T) + 15u) & ~15u;
            const uint32_t ib = (static_cast<uint32_t>(p.k) * (p.index_dtype == VKOP_I64 ? 8u : 4u) + 15u) & ~15u;
            ow.mail_idx_off = 16u + vb;
            ow.mail_stride = 16u + vb + ib;
            ow.mail = p.packets_out ? nullptr
                                    : reinterpret_cast<unsigned char *>(p.lists) + static_cast<size_t>(c_row) * kMailSlots * ow.mail_stride;
        }
        ow.need = !waited && !s_flag[0];
        ow.waited = waited;
        ow.deposited = false;
        select_and_emit<T, THREADS>(p, c_row, reinterpret_cast<uint64_t *>(mylist + 2), C, s_dyn, mz, S, nullptr, s_tmp, &ow);
        waited = ow.waited;
        if (p.packets_out && tid == 0) {
            uint32_t *pk = p.packets_out + static_cast<int64_t>(c_row) * packet_words(p.k);
            pk[0] = __float_as_uint(mz);
            pk[1] = __float_as_uint(S);
            pk[2] = static_cast<uint32_t>(C < p.k ? C : p.k);
            pk[3] = 0;
        }
        __syncthreads();
        if (warp == 0)
            row_order_finish<T>(p, ow, c_row);
    } else {
    // ---- announce the part; the last part of a row to arrive merges the row ----
        if (tid == 0) {
            mylist[0] = (static_cast<unsigned long long>(__float_as_uint(S)) << 32) | __float_as_uint(mz);
            mylist[1] = (static_cast<unsigned long long>(tpub) << 16) | static_cast<unsigned long long>(C);
            const uint32_t c_end = parts > 0 ? c_first + parts - 1
                                             : stream_owner(static_cast<uint32_t>(c_row + 1) * nvv - 1, grid, per, nvv, total, parts);
            const int nparts = static_cast<int>(c_end - c_first + 1);
            // release: the list (written by all threads before the barrier) and the header; acquire:
            // the lists of the parts that arrived earlier
            unsigned int arrived;
            unsigned int *ticket = p.counters + set * p.rows + c_row;
            asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(arrived) : "l"(ticket) : "memory");
            const bool last = arrived == static_cast<unsigned int>(nparts - 1);
            int in_order = 1;
            if (last) {
                *ticket = 0;  // ready for the next call that uses this set
                // results of one row are written in call order: has the previous call written its own?
                unsigned int d;
                asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(d) : "l"(row_done + c_row) : "memory");
                in_order = d == epoch;
            }
            s_flag[1] = last ? nparts : 0;
            s_flag[0] = in_order;
        }
        __syncthreads();
        const int nparts = s_flag[1];
        if (nparts > 0) {
            if (!waited && !s_flag[0]) {  // rare: the previous call is still merging this row
                asm volatile("griddepcontrol.wait;" ::: "memory");
                waited = true;
            }
            // the tile stage just consumed takes the gathered lists (the others may hold a copy
            // in flight), the two candidate regions serve the selection: 8 * THREADS slots each
            uint64_t *mbuf = reinterpret_cast<uint64_t *>(s_tile + stage * TV);
            merge_lists<T, THREADS>(p, c_row, rowlists, lstride, nparts, mbuf, s_cand, s_red, s_int, s_tmp);
            __syncthreads();
            // the row's result is written and its lists are read
            if (tid == 0) {
                const unsigned int d = epoch + 1u;
                asm volatile("st.release.gpu.u32 [%0], %1;" ::"l"(row_done + c_row), "r"(d) : "memory");
            }
        }
    }
    return waited;
}

template <typename T, int THREADS, int VECS, bool ALIGNED, bool CLUSTER, int STAGES = 2>
__global__ void __launch_bounds__(THREADS, 1024 / THREADS) softmax_topk_stream_kernel(const ChunkParams p) {
    constexpr int AHEAD = STAGES - 1;  // tiles in flight while one is processed
    constexpr int EPV = Elem<T>::kPerVec;
    constexpr int NW = THREADS / 32;
    constexpr int TV = THREADS * VECS;  // vectors per tile
    constexpr int CAP = kStreamSlots * THREADS;  // candidate slots of one row part
    extern __shared__ __align__(16) uint64_t s_dyn[];
    uint4 *s_tile = reinterpret_cast<uint4 *>(s_dyn);  // STAGES tile stages of TV vectors
    // First region: while a part streams, SLOTS private slots per thread (slot s of thread t at
    // s * THREADS + t), each (float bits << 32 | index in the row); after the part, the dense list.
    uint64_t *s_cand = s_dyn + STAGES * TV * 2;
    // Second region: while a part streams, the overflow list of threads whose slots are full
    // (s_count entries); after the part, scratch of the in-CTA selection.
    uint64_t *s_work = s_cand + CAP;
    constexpr int SLOTS = CAP / THREADS;
    static_assert(SLOTS * THREADS == CAP && SLOTS >= 1, "private slots tile the first region");
    __shared__ uint32_t s_wr[2][NW], s_wm[2][NW];
    __shared__ __align__(16) int s_thist[2][256];  // histograms of thread maxima (threshold refresh), used in turn
    __shared__ float s_red[NW];
    __shared__ int s_hist[256];
    __shared__ int s_pick[4];
    __shared__ int s_tmp[2];
    __shared__ int s_int[8 + (THREADS >= 512 ? 1024 : 64)];  // merge: per-part header fields (parts <= 1024 / 64)
    __shared__ int s_count;
    __shared__ uint32_t s_epoch, s_tnew;
    __shared__ int s_flag[2];

    const int tid = threadIdx.x;
    const uint32_t grid = gridDim.x;
    const uint32_t nvv = static_cast<uint32_t>(p.nvv);
    const uint32_t total = static_cast<uint32_t>(p.rows) * nvv;
    const uint32_t per = static_cast<uint32_t>(p.per_cta);
    const uint32_t parts = static_cast<uint32_t>(p.parts_per_row);
    const uint32_t Vs = stream_boundary(blockIdx.x, grid, per, nvv, total, parts);
    const uint32_t Ve = stream_boundary(blockIdx.x + 1, grid, per, nvv, total, parts);
    if (Ve <= Vs) {
        if (CLUSTER) {  // (the planner gives every CTA of a cluster a part; keep the barriers matched anyway)
            cooperative_groups::this_cluster().sync();
            cooperative_groups::this_cluster().sync();
        }
        return;
    }
    int remaining = static_cast<int>(Ve - Vs);
    // Whole rows in overlapping calls: the calls of one row are numbered by a ticket of that row alone,
    // drawn here, first thing, by one thread (CTA c holds row c).  One round trip, no other CTA involved.
    const bool row_tickets = !CLUSTER && parts == 1 && p.input_ready;
    unsigned int ticket = 0;
    if (row_tickets && tid == 0)
        asm volatile("atom.relaxed.gpu.global.add.u32 %0, [%1], 1;" : "=r"(ticket) : "l"(p.row_ticket + blockIdx.x) : "memory");
    bool waited = false;
    if (!p.input_ready) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        waited = true;
    }
    const uint32_t filler = Elem<T>::kNegInfWord;
    const float c1 = p.inv_t * kLog2e;
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

    // ---- tile iterators: (row, first vector slot, slots in the tile).  One walks in front and starts the
    // copies, AHEAD tiles before the other, which processes them. ----
    auto tile_len = [&](int tv0, int rem) {
        const int n = TV < static_cast<int>(nvv) - tv0 ? TV : static_cast<int>(nvv) - tv0;
        return n > rem ? rem : n;
    };
    int row = static_cast<int>(Vs / nvv);
    int v0 = static_cast<int>(Vs - static_cast<uint32_t>(row) * nvv);
    int nvt = tile_len(v0, remaining);
    bool part_last = (v0 + nvt == static_cast<int>(nvv)) || (nvt == remaining);  // last tile of the row part
    int i_row = row, i_v0 = v0, i_nvt = nvt, i_rem = remaining, i_stage = 0;  // the tile to copy next

    // this thread's first slot of stage 0, as a shared-memory address
    const uint32_t sdst0 = static_cast<uint32_t>(__cvta_generic_to_shared(s_tile + tid));
    auto issue_tile = [&](int stage, int r, int tv0, int tn) {
        if (ALIGNED && tn == TV) {
            // a full tile of an aligned row: four copies at fixed offsets, nothing to test
            const char *g = reinterpret_cast<const char *>(reinterpret_cast<const uint4 *>(p.logits) +
                                                           static_cast<int64_t>(r) * p.vstride + tv0 + tid);
            const uint32_t sdst = sdst0 + static_cast<uint32_t>(stage) * (TV * 16);
#pragma unroll
            for (int j = 0; j < VECS; j++)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sdst + j * THREADS * 16), "l"(g + j * THREADS * 16)
                             : "memory");
            asm volatile("cp.async.commit_group;" ::: "memory");
            return;
        }
        int head, nvr;
        const uint4 *vbase;
        row_geom(r, head, nvr, vbase);
        const int lim = tn < nvr - tv0 ? tn : nvr - tv0;
        const uint4 *src = vbase + tv0;
        uint4 *dst = s_tile + stage * TV;
#pragma unroll
        for (int j = 0; j < VECS; j++) {
            const int lv = j * THREADS + tid;
            if (lv < lim) {
                const uint32_t saddr = static_cast<uint32_t>(__cvta_generic_to_shared(dst + lv));
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(saddr), "l"(src + lv) : "memory");
            } else {
                dst[lv] = make_uint4(filler, filler, filler, filler);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // Starts the copy of the next tile that has none yet, or commits an empty group when the range is
    // exhausted: every call is one copy group, so that the wait below always counts the same.
    auto issue_next = [&]() {
        if (i_rem > 0) {
            issue_tile(i_stage, i_row, i_v0, i_nvt);
            i_rem -= i_nvt;
            if (i_rem > 0) {
                i_v0 += i_nvt;
                if (i_v0 >= static_cast<int>(nvv)) {
                    i_row++;
                    i_v0 = 0;
                }
                i_nvt = tile_len(i_v0, i_rem);
            }
        } else {
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
        i_stage = i_stage + 1 == STAGES ? 0 : i_stage + 1;
    };
    int stage = 0;
#pragma unroll
    for (int a = 0; a < AHEAD; a++)
        issue_next();

    // ---- the place of this call among the calls that share its workspace (the first tile is on its
    // way meanwhile).  Every CTA reads the workspace's call counter and then draws an arrival ticket;
    // the CTA that draws the last ticket of the call advances the counter.  The next call is let in
    // only after every CTA of this one has drawn (a barrier orders the draw before the signal), so
    // all CTAs of a call read the same number, whatever the grids of the calls.  Calls alternate between two sets
    // of scratch lists and arrival counters, so a call never waits for the row merges of the call
    // right before it, only for those of the call before that.
    // CLUSTER (the CTAs of one row form a thread-block cluster and hand their parts over in shared
    // memory) is used for calls that wait for their predecessor at once: nothing to number. ----
    if (row_tickets) {
        if (tid == 0)
            s_epoch = ticket;
    } else if (!CLUSTER && tid == 0) {
        unsigned int e, t;
        asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(e) : "l"(p.epoch_word) : "memory");
        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(t) : "l"(p.arrive_word) : "memory");
        if (t == grid - 1u) {  // the last CTA of this call to arrive numbers the next call
            *p.arrive_word = 0u;
            const unsigned int n = e + 1u;
            asm volatile("st.release.gpu.u32 [%0], %1;" ::"l"(p.epoch_word), "r"(n) : "memory");
            // The next call reads both words without any other ordering against this call than its start,
            // and it starts once every CTA here has passed the signal below: the two stores have to be
            // performed, not just ordered, before this thread signals.
            __threadfence();
        }
        s_epoch = e;
    }

    // ---- state of the current row part ----
    // Threshold groups: gs lanes form a group; the minimum over all groups (of full warps) of the group
    // maximum of the running thread maxima has at least one element per group at or above it, so gs is
    // the largest power of two that still gives k groups (0: the part is too small for a threshold).
    auto group_lanes = [&](int full_warps) {
        int g = 32;
        while (g >= 1 && full_warps * (32 / g) < p.k)
            g >>= 1;
        return g;
    };
    float m_t = -INFINITY, s_t = 0.0f;
    uint32_t tkey = 0;       // running threshold key (0 = none yet: every valid element is a candidate)
    float T_thr = key_to_float(0u);
    int part_v0 = v0;        // first slot of the part
    int part_tile = 0;       // tiles of the part processed so far
    int nfullw = (nvt < THREADS ? nvt : THREADS) / 32;  // warps whose threads all own data in this part
    int gs = group_lanes(nfullw);
    int parity = 0;
    // groups for the upper end of the histogram range: the smallest of their maxima should rank
    // well inside the best k thread maxima
    const int hgroups_k = p.k < 4 ? 1 : p.k < 10 ? 2 : p.k < 24 ? 4 : p.k < 56 ? 8 : 16;
    const int hgroups = hgroups_k < NW ? hgroups_k : NW;  // (a group is at least one warp)
    if (tid < 256)
        s_thist[0][tid] = 0;
    uint64_t *slot = s_cand + tid;  // this thread's next private slot; past slot_end the slots are full
    uint64_t *const slot_end = s_cand + CAP;
    // Keeps one element of the part: idx is its index in the row.
    auto keep = [&](float fv, int idx) {
        const uint64_t ent = (static_cast<uint64_t>(__float_as_uint(fv)) << 32) | static_cast<uint32_t>(idx);
        if (slot < slot_end) {
            *slot = ent;
        } else {
            const int pos = atomicAdd(&s_count, 1);
            if (pos < CAP)
                s_work[pos] = ent;
        }
        slot += THREADS;
    };
    if (tid == 0)
        s_count = 0;
    __syncthreads();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t epoch = CLUSTER ? 0u : s_epoch;
    for (;;) {
        const int c_row = row;
        const int c_v0 = v0, c_nvt = nvt;
        const bool c_last = part_last;
        int head, nvr;
        const uint4 *vbase;
        row_geom(c_row, head, nvr, vbase);
        // start the copy AHEAD tiles in front, wait for the current tile, advance the iterator
        remaining -= nvt;
        const bool has_next = remaining > 0;
        issue_next();
        asm volatile("cp.async.wait_group %0;" ::"n"(AHEAD) : "memory");  // everything but the AHEAD newest groups
        // the current tile: this thread's own slots of the stage
        uint4 d[VECS];
        uint4 *const cur = s_tile + stage * TV + tid;
#pragma unroll
        for (int j = 0; j < VECS; j++)
            d[j] = cur[j * THREADS];
        const int consumed = stage;
        stage = stage + 1 == STAGES ? 0 : stage + 1;
        if (has_next) {
            v0 += nvt;
            if (v0 >= static_cast<int>(nvv)) {
                row++;
                v0 = 0;
            }
            nvt = tile_len(v0, remaining);
            part_last = (v0 + nvt == static_cast<int>(nvv)) || (nvt == remaining);
        }

        bool edited = false;  // the words differ from what the stage holds
        if (p.negate) {
            edited = true;
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
            edited = true;
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

        // The candidate filter further down reads the tile from the stage again (keeping the words in
        // registers across the threshold refresh costs more than the few vectors it looks at).
        if (edited) {
#pragma unroll
            for (int j = 0; j < VECS; j++)
                cur[j * THREADS] = d[j];
        }

        // ---- maxima per vector and of the tile; online softmax statistics ----
        float vmax[VECS];
        float vm = -INFINITY;
#pragma unroll
        for (int j = 0; j < VECS; j++) {
            const float a = Elem<T>::vector_max(d[j]);
            vmax[j] = a;
            vm = fmaxf(vm, a);
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
        } else {
            // Nothing is summed here (no sum wanted, or no finite reference yet), and the maxima pass
            // NaN over: look for it and poison the sum, which sends the part to the exact fallback.
            bool has_nan = false;
#pragma unroll
            for (int j = 0; j < VECS; j++)
                has_nan |= Elem<T>::vector_has_nan(d[j]);
            if (has_nan)
                s_t = __int_as_float(0x7FC00000);
        }

        // ---- threshold refresh from the running thread maxima: on tiles 0, 1, 3, 7, ... of the part and
        // on its last tile (the threshold settles quickly); the other tiles need no barrier at all.
        // (stream_refresh_threshold) ----
        if ((part_tile & (part_tile + 1)) == 0 || c_last) {
            const uint32_t t_new = stream_refresh_threshold<THREADS>(m_t, p.k, gs, nfullw, hgroups, s_wr[parity], s_wm[parity],
                                                                     s_thist[parity], s_thist[parity ^ 1], &s_tnew);
            tkey = t_new > tkey ? t_new : tkey;
            T_thr = key_to_float(tkey);
            parity ^= 1;
        }
        part_tile++;
        const bool allpass = tkey == 0u || T_thr == -INFINITY;

        // ---- candidates of this tile ----
        if (!allpass) {
            // padding is -inf and T is above -inf: whatever passes is a valid element
            const int ibase = (c_v0 + tid) * EPV - head;
#pragma unroll
            for (int j = 0; j < VECS; j++) {
                if (!(vmax[j] < T_thr)) {
                    float f[EPV];
                    Elem<T>::unpack(cur[j * THREADS], f);
#pragma unroll
                    for (int e = 0; e < EPV; e++) {
                        if (!(f[e] < T_thr))
                            keep(f[e], ibase + j * THREADS * EPV + e);
                    }
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < VECS; j++) {
                float f[EPV];
                Elem<T>::unpack(cur[j * THREADS], f);
                const int lv = j * THREADS + tid;
#pragma unroll
                for (int e = 0; e < EPV; e++) {
                    const int i = (c_v0 + lv) * EPV + e - head;
                    if (lv < c_nvt && i >= 0 && i < cols)
                        keep(f[e], i);
                }
            }
        }

        if (c_last) {
            PartEnd e;
            e.m_t = m_t;
            e.s_t = s_t;
            e.tkey = tkey;
            e.slot = slot;
            e.c_row = c_row;
            e.c_v0 = c_v0;
            e.c_nvt = c_nvt;
            e.part_v0 = part_v0;
            e.head = head;
            e.nvr = nvr;
            e.vbase = vbase;
            e.stage = consumed;
            e.epoch = epoch;
            e.has_next = has_next;
            e.waited = waited;
            StreamShared sh;
            sh.wm0 = s_wm[0];
            sh.red = s_red;
            sh.hist = s_hist;
            sh.pick = s_pick;
            sh.tmp = s_tmp;
            sh.flag = s_flag;
            sh.sint = s_int;
            sh.count = &s_count;
            waited = stream_finish_part<T, THREADS, VECS, ALIGNED, CLUSTER, STAGES>(p, e, sh, s_dyn);
            if (has_next) {
                // ---- reset for the next row part ----
                __syncthreads();  // every thread is done with the candidate regions and the counters
                m_t = -INFINITY;
                s_t = 0.0f;
                tkey = 0;
                T_thr = key_to_float(0u);
                part_v0 = v0;
                part_tile = 0;
                nfullw = (nvt < THREADS ? nvt : THREADS) / 32;
                gs = group_lanes(nfullw);
                slot = s_cand + tid;
                if (tid == 0)
                    s_count = 0;
            }
        }
        if (!has_next)
            break;
    }
    // Overlapping calls: a kernel must not complete before its predecessor has (with whole rows a result may
    // have been left for a CTA of an earlier kernel to deliver; in every shape, whatever is enqueued behind a
    // call may overwrite the logits of the calls before it): one CTA waits for the previous kernel.
    if (!CLUSTER && blockIdx.x == 0 && !waited)
        asm volatile("griddepcontrol.wait;" ::: "memory");
}

// ---------------------------------------------------------------------------

int plan_stream(const vkop_softmax_topk_desc &d, bool base_aligned, StreamPlan *plan) {
    if (d.k > kChunkMaxK)
        return VKOP_UNSUPPORTED;
    const int esz = d.dtype == VKOP_F32 ? 4 : 2;
    const int epv = 16 / esz;
    const int64_t stride = d.row_stride ? d.row_stride : d.cols;
    // rows that all start on a 16-byte boundary: exact slot count and the cheaper address arithmetic
    const bool aligned = base_aligned && (stride * esz) % 16 == 0;
    const int64_t nvv = aligned ? (d.cols + epv - 1) / epv : (d.cols + 2 * (epv - 1)) / epv;
    if (d.rows <= 0 || d.rows >= (1ll << 31) || d.cols >= (1ll << 30) || d.rows * nvv >= (1ll << 32) - (1ll << 20))
        return VKOP_UNSUPPORTED;
    const int64_t total = d.rows * nvv;
    const int64_t slots = kNumSms * kStreamCtasPerSm;
    const int64_t tile = static_cast<int64_t>(kStreamThreads) * kStreamVecs;
    const int64_t tiles = (total + tile - 1) / tile;
    int64_t grid = slots < tiles ? slots : tiles;
    int parts_per_row = 0;
    // Calls that may overlap their predecessor (the caller vouches for the logits) fill the GPU
    // together: a call takes about 64 CTAs, a whole row per CTA when there are that many rows, so
    // that rows need no merge at all.  A call that waits for its predecessor spreads over all SMs.
    const bool overlapping = (d.flags & VKOP_FLAG_INPUT_READY) != 0;
    if (d.rows <= slots / 2) {  // (with more rows than that, byte-balanced ranges were measured faster than a CTA per row)
        int64_t s = slots / d.rows;
        if (overlapping) {
            const int64_t few = (64 + d.rows - 1) / d.rows;
            s = few < s ? few : s;
        }
        if (d.splits > 0)
            s = d.splits;  // the caller's choice of CTAs per row
        // (decided on the slot count of aligned rows whatever the pointer: calls with aligned and
        // unaligned logits may share a workspace, and the meaning of the rows' order words follows the shape)
        const int64_t nvv_a = (d.cols + epv - 1) / epv;
        const int64_t tiles_a = (d.rows * nvv_a + tile - 1) / tile;
        if (s <= slots && nvv_a / s >= 2 * kUnit && d.rows * s <= tiles_a) {
            parts_per_row = static_cast<int>(s);  // the same number of CTAs for every row: no CTA crosses a row
            grid = d.rows * s;
        }
    }
    // Several hundred rows (at least half of what the GPU holds as light CTAs, at most all of it): one
    // 256-thread CTA per row, four to an SM, in a single wave.  One call fills the GPU by itself, no row has
    // parts to merge, and no CTA crosses a row.
    bool many_whole_rows = false;
    {
        const int64_t light_slots = 4 * static_cast<int64_t>(kNumSms);
        const int64_t nvv_a = (d.cols + epv - 1) / epv;
        if (d.splits == 0 && parts_per_row == 0 && d.rows >= light_slots / 2 && d.rows <= light_slots &&
            nvv_a >= 2048) {  // (rows of 32 KB and more)
            many_whole_rows = true;
            parts_per_row = 1;
            grid = d.rows;
        }
    }
    const int64_t per = (total + grid - 1) / grid;
    // parts a row can be cut into: its share of the CTAs, plus one at either end
    const int64_t maxparts = parts_per_row > 0 ? parts_per_row : (nvv + per - 1) / per + 2;
    // Overlapping calls run as lighter CTAs, four to an SM: while some finish their row part, the
    // others keep streaming.  A call that waits for its predecessor anyway runs as two large CTAs
    // per SM, and with few parts per row the CTAs of a row form a cluster and hand their parts over
    // in shared memory.
    int threads = kStreamThreads;
    if ((overlapping || many_whole_rows) && parts_per_row > 0 && maxparts <= 64 && maxparts * d.k <= 8 * kStreamThreadsSmall)
        threads = kStreamThreadsSmall;
    // The CTA that merges a row gathers every part's list into one tile stage of its shared memory
    // (8 * threads slots) and selects in the two candidate regions (as many again).
    const int64_t merge_slots = 8 * static_cast<int64_t>(threads);
    static_assert(kStreamVecs * 16 == 8 * 8 && 2 * kStreamSlots == 8, "a tile stage and the candidate regions hold 8 slots per thread");
    if (maxparts * d.k > merge_slots || maxparts > 1024)
        return VKOP_UNSUPPORTED;
    int list_cap = static_cast<int>(merge_slots / maxparts);
    if (list_cap > kStreamListCap)
        list_cap = kStreamListCap;
    plan->threads = threads;
    plan->grid = static_cast<int>(grid);
    plan->per_cta = per;
    plan->nvv = nvv;
    plan->vstride = aligned ? stride * esz / 16 : 0;
    plan->aligned = aligned ? 1 : 0;
    plan->parts_per_row = parts_per_row;
    // few parts per row: the CTAs of a row form a cluster and hand their parts over in shared memory
    plan->cluster = (!overlapping && !many_whole_rows && parts_per_row >= 1 && parts_per_row <= kStreamMaxCluster) ? parts_per_row : 0;
    plan->maxparts = static_cast<int>(maxparts);
    plan->list_cap = list_cap;
    // per row: an arrival counter for each of the two sets of lists (the call counter and the rows'
    // counters of finished calls sit in the head of the workspace that the streaming kernels share)
    plan->counters_bytes = ((static_cast<size_t>(d.rows) * 2 * 4 + 255) / 256) * 256;
    plan->lists_bytes = 2 * static_cast<size_t>(d.rows) * maxparts * (2 + list_cap) * 8;
    if ((overlapping || many_whole_rows) && parts_per_row == 1) {
        // whole rows publish no lists; the region holds the rows' mailboxes (kMailSlots entries of two
        // addresses, k values and k indices, each block rounded up to 16 bytes)
        const size_t entry = 16 + ((static_cast<size_t>(d.k) * esz + 15) & ~static_cast<size_t>(15)) +
                             ((static_cast<size_t>(d.k) * (d.index_dtype == VKOP_I64 ? 8 : 4) + 15) & ~static_cast<size_t>(15));
        plan->lists_bytes = static_cast<size_t>(d.rows) * kMailSlots * entry;
    }
    // Whole rows of 16-bit logits in overlapping calls: eight-kilobyte tiles, four stages.  Such a CTA is one of a
    // few hundred that share the memory system, each limited by what it has in flight: three tiles instead of
    // one, at the same sixteen elements per thread and tile as 32-bit logits have in a sixteen-kilobyte tile
    // (measured: 8.4 -> 7.0 us a call for fp16; 32-bit logits, eight elements per tile, lose to the loop overhead).
    plan->deep = (esz == 2 && threads == kStreamThreadsSmall && parts_per_row == 1 && kStreamThreadsSmall != kStreamThreads) ? 1 : 0;
    const size_t stage_bytes = plan->deep ? static_cast<size_t>(kStreamDeepStages) * threads * kStreamDeepVecs * 16
                                          : 2 * static_cast<size_t>(threads) * kStreamVecs * 16;
    plan->smem_bytes = stage_bytes + 2 * static_cast<size_t>(kStreamSlots) * threads * 8;
    return VKOP_OK;
}

// cluster > 0: consecutive groups of `cluster` CTAs form thread-block clusters.
template <typename Kern, typename... Args>
static int launch_pdl(Kern kern, unsigned grid, unsigned block, size_t smem, unsigned cluster, cudaStream_t stream, Args... args) {
    if (smem > 32 * 1024 &&
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
        return VKOP_CUDA_ERROR;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 1;
    if (cluster > 0) {
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = cluster;
        attr[1].val.clusterDim.y = 1;
        attr[1].val.clusterDim.z = 1;
        cfg.numAttrs = 2;
    }
    cfg.attrs = attr;
    return cudaLaunchKernelEx(&cfg, kern, args...) == cudaSuccess ? VKOP_OK : VKOP_CUDA_ERROR;
}

template <typename T, bool ALIGNED>
static int launch_stream_t(const ChunkParams &p, const StreamPlan &plan, cudaStream_t stream) {
    const unsigned grid = static_cast<unsigned>(plan.grid);
    int rc;
    if (plan.cluster > 0)
        rc = launch_pdl(softmax_topk_stream_kernel<T, kStreamThreads, kStreamVecs, ALIGNED, true>, grid, kStreamThreads,
                        plan.smem_bytes, static_cast<unsigned>(plan.cluster), stream, p);
    else if (plan.deep)
        rc = launch_pdl(softmax_topk_stream_kernel<T, kStreamThreadsSmall, kStreamDeepVecs, ALIGNED, false, kStreamDeepStages>, grid,
                        kStreamThreadsSmall, plan.smem_bytes, 0u, stream, p);
    else if (plan.threads == kStreamThreadsSmall)
        rc = launch_pdl(softmax_topk_stream_kernel<T, kStreamThreadsSmall, kStreamVecs, ALIGNED, false>, grid,
                        kStreamThreadsSmall, plan.smem_bytes, 0u, stream, p);
    else
        rc = launch_pdl(softmax_topk_stream_kernel<T, kStreamThreads, kStreamVecs, ALIGNED, false>, grid, kStreamThreads,
                        plan.smem_bytes, 0u, stream, p);
    if (rc != VKOP_OK)
        return rc;
    note_launch(1);
    return check_launch();
}

int launch_stream(const vkop_softmax_topk_desc &d, const StreamPlan &plan, const void *logits, void *out_values,
                  void *out_indices, void *packets_out, void *common_ws, void *workspace, int need_sum, cudaStream_t stream) {
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
    p.arrive_word = reinterpret_cast<unsigned int *>(common_ws);
    p.epoch_word = reinterpret_cast<unsigned int *>(static_cast<char *>(common_ws) + 4);
    p.row_done = reinterpret_cast<unsigned int *>(static_cast<char *>(common_ws) + 256);
    p.row_ticket = p.row_done + ((static_cast<size_t>(d.rows) + 63) / 64) * 64;
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

