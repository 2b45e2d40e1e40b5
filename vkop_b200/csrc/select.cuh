// Device code shared by the fused Softmax + TopK kernels: parameters, the
// emission of a ranked survivor, the exact selection among candidates held in
// shared memory, the radix-select fallback over a range of a row, and the
// per-row merge of published candidate lists.
#pragma once

#include <cooperative_groups.h>
#include <type_traits>

#include "common.cuh"

namespace vkop_cuda {

constexpr unsigned long long kWaitLimitNs = 1000000000ull;  // every poll loop gives up after about a second

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Waits (bounded, about a second) until a row's counter of finished calls satisfies the test:
// exact: it shows `want`; otherwise: it has reached `want`.  The calls it waits for were launched
// before this one, have all their CTAs running (a call is let in only after every CTA of its
// predecessor has started) and never wait for a later call.  Called by one thread.
static __device__ __noinline__ bool wait_row_counter(const unsigned int *row_done, uint32_t want, bool exact,
                                                     uint32_t mask = 0xFFFFFFFFu) {
    const unsigned long long t0 = global_ns();
    want &= mask;
    for (;;) {
        for (int i = 0; i < 64; i++) {
            unsigned int dn;
            asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(dn) : "l"(row_done) : "memory");
            dn &= mask;
            if (exact ? dn == want : static_cast<int>(dn - want) >= 0)
                return true;
            __nanosleep(64);
        }
        if (global_ns() - t0 > kWaitLimitNs)
            return false;
    }
}

constexpr int kCandCap = 2048;        // candidate slots of the chunk filter
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
    // streaming kernel only
    int64_t nvv;       // vector slots per row (the same for every row; slots past a row's end are empty)
    int64_t per_cta;   // nominal vector slots per CTA
    int64_t vstride;   // vectors between the starts of consecutive rows (rows 16-byte aligned only)
    int parts_per_row; // > 0: every row is cut into this many CTAs and no CTA crosses a row
    int input_ready;   // the logits were complete before this launch was enqueued
    // calls on one workspace number themselves (streaming kernels): the call counter, the CTAs of the
    // current call that have drawn their arrival ticket, and per row the calls whose result is written
    unsigned int *epoch_word, *arrive_word, *row_done;
    unsigned int *row_ticket;  // per row: calls started on the row (whole rows in overlapping calls number themselves per row)
};


__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Results of one row reach the outputs in call order, and no CTA holds its place on an SM waiting for
// that.  A row has an order word: the number of calls that have finished the row (low 16 bits) and one
// bit per call that has deposited its result (bit 16 + call % 16), and a mailbox of kMailSlots entries
// (entry = the two addresses the result belongs at, then the k values and the k indices exactly as
// they would have been stored).  A CTA that has ranked its row and finds that the previous call has
// not finished the row yet writes its result into entry call % 16, sets its bit and leaves.  A CTA
// that finds it is its turn writes straight to the outputs, then delivers the entries that later calls
// have deposited meanwhile, in call order, and publishes the new count with a compare-and-swap that
// fails whenever a bit has appeared in between (row_order_finish).  A depositor whose bit lands after
// the count already names it delivers its own entry.  Either way the outputs receive the calls'
// results in call order.  Since a deposited result is delivered by a CTA of an earlier kernel, CTA 0 of
// every kernel waits for its predecessor kernel before it ends: a kernel has then completed only when
// every earlier one has.  Without a mailbox (packets as output), or when the entry is still taken,
// the CTA waits for its turn instead (bounded poll of the word, then the whole previous kernel).
constexpr int kMailSlots = 16;
struct OrderWait {
    unsigned int *word;   // the row's order word
    uint32_t epoch;       // number of this call
    int *flag;            // a word of shared memory
    unsigned char *mail;  // the row's mailbox (null: none)
    uint32_t mail_stride, mail_idx_off;  // bytes per entry; offset of the indices in an entry
    bool need;            // the previous call had not finished the row when this CTA last looked
    bool waited;          // in/out: this thread has waited for the whole previous kernel
    bool deposited;       // out: the result belongs in the mailbox entry, not at the outputs
};
__device__ __forceinline__ uint32_t mail_bit(uint32_t call) { return 0x10000u << (call & (kMailSlots - 1)); }

// Called by every thread of the selecting CTA right before its first store.
template <int BAR, int THREADS>
__device__ __forceinline__ void order_hook(OrderWait *ow) {
    if (ow == nullptr || !ow->need || ow->waited)
        return;
    if (threadIdx.x == 0) {
        unsigned int w;
        asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(w) : "l"(ow->word) : "memory");
        int f;
        if (((w ^ ow->epoch) & 0xFFFFu) == 0u)
            f = 1;  // its turn by now
        else if (ow->mail != nullptr && (w & mail_bit(ow->epoch)) == 0u && ((ow->epoch - w) & 0xFFFFu) < kMailSlots)
            f = 2;  // deposit (fewer than kMailSlots calls of the row are unfinished: nobody else has or takes this entry)
        else
            f = wait_row_counter(ow->word, ow->epoch, true, 0xFFFFu) ? 1 : 0;
        *ow->flag = f;
    }
    cta_sync<BAR, THREADS>();
    const int f = *ow->flag;
    if (f == 0) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        ow->waited = true;
    }
    ow->deposited = f == 2;
    ow->need = false;
}

// Where a ranked survivor goes: the final outputs, a packet, or a candidate list.
template <typename T>
__device__ __forceinline__ void emit(const ChunkParams &p, int64_t row, int rank, uint64_t comp, float m, float s,
                                     unsigned long long *list_out, const OrderWait *ow = nullptr) {
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
    // (a result that has to wait for its turn goes to the row's mailbox entry in the same form)
    const bool mailed = ow != nullptr && ow->deposited;
    unsigned char *const entry = mailed ? ow->mail + (ow->epoch & (kMailSlots - 1)) * ow->mail_stride : nullptr;
    void *const ov = mailed ? static_cast<void *>(entry + 16) : p.out_values;
    void *const oi = mailed ? static_cast<void *>(entry + ow->mail_idx_off) : p.out_indices;
    const int64_t o = mailed ? rank : row * p.k + rank;
    if (p.value_kind == VKOP_VALUE_RAW) {
        reinterpret_cast<T *>(ov)[o] = reinterpret_cast<const T *>(p.logits)[row * p.row_stride + idx];
    } else {
        store_value<T>(ov, o, softmax_prob(key_to_float(cand_key(comp)), p.inv_t, m, s));
    }
    store_index(oi, p.index_dtype, o, static_cast<int64_t>(idx) + p.index_offset);
}

// Copies a mailbox entry to the addresses in its header.  Executed by one warp.
template <typename T>
__device__ __forceinline__ void deliver_entry(const unsigned char *entry, uint32_t idx_off, int k, int index_dtype) {
    const int lane = threadIdx.x & 31;
    // (the entry was written by another SM: read it from the L2)
    const unsigned long long h0 = __ldcg(reinterpret_cast<const unsigned long long *>(entry));
    const unsigned long long h1 = __ldcg(reinterpret_cast<const unsigned long long *>(entry + 8));
    using Bits = typename std::conditional<sizeof(T) == 4, unsigned int, unsigned short>::type;
    Bits *const dv = reinterpret_cast<Bits *>(h0);
    void *const di = reinterpret_cast<void *>(h1);
    const Bits *const sv = reinterpret_cast<const Bits *>(entry + 16);
    for (int i = lane; i < k; i += 32) {
        dv[i] = __ldcg(sv + i);
        if (index_dtype == VKOP_I64)
            reinterpret_cast<long long *>(di)[i] = __ldcg(reinterpret_cast<const long long *>(entry + idx_off) + i);
        else
            reinterpret_cast<int *>(di)[i] = __ldcg(reinterpret_cast<const int *>(entry + idx_off) + i);
    }
}

// After the stores of a row's result (all threads, then a CTA barrier): settles the row's order word.
// Executed by warp 0 of the CTA.  See OrderWait.
template <typename T>
__device__ __noinline__ void row_order_finish(const ChunkParams &p, const OrderWait ow, int64_t row) {
    const int lane = threadIdx.x & 31;
    uint32_t cur = ow.epoch, cleared = 0u;
    if (ow.deposited) {
        unsigned char *const entry = ow.mail + (cur & (kMailSlots - 1)) * ow.mail_stride;
        unsigned int old = 0u;
        if (lane == 0) {
            const size_t isz = p.index_dtype == VKOP_I64 ? 8 : 4;
            *reinterpret_cast<void **>(entry) = static_cast<char *>(p.out_values) + row * p.k * sizeof(T);
            *reinterpret_cast<void **>(entry + 8) = static_cast<char *>(p.out_indices) + row * p.k * isz;
            __threadfence();  // the entry (written by the whole CTA before the barrier) before the bit
            asm volatile("atom.acq_rel.gpu.global.or.b32 %0, [%1], %2;" : "=r"(old) : "l"(ow.word), "r"(mail_bit(cur)) : "memory");
        }
        old = __shfl_sync(kFullMask, old, 0);
        if (((old ^ cur) & 0xFFFFu) != 0u)
            return;  // an earlier call of this row delivers it
        // the previous call published its count before the bit was there: this CTA delivers its own entry
        deliver_entry<T>(entry, ow.mail_idx_off, p.k, p.index_dtype);
        cleared = mail_bit(cur);
    }
    // this call's result is in place: deliver what later calls have deposited, in call order, then publish
    for (int it = 0; it < 256; it++) {
        unsigned int w = 0u;
        if (lane == 0)
            asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(w) : "l"(ow.word) : "memory");
        w = __shfl_sync(kFullMask, w, 0);
        const uint32_t nb = mail_bit(cur + 1u);
        if (ow.mail != nullptr && (w & nb) != 0u && (cleared & nb) == 0u) {
            deliver_entry<T>(ow.mail + ((cur + 1u) & (kMailSlots - 1)) * ow.mail_stride, ow.mail_idx_off, p.k, p.index_dtype);
            cleared |= nb;
            cur++;
            continue;
        }
        const uint32_t desired = ((w & 0xFFFF0000u) & ~cleared) | ((cur + 1u) & 0xFFFFu);
        unsigned int seen = 0u;
        __threadfence();  // the deliveries of all lanes before the count
        __syncwarp();
        if (lane == 0)
            asm volatile("atom.acq_rel.gpu.global.cas.b32 %0, [%1], %2, %3;" : "=r"(seen) : "l"(ow.word), "r"(w), "r"(desired) : "memory");
        seen = __shfl_sync(kFullMask, seen, 0);
        if (seen == w)
            return;
    }
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
// survivors are emitted at their rank.  Executed by THREADS threads (the whole
// CTA, or with BAR > 0 the threads 0 .. THREADS-1 that share named barrier
// BAR); list and work are clobbered.  ow (may be null): an order to keep
// between overlapping calls; it is waited for as late as possible, after the
// ranking and right before the first store, so that the stretch a successor
// may have to wait for is the stores alone.
template <typename T, int THREADS, int BAR = 0>
__device__ __noinline__ void select_and_emit(const ChunkParams &p, int64_t row, uint64_t *list, int n, uint64_t *work, float M,
                                float S, unsigned long long *list_out, int *s_tmp, OrderWait *ow = nullptr) {
    constexpr int NW = THREADS / 32;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int k = p.k;
    // ---- short lists (the usual case behind a tight threshold): the rank of a candidate is the number
    // of candidates that beat it; PER threads share the count of one candidate.  No sort, no barrier. ----
    constexpr int kSmall = 128;
    if (n <= kSmall) {
        constexpr int PER = THREADS / kSmall >= 1 ? THREADS / kSmall : 1;
        static_assert(PER <= 32 && (PER & (PER - 1)) == 0, "a power of two within a warp");
        if constexpr (THREADS / PER >= kSmall) {
            // every candidate has its threads: count first, wait for the order, then store
            const int c = tid / PER, sub = tid % PER;
            const uint64_t me = c < n ? list[c] : ~0ull;
            int beat = 0;
            for (int i = sub; i < n; i += PER)
                beat += list[i] > me ? 1 : 0;
#pragma unroll
            for (int o = 1; o < PER; o <<= 1)
                beat += __shfl_xor_sync(kFullMask, beat, o);
            order_hook<BAR, THREADS>(ow);
            if (c < n && sub == 0 && beat < k)
                emit<T>(p, row, beat, me, M, S, list_out, ow);
            return;
        }
        order_hook<BAR, THREADS>(ow);
        for (int c0 = 0; c0 < kSmall; c0 += THREADS / PER) {
            const int c = c0 + tid / PER, sub = tid % PER;
            const uint64_t me = c < n ? list[c] : ~0ull;
            int beat = 0;
            for (int i = sub; i < n; i += PER)
                beat += list[i] > me ? 1 : 0;
#pragma unroll
            for (int o = 1; o < PER; o <<= 1)
                beat += __shfl_xor_sync(kFullMask, beat, o);
            if (c < n && sub == 0 && beat < k)
                emit<T>(p, row, beat, me, M, S, list_out, ow);
        }
        return;
    }
    // ---- narrow: r-th largest key of every full group of 32, minimised over the groups; the survivors
    // are regrouped and narrowed again while that still removes a good share of them ----
    uint64_t *src = list;
    int n2 = n;
    for (int round = 0; round < 4; round++) {
        const int nfull = n2 / 32;
        const int r = nfull > 0 ? (k + nfull - 1) / nfull : 99;
        if (!(n2 > 2 * k + 32 && r <= 8))
            break;
        if (tid == 0) {
            s_tmp[0] = 0x7FFFFFFF;  // threshold key >> 1 (kept positive for atomicMin on int)
            s_tmp[1] = 0;
        }
        cta_sync<BAR, THREADS>();
        for (int g = warp; g < nfull; g += NW) {
            uint32_t cur = cand_key(src[g * 32 + lane]);
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
        cta_sync<BAR, THREADS>();
        const uint32_t tkey = static_cast<uint32_t>(s_tmp[0]) << 1;  // rounded down: keeps the bound valid
        for (int i = tid; i < n2; i += THREADS) {
            const uint64_t c = src[i];
            if (cand_key(c) >= tkey) {
                const int pos = atomicAdd(&s_tmp[1], 1);
                work[pos] = c;
            }
        }
        cta_sync<BAR, THREADS>();
        const int n3 = s_tmp[1];
        uint64_t *t = src;
        src = work;
        work = t;
        const bool progress = n3 * 4 <= n2 * 3;
        n2 = n3;
        cta_sync<BAR, THREADS>();  // s_tmp is reused by the next round
        if (!progress)
            break;
    }
    // ---- sort groups of 32, then rank every survivor against the other groups ----
    const int ng = (n2 + 31) / 32;
    for (int g = warp; g < ng; g += NW) {
        const int i = g * 32 + lane;
        uint64_t v = i < n2 ? src[i] : 0ull;
        v = warp_sort_desc(v, lane);
        work[i] = v;
    }
    cta_sync<BAR, THREADS>();
    order_hook<BAR, THREADS>(ow);
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
                emit<T>(p, row, rank, me, M, S, list_out, ow);
        }
    }
}

// Exact selection of the kk best (key, ~index) values of a chunk by an 8-bit
// most-significant-digit radix select over the 64-bit candidate value.  The
// chunk is re-read from memory.  Leaves exactly kk candidates in s_cand.
template <typename T, int THREADS, int BAR = 0>
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
        cta_sync<BAR, THREADS>();
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
                    uint64_t c = make_cand(order_key_sel(f[e], negate), static_cast<uint32_t>(i));
                    if ((c & mask) == prefix)
                        atomicAdd(&s_hist[static_cast<int>(c >> shift) & 255], 1);
                }
            }
        }
        cta_sync<BAR, THREADS>();
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
        cta_sync<BAR, THREADS>();
        prefix |= static_cast<uint64_t>(s_pick[0]) << shift;
        mask |= 0xFFull << shift;
        need = s_pick[1];
        if (s_pick[2] == need)
            break;  // the whole bin is taken: threshold = prefix
    }
    if (tid == 0)
        *s_count = 0;
    cta_sync<BAR, THREADS>();
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
                uint64_t c = make_cand(order_key_sel(f[e], negate), static_cast<uint32_t>(i));
                if (c >= prefix) {
                    int pos = atomicAdd(s_count, 1);
                    if (pos < kCandCap)
                        s_cand[pos] = c;
                }
            }
        }
    }
    cta_sync<BAR, THREADS>();
}

// Gathers the candidate lists of the G parts of one row into shared memory,
// merges their statistics and selects.  Executed by one whole CTA.
// lists: G blocks of `stride` 64-bit words: header word 0 = (m, s) as float
// bits; header word 1 = count in bits 0-15, then 32 bits of threshold key (at
// least k of the part's candidates reach it; 0 = none) and 16 bits the
// streaming kernel keeps for its slot state; then the candidates.
// s_buf holds the gathered candidates; s_sel is the scratch of the selection
// (as many slots again), or null to take it right behind the candidates.
// PEERS: the lists are not in global memory: list g sits at `lists` in the
// shared memory of CTA g of this thread-block cluster (at most 32 lists of at
// most 512 candidates).
template <typename T, int THREADS, bool PEERS = false, int BAR = 0>
__device__ __noinline__ void merge_lists(const ChunkParams &p, int64_t row, const unsigned long long *lists, int64_t stride, int G,
                            uint64_t *s_buf, uint64_t *s_sel, float *s_red, int *s_int, int *s_tmp) {
    constexpr int NW = THREADS / 32;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float M, S;
    int n;
    if (PEERS || (G <= NW && p.list_cap <= 512)) {
        // Few, short lists: warp g takes list g and fetches its header and its whole capacity in one
        // round trip (entries past the count are ignored).  One barrier later every warp knows all
        // headers: the largest of the parts' thresholds bounds the row's k-th best from below (that
        // part alone holds k candidates at or above it), so only candidates that reach it are kept.
        const int g = warp;
        unsigned long long regs[16];
        int cnt = 0;
        if (g < G) {
            unsigned long long h0, h1;
            if (PEERS) {
                const unsigned long long *L = cooperative_groups::this_cluster().map_shared_rank(lists, g);
                // header and the whole capacity in one round trip (entries past the count are ignored)
                h0 = L[0];
                h1 = L[1];
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const int i = lane + 32 * j;
                    regs[j] = i < p.list_cap ? L[2 + i] : 0ull;
                }
                cnt = static_cast<int>(h1 & 0xFFFFu);
            } else {
                const unsigned long long *L = lists + g * stride;
                h0 = __ldcg(L);
                h1 = __ldcg(L + 1);
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const int i = lane + 32 * j;
                    regs[j] = i < p.list_cap ? __ldcg(L + 2 + i) : 0ull;
                }
                cnt = static_cast<int>(h1 & 0xFFFFu);
            }
            if (lane == 0) {
                s_int[8 + g] = static_cast<int>(static_cast<uint32_t>(h1 >> 16));       // threshold key of the part
                s_int[8 + NW + g] = static_cast<int>(static_cast<uint32_t>(h0));         // max z bits
                s_int[8 + 2 * NW + g] = static_cast<int>(static_cast<uint32_t>(h0 >> 32));  // sum bits
            }
        }
        if (tid == 0)
            s_tmp[0] = 0;
        cta_sync<BAR, THREADS>();
        uint32_t trow = 0;
        M = -INFINITY;
        for (int q = 0; q < G; q++) {
            const uint32_t tq = static_cast<uint32_t>(s_int[8 + q]);
            trow = tq > trow ? tq : trow;
            M = fmaxf(M, __int_as_float(s_int[8 + NW + q]));
        }
        S = 0.0f;
        for (int q = 0; q < G; q++) {
            const float sg = __int_as_float(s_int[8 + 2 * NW + q]);
            if (sg != 0.0f)  // an all -inf part has sum 0 and no defined maximum
                S += sg * expf(__int_as_float(s_int[8 + NW + q]) - M);
        }
        if (g < G) {
#pragma unroll
            for (int j = 0; j < 16; j++) {
                const int i = lane + 32 * j;
                const bool pass = i < cnt && cand_key(regs[j]) >= trow;
                const unsigned b = __ballot_sync(kFullMask, pass);
                if (b != 0u) {
                    int base = 0;
                    if (lane == 0)
                        base = atomicAdd(&s_tmp[0], __popc(b));
                    base = __shfl_sync(kFullMask, base, 0);
                    if (pass)
                        s_buf[base + __popc(b & ((1u << lane) - 1u))] = regs[j];
                }
            }
        }
        cta_sync<BAR, THREADS>();
        n = s_tmp[0];
        cta_sync<BAR, THREADS>();  // s_tmp is reused by the selection
    } else {
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
                    cnt = static_cast<int>(__ldcg(lists + g * stride + 1) & 0xFFFFu);
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
        cta_sync<BAR, THREADS>();
        M = s_red[0];
        S = s_red[1];
        n = s_int[0];
        // gather: warp per list
        for (int g = warp; g < G; g += NW) {
            const int off = s_int[8 + g];
            const int end = (g + 1 < G) ? s_int[8 + g + 1] : n;
            const unsigned long long *src = lists + g * stride + 2;
            for (int i = lane; i < end - off; i += 32)
                s_buf[off + i] = __ldcg(src + i);
        }
        cta_sync<BAR, THREADS>();
    }
    const int nsel = n < p.k ? n : p.k;
    if (p.packets_out && tid == 0) {
        uint32_t *pk = p.packets_out + row * packet_words(p.k);
        pk[0] = __float_as_uint(M);
        pk[1] = __float_as_uint(S);
        pk[2] = static_cast<uint32_t>(nsel);
        pk[3] = 0;
    }
    select_and_emit<T, THREADS, BAR>(p, row, s_buf, n, s_sel ? s_sel : s_buf + ((n + 31) & ~31), M, S, nullptr, s_tmp);
}

}  // namespace vkop_cuda
