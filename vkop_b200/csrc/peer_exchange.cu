// Packet exchange of the vocabulary-sharded path over peer memory (NVLink), without a collective
// library: every GPU stores its per-row packets straight into a receive buffer in each peer's
// memory and then raises a flag there; before it merges, a GPU waits until the flags of all
// ranks show the current step.
//
// Receive buffers are two steps deep (slot = step & 1).  That is enough without any back-pressure:
// a rank pushes step n+2 only after it has merged step n+1, which needed the peer's packets of step
// n+1, which the peer pushed after it had merged step n -- so the slot is free by then.
//
// The wait is a bounded poll: after max_polls looks it gives up, writes VKOP_TIMEOUT to the
// status word and returns, so a missing peer shows as a status, never as a hang.
#include "common.cuh"
#include "launchers.h"

namespace vkop_cuda {

// Stores `words` 32-bit words of this rank's packets into slot [seq & 1][rank] of peer `peer`; the last of
// the `nblocks` blocks that share the copy (ticket counter) raises the flag there.  block: 0 .. nblocks-1.
__device__ __forceinline__ void push_to_peer(const uint32_t *src, uint32_t *const *peer_slots, uint32_t *const *peer_flags, int rank,
                                             int world, int peer, size_t words, uint32_t seq, unsigned int *tickets,
                                             unsigned block, unsigned nblocks) {
    uint32_t *dst = peer_slots[peer] + (static_cast<size_t>(seq & 1u) * world + rank) * words;
    const size_t stride = static_cast<size_t>(nblocks) * blockDim.x;
    if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0) {
        const uint4 *s4 = reinterpret_cast<const uint4 *>(src);
        uint4 *d4 = reinterpret_cast<uint4 *>(dst);
        const size_t n4 = words / 4;
        for (size_t i = static_cast<size_t>(block) * blockDim.x + threadIdx.x; i < n4; i += stride)
            d4[i] = s4[i];
        for (size_t i = n4 * 4 + static_cast<size_t>(block) * blockDim.x + threadIdx.x; i < words; i += stride)
            dst[i] = src[i];
    } else {
        for (size_t i = static_cast<size_t>(block) * blockDim.x + threadIdx.x; i < words; i += stride)
            dst[i] = src[i];
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int t = atomicAdd(&tickets[peer], 1u);
        if (t == nblocks - 1) {  // every block of this peer's copy has stored and fenced
            tickets[peer] = 0;
            __threadfence_system();
            uint32_t *flag = peer_flags[peer] + static_cast<size_t>(seq & 1u) * world + rank;
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(seq) : "memory");
        }
    }
}

// Thread s < world waits (bounded) for the flag of rank s in the local flags to show seq.
__device__ __forceinline__ void wait_for_ranks(const uint32_t *flags, int world, uint32_t seq, uint32_t max_polls, int *status) {
    const int s = threadIdx.x;
    if (s >= world)
        return;
    const uint32_t *flag = flags + static_cast<size_t>(seq & 1u) * world + s;
    for (uint32_t it = 0; it < max_polls; ++it) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if (v == seq)
            return;
        __nanosleep(it < 64 ? 100 : 1000);
    }
    *status = VKOP_TIMEOUT;  // the caller reads it after synchronising; the context stays usable
}

// grid (blocks per peer, world).  words: 32-bit words of this rank's packets.
__global__ void __launch_bounds__(256) packets_push_kernel(const uint32_t *src, uint32_t *const *peer_slots,
                                                          uint32_t *const *peer_flags, int rank, int world, size_t words,
                                                          uint32_t seq, unsigned int *tickets) {
    push_to_peer(src, peer_slots, peer_flags, rank, world, blockIdx.y, words, seq, tickets, blockIdx.x, gridDim.x);
}

// One CTA; thread s waits for the packets of rank s.
__global__ void packets_wait_kernel(const uint32_t *flags, int world, uint32_t seq, uint32_t max_polls, int *status) {
    wait_for_ranks(flags, world, seq, max_polls, status);
}

// All ranks of one exchange step in ONE launch, for a machine with fewer GPUs than ranks: kernels that
// wait for one another must not be separate launches on one GPU (nothing makes them run at the same
// time), so here the ranks are groups of blocks of a single cooperative launch (all blocks resident).
// grid (blocks per peer, world peers, world ranks): block (b, p, r) is block b of rank r's copy to peer p;
// then block (0, 0, r) waits, as rank r, for the flags of all ranks in rank r's buffer -- while the other
// ranks' blocks are still storing and raising theirs: the stores, fences and flags of the real exchange,
// running concurrently.  srcs[r], tickets[r], flags_of[r], status[r]: rank r's packets, tickets, flags, status.
__global__ void __launch_bounds__(256) packets_exchange_all_ranks_kernel(const uint32_t *const *srcs, uint32_t *const *peer_slots,
                                                                        uint32_t *const *peer_flags, int world, size_t words,
                                                                        uint32_t seq, unsigned int *const *tickets,
                                                                        uint32_t max_polls, int *status) {
    const int rank = blockIdx.z;
    push_to_peer(srcs[rank], peer_slots, peer_flags, rank, world, blockIdx.y, words, seq, tickets[rank], blockIdx.x, gridDim.x);
    if (blockIdx.x == 0 && blockIdx.y == 0)
        wait_for_ranks(peer_flags[rank], world, seq, max_polls, status + rank);
}

int launch_packets_push(const void *packets, size_t bytes, void *const *peer_slots, void *const *peer_flags, int rank,
                        int world, uint32_t seq, void *tickets, cudaStream_t stream) {
    if (bytes == 0)
        return VKOP_OK;
    const size_t words = bytes / 4;
    unsigned blocks = static_cast<unsigned>((words / 4 + 255) / 256);
    blocks = blocks < 1 ? 1 : (blocks > 64 ? 64 : blocks);
    packets_push_kernel<<<dim3(blocks, static_cast<unsigned>(world)), 256, 0, stream>>>(
        static_cast<const uint32_t *>(packets), reinterpret_cast<uint32_t *const *>(peer_slots),
        reinterpret_cast<uint32_t *const *>(peer_flags), rank, world, words, seq, static_cast<unsigned int *>(tickets));
    note_launch(1);
    return check_launch();
}

int launch_packets_wait(const void *flags, int world, uint32_t seq, uint32_t max_polls, int *status, cudaStream_t stream) {
    packets_wait_kernel<<<1, 32 * ((world + 31) / 32), 0, stream>>>(static_cast<const uint32_t *>(flags), world, seq, max_polls,
                                                                   status);
    note_launch(1);
    return check_launch();
}

int launch_packets_exchange_all_ranks(const void *const *srcs, size_t bytes, void *const *peer_slots, void *const *peer_flags,
                                      int world, uint32_t seq, void *const *tickets, uint32_t max_polls, int *status,
                                      cudaStream_t stream) {
    if (bytes == 0)
        return VKOP_OK;
    size_t words = bytes / 4;
    unsigned blocks = static_cast<unsigned>((words / 4 + 255) / 256);
    blocks = blocks < 1 ? 1 : (blocks > 4 ? 4 : blocks);
    // every block must be resident at once (the waiting blocks wait for the storing ones): a cooperative launch
    // checks that and fails cleanly otherwise
    int dev = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, packets_exchange_all_ranks_kernel, 256, 0) != cudaSuccess)
        return VKOP_CUDA_ERROR;
    if (static_cast<long long>(blocks) * world * world > static_cast<long long>(sms) * per_sm)
        return VKOP_UNSUPPORTED;
    const uint32_t *const *a0 = reinterpret_cast<const uint32_t *const *>(srcs);
    uint32_t *const *a1 = reinterpret_cast<uint32_t *const *>(peer_slots);
    uint32_t *const *a2 = reinterpret_cast<uint32_t *const *>(peer_flags);
    unsigned int *const *a6 = reinterpret_cast<unsigned int *const *>(tickets);
    void *args[] = {&a0, &a1, &a2, &world, &words, &seq, &a6, &max_polls, &status};
    if (cudaLaunchCooperativeKernel(reinterpret_cast<void *>(packets_exchange_all_ranks_kernel),
                                    dim3(blocks, static_cast<unsigned>(world), static_cast<unsigned>(world)), dim3(256), args, 0,
                                    stream) != cudaSuccess)
        return VKOP_CUDA_ERROR;
    note_launch(1);
    return check_launch();
}

}  // namespace vkop_cuda
