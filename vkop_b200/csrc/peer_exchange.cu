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

// grid (blocks per peer, world).  words: 32-bit words of this rank's packets.
__global__ void __launch_bounds__(256) packets_push_kernel(const uint32_t *src, uint32_t *const *peer_slots,
                                                          uint32_t *const *peer_flags, int rank, int world, size_t words,
                                                          uint32_t seq, unsigned int *tickets) {
    const int peer = blockIdx.y;
    uint32_t *dst = peer_slots[peer] + (static_cast<size_t>(seq & 1u) * world + rank) * words;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0) {
        const uint4 *s4 = reinterpret_cast<const uint4 *>(src);
        uint4 *d4 = reinterpret_cast<uint4 *>(dst);
        const size_t n4 = words / 4;
        for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride)
            d4[i] = s4[i];
        for (size_t i = n4 * 4 + static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < words; i += stride)
            dst[i] = src[i];
    } else {
        for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < words; i += stride)
            dst[i] = src[i];
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int t = atomicAdd(&tickets[peer], 1u);
        if (t == gridDim.x - 1) {  // every block of this peer's copy has stored and fenced
            tickets[peer] = 0;
            __threadfence_system();
            uint32_t *flag = peer_flags[peer] + static_cast<size_t>(seq & 1u) * world + rank;
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(seq) : "memory");
        }
    }
}

// One CTA; thread s waits for the packets of rank s.
__global__ void packets_wait_kernel(const uint32_t *flags, int world, uint32_t seq, uint32_t max_polls, int *status) {
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

}  // namespace vkop_cuda
