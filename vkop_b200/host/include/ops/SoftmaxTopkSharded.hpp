// Fused Softmax + TopK over logits whose columns (the vocabulary) are split
// over the GPUs of one node, one rank per GPU: the native owner of what a
// vocabulary-sharded step needs -- the per-rank scratch, the receive buffer
// that the other ranks store into over NVLink, its CUDA IPC handle, the mapping
// of the peers' buffers, the step numbers, and the chain of launches
//   partial (this rank's columns -> one packet per row)
//   push    (the packets into every rank's receive buffer, then a flag)
//   wait    (bounded, for the flags of all ranks)      merge (k best of all).
// The reference runs on a single device (benchmark/main.cpp:49-50) and has no
// counterpart; the operator extends its Softmax -> TopK post-processing
// (benchmark/main.cpp:85-101) to a sharded classifier head.
//
// How the ranks find each other is the caller's business (MPI, a process
// group, a file): every rank calls ipc_handle(), the 64-byte handles travel by
// whatever means, every rank calls connect() with all of them in rank order,
// and after a barrier of the caller's the ranks may run.  Ranks that live in
// ONE process (one thread or one loop driving several GPUs) use connect_local()
// with the peers' objects instead: a process cannot open its own IPC handles.
//
// A step is run(), or begin() on every rank followed by finish(): begin()
// enqueues partial + push, finish() wait + merge.  The wait is bounded (about a
// second); timed_out() tells after a synchronisation whether one gave up.
// Receive slots are two steps deep, which needs no back-pressure: a rank
// pushes step n + 2 only after it merged n + 1, which needed the peer's n + 1
// packets, which the peer pushed after it had merged n.
#ifndef VKOP_HOST_OPS_SOFTMAXTOPKSHARDED_HPP_
#define VKOP_HOST_OPS_SOFTMAXTOPKSHARDED_HPP_

#include <cuda_runtime_api.h>

#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "vkop_cuda.h"

namespace vkop {
namespace ops {

class SoftmaxTopkSharded {
  public:
    struct Config {
        int device = 0;
        int rank = 0, world = 1;
        int64_t rows = 0;
        int64_t cols_local = 0;   // columns this rank holds
        int64_t col_offset = 0;   // index of its first column in the whole vocabulary
        int k = 1;
        int dtype = VKOP_F32;           // vkop_dtype of logits and values
        int index_dtype = VKOP_I32;     // vkop_index_dtype of the result
        float inv_temperature = 1.0f;
        uint32_t max_polls = 1u << 20;  // looks of the bounded wait (about a microsecond each)
    };

    explicit SoftmaxTopkSharded(const Config &c) : c_(c) {
        if (c.world < 1 || c.rank < 0 || c.rank >= c.world || c.rows < 1 || c.cols_local < 1 || c.k < 1)
            throw std::invalid_argument("SoftmaxTopkSharded: bad configuration");
        DeviceGuard g(c_.device);
        desc_ = vkop_softmax_topk_desc{};
        desc_.rows = c.rows;
        desc_.cols = c.cols_local;
        desc_.row_stride = c.cols_local;
        desc_.dtype = c.dtype;
        desc_.k = c.k;
        desc_.index_dtype = c.index_dtype;
        desc_.value_kind = VKOP_VALUE_PROBABILITY;
        desc_.inv_temperature = c.inv_temperature;
        desc_.largest = 1;
        desc_.index_offset = c.col_offset;
        packet_bytes_ = vkop_cuda_packet_bytes(c.k);
        packets_bytes_ = static_cast<size_t>(c.rows) * packet_bytes_;
        check(vkop_cuda_softmax_topk_workspace(&desc_, &ws_bytes_), "vkop_cuda_softmax_topk_workspace");
        // one allocation per rank for what the peers write: the receive slots [2][world][rows][packet], then the
        // flags [2][world] (a handle names a whole allocation)
        flag_offset_ = (2 * static_cast<size_t>(c.world) * packets_bytes_ + 255) / 256 * 256;
        recv_bytes_ = flag_offset_ + (2 * static_cast<size_t>(c.world) * 4 + 255) / 256 * 256;
        cuda(cudaMalloc(&recv_, recv_bytes_), "cudaMalloc");
        cuda(cudaMemset(recv_, 0, recv_bytes_), "cudaMemset");
        cuda(cudaMalloc(&packets_, packets_bytes_), "cudaMalloc");
        cuda(cudaMalloc(&ws_, ws_bytes_ ? ws_bytes_ : 16), "cudaMalloc");
        check(vkop_cuda_workspace_init(ws_, ws_bytes_, nullptr), "vkop_cuda_workspace_init");
        const size_t small = 256 + 256 + 2 * 8 * static_cast<size_t>(c.world);
        cuda(cudaMalloc(&small_, small), "cudaMalloc");
        cuda(cudaMemset(small_, 0, small), "cudaMemset");
        cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
        connected_ = c.world == 1;
    }
    SoftmaxTopkSharded(const SoftmaxTopkSharded &) = delete;
    SoftmaxTopkSharded &operator=(const SoftmaxTopkSharded &) = delete;

    ~SoftmaxTopkSharded() {
        cudaSetDevice(c_.device);
        cudaDeviceSynchronize();
        for (void *p : opened_)
            cudaIpcCloseMemHandle(p);
        cudaFree(small_);
        cudaFree(ws_);
        cudaFree(packets_);
        cudaFree(recv_);
    }

    // The 64-byte CUDA IPC handle of this rank's receive buffer.
    void ipc_handle(void *out64) const {
        DeviceGuard g(c_.device);
        cudaIpcMemHandle_t h;
        cuda(cudaIpcGetMemHandle(&h, recv_), "cudaIpcGetMemHandle");
        static_assert(sizeof(h) == 64, "CUDA IPC handles are 64 bytes");
        std::memcpy(out64, &h, 64);
    }

    // handles: world x 64 bytes, in rank order (this rank's own entry is not opened).  Every rank opens the
    // peers' handles with ITS OWN device current and lazy peer access: that maps a peer's buffer for this
    // device's kernels.  Synchronise all ranks (the caller's barrier) between connect() and the first step.
    void connect(const void *handles) {
        DeviceGuard g(c_.device);
        std::vector<void *> bases(c_.world, nullptr);
        for (int r = 0; r < c_.world; r++) {
            if (r == c_.rank) {
                bases[r] = recv_;
                continue;
            }
            cudaIpcMemHandle_t h;
            std::memcpy(&h, static_cast<const char *>(handles) + 64 * static_cast<size_t>(r), 64);
            void *p = nullptr;
            cuda(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
            opened_.push_back(p);
            bases[r] = p;
        }
        set_peers(bases);
    }

    // Ranks of one process: peers[r] is rank r's object (this rank's own entry is ignored).
    void connect_local(SoftmaxTopkSharded *const *peers) {
        DeviceGuard g(c_.device);
        std::vector<void *> bases(c_.world, nullptr);
        for (int r = 0; r < c_.world; r++) {
            if (r == c_.rank) {
                bases[r] = recv_;
                continue;
            }
            if (peers[r] == nullptr || peers[r]->c_.world != c_.world || peers[r]->c_.rank != r ||
                peers[r]->packets_bytes_ != packets_bytes_)
                throw std::invalid_argument("SoftmaxTopkSharded: peers do not match");
            if (peers[r]->c_.device != c_.device) {
                int can = 0;
                cuda(cudaDeviceCanAccessPeer(&can, c_.device, peers[r]->c_.device), "cudaDeviceCanAccessPeer");
                if (!can)
                    throw std::runtime_error("SoftmaxTopkSharded: no peer access between the devices");
                const cudaError_t e = cudaDeviceEnablePeerAccess(peers[r]->c_.device, 0);
                if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled)
                    cuda(e, "cudaDeviceEnablePeerAccess");
                cudaGetLastError();
            }
            bases[r] = peers[r]->recv_;
        }
        set_peers(bases);
    }

    // partial + push.  logits_local: [rows, cols_local] on this rank's device.
    void begin(const void *logits_local, cudaStream_t stream) {
        if (!connected_)
            throw std::logic_error("SoftmaxTopkSharded: connect() first");
        check(vkop_cuda_softmax_topk_partial(&desc_, logits_local, packets_, ws_, ws_bytes_, stream), "vkop_cuda_softmax_topk_partial");
        if (c_.world == 1)
            return;
        seq_ = seq_ + 1u == 0u ? 1u : seq_ + 1u;  // (0 is "no step")
        check(vkop_cuda_packets_push(packets_, packets_bytes_, slot_ptrs(), flag_ptrs(), c_.rank, c_.world, seq_, tickets(), stream),
              "vkop_cuda_packets_push");
    }

    // wait + merge.  out_values [rows, k] (logits' type), out_indices [rows, k].
    void finish(void *out_values, void *out_indices, cudaStream_t stream) {
        const void *gathered = packets_;
        if (c_.world > 1) {
            check(vkop_cuda_packets_wait(static_cast<char *>(recv_) + flag_offset_, c_.world, seq_, c_.max_polls, status(), stream),
                  "vkop_cuda_packets_wait");
            gathered = static_cast<char *>(recv_) + (seq_ & 1u) * static_cast<size_t>(c_.world) * packets_bytes_;
        }
        vkop_softmax_topk_desc d = desc_;
        d.index_offset = 0;  // (the packets carry indices into the whole vocabulary already)
        check(vkop_cuda_softmax_topk_merge(&d, gathered, c_.world, out_values, out_indices, stream), "vkop_cuda_softmax_topk_merge");
    }

    void run(const void *logits_local, void *out_values, void *out_indices, cudaStream_t stream) {
        begin(logits_local, stream);
        finish(out_values, out_indices, stream);
    }

    // After a synchronisation: has a bounded wait ever given up?
    bool timed_out() const {
        DeviceGuard g(c_.device);
        int s = 0;
        cuda(cudaMemcpy(&s, small_, sizeof(int), cudaMemcpyDeviceToHost), "cudaMemcpy");
        return s != 0;
    }

    const Config &config() const { return c_; }

  private:
    struct DeviceGuard {
        int prev = 0;
        explicit DeviceGuard(int dev) {
            cudaGetDevice(&prev);
            if (cudaSetDevice(dev) != cudaSuccess)
                throw std::runtime_error("SoftmaxTopkSharded: cudaSetDevice failed");
        }
        ~DeviceGuard() { cudaSetDevice(prev); }
    };
    static void cuda(cudaError_t e, const char *what) {
        if (e != cudaSuccess)
            throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
    }
    static void check(int status, const char *what) {
        if (status == VKOP_INVALID_ARG || status == VKOP_UNSUPPORTED)
            throw std::invalid_argument(std::string(what) + ": " + vkop_cuda_status_string(status));
        if (status != VKOP_OK)
            throw std::runtime_error(std::string(what) + ": " + vkop_cuda_status_string(status));
    }
    // small_: status word | tickets [world] at 256 | slot pointers [world] at 512 | flag pointers [world]
    int32_t *status() const { return static_cast<int32_t *>(small_); }
    void *tickets() const { return static_cast<char *>(small_) + 256; }
    void *const *slot_ptrs() const { return reinterpret_cast<void *const *>(static_cast<char *>(small_) + 512); }
    void *const *flag_ptrs() const {
        return reinterpret_cast<void *const *>(static_cast<char *>(small_) + 512 + 8 * static_cast<size_t>(c_.world));
    }
    void set_peers(const std::vector<void *> &bases) {
        std::vector<void *> ptrs(2 * static_cast<size_t>(c_.world));
        for (int r = 0; r < c_.world; r++) {
            ptrs[r] = bases[r];
            ptrs[c_.world + r] = static_cast<char *>(bases[r]) + flag_offset_;
        }
        cuda(cudaMemcpy(static_cast<char *>(small_) + 512, ptrs.data(), ptrs.size() * sizeof(void *), cudaMemcpyHostToDevice), "cudaMemcpy");
        connected_ = true;
    }

    Config c_;
    vkop_softmax_topk_desc desc_;
    size_t packet_bytes_ = 0, packets_bytes_ = 0, ws_bytes_ = 0, flag_offset_ = 0, recv_bytes_ = 0;
    void *recv_ = nullptr, *packets_ = nullptr, *ws_ = nullptr, *small_ = nullptr;
    std::vector<void *> opened_;
    uint32_t seq_ = 0;
    bool connected_ = false;
};

}  // namespace ops
}  // namespace vkop
#endif  // VKOP_HOST_OPS_SOFTMAXTOPKSHARDED_HPP_
