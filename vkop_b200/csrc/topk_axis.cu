// TopK along any axis of a row-major [outer, axis_len, inner] view, and the "sorted = 0" output order.
//
// The selection kernels of this library work on rows whose elements are consecutive.  For an inner extent
// above 1 the tensor is first turned so that the selected axis is the last one (a tiled transpose through
// shared memory, both sides coalesced), the rows are selected as usual into a [outer * inner, k] scratch, and
// a last kernel puts the results where the output layout [outer, k, inner] wants them.  That last kernel also
// produces the unsorted order: the k results of a row by ascending index (ONNX leaves the order open when
// sorted = 0; ascending index is the order the CPU oracle fixes).
#include "common.cuh"
#include "launchers.h"

namespace vkop_cuda {

constexpr int kTile = 32;

// in: [outer][A][I]  ->  out: [outer][I][A]; one CTA of 32 x 8 threads per 32 x 32 tile.
template <typename T>
__global__ void __launch_bounds__(256) transpose_axis_kernel(const T *__restrict__ in, T *__restrict__ out, int64_t A, int64_t I,
                                                             int64_t tiles_a, int64_t tiles_i, int64_t tiles) {
    __shared__ T tile[kTile][kTile + 1];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int64_t t = blockIdx.x; t < tiles; t += gridDim.x) {
        const int64_t o = t / (tiles_a * tiles_i);
        const int64_t r = t - o * tiles_a * tiles_i;
        const int64_t ta = r / tiles_i, ti = r - ta * tiles_i;
        const T *src = in + o * A * I;
        T *dst = out + o * A * I;
        const int64_t a0 = ta * kTile, i0 = ti * kTile;
#pragma unroll
        for (int y = ty; y < kTile; y += 8)
            if (a0 + y < A && i0 + tx < I)
                tile[y][tx] = src[(a0 + y) * I + i0 + tx];
        __syncthreads();
#pragma unroll
        for (int y = ty; y < kTile; y += 8)
            if (i0 + y < I && a0 + tx < A)
                dst[(i0 + y) * A + a0 + tx] = tile[tx][y];
        __syncthreads();
    }
}

// One CTA per selected row r = o * inner + i: its k (value, index) results go to out[(o * k + j) * inner + i];
// with by_index they are first put in ascending index order (bitonic sort of (index << 32 | rank) in shared memory).
template <typename T, typename IDX>
__global__ void __launch_bounds__(128) place_results_kernel(const T *__restrict__ vals, const int32_t *__restrict__ idx,
                                                            T *__restrict__ out_vals, IDX *__restrict__ out_idx, int k, int kpow2,
                                                            int64_t inner, int by_index) {
    extern __shared__ __align__(16) unsigned char s_raw[];
    uint64_t *s = reinterpret_cast<uint64_t *>(s_raw);
    const int64_t r = blockIdx.x;
    const int64_t o = r / inner, i = r - o * inner;
    const T *v = vals + r * k;
    const int32_t *x = idx + r * k;
    T *ov = out_vals + o * k * inner + i;
    IDX *oi = out_idx + o * k * inner + i;
    if (!by_index) {
        for (int j = threadIdx.x; j < k; j += blockDim.x) {
            ov[static_cast<int64_t>(j) * inner] = v[j];
            oi[static_cast<int64_t>(j) * inner] = static_cast<IDX>(x[j]);
        }
        return;
    }
    for (int j = threadIdx.x; j < kpow2; j += blockDim.x)
        s[j] = j < k ? (static_cast<uint64_t>(static_cast<uint32_t>(x[j])) << 32) | static_cast<uint32_t>(j) : ~0ull;
    __syncthreads();
    for (int size = 2; size <= kpow2; size <<= 1)
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int t = threadIdx.x; t < kpow2 / 2; t += blockDim.x) {
                const int lo = 2 * t - (t & (stride - 1)), hi = lo + stride;
                const bool asc = (lo & size) == 0;
                const uint64_t a = s[lo], c = s[hi];
                if (asc ? (a > c) : (a < c)) {
                    s[lo] = c;
                    s[hi] = a;
                }
            }
            __syncthreads();
        }
    for (int j = threadIdx.x; j < k; j += blockDim.x) {
        const uint64_t e = s[j];
        ov[static_cast<int64_t>(j) * inner] = v[static_cast<uint32_t>(e)];
        oi[static_cast<int64_t>(j) * inner] = static_cast<IDX>(static_cast<int32_t>(e >> 32));
    }
}

size_t topk_axis_transposed_bytes(const vkop_topk_axis_desc &d) {
    if (d.inner <= 1)
        return 0;
    const size_t esize = d.dtype == VKOP_F32 ? 4 : 2;
    return (static_cast<size_t>(d.outer) * d.axis_len * d.inner * esize + 255) / 256 * 256;
}

size_t topk_axis_values_bytes(const vkop_topk_axis_desc &d) {
    const size_t esize = d.dtype == VKOP_F32 ? 4 : 2;
    return (static_cast<size_t>(d.outer) * d.inner * d.k * esize + 255) / 256 * 256;
}

size_t topk_axis_indices_bytes(const vkop_topk_axis_desc &d) {
    return (static_cast<size_t>(d.outer) * d.inner * d.k * 4 + 255) / 256 * 256;
}

template <typename T>
static int transpose_typed(const vkop_topk_axis_desc &d, const void *in, void *out, cudaStream_t stream) {
    const int64_t ta = (d.axis_len + kTile - 1) / kTile, ti = (d.inner + kTile - 1) / kTile;
    const int64_t tiles = d.outer * ta * ti;
    const int64_t grid = tiles < (1 << 20) ? tiles : (1 << 20);
    transpose_axis_kernel<T><<<static_cast<unsigned>(grid), 256, 0, stream>>>(reinterpret_cast<const T *>(in),
                                                                              reinterpret_cast<T *>(out), d.axis_len, d.inner, ta,
                                                                              ti, tiles);
    note_launch();
    return check_launch();
}

int launch_transpose_axis(const vkop_topk_axis_desc &d, const void *in, void *out, cudaStream_t stream) {
    if (d.outer == 0 || d.axis_len == 0 || d.inner == 0)
        return VKOP_OK;
    return d.dtype == VKOP_F32 ? transpose_typed<uint32_t>(d, in, out, stream) : transpose_typed<uint16_t>(d, in, out, stream);
}

template <typename T, typename IDX>
static int place_typed(const vkop_topk_axis_desc &d, const void *vals, const void *idx, void *ov, void *oi, cudaStream_t stream) {
    int kpow2 = 1;
    while (kpow2 < d.k)
        kpow2 <<= 1;
    const int by_index = d.sorted ? 0 : 1;
    const size_t smem = by_index ? static_cast<size_t>(kpow2) * 8 : 0;
    int threads = kpow2 / 2;
    threads = threads < 32 ? 32 : (threads > 128 ? 128 : threads);
    const int64_t rows = d.outer * d.inner;
    if (rows > 0x7FFFFFFFll)
        return VKOP_UNSUPPORTED;
    place_results_kernel<T, IDX><<<static_cast<unsigned>(rows), threads, smem, stream>>>(
        reinterpret_cast<const T *>(vals), reinterpret_cast<const int32_t *>(idx), reinterpret_cast<T *>(ov),
        reinterpret_cast<IDX *>(oi), d.k, kpow2, d.inner, by_index);
    note_launch();
    return check_launch();
}

int launch_place_results(const vkop_topk_axis_desc &d, const void *vals, const void *idx, void *out_values, void *out_indices,
                         cudaStream_t stream) {
    if (d.outer == 0 || d.inner == 0)
        return VKOP_OK;
    const bool wide = d.index_dtype == VKOP_I64;
    if (d.dtype == VKOP_F32)
        return wide ? place_typed<uint32_t, int64_t>(d, vals, idx, out_values, out_indices, stream)
                    : place_typed<uint32_t, int32_t>(d, vals, idx, out_values, out_indices, stream);
    return wide ? place_typed<uint16_t, int64_t>(d, vals, idx, out_values, out_indices, stream)
                : place_typed<uint16_t, int32_t>(d, vals, idx, out_values, out_indices, stream);
}

}  // namespace vkop_cuda
