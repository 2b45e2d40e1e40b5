// Unfused Softmax with the full probability tensor as output, along the middle
// axis of a row-major [outer, axis_len, inner] view.
//
//  inner == 1: one CTA per row.  Each thread keeps a running (max, sum) pair
//  over a strided sweep of the row, the pairs are merged across the CTA, and a
//  second sweep (served from L2 for rows that fit) writes exp(z - max) / sum.
//  inner  > 1: one thread per (outer, inner) position walks the axis; adjacent
//  threads touch adjacent addresses, so every step is a coalesced access.
#include "common.cuh"
#include "launchers.h"

namespace vkop_cuda {

__device__ __forceinline__ void online_update(float &m, float &s, float z) {
    if (z > m) {
        s = s * expf(m - z) + 1.0f;  // m == -inf gives s * 0 + 1
        m = z;
    } else {
        s += expf(z - m);
    }
}

__device__ __forceinline__ void online_merge(float &m, float &s, float m2, float s2) {
    float mm = fmaxf(m, m2);
    float a = (s == 0.0f) ? 0.0f : s * expf(m - mm);
    float b = (s2 == 0.0f) ? 0.0f : s2 * expf(m2 - mm);
    m = mm;
    s = a + b;
}

template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS) softmax_rows_kernel(const T *__restrict__ in, T *__restrict__ out,
                                                              int64_t cols, float inv_t) {
    __shared__ float s_m[THREADS / 32], s_s[THREADS / 32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const T *row = in + static_cast<int64_t>(blockIdx.x) * cols;
    T *orow = out + static_cast<int64_t>(blockIdx.x) * cols;
    float m = -INFINITY, s = 0.0f;
    for (int64_t i = tid; i < cols; i += THREADS) {
        float z = __fmul_rn(Elem<T>::from_storage(row[i]), inv_t);
        if (z == z && z != -INFINITY)
            online_update(m, s, z);
        else if (z != z)
            s = z;  // NaN poisons the row, as in the reference arithmetic
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float m2 = __shfl_xor_sync(kFullMask, m, o), s2 = __shfl_xor_sync(kFullMask, s, o);
        online_merge(m, s, m2, s2);
    }
    if (lane == 0) {
        s_m[warp] = m;
        s_s[warp] = s;
    }
    __syncthreads();
    m = s_m[0];
    s = s_s[0];
#pragma unroll
    for (int w = 1; w < THREADS / 32; w++)
        online_merge(m, s, s_m[w], s_s[w]);
    for (int64_t i = tid; i < cols; i += THREADS)
        orow[i] = Elem<T>::to_storage(softmax_prob(Elem<T>::from_storage(row[i]), inv_t, m, s));
}

template <typename T>
__global__ void softmax_strided_kernel(const T *__restrict__ in, T *__restrict__ out, int64_t outer, int64_t axis_len,
                                       int64_t inner, float inv_t) {
    int64_t g = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (g >= outer * inner)
        return;
    int64_t o = g / inner, in_i = g - o * inner;
    const T *p = in + o * axis_len * inner + in_i;
    T *q = out + o * axis_len * inner + in_i;
    float m = -INFINITY;
    for (int64_t a = 0; a < axis_len; a++)
        m = fmaxf(m, __fmul_rn(Elem<T>::from_storage(p[a * inner]), inv_t));
    float s = 0.0f;
    for (int64_t a = 0; a < axis_len; a++)
        s += expf(__fsub_rn(__fmul_rn(Elem<T>::from_storage(p[a * inner]), inv_t), m));
    for (int64_t a = 0; a < axis_len; a++)
        q[a * inner] = Elem<T>::to_storage(softmax_prob(Elem<T>::from_storage(p[a * inner]), inv_t, m, s));
}

template <typename T>
static int launch_softmax_t(const vkop_softmax_desc &d, const void *input, void *output, cudaStream_t stream) {
    const T *in = reinterpret_cast<const T *>(input);
    T *out = reinterpret_cast<T *>(output);
    if (d.inner == 1) {
        if (d.outer > 0x7FFFFFFFll)
            return VKOP_UNSUPPORTED;
        if (d.axis_len <= 2048)
            softmax_rows_kernel<T, 128><<<static_cast<unsigned>(d.outer), 128, 0, stream>>>(in, out, d.axis_len, d.inv_temperature);
        else
            softmax_rows_kernel<T, 512><<<static_cast<unsigned>(d.outer), 512, 0, stream>>>(in, out, d.axis_len, d.inv_temperature);
    } else {
        const int64_t n = d.outer * d.inner;
        const int64_t blocks = (n + 127) / 128;
        if (blocks > 0x7FFFFFFFll)
            return VKOP_UNSUPPORTED;
        softmax_strided_kernel<T><<<static_cast<unsigned>(blocks), 128, 0, stream>>>(in, out, d.outer, d.axis_len, d.inner,
                                                                                    d.inv_temperature);
    }
    note_launch();
    return check_launch();
}

int launch_softmax(const vkop_softmax_desc &d, const void *input, void *output, cudaStream_t stream) {
    if (d.outer == 0)
        return VKOP_OK;
    switch (d.dtype) {
    case VKOP_F32: return launch_softmax_t<float>(d, input, output, stream);
    case VKOP_F16: return launch_softmax_t<__half>(d, input, output, stream);
    case VKOP_BF16: return launch_softmax_t<__nv_bfloat16>(d, input, output, stream);
    default: return VKOP_INVALID_ARG;
    }
}

}  // namespace vkop_cuda
