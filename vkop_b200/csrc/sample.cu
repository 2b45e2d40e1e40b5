// Sampling tail over the k survivors of a fused Softmax + TopK call: nucleus (top-p) cut and one
// draw per row by inverse CDF from a caller-supplied uniform number.  The data is tiny ([rows, k]),
// so one thread walks one row, sequentially in fp32 -- the order the CPU restatement uses, which
// makes the choice reproducible bit for bit.
#include "common.cuh"
#include "launchers.h"

namespace vkop_cuda {

template <typename T>
__global__ void sample_topk_kernel(const T *values, const void *indices, int index_dtype, int64_t rows, int k, float top_p,
                                   const float *u, int32_t *out_choice, void *out_token) {
    const int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (r >= rows)
        return;
    const T *v = values + r * k;
    float total = 0.0f;
    for (int j = 0; j < k; j++)
        total = __fadd_rn(total, Elem<T>::from_storage(v[j]));
    int n = k;
    if (top_p < 1.0f) {
        const float want = __fmul_rn(top_p, total);
        float acc = 0.0f;
        for (int j = 0; j < k; j++) {
            acc = __fadd_rn(acc, Elem<T>::from_storage(v[j]));
            if (acc >= want) {
                n = j + 1;
                break;
            }
        }
    }
    float mass = 0.0f;
    for (int j = 0; j < n; j++)
        mass = __fadd_rn(mass, Elem<T>::from_storage(v[j]));
    const float target = __fmul_rn(u[r], mass);
    int pick = n - 1;
    float acc = 0.0f;
    for (int j = 0; j < n; j++) {
        acc = __fadd_rn(acc, Elem<T>::from_storage(v[j]));
        if (acc > target) {
            pick = j;
            break;
        }
    }
    out_choice[r] = pick;
    if (index_dtype == VKOP_I64)
        static_cast<int64_t *>(out_token)[r] = static_cast<const int64_t *>(indices)[r * k + pick];
    else
        static_cast<int32_t *>(out_token)[r] = static_cast<const int32_t *>(indices)[r * k + pick];
}

int launch_sample_topk(const void *values, int dtype, const void *indices, int index_dtype, int64_t rows, int k, float top_p,
                       const float *u, int32_t *out_choice, void *out_token, cudaStream_t stream) {
    if (rows == 0)
        return VKOP_OK;
    const unsigned block = 128, grid = static_cast<unsigned>((rows + block - 1) / block);
    switch (dtype) {
    case VKOP_F32:
        sample_topk_kernel<float><<<grid, block, 0, stream>>>(static_cast<const float *>(values), indices, index_dtype, rows, k,
                                                              top_p, u, out_choice, out_token);
        break;
    case VKOP_F16:
        sample_topk_kernel<__half><<<grid, block, 0, stream>>>(static_cast<const __half *>(values), indices, index_dtype, rows,
                                                               k, top_p, u, out_choice, out_token);
        break;
    case VKOP_BF16:
        sample_topk_kernel<__nv_bfloat16><<<grid, block, 0, stream>>>(static_cast<const __nv_bfloat16 *>(values), indices,
                                                                      index_dtype, rows, k, top_p, u, out_choice, out_token);
        break;
    default:
        return VKOP_INVALID_ARG;
    }
    note_launch(1);
    return check_launch();
}

}  // namespace vkop_cuda
