#include "common.cuh"
#include "launchers.h"
namespace vkop_cuda {
int plan_radix(const vkop_softmax_topk_desc &, RadixPlan *) { return VKOP_UNSUPPORTED; }
int launch_radix(const vkop_softmax_topk_desc &, const RadixPlan &, const void *, void *, void *, void *, void *, int,
                 cudaStream_t) { return VKOP_UNSUPPORTED; }
}
