#include "common.cuh"
#include "launchers.h"
namespace vkop_cuda {
int plan_nms(const vkop_nms_desc &, size_t *) { return VKOP_UNSUPPORTED; }
int launch_nms(const vkop_nms_desc &, const void *, const void *, int32_t *, int32_t *, void *, cudaStream_t) { return VKOP_UNSUPPORTED; }
}
