// Shared device helpers: order-preserving keys, 16-byte vector unpacking,
// packet layout, launch accounting.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "vkop_cuda.h"

namespace vkop_cuda {

constexpr float kLog2e = 1.4426950408889634f;
constexpr unsigned kFullMask = 0xFFFFFFFFu;

// Counts kernel launches issued by this library (read by vkop_cuda_launch_count).
void note_launch(int n = 1);

inline int check_launch() { return cudaGetLastError() == cudaSuccess ? VKOP_OK : VKOP_CUDA_ERROR; }

// Barrier over the whole CTA (BAR == 0) or over the N threads that share named barrier BAR.
template <int BAR, int N>
__device__ __forceinline__ void cta_sync() {
    if constexpr (BAR == 0)
        __syncthreads();
    else
        asm volatile("bar.sync %0, %1;" ::"n"(BAR), "n"(N) : "memory");
}

// float -> uint32 such that a > b <=> key(a) > key(b); -0 maps with +0, every
// NaN maps to the largest key.  No valid value maps to key 0.
__device__ __forceinline__ uint32_t order_key(float x) {
    uint32_t u = __float_as_uint(x + 0.0f);
    uint32_t k = u ^ (static_cast<uint32_t>(static_cast<int32_t>(u) >> 31) | 0x80000000u);
    return (x != x) ? 0xFFFFFFFFu : k;
}

// Key of an element AFTER the sign flip that turns "smallest" into "largest" (flipped != 0): the
// flip leaves a NaN a NaN, which must then rank last, not first (NaN is the largest value whichever
// way the selection goes): key 1 lies below the key of -inf, and no number maps to it.
__device__ __forceinline__ uint32_t order_key_sel(float x, int flipped) {
    return (flipped && x != x) ? 1u : order_key(x);
}

__device__ __forceinline__ float key_to_float(uint32_t k) {
    uint32_t u = (k & 0x80000000u) ? (k ^ 0x80000000u) : ~k;
    return __uint_as_float(u);
}

// Candidate = (key, index) packed so that a larger 64-bit value ranks first:
// key descending, then index ascending.
__device__ __forceinline__ uint64_t make_cand(uint32_t key, uint32_t idx) {
    return (static_cast<uint64_t>(key) << 32) | static_cast<uint32_t>(~idx);
}
__device__ __forceinline__ uint32_t cand_key(uint64_t c) { return static_cast<uint32_t>(c >> 32); }
__device__ __forceinline__ uint32_t cand_idx(uint64_t c) { return ~static_cast<uint32_t>(c); }

// ---- element types: 16-byte vectors -------------------------------------
template <typename T>
struct Elem;

template <>
struct Elem<float> {
    static constexpr int kPerVec = 4;
    static constexpr uint32_t kNegInfWord = 0xFF800000u;
    __device__ static __forceinline__ void unpack(const uint4 &v, float (&f)[4]) {
        f[0] = __uint_as_float(v.x);
        f[1] = __uint_as_float(v.y);
        f[2] = __uint_as_float(v.z);
        f[3] = __uint_as_float(v.w);
    }
    // largest element of the vector (NaN elements are passed over, as fmaxf does)
    __device__ static __forceinline__ float vector_max(const uint4 &v) {
        return fmaxf(fmaxf(__uint_as_float(v.x), __uint_as_float(v.y)), fmaxf(__uint_as_float(v.z), __uint_as_float(v.w)));
    }
    __device__ static __forceinline__ bool vector_has_nan(const uint4 &v) {
        const float a = __uint_as_float(v.x), b = __uint_as_float(v.y), c = __uint_as_float(v.z), e = __uint_as_float(v.w);
        return (a != a) | (b != b) | (c != c) | (e != e);
    }
    __device__ static __forceinline__ float from_storage(float v) { return v; }
    __device__ static __forceinline__ float to_storage(float v) { return v; }
};

template <>
struct Elem<__half> {
    static constexpr int kPerVec = 8;
    static constexpr uint32_t kNegInfWord = 0xFC00FC00u;
    __device__ static __forceinline__ void unpack(const uint4 &v, float (&f)[8]) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            __half2 h = *reinterpret_cast<const __half2 *>(&w[i]);
            float2 p = __half22float2(h);
            f[2 * i] = p.x;
            f[2 * i + 1] = p.y;
        }
    }
    // packed maxima: three instructions for eight elements, then the two halves of the last word
    __device__ static __forceinline__ float vector_max(const uint4 &v) {
        const __half2 a = *reinterpret_cast<const __half2 *>(&v.x), b = *reinterpret_cast<const __half2 *>(&v.y);
        const __half2 c = *reinterpret_cast<const __half2 *>(&v.z), e = *reinterpret_cast<const __half2 *>(&v.w);
        const float2 f = __half22float2(__hmax2(__hmax2(a, b), __hmax2(c, e)));
        return fmaxf(f.x, f.y);
    }
    // a half is NaN when its magnitude bits exceed 0x7C00: adding 0x03FF then carries into bit 15
    __device__ static __forceinline__ bool vector_has_nan(const uint4 &v) {
        const uint32_t m = 0x7FFF7FFFu, a = 0x03FF03FFu;
        return ((((v.x & m) + a) | ((v.y & m) + a) | ((v.z & m) + a) | ((v.w & m) + a)) & 0x80008000u) != 0u;
    }
    __device__ static __forceinline__ float from_storage(__half v) { return __half2float(v); }
    __device__ static __forceinline__ __half to_storage(float v) { return __float2half_rn(v); }
};

template <>
struct Elem<__nv_bfloat16> {
    static constexpr int kPerVec = 8;
    static constexpr uint32_t kNegInfWord = 0xFF80FF80u;
    __device__ static __forceinline__ void unpack(const uint4 &v, float (&f)[8]) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
    }
    __device__ static __forceinline__ float vector_max(const uint4 &v) {
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162 *>(&v.x), b = *reinterpret_cast<const __nv_bfloat162 *>(&v.y);
        const __nv_bfloat162 c = *reinterpret_cast<const __nv_bfloat162 *>(&v.z), e = *reinterpret_cast<const __nv_bfloat162 *>(&v.w);
        const float2 f = __bfloat1622float2(__hmax2(__hmax2(a, b), __hmax2(c, e)));
        return fmaxf(f.x, f.y);
    }
    // a bfloat16 is NaN when its magnitude bits exceed 0x7F80: adding 0x007F then carries into bit 15
    __device__ static __forceinline__ bool vector_has_nan(const uint4 &v) {
        const uint32_t m = 0x7FFF7FFFu, a = 0x007F007Fu;
        return ((((v.x & m) + a) | ((v.y & m) + a) | ((v.z & m) + a) | ((v.w & m) + a)) & 0x80008000u) != 0u;
    }
    __device__ static __forceinline__ float from_storage(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ static __forceinline__ __nv_bfloat16 to_storage(float v) { return __float2bfloat16_rn(v); }
};

// Streaming 16-byte load: read once, do not keep in L1.
__device__ __forceinline__ uint4 load_stream(const uint4 *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// Replaces the elements of a vector outside [lo, hi) by -inf.
template <typename T>
__device__ __forceinline__ void mask_vector(uint4 &v, int lo, int hi) {
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
    if constexpr (sizeof(T) == 4) {
#pragma unroll
        for (int e = 0; e < 4; e++)
            if (e < lo || e >= hi)
                w[e] = Elem<T>::kNegInfWord;
    } else {
#pragma unroll
        for (int e = 0; e < 8; e++) {
            if (e < lo || e >= hi) {
                uint32_t ninf = Elem<T>::kNegInfWord & 0xFFFFu;
                if (e & 1)
                    w[e >> 1] = (w[e >> 1] & 0x0000FFFFu) | (ninf << 16);
                else
                    w[e >> 1] = (w[e >> 1] & 0xFFFF0000u) | ninf;
            }
        }
    }
    v = make_uint4(w[0], w[1], w[2], w[3]);
}

// ---- packet: per-(row, part) softmax statistics + k best candidates -------
// words: [0] m (float bits), [1] s (float bits), [2] count, [3] reserved,
//        [4 .. 4+k) keys, [4+k .. 4+2k) indices.  Entries are sorted best first.
__host__ __device__ inline int packet_words(int k) { return 4 + 2 * k; }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        v += __shfl_xor_sync(kFullMask, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        v = fmaxf(v, __shfl_xor_sync(kFullMask, v, o));
    return v;
}

// Softmax probability of one stored logit given the row maximum of
// z = x * inv_t and the row sum: separately rounded multiply, subtract,
// exp and a true division, as the restated reference arithmetic has them.
__device__ __forceinline__ float softmax_prob(float x, float inv_t, float m, float s) {
    float z = __fmul_rn(x, inv_t);
    return __fdiv_rn(expf(__fsub_rn(z, m)), s);
}

template <typename T>
__device__ __forceinline__ void store_value(void *base, int64_t i, float v) {
    reinterpret_cast<T *>(base)[i] = Elem<T>::to_storage(v);
}

__device__ __forceinline__ void store_index(void *base, int index_dtype, int64_t i, int64_t v) {
    if (index_dtype == VKOP_I64)
        reinterpret_cast<int64_t *>(base)[i] = v;
    else
        reinterpret_cast<int32_t *>(base)[i] = static_cast<int32_t>(v);
}

}  // namespace vkop_cuda
