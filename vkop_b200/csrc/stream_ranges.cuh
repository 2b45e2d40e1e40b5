// Ranges of 16-byte vector slots that the CTAs of the streaming kernels own.
//
// The [rows, nvv] grid of vector slots is cut into `grid` consecutive ranges, either a fixed number
// of parts per row or byte-balanced ranges that may run across rows; boundaries inside a row are
// snapped to multiples of kUnit vectors so that no CTA holds a sliver of a row.
#pragma once

#include <stdint.h>

namespace vkop_cuda {

constexpr int kUnit = 256;  // range boundaries inside a row are multiples of this many vectors

// Snaps a slot offset inside a row to the nearest allowed boundary.
__host__ __device__ inline uint32_t snap_in_row(uint32_t v, uint32_t nvv) {
    const uint32_t units = nvv / kUnit > 0 ? nvv / kUnit : 1;
    const uint32_t u = (v + kUnit / 2) / kUnit;
    return u >= units ? nvv : u * kUnit;
}

// First slot of CTA c (all arithmetic in 32 bits: rows * nvv < 2^32).
// parts > 0: CTA c serves part c % parts of row c / parts.
__host__ __device__ inline uint32_t stream_boundary(uint32_t c, uint32_t grid, uint32_t per, uint32_t nvv, uint32_t total,
                                                    uint32_t parts) {
    if (c >= grid)
        return total;
    if (parts > 0) {
        const uint32_t r = c / parts, j = c - r * parts;
        return r * nvv + snap_in_row(static_cast<uint32_t>(static_cast<uint64_t>(j) * nvv / parts), nvv);
    }
    const uint64_t v64 = static_cast<uint64_t>(c) * per;
    if (v64 >= total)
        return total;
    const uint32_t V = static_cast<uint32_t>(v64);
    const uint32_t r = V / nvv;
    return r * nvv + snap_in_row(V - r * nvv, nvv);
}

// Largest CTA index whose range starts at or before slot V (V < total).
__host__ __device__ inline uint32_t stream_owner(uint32_t V, uint32_t grid, uint32_t per, uint32_t nvv, uint32_t total, uint32_t parts) {
    uint32_t c;
    if (parts > 0) {
        const uint32_t r = V / nvv;
        c = r * parts + static_cast<uint32_t>(static_cast<uint64_t>(V - r * nvv) * parts / nvv);
    } else {
        c = V / per;
    }
    if (c >= grid)
        c = grid - 1;
    while (c + 1 < grid && stream_boundary(c + 1, grid, per, nvv, total, parts) <= V)
        c++;
    while (c > 0 && stream_boundary(c, grid, per, nvv, total, parts) > V)
        c--;
    return c;
}

}  // namespace vkop_cuda
