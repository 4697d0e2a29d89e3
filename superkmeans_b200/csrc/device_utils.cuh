// Small device-side helpers shared by the kernel files.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace skmb {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Monotone map float -> uint32 (preserves <), so that (key << 32 | index) orders by distance then
// by index under an unsigned 64-bit minimum.
__device__ __forceinline__ uint32_t float_to_ordered(float f) {
    const uint32_t b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float ordered_to_float(uint32_t o) {
    const uint32_t b = (o & 0x80000000u) ? (o & 0x7fffffffu) : ~o;
    return __uint_as_float(b);
}

} // namespace skmb
