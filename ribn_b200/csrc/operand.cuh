// Device helpers for turning activations into signed 8-bit digits for the integer MMA.
#pragma once
#include <stdint.h>

#include "gemv.cuh"

namespace ribn {

__device__ __forceinline__ float operand_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ float operand_half_sum(float v) {  // sum over each 16-lane half
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float operand_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Three signed digits of v * inv (|v * inv| <= 127): returns d1 + d2/128 + d3/16384.
__device__ __forceinline__ float operand_digits(float v, float inv, int& d1, int& d2, int& d3) {
    const float r0 = v * inv;
    const float f1 = fminf(fmaxf(rintf(r0), -127.0f), 127.0f);
    const float r1 = (r0 - f1) * 128.0f;
    const float f2 = fminf(fmaxf(rintf(r1), -127.0f), 127.0f);
    const float r2 = (r1 - f2) * 128.0f;
    const float f3 = fminf(fmaxf(rintf(r2), -127.0f), 127.0f);
    d1 = (int)f1; d2 = (int)f2; d3 = (int)f3;
    return f1 + f2 * (1.0f / 128.0f) + f3 * (1.0f / 16384.0f);
}

}  // namespace ribn
