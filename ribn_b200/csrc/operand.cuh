// Device helpers that write activations in the integer-MMA operand form
// (see ActOperand): one warp handles one 32-span, lane = input within the span.
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

// All 32 lanes call this with their input `v` of span `span` (inputs span * 32 + lane) of member
// `member`; `square` is the lane's contribution to the RMSNorm sum of squares (ignored when the
// operand has no ss32).  `k` is the operand's input count.
__device__ __forceinline__ void operand_store_span(const ActOperand& op, int member, int k, int span, int lane, float v,
                                                   float square) {
    const float amax = operand_warp_max(fabsf(v));
    const float sx = amax / 127.0f;
    const float inv = amax > 0.0f ? 127.0f / amax : 0.0f;
    int d1, d2, d3;
    const float value = operand_digits(v, inv, d1, d2, d3);
    const float half = operand_half_sum(value);
    signed char* base = op.dig + (size_t)member * 3 * k + operand_position(span * 32 + lane);
    base[0] = (signed char)d1;
    base[k] = (signed char)d2;
    base[2 * (size_t)k] = (signed char)d3;
    if ((lane & 15) == 0) op.sxs16[(size_t)member * (k / 16) + span * 2 + (lane >> 4)] = sx * half;
    if (lane == 0) op.sx[(size_t)member * (k / 32) + span] = sx;
    if (op.ss32 != nullptr) {
        const float ss = operand_warp_sum(square);
        if (lane == 0) op.ss32[(size_t)member * (k / 32) + span] = ss;
    }
}

}  // namespace ribn
