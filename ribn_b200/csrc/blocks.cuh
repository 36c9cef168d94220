// GGUF block formats (Q8_0, Q4_K, Q6_K) and their bit-exact device decoders.
//
// The decoded value of every element follows the reference's host decoder
// (crates/gguf/src/lib.rs:561-649) operation by operation, with explicit
// round-to-nearest intrinsics so that no multiply/subtract pair is ever
// contracted into an FMA:
//   Q8_0: d * q
//   Q4_K: (d * scale6) * q - (dmin * min6)      three roundings
//   Q6_K: (d * scale8) * (q - 32)               two roundings
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace ribn {

enum GgmlType : int { kF32 = 0, kF16 = 1, kQ8_0 = 8, kQ4_K = 12, kQ6_K = 14 };

__host__ __device__ inline int block_elems(int type) {
    switch (type) {
        case kF32: case kF16: return 1;
        case kQ8_0: return 32;
        case kQ4_K: case kQ6_K: return 256;
        default: return 0;
    }
}

__host__ __device__ inline int block_bytes(int type) {
    switch (type) {
        case kF32: return 4;
        case kF16: return 2;
        case kQ8_0: return 34;
        case kQ4_K: return 144;
        case kQ6_K: return 210;
        default: return 0;
    }
}

__device__ __forceinline__ float f16_bits_to_f32(unsigned short bits) {
    return __half2float(__ushort_as_half(bits));
}

__device__ __forceinline__ float load_f16(const unsigned char* p) {
    return f16_bits_to_f32((unsigned short)(p[0] | ((unsigned short)p[1] << 8)));
}

// Six-bit scale / minimum of group `g` from the 12 packed bytes that start at
// byte 4 of a Q4_K block (crates/gguf/src/lib.rs:561-575).
__device__ __forceinline__ int q4k_scale(const unsigned char* p, int g) {
    return g < 4 ? (p[g] & 0x3f) : ((p[8 + g - 4] & 0x0f) | ((p[g - 4] >> 2) & 0x30));
}
__device__ __forceinline__ int q4k_min(const unsigned char* p, int g) {
    return g < 4 ? (p[4 + g] & 0x3f) : ((p[8 + g - 4] >> 4) | ((p[4 + g - 4] >> 2) & 0x30));
}

// Element `i` (0..255) of a raw 144-byte Q4_K block.
__device__ __forceinline__ float q4k_element(const unsigned char* b, int i) {
    const float d = load_f16(b), dmin = load_f16(b + 2);
    const int g = i >> 5, l = i & 31;
    const float gs = __fmul_rn(d, (float)q4k_scale(b + 4, g));
    const float gm = __fmul_rn(dmin, (float)q4k_min(b + 4, g));
    const int q = (b[16 + (g >> 1) * 32 + l] >> ((g & 1) * 4)) & 0x0f;
    return __fsub_rn(__fmul_rn(gs, (float)q), gm);
}

// Element `i` (0..255) of a raw 210-byte Q6_K block
// (crates/gguf/src/lib.rs:623-649).
__device__ __forceinline__ float q6k_element(const unsigned char* b, int i) {
    const int g = i >> 5, l = i & 31;
    const int chunk = g >> 2, variant = g & 3;
    const int low = (b[chunk * 64 + (variant & 1) * 32 + l] >> (variant < 2 ? 0 : 4)) & 0x0f;
    const int high = (b[128 + chunk * 32 + l] >> (variant * 2)) & 0x03;
    const int q = (low | (high << 4)) - 32;
    const float d = load_f16(b + 208);
    const float gs = __fmul_rn(d, (float)(signed char)b[192 + g * 2 + (l >> 4)]);
    return __fmul_rn(gs, (float)q);
}

// Element `i` (0..31) of a raw 34-byte Q8_0 block (crates/gguf/src/lib.rs:577-582).
__device__ __forceinline__ float q8_0_element(const unsigned char* b, int i) {
    return __fmul_rn(load_f16(b), (float)(signed char)b[2 + i]);
}

// Element `k` of an encoded row of any supported type.
__device__ __forceinline__ float row_element(int type, const unsigned char* row, long long k) {
    switch (type) {
        case kF32: return reinterpret_cast<const float*>(row)[k];
        case kF16: return f16_bits_to_f32(reinterpret_cast<const unsigned short*>(row)[k]);
        case kQ8_0: return q8_0_element(row + (k >> 5) * 34, (int)(k & 31));
        case kQ4_K: return q4k_element(row + (k >> 8) * 144, (int)(k & 255));
        case kQ6_K: return q6k_element(row + (k >> 8) * 210, (int)(k & 255));
        default: return 0.0f;
    }
}

}  // namespace ribn
