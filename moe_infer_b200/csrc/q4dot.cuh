// In-register 4-bit dequant dot products shared by the matvec and decode kernels.
//
// A "chunk" is one 128-bit load: 4 u32 words = 32 nibbles = half of a 64-column
// quantisation group.  Nibble n of word p is column p*8+n (reference
// src/dtype.rs:123-131).  A nibble is turned into the float 16+n with one shift
// and one LOP3 (mask, then OR the exponent of 16.0f), so no integer-to-float
// conversion is issued; the offset is removed with the chunk's pre-computed
// sum of activations:
//     sum_i (n_i*s + b) x_i = s * sum_i (16+n_i) x_i + (b - 16 s) * sum_i x_i
//
// Activations live in shared memory "chunk-transposed": float4 j (0..7) of chunk
// c is at xs[j * n_chunks + c], so that the 32 lanes of a warp, which own 32
// consecutive chunks, read 32 consecutive float4 (no bank conflicts).
#pragma once
#include "common.cuh"

namespace moe {

template <int N>
__device__ __forceinline__ float nib_f16plus(uint32_t w) {
    // (16 + nibble N of w) as f32: nibble moved to mantissa bits 19..22.
    uint32_t t;
    if constexpr (N * 4 < 19) t = w << (19 - N * 4);
    else t = w >> (N * 4 - 19);
    return __uint_as_float((t & 0x00780000u) | 0x41800000u);
}

__device__ __forceinline__ float dot8(uint32_t w, const float4& a, const float4& b, float acc) {
    acc = fmaf(nib_f16plus<0>(w), a.x, acc);
    acc = fmaf(nib_f16plus<1>(w), a.y, acc);
    acc = fmaf(nib_f16plus<2>(w), a.z, acc);
    acc = fmaf(nib_f16plus<3>(w), a.w, acc);
    acc = fmaf(nib_f16plus<4>(w), b.x, acc);
    acc = fmaf(nib_f16plus<5>(w), b.y, acc);
    acc = fmaf(nib_f16plus<6>(w), b.z, acc);
    acc = fmaf(nib_f16plus<7>(w), b.w, acc);
    return acc;
}

// sum_i (16 + n_i) * x_i over the 32 nibbles of q; xv = the chunk's 8 float4.
__device__ __forceinline__ float dot32(const uint4& q, const float4 (&xv)[8]) {
    float a0 = dot8(q.x, xv[0], xv[1], 0.0f);
    float a1 = dot8(q.y, xv[2], xv[3], 0.0f);
    a0 = dot8(q.z, xv[4], xv[5], a0);
    a1 = dot8(q.w, xv[6], xv[7], a1);
    return a0 + a1;
}

// Contribution of one chunk of one row: s * dot + (b - 16 s) * sumx.
__device__ __forceinline__ float chunk_term(const uint4& q, const float4 (&xv)[8], float sumx,
                                            uint16_t s_bits, uint16_t b_bits) {
    const float s = bf16_bits_to_f32(s_bits);
    const float b = bf16_bits_to_f32(b_bits);
    return fmaf(s, dot32(q, xv), (b - 16.0f * s) * sumx);
}

}  // namespace moe
