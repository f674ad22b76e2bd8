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

// ─── integer dot products ───────────────────────────────────────────────────
// The 4-bit weights are small integers, so the dot product of a row with a vector is done in
// integer arithmetic: every 32-element chunk of the vector is written as X * delta with
// integers |X| <= 2^22 (delta = chunk maximum / 2^22), X is split into three signed base-256
// digits, and dp4a (four byte products summed into 32 bits) multiplies them with the nibbles,
// four at a time.  Sums are exact; the only rounding is that of x to 23 bits relative to its
// chunk's maximum, the same order as the f32 mantissa the reference multiplies with.
// Byte order: the nibbles of a weight word are split as (w & 0x0F0F0F0F) = columns 0,2,4,6 and
// ((w >> 4) & 0x0F0F0F0F) = columns 1,3,5,7, so digit words are stored "even" and "odd".
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// One thread's float4 (elements 4 j .. 4 j + 3 of chunk c; the 8 threads of a chunk are
// consecutive lanes): writes its digits into planes[(p * 2 + odd) * n_chunks + c] and, from
// lane j == 0, the chunk's delta.
__device__ __forceinline__ void stage_digits(uint4* planes, float* deltas, int n_chunks, int c, int j, const float4& o) {
    float mx = fmaxf(fmaxf(fabsf(o.x), fabsf(o.y)), fmaxf(fabsf(o.z), fabsf(o.w)));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
    const float inv = mx > 0.0f ? 4194304.0f / mx : 0.0f;
    if (j == 0) deltas[c] = mx * (1.0f / 4194304.0f);
    const int X[4] = {__float2int_rn(o.x * inv), __float2int_rn(o.y * inv), __float2int_rn(o.z * inv), __float2int_rn(o.w * inv)};
    uint32_t d[3][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int d0 = (X[i] << 24) >> 24;
        const int X1 = (X[i] - d0) >> 8;
        const int d1 = (X1 << 24) >> 24;
        const int d2 = (X1 - d1) >> 8;
        d[0][i] = (uint32_t)d0 & 0xFFu;
        d[1][i] = (uint32_t)d1 & 0xFFu;
        d[2][i] = (uint32_t)d2 & 0xFFu;
    }
    // this thread holds columns (4 half .. 4 half + 3) of word k: two even and two odd bytes
    const int k = j >> 1, half = j & 1;
#pragma unroll
    for (int p = 0; p < 3; ++p) {
        const uint16_t ev = (uint16_t)(d[p][0] | (d[p][2] << 8));
        const uint16_t od = (uint16_t)(d[p][1] | (d[p][3] << 8));
        uint16_t* e16 = reinterpret_cast<uint16_t*>(planes + (size_t)(p * 2 + 0) * n_chunks + c);
        uint16_t* o16 = reinterpret_cast<uint16_t*>(planes + (size_t)(p * 2 + 1) * n_chunks + c);
        e16[k * 2 + half] = ev;
        o16[k * 2 + half] = od;
    }
}

// sum over the 32 nibbles of q of nibble * X, as a float (X = the chunk's integers)
__device__ __forceinline__ float dot32_int(const uint4& q, const uint4 (&xe)[3], const uint4 (&xo)[3]) {
    int a[3] = {0, 0, 0};
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t lo = w[k] & 0x0F0F0F0Fu, hi = (w[k] >> 4) & 0x0F0F0F0Fu;
#pragma unroll
        for (int p = 0; p < 3; ++p) {
            const uint32_t e = k == 0 ? xe[p].x : k == 1 ? xe[p].y : k == 2 ? xe[p].z : xe[p].w;
            const uint32_t o = k == 0 ? xo[p].x : k == 1 ? xo[p].y : k == 2 ? xo[p].z : xo[p].w;
            a[p] = dp4a_us(lo, e, a[p]);
            a[p] = dp4a_us(hi, o, a[p]);
        }
    }
    return fmaf((float)a[2], 65536.0f, fmaf((float)a[1], 256.0f, (float)a[0]));
}

// int -> float for |v| < 2^22 with one integer and one floating-point add (both full-rate pipes)
__device__ __forceinline__ float small_int_to_float(int v) { return __int_as_float(v + 0x4B400000) - 12582912.0f; }

// dot32_int for digit planes that already sit in registers, converting through small_int_to_float
// (|sum of a plane| <= 8 * 4 * 15 * 128 < 2^22)
__device__ __forceinline__ float dot32_regs(const uint4& q, const uint4 (&xe)[3], const uint4 (&xo)[3]) {
    int a[3] = {0, 0, 0};
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t lo = w[k] & 0x0F0F0F0Fu, hi = (w[k] >> 4) & 0x0F0F0F0Fu;
#pragma unroll
        for (int p = 0; p < 3; ++p) {
            const uint32_t e = k == 0 ? xe[p].x : k == 1 ? xe[p].y : k == 2 ? xe[p].z : xe[p].w;
            const uint32_t o = k == 0 ? xo[p].x : k == 1 ? xo[p].y : k == 2 ? xo[p].z : xo[p].w;
            a[p] = dp4a_us(lo, e, a[p]);
            a[p] = dp4a_us(hi, o, a[p]);
        }
    }
    return fmaf(small_int_to_float(a[2]), 65536.0f, fmaf(small_int_to_float(a[1]), 256.0f, small_int_to_float(a[0])));
}

}  // namespace moe
