// The model head around the layer stack: token embedding rows, final RMS norm, lm_head.
//
// Replaces embed_lookup and final_norm (reference src/math_util.rs:205-247), the
// lm_head matvec (src/engine/qwen35_moe/fused_exp1.rs:860-879 -> matvec_int8,
// src/engine/shaders.metal:2435-2471, for the BQ4 scheme's INT8 head; the 4-bit
// dequant-matvec for the INT4 scheme) and the INT8 codec's reader side
// (src/dtype.rs:164-179: one f32 scale per output row).  lm_head is the largest
// single read of a decode step (vocab x hidden: 0.5 GB as INT8, 0.29 GB as 4-bit):
// HBM-bound streaming kernels, x kept in registers as exact integer digit planes.
#include "q4dot.cuh"
#include "stage.cuh"

namespace moe {

// ─── embedding rows ─────────────────────────────────────────────────────────
// (nibble as f32) * scale + bias with separately rounded multiply and add, as the reference computes it.
__global__ void __launch_bounds__(256) embed_rows_kernel(const uint32_t* __restrict__ w, const uint16_t* __restrict__ s,
                                                         const uint16_t* __restrict__ b, const int64_t* __restrict__ ids,
                                                         int hidden, int64_t vocab, float* __restrict__ out,
                                                         unsigned int* err) {
    const int t = blockIdx.x;
    int64_t id = ids[t];
    if (id < 0 || id >= vocab) {  // reported, never dereferenced: the row becomes zeros
        if (threadIdx.x == 0) atomicExch(err, 11u);
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[(size_t)t * hidden + i] = 0.0f;
        return;
    }
    const int words = hidden / 8, groups = hidden / kGroup;
    for (int p = threadIdx.x; p < words; p += blockDim.x) {
        const uint32_t packed = w[(size_t)id * words + p];
        const int g = p / (kGroup / 8);
        const float scale = bf16_bits_to_f32(s[(size_t)id * groups + g]), bias = bf16_bits_to_f32(b[(size_t)id * groups + g]);
        float v[8];
#pragma unroll
        for (int n = 0; n < 8; ++n) v[n] = __fadd_rn(__fmul_rn((float)((packed >> (4 * n)) & 0xFu), scale), bias);
        float4* dst = reinterpret_cast<float4*>(out + (size_t)t * hidden + p * 8);
        dst[0] = make_float4(v[0], v[1], v[2], v[3]);
        dst[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
}

// ─── final norm: x = h * (inv_rms * w), one CTA per token ───────────────────
__global__ void __launch_bounds__(256) final_norm_kernel(const float* __restrict__ h, const uint16_t* __restrict__ w, int hidden,
                                                         float* __restrict__ x) {
    __shared__ float red[8];
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* row = h + (size_t)t * hidden;
    float ss = 0.0f;
    for (int i = tid; i < hidden; i += 256) ss = fmaf(row[i], row[i], ss);
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float inv_rms = 1.0f / sqrtf(tot / (float)hidden + 1e-6f);  // RMS_NORM_EPS (src/constants.rs:15)
    for (int i = tid; i < hidden; i += 256) x[(size_t)t * hidden + i] = row[i] * (inv_rms * bf16_bits_to_f32(w[i]));
}

// ─── INT8 lm_head, streaming, rows of 2,048 columns ─────────────────────────
// out[row] = scale[row] * sum_c w[row][c] * x[c].  x is staged once per CTA as three signed-byte digit planes per
// 32-element chunk (exact integer sums, 23 bits relative to the chunk's maximum); a lane keeps the planes of its own
// 64 columns in registers, so a row costs it four 128-bit loads and 48 dp4a.
constexpr int kI8Cols = 2048;
constexpr int kI8Warps = 8;
constexpr int kI8Unroll = 2;

__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__global__ void __launch_bounds__(kI8Warps * 32, 2)
matvec_int8_stream_kernel(const int8_t* __restrict__ w, const float* __restrict__ scales, const float* __restrict__ x,
                          float* __restrict__ y, int rows, unsigned int* err_flag) {
    constexpr int nch = kI8Cols / 32;
    __shared__ __align__(128) float raw[kI8Cols];
    __shared__ __align__(16) uint32_t xd[3][nch][8];  // digit planes in column order: word k of a chunk = columns 4k .. 4k + 3
    __shared__ float xdl[nch];
    __shared__ uint64_t bar;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    if (tid == 0) {
        mbar_expect_tx(&bar, kI8Cols * 4u);
        bulk_g2s(raw, x, kI8Cols * 4u, &bar);
    }
    const int ok = __syncthreads_and(mbar_wait(&bar, 0) ? 1 : 0);
    if (!ok) {
        if (tid == 0) atomicExch(err_flag, 1u);
        return;
    }
#pragma unroll
    for (int it = 0; it < kI8Cols / 4 / (kI8Warps * 32); ++it) {
        const int f = tid + it * kI8Warps * 32, c = f >> 3, j = f & 7;  // eight consecutive lanes per chunk
        const float4 o = reinterpret_cast<const float4*>(raw)[f];
        float mx = fmaxf(fmaxf(fabsf(o.x), fabsf(o.y)), fmaxf(fabsf(o.z), fabsf(o.w)));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
        const float inv = mx > 0.0f ? 4194304.0f / mx : 0.0f;
        if (j == 0) xdl[c] = mx * (1.0f / 4194304.0f);
        const int X[4] = {__float2int_rn(o.x * inv), __float2int_rn(o.y * inv), __float2int_rn(o.z * inv), __float2int_rn(o.w * inv)};
        uint32_t pk[3] = {0u, 0u, 0u};
#pragma unroll
        for (int i = 0; i < 4; ++i) {  // three signed base-256 digits of each integer
            const int d0 = (X[i] << 24) >> 24;
            const int X1 = (X[i] - d0) >> 8;
            const int d1 = (X1 << 24) >> 24;
            const int d2 = (X1 - d1) >> 8;
            pk[0] |= ((uint32_t)d0 & 0xFFu) << (8 * i);
            pk[1] |= ((uint32_t)d1 & 0xFFu) << (8 * i);
            pk[2] |= ((uint32_t)d2 & 0xFFu) << (8 * i);
        }
#pragma unroll
        for (int p = 0; p < 3; ++p) xd[p][c][j] = pk[p];
    }
    __syncthreads();
    uint32_t xr[2][3][8];  // this lane's columns 64 lane .. 64 lane + 63: chunks 2 lane and 2 lane + 1
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int p = 0; p < 3; ++p)
#pragma unroll
            for (int k = 0; k < 8; ++k) xr[h][p][k] = xd[p][2 * lane + h][k];
    const float dl0 = xdl[2 * lane], dl1 = xdl[2 * lane + 1];

    const int stride = gridDim.x * kI8Warps;
    for (int row0 = blockIdx.x * kI8Warps + warp; row0 < rows; row0 += stride * kI8Unroll) {
        uint4 q[kI8Unroll][4];
        float sc[kI8Unroll];
#pragma unroll
        for (int u = 0; u < kI8Unroll; ++u) {
            const int row = row0 + u * stride;
            if (row < rows) {
                const uint4* wrow = reinterpret_cast<const uint4*>(w + (size_t)row * kI8Cols) + 4 * lane;
#pragma unroll
                for (int i = 0; i < 4; ++i) q[u][i] = ld_stream_u4(wrow + i);
                sc[u] = __ldg(scales + row);
            }
        }
#pragma unroll
        for (int u = 0; u < kI8Unroll; ++u) {
            const int row = row0 + u * stride;
            if (row < rows) {  // uniform per warp
                float d[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    int a[3] = {0, 0, 0};
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        const uint4 v = q[u][h * 2 + (k >> 2)];
                        const uint32_t wv = (k & 3) == 0 ? v.x : (k & 3) == 1 ? v.y : (k & 3) == 2 ? v.z : v.w;
#pragma unroll
                        for (int p = 0; p < 3; ++p) a[p] = dp4a_ss(wv, xr[h][p][k], a[p]);
                    }
                    // |a[p]| <= 8 * 4 * 127 * 128 < 2^22
                    d[h] = fmaf(small_int_to_float(a[2]), 65536.0f, fmaf(small_int_to_float(a[1]), 256.0f, small_int_to_float(a[0])));
                }
                float acc = sc[u] * fmaf(dl0, d[0], dl1 * d[1]);
                acc = warp_sum(acc);
                if (lane == 0) y[row] = acc;
            }
        }
    }
}

// Generic INT8 matvec for other widths (cols a multiple of 16, at most 16,384): one warp per row, x in shared memory.
__global__ void __launch_bounds__(256) matvec_int8_kernel(const int8_t* __restrict__ w, const float* __restrict__ scales,
                                                          const float* __restrict__ x, float* __restrict__ y, int rows, int cols) {
    extern __shared__ __align__(16) float xs[];
    for (int i = threadIdx.x; i < cols; i += 256) xs[i] = x[i];
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int row = blockIdx.x * 8 + warp; row < rows; row += gridDim.x * 8) {
        const uint4* wrow = reinterpret_cast<const uint4*>(w + (size_t)row * cols);
        float acc = 0.0f;
        for (int c = lane; c < cols / 16; c += 32) {
            const uint4 v = ld_stream_u4(wrow + c);
            const uint32_t ws[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 4; ++k)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc = fmaf((float)(int8_t)(ws[k] >> (8 * i)), xs[c * 16 + k * 4 + i], acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) y[row] = acc * scales[row];
    }
}

// ─── host side ──────────────────────────────────────────────────────────────

static size_t al256h(size_t v) { return (v + 255) / 256 * 256; }

void head_destroy(moe_engine* e) {
    HeadState& hs = e->head;
    if (hs.embed) cudaFree(hs.embed);
    if (hs.final_norm) cudaFree(hs.final_norm);
    if (hs.lm_head) cudaFree(hs.lm_head);
    if (hs.work) cudaFree(hs.work);
    hs = HeadState{};
}

int head_load_tensor(moe_engine* e, int which, const void* w, const void* s, const void* b, int dtype) {
    const moe_dims_t& d = e->dims;
    HeadState& hs = e->head;
    MOE_REQUIRE(w, "null tensor");
    MOE_REQUIRE(d.vocab > 0, "the engine was created with vocab == 0: it has no head");
    const size_t V = (size_t)d.vocab, H = (size_t)d.hidden, G = H / d.group;
    auto put = [&](uint8_t* dst, const void* src, size_t bytes) -> int {
        MOE_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, e->stream));
        return MOE_OK;
    };
    int rc = MOE_OK;
    if (which == MOE_H_EMBED) {
        MOE_REQUIRE(dtype == MOE_DT_INT4 && s && b, "the embedding table is an INT4 triple (weight, scales, biases)");
        const size_t wb = al256h(V * H / 2), sb = al256h(V * G * 2);
        if (!hs.embed) {
            MOE_CUDA(cudaMalloc(&hs.embed, wb + 2 * sb));
            e->resident += wb + 2 * sb;
        }
        hs.embed_s = wb; hs.embed_b = wb + sb;
        if ((rc = put(hs.embed, w, V * H / 2)) || (rc = put(hs.embed + hs.embed_s, s, V * G * 2)) ||
            (rc = put(hs.embed + hs.embed_b, b, V * G * 2)))
            return rc;
        MOE_CUDA(cudaStreamSynchronize(e->stream));
        hs.embed_loaded = true;
    } else if (which == MOE_H_FINAL_NORM) {
        MOE_REQUIRE(dtype == MOE_DT_BF16, "the final norm weight is bf16");
        if (!hs.final_norm) MOE_CUDA(cudaMalloc(&hs.final_norm, al256h(H * 2)));
        if ((rc = put((uint8_t*)hs.final_norm, w, H * 2))) return rc;
        MOE_CUDA(cudaStreamSynchronize(e->stream));
        hs.norm_loaded = true;
    } else if (which == MOE_H_LM_HEAD) {
        MOE_REQUIRE(dtype == MOE_DT_INT8 || dtype == MOE_DT_INT4, "lm_head is INT8 (per-row f32 scales) or an INT4 triple");
        MOE_REQUIRE(s && (dtype == MOE_DT_INT8 || b), "lm_head: scales (and biases for INT4) missing");
        const size_t wb = al256h(dtype == MOE_DT_INT8 ? V * H : V * H / 2);
        const size_t sb = al256h(dtype == MOE_DT_INT8 ? V * 4 : V * G * 2);
        const size_t total = wb + 2 * sb;
        if (hs.lm_head && hs.lm_bytes != total) {
            MOE_CUDA(cudaStreamSynchronize(e->stream));
            cudaFree(hs.lm_head);
            hs.lm_head = nullptr;
            e->resident -= hs.lm_bytes;
        }
        if (!hs.lm_head) {
            MOE_CUDA(cudaMalloc(&hs.lm_head, total));
            hs.lm_bytes = total;
            e->resident += total;
        }
        hs.lm_s = wb; hs.lm_b = wb + sb;
        hs.lm_dtype = dtype;
        if ((rc = put(hs.lm_head, w, dtype == MOE_DT_INT8 ? V * H : V * H / 2)) ||
            (rc = put(hs.lm_head + hs.lm_s, s, dtype == MOE_DT_INT8 ? V * 4 : V * G * 2)))
            return rc;
        if (dtype == MOE_DT_INT4 && (rc = put(hs.lm_head + hs.lm_b, b, V * G * 2))) return rc;
        MOE_CUDA(cudaStreamSynchronize(e->stream));
        hs.lm_loaded = true;
    } else {
        set_error("unknown head tensor %d", which);
        return MOE_ERR_INVALID;
    }
    return MOE_OK;
}

// normalised hidden states [n, H], followed by int64 token ids [n]
int head_reserve(moe_engine* e, int32_t n) {
    HeadState& hs = e->head;
    if (n <= hs.cap) return MOE_OK;
    MOE_CUDA(cudaStreamSynchronize(e->stream));
    if (hs.work) cudaFree(hs.work);
    hs.work = nullptr;
    hs.cap = 0;
    const size_t xb = al256h((size_t)n * e->dims.hidden * 4);
    MOE_CUDA(cudaMalloc(&hs.work, xb + al256h((size_t)n * 8)));
    hs.x = reinterpret_cast<float*>(hs.work);
    hs.ids = reinterpret_cast<int64_t*>(hs.work + xb);
    hs.cap = n;
    return MOE_OK;
}

int launch_embed(moe_engine* e, const int64_t* ids_dev, int32_t n, float* out_dev) {
    const HeadState& hs = e->head;
    if (!hs.embed_loaded) {
        set_error("the embedding table (model.embed_tokens) is not loaded");
        return MOE_ERR_STATE;
    }
    MOE_REQUIRE(e->dims.hidden % 8 == 0 && (((uintptr_t)out_dev) & 15) == 0, "embed: output must be 16-byte aligned");
    embed_rows_kernel<<<n, 256, 0, e->stream>>>(reinterpret_cast<const uint32_t*>(hs.embed),
                                                reinterpret_cast<const uint16_t*>(hs.embed + hs.embed_s),
                                                reinterpret_cast<const uint16_t*>(hs.embed + hs.embed_b), ids_dev,
                                                e->dims.hidden, e->dims.vocab, out_dev, e->dec_sync + 2);
    e->launches++;
    MOE_CUDA(cudaGetLastError());
    return MOE_OK;
}

// logits[t] = lm_head . final_norm(hidden[t]) for n tokens; all device pointers
int launch_logits(moe_engine* e, const float* hidden_dev, int32_t n, float* logits_dev) {
    return launch_logits_norm(e, hidden_dev, n, logits_dev, nullptr);
}

int launch_logits_norm(moe_engine* e, const float* hidden_dev, int32_t n, float* logits_dev, const uint16_t* norm_w) {
    HeadState& hs = e->head;
    const moe_dims_t& d = e->dims;
    if ((!norm_w && !hs.norm_loaded) || !hs.lm_loaded) {
        set_error("the model head is not loaded (%s missing)", !hs.lm_loaded ? "lm_head" : "model.norm.weight");
        return MOE_ERR_STATE;
    }
    int rc = head_reserve(e, n);
    if (rc) return rc;
    final_norm_kernel<<<n, 256, 0, e->stream>>>(hidden_dev, norm_w ? norm_w : hs.final_norm, d.hidden, hs.x);
    e->launches++;
    for (int t = 0; t < n; ++t) {
        const float* x = hs.x + (size_t)t * d.hidden;
        float* y = logits_dev + (size_t)t * d.vocab;
        if (hs.lm_dtype == MOE_DT_INT4) {
            rc = launch_matvec(e, hs.lm_head, hs.lm_head + hs.lm_s, hs.lm_head + hs.lm_b, x, y, d.vocab, d.hidden);
            if (rc) return rc;
        } else if (d.hidden == kI8Cols) {
            int blocks = (d.vocab + kI8Warps * kI8Unroll - 1) / (kI8Warps * kI8Unroll);
            if (blocks > e->sm_count * 2) blocks = e->sm_count * 2;
            matvec_int8_stream_kernel<<<blocks, kI8Warps * 32, 0, e->stream>>>(
                reinterpret_cast<const int8_t*>(hs.lm_head), reinterpret_cast<const float*>(hs.lm_head + hs.lm_s), x, y, d.vocab,
                e->dec_sync + 2);
            e->launches++;
        } else {
            MOE_REQUIRE(d.hidden % 16 == 0 && d.hidden <= 16384, "INT8 lm_head: hidden (%d) must be a multiple of 16 up to 16384", d.hidden);
            if (!hs.i8_attr_set) {
                MOE_CUDA(cudaFuncSetAttribute(matvec_int8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 16384 * 4));
                hs.i8_attr_set = true;
            }
            int blocks = (d.vocab + 7) / 8;
            if (blocks > e->sm_count * 8) blocks = e->sm_count * 8;
            matvec_int8_kernel<<<blocks, 256, (size_t)d.hidden * 4, e->stream>>>(
                reinterpret_cast<const int8_t*>(hs.lm_head), reinterpret_cast<const float*>(hs.lm_head + hs.lm_s), x, y, d.vocab,
                d.hidden);
            e->launches++;
        }
    }
    MOE_CUDA(cudaGetLastError());
    return MOE_OK;
}

}  // namespace moe
