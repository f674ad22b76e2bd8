// Batch-1 decode of the MoE stack: one persistent cooperative kernel walks the
// layers, three grid-wide phases per layer, weights streamed from the resident
// HBM store with 128-bit loads and dequantised in registers.
//
// Replaces, per layer, the tail of op1 (post-attention norm, router matvec,
// shared-expert gate/up, shared_expert_gate), the CPU route_experts round trip and
// op2 (8 x gate/up/SwiGLU/down, shared down, moe_combine_residual) of the
// reference's decode engines (src/engine/qwen35_moe/fused_exp1.rs:149-365,
// 734-856; CPU statement src/engine/qwen35_moe/cpu.rs:187-205, 78-85, 398-483).
// Where the reference commits 41 command buffers per token with a blocking
// GPU->CPU wait each, this is one launch for the whole stack; top-k runs on
// the device.
//
//   phase A  x = rmsnorm(h) (every CTA, redundantly); router logits, shared
//            expert gate/up + SwiGLU, shared gate score          [~2.2 MB]
//   phase B  softmax + top-k (every CTA, redundantly, one warp); gate/up/SwiGLU
//            of the K chosen experts                               [~9.4 MB]
//   phase C  down projections of the K experts and the shared expert, combine
//            with the residual: one warp owns one output element   [~5.3 MB]
//
// HBM-bound: 16,974,976 weight bytes per layer-token at the reference sizes.
// Between phases the CTAs meet at a grid barrier built on one global counter;
// the wait is bounded and a timeout raises an error word instead of hanging.
#include "q4dot.cuh"
#include "stage.cuh"

namespace moe {

constexpr int kH = 2048;        // hidden (both reference models)
constexpr int kI = 512;         // moe_intermediate_size == shared_expert_intermediate_size
constexpr int kDecWarps = 16;
constexpr int kDecThreads = kDecWarps * 32;
constexpr int kChH = kH / 32;   // 64 chunks per hidden row
constexpr int kChI = kI / 32;   // 16 chunks per intermediate row
constexpr int kMaxEPerLane = 16;  // top-k supports E <= 512

struct DecodeParams {
    const LayerDev* layers;
    int l0, l1;
    const float* h_in;
    float* h_out;
    float* h_buf0;
    float* h_buf1;
    float* logits;      // [E]
    float* act;         // [(K + 1) * I]
    float* misc;        // [0] shared gate score
    const float* logit_bias;
    const int32_t* forced_idx;
    int32_t* out_idx;
    float* out_w;
    unsigned int* sync; // [0] arrivals, [1] exits, [2] error word
    int E, K;
    moe_expert_layout_t lay;
};

struct __align__(16) DecodeSmem {
    float raw[kH];              // bulk-copy landing zone for h
    float xn[kH];               // normalised x, plain order (bf16 router rows)
    float4 xs[8 * kChH];        // normalised x, chunk-transposed
    float sumx[kChH];
    float4 acts[(kMaxK + 1) * 8 * kChI];  // SwiGLU outputs, chunk-transposed per expert
    float suma[(kMaxK + 1) * kChI];
    float red[kDecWarps];
    float topw[kMaxK + 1];      // combine weights; [K] = sigmoid(shared gate)
    int topi[kMaxK];
    int flag;
    uint64_t bar;
};

// ─── grid barrier with a bounded wait ───────────────────────────────────────
// Arrivals are counted on one monotonically increasing word; `target` is the
// count that completes this barrier.  Returns false (for the whole CTA) when
// the wait gave up or another CTA already raised the error word.
__device__ __forceinline__ bool grid_barrier(unsigned int* sync, unsigned int target, DecodeSmem* sm) {
    // h is written with generic stores and read back by bulk (async-proxy) copies
    asm volatile("fence.proxy.async;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(&sync[0], 1u);
        int ok = 0;
        for (uint32_t i = 0; i < kWaitLimit; ++i) {
            unsigned int v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(sync) : "memory");
            if (v >= target) { ok = 1; break; }
            if ((i & 255u) == 255u) {
                unsigned int err;
                asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(err) : "l"(sync + 2) : "memory");
                if (err) break;
            }
        }
        if (!ok) atomicExch(&sync[2], 2u);
        sm->flag = ok;
        asm volatile("fence.proxy.async;" ::: "memory");
    }
    __syncthreads();
    return sm->flag != 0;
}

// ─── x = rmsnorm(h) * w, staged three ways (plain, chunk-transposed, chunk sums) ──
// rms_norm_bf16 (reference src/math_util.rs:282-288), eps 1e-6.
__device__ __forceinline__ bool stage_norm(DecodeSmem* sm, const float* h, const uint16_t* norm_w,
                                           uint32_t parity) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        mbar_expect_tx(&sm->bar, kH * 4u);
        bulk_g2s(sm->raw, h, kH * 4u, &sm->bar);
    }
    if (!__syncthreads_and(mbar_wait(&sm->bar, parity) ? 1 : 0)) return false;
    static_assert(kH == kDecThreads * 4, "one float4 per thread");
    const float4 v = reinterpret_cast<const float4*>(sm->raw)[tid];
    float ss = warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w);
    if (lane == 0) sm->red[warp] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < kDecWarps; ++i) tot += sm->red[i];
    const float inv_rms = 1.0f / sqrtf(tot / (float)kH + 1e-6f);
    const uint2 wb = reinterpret_cast<const uint2*>(norm_w)[tid];  // 4 bf16
    float4 o;
    o.x = v.x * inv_rms * __uint_as_float(wb.x << 16);
    o.y = v.y * inv_rms * __uint_as_float(wb.x & 0xFFFF0000u);
    o.z = v.z * inv_rms * __uint_as_float(wb.y << 16);
    o.w = v.w * inv_rms * __uint_as_float(wb.y & 0xFFFF0000u);
    reinterpret_cast<float4*>(sm->xn)[tid] = o;
    const int c = tid >> 3, j = tid & 7;   // float4 j of chunk c
    sm->xs[j * kChH + c] = o;
    float s = (o.x + o.y) + (o.z + o.w);
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 4);
    if (j == 0) sm->sumx[c] = s;
    __syncthreads();
    return true;
}

// Dot products of NR 4-bit rows of length kH with the staged x.  All loads are
// issued before the first use so that NR*2 128-bit loads per lane are in flight.
template <int NR>
__device__ __forceinline__ void rows_dot_h(const DecodeSmem* sm, const uint32_t* const (&w)[NR],
                                           const uint16_t* const (&s)[NR],
                                           const uint16_t* const (&b)[NR], float (&out)[NR], int lane) {
    uint4 q[NR][2];
    uint16_t sc[NR][2], bi[NR][2];
#pragma unroll
    for (int r = 0; r < NR; ++r) {
#pragma unroll
        for (int it = 0; it < 2; ++it) {
            const int c = lane + 32 * it;
            q[r][it] = ld_stream_u4(reinterpret_cast<const uint4*>(w[r]) + c);
            sc[r][it] = __ldg(s[r] + (c >> 1));
            bi[r][it] = __ldg(b[r] + (c >> 1));
        }
    }
#pragma unroll
    for (int r = 0; r < NR; ++r) out[r] = 0.0f;
#pragma unroll
    for (int it = 0; it < 2; ++it) {
        const int c = lane + 32 * it;
        float4 xv[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) xv[j] = sm->xs[j * kChH + c];
        const float sx = sm->sumx[c];
#pragma unroll
        for (int r = 0; r < NR; ++r) out[r] += chunk_term(q[r][it], xv, sx, sc[r][it], bi[r][it]);
    }
#pragma unroll
    for (int r = 0; r < NR; ++r) out[r] = warp_sum(out[r]);
}

// One bf16 row of length kH (BQ4-scheme router; reference matvec_bf16,
// src/engine/shaders.metal:2392).
__device__ __forceinline__ float row_dot_bf16(const DecodeSmem* sm, const uint16_t* wrow, int lane) {
    uint4 q[kH / 8 / 32];
#pragma unroll
    for (int it = 0; it < kH / 256; ++it)
        q[it] = ld_stream_u4(reinterpret_cast<const uint4*>(wrow) + lane + 32 * it);
    float acc = 0.0f;
#pragma unroll
    for (int it = 0; it < kH / 256; ++it) {
        const int base = (lane + 32 * it) * 8;
        const float4 x0 = *reinterpret_cast<const float4*>(sm->xn + base);
        const float4 x1 = *reinterpret_cast<const float4*>(sm->xn + base + 4);
        acc = fmaf(__uint_as_float(q[it].x << 16), x0.x, acc);
        acc = fmaf(__uint_as_float(q[it].x & 0xFFFF0000u), x0.y, acc);
        acc = fmaf(__uint_as_float(q[it].y << 16), x0.z, acc);
        acc = fmaf(__uint_as_float(q[it].y & 0xFFFF0000u), x0.w, acc);
        acc = fmaf(__uint_as_float(q[it].z << 16), x1.x, acc);
        acc = fmaf(__uint_as_float(q[it].z & 0xFFFF0000u), x1.y, acc);
        acc = fmaf(__uint_as_float(q[it].w << 16), x1.z, acc);
        acc = fmaf(__uint_as_float(q[it].w & 0xFFFF0000u), x1.w, acc);
    }
    return warp_sum(acc);
}

// swiglu_fused (reference src/math_util.rs:254-259): silu(gate) * up.
__device__ __forceinline__ float swiglu(float g, float u) { return g / (1.0f + expf(-g)) * u; }

// ─── softmax + top-k + renormalise, one warp ────────────────────────────────
// route_experts (reference src/engine/qwen35_moe/cpu.rs:78-85): softmax over all
// E logits (src/math_util.rs:77-88), the K largest probabilities (ties: lower
// index first, matching the strict `>` of src/math_util.rs:101), divided by their
// sum (:120-126).  Results in descending order.
__device__ __forceinline__ void route_warp(const float* logits, const float* bias, const int32_t* forced,
                                           int E, int K, int* topi, float* topw, int lane) {
    float p[kMaxEPerLane];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < kMaxEPerLane; ++i) {
        const int e = lane + 32 * i;
        float v = -INFINITY;
        if (e < E) {
            v = __ldcg(logits + e);  // written by other CTAs: read through L2
            if (bias) v += bias[e];
        }
        p[i] = v;
        mx = fmaxf(mx, v);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < kMaxEPerLane; ++i) {
        const int e = lane + 32 * i;
        p[i] = (e < E) ? expf(p[i] - mx) : 0.0f;
        sum += p[i];
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
#pragma unroll
    for (int i = 0; i < kMaxEPerLane; ++i) p[i] = (lane + 32 * i < E) ? p[i] * inv : -1.0f;

    float myw = 0.0f;
    int myi = 0;
    if (forced) {
        for (int k = 0; k < K; ++k) {
            const int e = forced[k];
            float v = 0.0f;
#pragma unroll
            for (int i = 0; i < kMaxEPerLane; ++i)
                if (lane + 32 * i == e) v = p[i];
            v = __shfl_sync(0xffffffffu, v, e & 31);
            if (lane == k) { myw = v; myi = e; }
        }
    } else {
        for (int k = 0; k < K; ++k) {
            float bv = -2.0f;
            int be = 0x7fffffff;
#pragma unroll
            for (int i = 0; i < kMaxEPerLane; ++i) {
                const int e = lane + 32 * i;
                if (p[i] > bv) { bv = p[i]; be = e; }  // ascending e inside a lane: first max wins
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oe = __shfl_xor_sync(0xffffffffu, be, o);
                if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
            }
            if (lane == k) { myw = bv; myi = be; }
#pragma unroll
            for (int i = 0; i < kMaxEPerLane; ++i)
                if (lane + 32 * i == be) p[i] = -1.0f;  // taken
        }
    }
    // normalize_weights: divide by the sum of the K selected probabilities
    float ws = warp_sum(lane < K ? myw : 0.0f);
    if (ws > 0.0f) myw *= (1.0f / ws);
    if (lane < K) { topi[lane] = myi; topw[lane] = myw; }
}

// ─── the persistent kernel ──────────────────────────────────────────────────
__global__ void __launch_bounds__(kDecThreads, 1) decode_stack_kernel(DecodeParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    DecodeSmem* sm = reinterpret_cast<DecodeSmem*>(smem_raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = gridDim.x;
    const int cta = blockIdx.x;
    const int E = p.E, K = p.K;
    const moe_expert_layout_t L = p.lay;

    if (tid == 0) {
        mbar_init(&sm->bar, 1);
        mbar_fence_init();
    }
    __syncthreads();

    unsigned int bar_target = 0;
    uint32_t parity = 0;
    bool alive = true;

    for (int l = p.l0; l < p.l1 && alive; ++l) {
        const LayerDev ly = p.layers[l];
        const float* h_cur = (l == p.l0) ? p.h_in : (((l - p.l0) & 1) ? p.h_buf0 : p.h_buf1);
        float* h_nxt = (l == p.l1 - 1) ? p.h_out : (((l - p.l0) & 1) ? p.h_buf1 : p.h_buf0);

        // ── phase A ────────────────────────────────────────────────────────
        if (!stage_norm(sm, h_cur, ly.post_norm, parity)) {
            if (tid == 0) atomicExch(&p.sync[2], 3u);
            alive = false;
            break;
        }
        parity ^= 1u;
        {
            // items: [0, E) router rows, [E, E + I) shared gate/up row pairs, E + I: shared gate score
            const int n_items = E + kI + 1;
            for (int item = warp * G + cta; item < n_items; item += kDecWarps * G) {
                if (item < E) {
                    float v;
                    if (ly.router_bf16) {
                        v = row_dot_bf16(sm, ly.router_bf16 + (size_t)item * kH, lane);
                    } else {
                        const uint32_t* const w[1] = {ly.router_q4.w + (size_t)item * (kH / 8)};
                        const uint16_t* const s[1] = {ly.router_q4.s + (size_t)item * (kH / kGroup)};
                        const uint16_t* const b[1] = {ly.router_q4.b + (size_t)item * (kH / kGroup)};
                        float o[1];
                        rows_dot_h<1>(sm, w, s, b, o, lane);
                        v = o[0];
                    }
                    if (lane == 0) p.logits[item] = v;
                } else if (item < E + kI) {
                    const int r = item - E;
                    const moe_expert_layout_t& S = L;  // shared expert uses the same layout (kI rows)
                    const uint8_t* ex = ly.shared;
                    const uint32_t* const w[2] = {
                        reinterpret_cast<const uint32_t*>(ex + S.gate_w) + (size_t)r * (kH / 8),
                        reinterpret_cast<const uint32_t*>(ex + S.up_w) + (size_t)r * (kH / 8)};
                    const uint16_t* const s[2] = {
                        reinterpret_cast<const uint16_t*>(ex + S.gate_s) + (size_t)r * (kH / kGroup),
                        reinterpret_cast<const uint16_t*>(ex + S.up_s) + (size_t)r * (kH / kGroup)};
                    const uint16_t* const b[2] = {
                        reinterpret_cast<const uint16_t*>(ex + S.gate_b) + (size_t)r * (kH / kGroup),
                        reinterpret_cast<const uint16_t*>(ex + S.up_b) + (size_t)r * (kH / kGroup)};
                    float o[2];
                    rows_dot_h<2>(sm, w, s, b, o, lane);
                    if (lane == 0) p.act[K * kI + r] = swiglu(o[0], o[1]);
                } else {
                    const uint32_t* const w[1] = {ly.sgate.w};
                    const uint16_t* const s[1] = {ly.sgate.s};
                    const uint16_t* const b[1] = {ly.sgate.b};
                    float o[1];
                    rows_dot_h<1>(sm, w, s, b, o, lane);
                    if (lane == 0) p.misc[0] = o[0];
                }
            }
        }
        bar_target += G;
        if (!grid_barrier(p.sync, bar_target, sm)) { alive = false; break; }

        // ── phase B ────────────────────────────────────────────────────────
        if (warp == 0) {
            const int32_t* forced = p.forced_idx;
            route_warp(p.logits, p.logit_bias, forced, E, K, sm->topi, sm->topw, lane);
            if (lane == 0) {
                // sigmoid (reference src/math_util.rs:67-69) of the shared gate score
                sm->topw[K] = 1.0f / (1.0f + expf(-__ldcg(p.misc)));
            }
            if (cta == 0 && lane < K) {
                if (p.out_idx) p.out_idx[lane] = sm->topi[lane];
                if (p.out_w) p.out_w[lane] = sm->topw[lane];
            }
        }
        __syncthreads();
        {
            const int n_items = K * kI;  // (expert slot k, row r): gate row r and up row r
            for (int item0 = warp * G + cta; item0 < n_items; item0 += 2 * kDecWarps * G) {
                const int item1 = item0 + kDecWarps * G;
                const bool two = item1 < n_items;
                const int it[2] = {item0, two ? item1 : item0};
                const uint32_t* w[4];
                const uint16_t* s[4];
                const uint16_t* b[4];
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const int k = it[q] / kI, r = it[q] - k * kI;
                    const uint8_t* ex = ly.experts + (size_t)sm->topi[k] * L.expert_size;
                    w[2 * q] = reinterpret_cast<const uint32_t*>(ex + L.gate_w) + (size_t)r * (kH / 8);
                    w[2 * q + 1] = reinterpret_cast<const uint32_t*>(ex + L.up_w) + (size_t)r * (kH / 8);
                    s[2 * q] = reinterpret_cast<const uint16_t*>(ex + L.gate_s) + (size_t)r * (kH / kGroup);
                    s[2 * q + 1] = reinterpret_cast<const uint16_t*>(ex + L.up_s) + (size_t)r * (kH / kGroup);
                    b[2 * q] = reinterpret_cast<const uint16_t*>(ex + L.gate_b) + (size_t)r * (kH / kGroup);
                    b[2 * q + 1] = reinterpret_cast<const uint16_t*>(ex + L.up_b) + (size_t)r * (kH / kGroup);
                }
                const uint32_t* const wc[4] = {w[0], w[1], w[2], w[3]};
                const uint16_t* const sc[4] = {s[0], s[1], s[2], s[3]};
                const uint16_t* const bc[4] = {b[0], b[1], b[2], b[3]};
                float o[4];
                rows_dot_h<4>(sm, wc, sc, bc, o, lane);
                if (lane == 0) {
                    p.act[it[0]] = swiglu(o[0], o[1]);
                    if (two) p.act[it[1]] = swiglu(o[2], o[3]);
                }
            }
        }
        bar_target += G;
        if (!grid_barrier(p.sync, bar_target, sm)) { alive = false; break; }

        // ── phase C ────────────────────────────────────────────────────────
        {
            // stage the (K + 1) x I SwiGLU outputs chunk-transposed, with chunk sums
            const int n_f4 = (K + 1) * (kI / 4);
            for (int i = tid; i < n_f4; i += kDecThreads) {
                const float4 v = __ldcg(reinterpret_cast<const float4*>(p.act) + i);
                const int m = i / (kI / 4), f = i - m * (kI / 4);
                const int c = f >> 3, j = f & 7;
                sm->acts[(m * 8 + j) * kChI + c] = v;
                float sv = (v.x + v.y) + (v.z + v.w);
                sv += __shfl_xor_sync(0xffffffffu, sv, 1);
                sv += __shfl_xor_sync(0xffffffffu, sv, 2);
                sv += __shfl_xor_sync(0xffffffffu, sv, 4);
                if (j == 0) sm->suma[m * kChI + c] = sv;
            }
            __syncthreads();
            // one warp per output element i: half-warp `sub` takes matrices sub, sub+2, ...
            const int sub = lane >> 4, c = lane & 15;
            constexpr int kMats = (kMaxK + 2) / 2;  // 5 matrix slots per half-warp
            for (int i = warp * G + cta; i < kH; i += kDecWarps * G) {
                uint4 q[kMats];
                uint16_t scv[kMats], biv[kMats];
#pragma unroll
                for (int jm = 0; jm < kMats; ++jm) {
                    const int m = sub + 2 * jm;
                    if (m <= K) {
                        const uint8_t* ex = (m < K) ? ly.experts + (size_t)sm->topi[m] * L.expert_size : ly.shared;
                        q[jm] = ld_stream_u4(reinterpret_cast<const uint4*>(ex + L.down_w) + (size_t)i * kChI + c);
                        scv[jm] = __ldg(reinterpret_cast<const uint16_t*>(ex + L.down_s) + (size_t)i * (kI / kGroup) + (c >> 1));
                        biv[jm] = __ldg(reinterpret_cast<const uint16_t*>(ex + L.down_b) + (size_t)i * (kI / kGroup) + (c >> 1));
                    } else {
                        q[jm] = make_uint4(0, 0, 0, 0);
                        scv[jm] = 0;
                        biv[jm] = 0;
                    }
                }
                float acc = 0.0f;
#pragma unroll
                for (int jm = 0; jm < kMats; ++jm) {
                    const int m = sub + 2 * jm;
                    if (m <= K) {
                        float4 xv[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) xv[j] = sm->acts[(m * 8 + j) * kChI + c];
                        acc = fmaf(sm->topw[m], chunk_term(q[jm], xv, sm->suma[m * kChI + c], scv[jm], biv[jm]), acc);
                    }
                }
                acc = warp_sum(acc);
                // moe_combine_residual (reference src/math_util.rs:599-612)
                if (lane == 0) h_nxt[i] = sm->raw[i] + acc;
            }
        }
        if (l + 1 < p.l1) {
            bar_target += G;
            if (!grid_barrier(p.sync, bar_target, sm)) { alive = false; break; }
        }
    }

    // Last CTA out rewinds the barrier words for the next launch.
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        const unsigned int done = atomicAdd(&p.sync[1], 1u) + 1u;
        if (done == (unsigned int)G) {
            p.sync[0] = 0u;
            p.sync[1] = 0u;
            __threadfence();
        }
    }
}

// ─── host side ──────────────────────────────────────────────────────────────

int decode_init(moe_engine* e) {
    const moe_dims_t& d = e->dims;
    MOE_CUDA(cudaMalloc(&e->dec_h[0], d.hidden * sizeof(float)));
    MOE_CUDA(cudaMalloc(&e->dec_h[1], d.hidden * sizeof(float)));
    MOE_CUDA(cudaMalloc(&e->dec_logits, d.num_experts * sizeof(float)));
    MOE_CUDA(cudaMalloc(&e->dec_act, (size_t)(kMaxK + 1) * d.inter * sizeof(float)));
    MOE_CUDA(cudaMalloc(&e->dec_misc, 16 * sizeof(float)));
    MOE_CUDA(cudaMalloc(&e->dec_idx, kMaxK * sizeof(int32_t)));
    MOE_CUDA(cudaMalloc(&e->dec_w, kMaxK * sizeof(float)));
    MOE_CUDA(cudaMalloc(&e->dec_sync, 16 * sizeof(unsigned int)));
    MOE_CUDA(cudaMemset(e->dec_sync, 0, 16 * sizeof(unsigned int)));
    MOE_CUDA(cudaMallocHost(&e->stage_host, (size_t)2 * d.hidden * sizeof(float)));
    MOE_CUDA(cudaFuncSetAttribute(decode_stack_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)sizeof(DecodeSmem)));
    int per_sm = 0;
    MOE_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_stack_kernel, kDecThreads,
                                                           sizeof(DecodeSmem)));
    MOE_REQUIRE(per_sm >= 1, "decode kernel does not fit on an SM");
    e->dec_grid = e->sm_count;  // one CTA per SM, all co-resident (cooperative launch)
    return MOE_OK;
}

void decode_destroy(moe_engine* e) {
    cudaFree(e->dec_h[0]); cudaFree(e->dec_h[1]); cudaFree(e->dec_logits); cudaFree(e->dec_act);
    cudaFree(e->dec_misc); cudaFree(e->dec_idx); cudaFree(e->dec_w); cudaFree(e->dec_sync);
    if (e->stage_host) cudaFreeHost(e->stage_host);
}

int launch_decode(moe_engine* e, int l0, int l1, const float* h_in, float* h_out,
                  const float* logit_bias, const int32_t* forced_idx, int32_t* out_idx, float* out_w) {
    const moe_dims_t& d = e->dims;
    MOE_REQUIRE(d.hidden == kH && d.inter == kI && d.shared_inter == kI,
                "decode path is built for hidden=%d, inter=shared_inter=%d (got %d/%d/%d)", kH, kI,
                d.hidden, d.inter, d.shared_inter);
    MOE_REQUIRE(d.num_experts <= 32 * kMaxEPerLane, "decode path supports at most %d experts", 32 * kMaxEPerLane);
    MOE_REQUIRE(l0 >= 0 && l1 > l0 && l1 <= (int)e->layers.size(), "decode: bad layer range [%d, %d)", l0, l1);
    MOE_REQUIRE((((uintptr_t)h_in) & 15) == 0 && (((uintptr_t)h_out) & 15) == 0, "decode: h must be 16-byte aligned");
    for (int l = l0; l < l1; ++l) {
        int rc = check_layer_ready(e, l);
        if (rc != MOE_OK) return rc;
    }
    int rc = refresh_layer_table(e);
    if (rc != MOE_OK) return rc;
    DecodeParams p{};
    p.layers = e->layers_dev;
    p.l0 = l0; p.l1 = l1;
    p.h_in = h_in; p.h_out = h_out;
    p.h_buf0 = e->dec_h[0]; p.h_buf1 = e->dec_h[1];
    p.logits = e->dec_logits; p.act = e->dec_act; p.misc = e->dec_misc;
    p.logit_bias = logit_bias; p.forced_idx = forced_idx;
    p.out_idx = out_idx; p.out_w = out_w;
    p.sync = e->dec_sync;
    p.E = d.num_experts; p.K = d.top_k;
    p.lay = e->lay;
    void* args[] = {&p};
    MOE_CUDA(cudaLaunchCooperativeKernel((const void*)decode_stack_kernel, dim3(e->dec_grid), dim3(kDecThreads),
                                         args, sizeof(DecodeSmem), e->stream));
    e->launches++;
    return MOE_OK;
}

}  // namespace moe
