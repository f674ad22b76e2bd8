// Batch-1 decode of the MoE stack: one persistent cooperative kernel walks the
// layers; every CTA owns a fixed, contiguous slice of each weight matrix and
// pulls it from the resident HBM store into shared memory with bulk (TMA)
// copies issued as early as the data dependencies allow; nibbles are
// dequantised in registers and reduced with warp shuffles.
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
//            expert gate/up + SwiGLU, shared gate score            [~2.2 MB]
//            -- does not depend on routing: its weights are requested one
//               layer ahead
//   phase B  softmax + top-k (every CTA, redundantly); gate/up/SwiGLU of the K
//            chosen experts                                         [~9.4 MB]
//   phase C  down projections of the K experts and the shared expert, combine
//            with the residual: one warp owns one output element    [~5.3 MB]
//            -- requested together with phase B's weights, right after top-k
//
// HBM-bound: 16,974,976 weight bytes per layer-token at the reference sizes.
// Between phases the CTAs meet at a grid barrier built on one global counter;
// every wait (barrier, mbarrier) is bounded and a timeout raises an error word
// instead of hanging.
#include "q4dot.cuh"
#include "stage.cuh"

namespace moe {

constexpr int kH = 2048;        // hidden (both reference models)
constexpr int kI = 512;         // moe_intermediate_size == shared_expert_intermediate_size
constexpr int kDecWarps = 16;
constexpr int kDecThreads = kDecWarps * 32;
constexpr int kChH = kH / 32;   // 64 chunks (128-bit loads) per hidden row
constexpr int kChI = kI / 32;   // 16 chunks per intermediate row
constexpr int kMaxE = 512;      // routing supports up to 512 experts
constexpr int kProfPoints = 12;

// Per-CTA slice capacities; the host checks that the grid is large enough.
constexpr int kMaxRouterRows = 4;   // ceil(E / grid)
constexpr int kMaxSharedRows = 4;   // ceil(I / grid) gate/up row pairs of the shared expert
constexpr int kMaxBItems = 28;      // ceil(K * I / grid) gate/up row pairs of routed experts
constexpr int kMaxCRows = 14;       // ceil(H / grid) output elements

#define PROF(idx)                                                                                  \
    do {                                                                                           \
        if (p.prof && cta == 0 && tid == 0) p.prof[(l - p.l0) * kProfPoints + (idx)] = clock64();  \
    } while (0)

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
    long long* prof;    // nullable: [layer][kProfPoints] SM-clock stamps taken by CTA 0
    int E, K;
    moe_expert_layout_t lay;
};

struct __align__(128) DecodeSmem {
    // prefetched weight slices (destinations of bulk copies: 16-byte aligned offsets)
    uint4 a_router[kMaxRouterRows * (kH * 2 / 16)];      // bf16 rows (4096 B each) or 4-bit rows (1024 B each)
    uint4 a_shw[2][kMaxSharedRows][kChH];                // shared expert gate / up rows
    uint4 a_sgw[kChH];                                   // shared_expert_gate row
    uint4 b_w[2][kMaxBItems][kChH];                      // routed gate / up rows
    uint4 c_w[kMaxK + 1][kMaxCRows][kChI];               // down rows of the K experts + shared expert
    uint16_t a_router_s[kMaxRouterRows][kH / kGroup];
    uint16_t a_router_b[kMaxRouterRows][kH / kGroup];
    uint16_t a_shs[2][kMaxSharedRows][kH / kGroup];
    uint16_t a_shb[2][kMaxSharedRows][kH / kGroup];
    uint16_t a_sgs[kH / kGroup];
    uint16_t a_sgb[kH / kGroup];
    uint16_t b_s[2][kMaxBItems][kH / kGroup];
    uint16_t b_b[2][kMaxBItems][kH / kGroup];
    uint16_t c_s[kMaxK + 1][kMaxCRows][kI / kGroup];
    uint16_t c_b[kMaxK + 1][kMaxCRows][kI / kGroup];
    // activations
    float raw[kH];              // bulk-copy landing zone for h
    float xn[kH];               // normalised x, plain order (bf16 router rows)
    float4 xs[8 * kChH];        // normalised x, chunk-transposed
    float sumx[kChH];
    float4 acts[(kMaxK + 1) * 8 * kChI];  // SwiGLU outputs, chunk-transposed per expert
    float suma[(kMaxK + 1) * kChI];
    float prob[kMaxE];
    float red[kDecWarps];
    float red2[kDecWarps];
    float cand_p[kMaxE];
    int cand_i[kMaxE];
    int ncand;
    float topw[kMaxK + 1];      // combine weights; [K] = sigmoid(shared gate)
    float topp[kMaxK];
    int topi[kMaxK];
    int flag;
    uint64_t bar_h;
};
static_assert(sizeof(DecodeSmem) <= 227 * 1024, "decode staging exceeds shared memory");
static_assert((sizeof(uint16_t) * (kMaxK + 1) * kMaxCRows * (kI / kGroup)) % 16 == 0, "bulk-copy destinations stay aligned");

__device__ __forceinline__ int slice_lo(int c, int n, int G) { return (int)(((long long)c * n) / G); }

// ─── grid barrier with a bounded wait ───────────────────────────────────────
// Arrivals are counted on one monotonically increasing word; `target` is the
// count that completes this barrier.  Returns false (for the whole CTA) when
// the wait gave up or another CTA already raised the error word.
__device__ __forceinline__ bool grid_barrier(unsigned int* sync, unsigned int target, DecodeSmem* sm) {
    // h is written with generic stores and read back by bulk (async-proxy) copies
    asm volatile("fence.proxy.async;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0) {
        // release: publishes this CTA's writes (ordered before it by the bar.sync above)
        asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(sync), "r"(1u) : "memory");
        int ok = 0;
        const long long t0 = clock64();
        for (uint32_t i = 0;; ++i) {
            unsigned int v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(sync) : "memory");
            if (v >= target) { ok = 1; break; }
            if ((i & 63u) == 63u) {
                unsigned int err;
                asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(err) : "l"(sync + 2) : "memory");
                if (err || clock64() - t0 > kWaitCycles) break;
            }
        }
        if (!ok) atomicExch(&sync[2], 2u);
        sm->flag = ok;
        asm volatile("fence.proxy.async;" ::: "memory");
    }
    __syncthreads();
    return sm->flag != 0;
}

// ─── weight prefetch with per-thread 16-byte asynchronous copies ─────────────
// Every thread of the CTA copies pieces p = tid, tid + 512, ... of a slice;
// completion is tracked with cp.async groups (one group per slice), then a CTA
// barrier makes the bytes visible to every warp.
__device__ __forceinline__ void cp16(void* dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void copy_flat(void* dst, const void* src, int pieces, int tid) {
    for (int q = tid; q < pieces; q += kDecThreads)
        cp16(reinterpret_cast<uint8_t*>(dst) + (size_t)q * 16, reinterpret_cast<const uint8_t*>(src) + (size_t)q * 16);
}

// phase A slice: router rows [e0, e0+ne), shared gate/up pairs [p0, p0+np), shared gate (last CTA)
__device__ __forceinline__ void prefetch_A(DecodeSmem* sm, const LayerDev& ly, const moe_expert_layout_t& S,
                                           int cta, int G, int E, int tid) {
    const int e0 = slice_lo(cta, E, G), ne = slice_lo(cta + 1, E, G) - e0;
    const int p0 = slice_lo(cta, kI, G), np = slice_lo(cta + 1, kI, G) - p0;
    constexpr int kRowW = kH / 2, kRowS = (kH / kGroup) * 2;  // bytes of one 4-bit row / of its scales
    if (ly.router_bf16) {
        copy_flat(sm->a_router, ly.router_bf16 + (size_t)e0 * kH, ne * (kH * 2 / 16), tid);
    } else {
        copy_flat(sm->a_router, ly.router_q4.w + (size_t)e0 * (kH / 8), ne * (kRowW / 16), tid);
        copy_flat(sm->a_router_s, ly.router_q4.s + (size_t)e0 * (kH / kGroup), ne * (kRowS / 16), tid);
        copy_flat(sm->a_router_b, ly.router_q4.b + (size_t)e0 * (kH / kGroup), ne * (kRowS / 16), tid);
    }
    const uint8_t* sh = ly.shared;
    copy_flat(sm->a_shw[0], sh + S.gate_w + (size_t)p0 * kRowW, np * (kRowW / 16), tid);
    copy_flat(sm->a_shw[1], sh + S.up_w + (size_t)p0 * kRowW, np * (kRowW / 16), tid);
    // the four small arrays: one piece per thread at most
    {
        const int per = np * (kRowS / 16);
        if (tid < 4 * per) {
            const int a = tid / per, q = tid - a * per;
            const int64_t off = a == 0 ? S.gate_s : a == 1 ? S.up_s : a == 2 ? S.gate_b : S.up_b;
            uint16_t* d = a == 0 ? sm->a_shs[0][0] : a == 1 ? sm->a_shs[1][0] : a == 2 ? sm->a_shb[0][0] : sm->a_shb[1][0];
            cp16(reinterpret_cast<uint8_t*>(d) + q * 16, sh + off + (size_t)p0 * kRowS + q * 16);
        }
    }
    if (cta == G - 1) {
        copy_flat(sm->a_sgw, ly.sgate.w, kRowW / 16, tid);
        if (tid < kRowS / 16) cp16(reinterpret_cast<uint8_t*>(sm->a_sgs) + tid * 16, reinterpret_cast<const uint8_t*>(ly.sgate.s) + tid * 16);
        else if (tid < 2 * (kRowS / 16))
            cp16(reinterpret_cast<uint8_t*>(sm->a_sgb) + (tid - kRowS / 16) * 16,
                 reinterpret_cast<const uint8_t*>(ly.sgate.b) + (tid - kRowS / 16) * 16);
    }
    cp_commit();
}

// phase B: a warp copies the items it will compute itself, j = warp and warp + 16
// of this CTA's [i0, i0 + nb) (item = slot k * I + row r: gate row r and up row r of
// the k-th chosen expert).  Warp-private, so only a __syncwarp is needed before use
// and warps start computing as soon as their own bytes land.
__device__ __forceinline__ void prefetch_B_warp(DecodeSmem* sm, const LayerDev& ly, const moe_expert_layout_t& L,
                                                int i0, int nb, int warp, int lane) {
    constexpr int kPW = kH / 2 / 16;  // 64 pieces per weight row; scales/biases: 4 pieces per row
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        const int j = warp + t * kDecWarps;
        if (j < nb) {
            const int i = i0 + j, k = i / kI, r = i - k * kI;
            const uint8_t* ex = ly.experts + (size_t)sm->topi[k] * L.expert_size;
            const uint8_t* gw = ex + L.gate_w + (size_t)r * (kH / 2);
            const uint8_t* uw = ex + L.up_w + (size_t)r * (kH / 2);
            cp16(&sm->b_w[0][j][lane], gw + lane * 16);
            cp16(&sm->b_w[0][j][lane + 32], gw + (lane + 32) * 16);
            cp16(&sm->b_w[1][j][lane], uw + lane * 16);
            cp16(&sm->b_w[1][j][lane + 32], uw + (lane + 32) * 16);
            if (lane < 16) {
                const int a = lane >> 2, c = lane & 3;
                const int64_t off = a == 0 ? L.gate_s : a == 1 ? L.up_s : a == 2 ? L.gate_b : L.up_b;
                uint16_t* d = a == 0 ? sm->b_s[0][j] : a == 1 ? sm->b_s[1][j] : a == 2 ? sm->b_b[0][j] : sm->b_b[1][j];
                cp16(reinterpret_cast<uint8_t*>(d) + c * 16, ex + off + (size_t)r * (kH / kGroup) * 2 + c * 16);
            }
        }
    }
    static_assert(kPW == 64, "two pieces per lane per row");
    cp_commit();
}

// phase C: a warp copies the down rows of the output element it owns (row r0 + warp)
// for the K chosen experts and the shared expert.
__device__ __forceinline__ void prefetch_C_warp(DecodeSmem* sm, const LayerDev& ly, const moe_expert_layout_t& L,
                                                int r0, int nc, int K, int warp, int lane) {
    for (int j = warp; j < nc; j += kDecWarps) {
        const int pw = (K + 1) * kChI;  // 16 pieces per row
        for (int q = lane; q < pw; q += 32) {
            const int m = q / kChI, c = q - m * kChI;
            const uint8_t* ex = (m < K) ? ly.experts + (size_t)sm->topi[m] * L.expert_size : ly.shared;
            cp16(&sm->c_w[m][j][c], ex + L.down_w + (size_t)(r0 + j) * (kI / 2) + c * 16);
        }
        if (lane < 2 * (K + 1)) {
            const int m = lane >> 1, a = lane & 1;
            const uint8_t* ex = (m < K) ? ly.experts + (size_t)sm->topi[m] * L.expert_size : ly.shared;
            cp16(a ? sm->c_b[m][j] : sm->c_s[m][j], ex + (a ? L.down_b : L.down_s) + (size_t)(r0 + j) * (kI / kGroup) * 2);
        }
    }
    cp_commit();
}

// ─── x = rmsnorm(h) * w, staged three ways (plain, chunk-transposed, chunk sums) ──
// rms_norm_bf16 (reference src/math_util.rs:282-288), eps 1e-6.
__device__ __forceinline__ bool stage_norm(DecodeSmem* sm, const float* h, const uint16_t* norm_w,
                                           uint32_t parity) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        mbar_expect_tx(&sm->bar_h, kH * 4u);
        bulk_g2s(sm->raw, h, kH * 4u, &sm->bar_h);
    }
    const uint2 wb = __ldg(reinterpret_cast<const uint2*>(norm_w) + tid);  // 4 bf16, in flight during the wait
    if (!__syncthreads_and(mbar_wait(&sm->bar_h, parity) ? 1 : 0)) return false;
    static_assert(kH == kDecThreads * 4, "one float4 per thread");
    const float4 v = reinterpret_cast<const float4*>(sm->raw)[tid];
    float ss = warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w);
    if (lane == 0) sm->red[warp] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < kDecWarps; ++i) tot += sm->red[i];
    const float inv_rms = 1.0f / sqrtf(tot / (float)kH + 1e-6f);
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

// Dot products of NR 4-bit rows of length kH (staged in shared memory) with the staged x.
template <int NR>
__device__ __forceinline__ void rows_dot_h(const DecodeSmem* sm, const uint4* const (&w)[NR],
                                           const uint16_t* const (&s)[NR], const uint16_t* const (&b)[NR],
                                           float (&out)[NR], int lane) {
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
        for (int r = 0; r < NR; ++r) out[r] += chunk_term(w[r][c], xv, sx, s[r][c >> 1], b[r][c >> 1]);
    }
#pragma unroll
    for (int r = 0; r < NR; ++r) out[r] = warp_sum(out[r]);
}

// One bf16 row of length kH (BQ4-scheme router; reference matvec_bf16,
// src/engine/shaders.metal:2392), the row staged in shared memory.
__device__ __forceinline__ float row_dot_bf16(const DecodeSmem* sm, const uint4* wrow, int lane) {
    float acc = 0.0f;
#pragma unroll
    for (int it = 0; it < kH / 256; ++it) {
        const uint4 q = wrow[lane + 32 * it];
        const int base = (lane + 32 * it) * 8;
        const float4 x0 = *reinterpret_cast<const float4*>(sm->xn + base);
        const float4 x1 = *reinterpret_cast<const float4*>(sm->xn + base + 4);
        acc = fmaf(__uint_as_float(q.x << 16), x0.x, acc);
        acc = fmaf(__uint_as_float(q.x & 0xFFFF0000u), x0.y, acc);
        acc = fmaf(__uint_as_float(q.y << 16), x0.z, acc);
        acc = fmaf(__uint_as_float(q.y & 0xFFFF0000u), x0.w, acc);
        acc = fmaf(__uint_as_float(q.z << 16), x1.x, acc);
        acc = fmaf(__uint_as_float(q.z & 0xFFFF0000u), x1.y, acc);
        acc = fmaf(__uint_as_float(q.w << 16), x1.z, acc);
        acc = fmaf(__uint_as_float(q.w & 0xFFFF0000u), x1.w, acc);
    }
    return warp_sum(acc);
}

// swiglu_fused (reference src/math_util.rs:254-259): silu(gate) * up.
__device__ __forceinline__ float swiglu(float g, float u) { return g / (1.0f + expf(-g)) * u; }

// ─── softmax + top-k + renormalise, whole CTA ───────────────────────────────
// route_experts (reference src/engine/qwen35_moe/cpu.rs:78-85): softmax over all
// E logits (src/math_util.rs:77-88), the K largest probabilities (ties: lower
// index first, matching the strict `>` of src/math_util.rs:101), divided by their
// sum (:120-126).  Thread t owns expert t.  The K-th largest of the 16 per-warp
// maxima is a lower bound of the K-th largest probability, so only experts at
// or above it are candidates; each candidate finds its rank by counting the
// candidates that beat it.  Results come out in descending order.
__device__ __forceinline__ void route_cta(DecodeSmem* sm, const float* logits, const float* bias,
                                          const int32_t* forced, int E, int K) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float v = -INFINITY;
    if (tid < E) {
        v = __ldcg(logits + tid);  // written by other CTAs: read through L2
        if (bias) v += bias[tid];
    }
    float mx = v;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) sm->red[warp] = mx;
    if (tid == 0) sm->ncand = 0;
    __syncthreads();
    const float wmx = mx;  // this warp's max logit
    mx = sm->red[0];
#pragma unroll
    for (int i = 1; i < kDecWarps; ++i) mx = fmaxf(mx, sm->red[i]);
    const float ex = (tid < E) ? expf(v - mx) : 0.0f;
    const float ws = warp_sum(ex);
    __syncthreads();
    if (lane == 0) { sm->red[warp] = ws; sm->red2[warp] = (warp * 32 < E) ? expf(wmx - mx) : -1.0f; }
    __syncthreads();
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < kDecWarps; ++i) sum += sm->red[i];
    const float inv = 1.0f / sum;
    const float pr = ex * inv;
    static_assert(kMaxE == kDecThreads, "one thread per expert slot");
    sm->prob[tid] = (tid < E) ? pr : -1.0f;
    if (forced) {
        __syncthreads();
        if (tid < K) { sm->topi[tid] = forced[tid]; sm->topp[tid] = sm->prob[forced[tid]]; }
    } else {
        // threshold = K-th largest warp maximum (as a probability); -1 when fewer than K warps hold experts
        float tau;
        {
            const int me = lane & (kDecWarps - 1);
            const float mine = sm->red2[me] * inv;  // bit-identical to the owning thread's pr; negative for empty warps
            int cnt = 0;
#pragma unroll
            for (int j = 0; j < kDecWarps; ++j) {
                const float o = __shfl_sync(0xffffffffu, mine, j);
                cnt += (o > mine) || (o == mine && j < me);
            }
            // exactly one of lanes 0..15 has K-1 warp maxima ahead of it
            const unsigned hit = __ballot_sync(0xffffffffu, cnt == K - 1 && lane < kDecWarps);
            tau = __shfl_sync(0xffffffffu, mine, __ffs(hit) - 1);
            if (tau < 0.0f) tau = -1.0f;  // fewer than K warps hold experts: everything is a candidate
        }
        if (tid < E && pr >= tau) {
            const int slot = atomicAdd(&sm->ncand, 1);
            sm->cand_p[slot] = pr;
            sm->cand_i[slot] = tid;
        }
        __syncthreads();
        const int nc = sm->ncand;
        if (tid < nc) {
            const float cp = sm->cand_p[tid];
            const int ci = sm->cand_i[tid];
            int rank = 0;
            for (int j = 0; j < nc; ++j) {
                const float q = sm->cand_p[j];
                rank += (q > cp) || (q == cp && sm->cand_i[j] < ci);
            }
            if (rank < K) { sm->topi[rank] = ci; sm->topp[rank] = cp; }
        }
    }
    __syncthreads();
    if (tid == 0) {
        // normalize_weights: divide by the sum of the K selected probabilities
        float s = 0.0f;
        for (int k = 0; k < K; ++k) s += sm->topp[k];
        const float invs = s > 0.0f ? 1.0f / s : 1.0f;
        for (int k = 0; k < K; ++k) sm->topw[k] = sm->topp[k] * invs;
    }
    __syncthreads();
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
        mbar_init(&sm->bar_h, 1);
        mbar_fence_init();
    }
    __syncthreads();

    // this CTA's slices
    const int e0 = slice_lo(cta, E, G), ne = slice_lo(cta + 1, E, G) - e0;
    const int p0 = slice_lo(cta, kI, G), np = slice_lo(cta + 1, kI, G) - p0;
    const int i0 = slice_lo(cta, K * kI, G), nb = slice_lo(cta + 1, K * kI, G) - i0;
    const int r0 = slice_lo(cta, kH, G), nc = slice_lo(cta + 1, kH, G) - r0;

    unsigned int bar_target = 0;
    uint32_t parity = 0;
    bool alive = true;

    prefetch_A(sm, p.layers[p.l0], L, cta, G, E, tid);

    for (int l = p.l0; l < p.l1 && alive; ++l) {
        const LayerDev ly = p.layers[l];
        const float* h_cur = (l == p.l0) ? p.h_in : (((l - p.l0) & 1) ? p.h_buf0 : p.h_buf1);
        float* h_nxt = (l == p.l1 - 1) ? p.h_out : (((l - p.l0) & 1) ? p.h_buf1 : p.h_buf0);

        // ── phase A ────────────────────────────────────────────────────────
        PROF(0);
        if (!stage_norm(sm, h_cur, ly.post_norm, parity)) {
            if (tid == 0) atomicExch(&p.sync[2], 3u);
            alive = false;
            break;
        }
        cp_wait<0>();  // this layer's phase-A slice (requested one layer ago)
        __syncthreads();
        PROF(1);
        {
            // warps [0, ne): router rows; [4, 4 + np): shared gate/up pairs; 8: shared gate score
            if (warp < ne) {
                float v;
                if (ly.router_bf16) {
                    v = row_dot_bf16(sm, sm->a_router + warp * (kH * 2 / 16), lane);
                } else {
                    const uint4* const w[1] = {sm->a_router + warp * kChH};
                    const uint16_t* const s[1] = {sm->a_router_s[warp]};
                    const uint16_t* const b[1] = {sm->a_router_b[warp]};
                    float o[1];
                    rows_dot_h<1>(sm, w, s, b, o, lane);
                    v = o[0];
                }
                if (lane == 0) p.logits[e0 + warp] = v;
            } else if (warp >= 4 && warp < 4 + np) {
                const int j = warp - 4;
                const uint4* const w[2] = {sm->a_shw[0][j], sm->a_shw[1][j]};
                const uint16_t* const s[2] = {sm->a_shs[0][j], sm->a_shs[1][j]};
                const uint16_t* const b[2] = {sm->a_shb[0][j], sm->a_shb[1][j]};
                float o[2];
                rows_dot_h<2>(sm, w, s, b, o, lane);
                if (lane == 0) p.act[K * kI + p0 + j] = swiglu(o[0], o[1]);
            } else if (warp == 8 && cta == G - 1) {
                const uint4* const w[1] = {sm->a_sgw};
                const uint16_t* const s[1] = {sm->a_sgs};
                const uint16_t* const b[1] = {sm->a_sgb};
                float o[1];
                rows_dot_h<1>(sm, w, s, b, o, lane);
                if (lane == 0) p.misc[0] = o[0];
            }
        }
        PROF(2);
        bar_target += G;
        if (!grid_barrier(p.sync, bar_target, sm)) { alive = false; break; }
        PROF(3);
        PROF(4);

        // ── phase B ────────────────────────────────────────────────────────
        route_cta(sm, p.logits, p.logit_bias, p.forced_idx, E, K);
        PROF(5);
        // request this warp's gate/up rows now; its down rows and the next layer's
        // phase-A slice are requested after the gate/up arithmetic, so that their
        // issue (which stalls while the load queues are full) overlaps barrier 2
        prefetch_B_warp(sm, ly, L, i0, nb, warp, lane);
        if (warp == 0) {
            if (lane == 0) {
                // sigmoid (reference src/math_util.rs:67-69) of the shared gate score
                sm->topw[K] = 1.0f / (1.0f + expf(-__ldcg(p.misc)));
            }
            if (cta == 0 && lane < K) {
                if (p.out_idx) p.out_idx[lane] = sm->topi[lane];
                if (p.out_w) p.out_w[lane] = sm->topw[lane];
            }
        }
        PROF(6);
        cp_wait<0>();  // this warp's gate/up rows landed
        __syncwarp();
        PROF(7);
        {
            // item j of this CTA = (gate row, up row) pair; two items per warp pass
            for (int j = warp; j < nb; j += 2 * kDecWarps) {
                const int j2 = j + kDecWarps;
                const bool two = j2 < nb;
                const int jb = two ? j2 : j;
                const uint4* const w[4] = {sm->b_w[0][j], sm->b_w[1][j], sm->b_w[0][jb], sm->b_w[1][jb]};
                const uint16_t* const s[4] = {sm->b_s[0][j], sm->b_s[1][j], sm->b_s[0][jb], sm->b_s[1][jb]};
                const uint16_t* const b[4] = {sm->b_b[0][j], sm->b_b[1][j], sm->b_b[0][jb], sm->b_b[1][jb]};
                float o[4];
                rows_dot_h<4>(sm, w, s, b, o, lane);
                if (lane == 0) {
                    p.act[i0 + j] = swiglu(o[0], o[1]);
                    if (two) p.act[i0 + j2] = swiglu(o[2], o[3]);
                }
            }
        }
        prefetch_C_warp(sm, ly, L, r0, nc, K, warp, lane);
        if (l + 1 < p.l1) prefetch_A(sm, p.layers[l + 1], L, cta, G, E, tid);
        else cp_commit();  // keep the group count per layer fixed
        PROF(8);
        bar_target += G;
        if (!grid_barrier(p.sync, bar_target, sm)) { alive = false; break; }
        PROF(9);

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
            cp_wait<1>();  // this warp's down rows landed
            __syncthreads();  // the staged activations above are shared by all warps
            PROF(10);
            // one warp per output element: half-warp `sub` takes matrices sub, sub+2, ...
            const int sub = lane >> 4, c = lane & 15;
            constexpr int kMats = (kMaxK + 2) / 2;  // 5 matrix slots per half-warp
            for (int j = warp; j < nc; j += kDecWarps) {
                float acc = 0.0f;
#pragma unroll
                for (int jm = 0; jm < kMats; ++jm) {
                    const int m = sub + 2 * jm;
                    if (m <= K) {
                        float4 xv[8];
#pragma unroll
                        for (int q = 0; q < 8; ++q) xv[q] = sm->acts[(m * 8 + q) * kChI + c];
                        acc = fmaf(sm->topw[m],
                                   chunk_term(sm->c_w[m][j][c], xv, sm->suma[m * kChI + c], sm->c_s[m][j][c >> 1],
                                              sm->c_b[m][j][c >> 1]),
                                   acc);
                    }
                }
                acc = warp_sum(acc);
                // moe_combine_residual (reference src/math_util.rs:599-612)
                if (lane == 0) h_nxt[r0 + j] = sm->raw[r0 + j] + acc;
            }
        }
        PROF(11);
        parity ^= 1u;
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
    e->dec_prof = nullptr;
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

// Turns the per-phase clock stamps on or off (a device buffer of
// layers x kProfPoints stamps, written by CTA 0 of the decode kernel).
int decode_profile_enable(moe_engine* e, bool on) {
    if (on && !e->dec_prof) {
        MOE_CUDA(cudaMalloc(&e->dec_prof, e->layers.size() * kProfPoints * sizeof(long long)));
        MOE_CUDA(cudaMemset(e->dec_prof, 0, e->layers.size() * kProfPoints * sizeof(long long)));
    } else if (!on && e->dec_prof) {
        MOE_CUDA(cudaStreamSynchronize(e->stream));
        cudaFree(e->dec_prof);
        e->dec_prof = nullptr;
    }
    return MOE_OK;
}

int decode_profile_read(moe_engine* e, long long* out, int max_layers, int* points) {
    *points = kProfPoints;
    if (!e->dec_prof) { set_error("decode profiling is off"); return MOE_ERR_STATE; }
    int n = (int)e->layers.size() < max_layers ? (int)e->layers.size() : max_layers;
    MOE_CUDA(cudaMemcpyAsync(out, e->dec_prof, (size_t)n * kProfPoints * sizeof(long long), cudaMemcpyDeviceToHost, e->stream));
    MOE_CUDA(cudaStreamSynchronize(e->stream));
    return MOE_OK;
}

void decode_destroy(moe_engine* e) {
    if (e->dec_prof) cudaFree(e->dec_prof);
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
    MOE_REQUIRE(d.num_experts <= kMaxE, "decode path supports at most %d experts", kMaxE);
    const int G = e->dec_grid;
    auto cdiv = [](int a, int b) { return (a + b - 1) / b; };
    // every CTA's weight slice must fit its shared-memory staging area
    MOE_REQUIRE(cdiv(d.num_experts, G) <= kMaxRouterRows && cdiv(kI, G) <= kMaxSharedRows &&
                    cdiv(d.top_k * kI, G) <= kMaxBItems && cdiv(kH, G) <= kMaxCRows,
                "decode kernel needs at least 147 SMs for these dimensions (device has %d)", G);
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
    p.prof = e->dec_prof;
    p.E = d.num_experts; p.K = d.top_k;
    p.lay = e->lay;
    void* args[] = {&p};
    MOE_CUDA(cudaLaunchCooperativeKernel((const void*)decode_stack_kernel, dim3(e->dec_grid), dim3(kDecThreads),
                                         args, sizeof(DecodeSmem), e->stream));
    e->launches++;
    return MOE_OK;
}

// ─── decode of one block for callers that must not allocate ─────────────────
//
// Some hosts cannot let a library call cudaMalloc: a serving process whose device
// memory is carved up once at start-up and owned by its own pool, a plug-in
// running inside such a process, or a latency-critical loop in which cudaMalloc /
// cudaFree (which synchronise the device and can fail when memory is fragmented)
// are banned after initialisation.  For them the decode kernel's work areas (the
// router logits, the SwiGLU outputs, the grid-barrier words, one layer
// descriptor) live in the fixed array below instead of in engine-owned
// allocations.  The array is part of the library image: every GPU that loads
// the library holds these 40 KiB until the process exits.
constexpr size_t kNaSync = 0;        // 16 barrier / error words
constexpr size_t kNaLayer = 256;     // one LayerDev
constexpr size_t kNaMisc = 512;      // float[16]
constexpr size_t kNaLogits = 1024;   // float[kMaxE + 4]
constexpr size_t kNaAct = 3328;      // float[(kMaxK + 1) * kI]
constexpr size_t kNaH0 = kNaAct + sizeof(float) * (kMaxK + 1) * kI;
constexpr size_t kNaH1 = kNaH0 + sizeof(float) * kH;
constexpr size_t kNoAllocScratchBytes = 40960;
static_assert(kNaH1 + sizeof(float) * kH <= kNoAllocScratchBytes, "scratch layout exceeds the array");
static_assert(kNaLogits + sizeof(float) * (kMaxE + 4) <= kNaAct && sizeof(LayerDev) <= kNaMisc - kNaLayer, "scratch layout overlaps");
static_assert(kNaAct % 256 == 0 && kNaH0 % 256 == 0 && kNaH1 % 256 == 0, "scratch parts stay 256-byte aligned");

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

constexpr int kNaMaxDevices = 64;
// In host code `g_noalloc_scratch` is only a handle for the runtime, not an address a
// kernel can use; the device address is looked up once per device and kept here.
static unsigned char* g_noalloc_dev_ptr[kNaMaxDevices] = {};
static int g_noalloc_grid[kNaMaxDevices] = {};

}  // namespace moe

using namespace moe;

extern "C" int moe_layer_decode_noalloc(const moe_dims_t* dims, int device, const moe_layer_ptrs_t* lp,
                                        const float* h_in_dev, float* h_out_dev, int32_t* out_idx_dev,
                                        float* out_w_dev, void* cuda_stream, int wait) {
    MOE_REQUIRE(dims && lp && h_in_dev && h_out_dev, "null argument");
    const moe_dims_t& d = *dims;
    MOE_REQUIRE(d.hidden == kH && d.inter == kI && d.shared_inter == kI && d.group == kGroup,
                "no-alloc decode is built for hidden=%d, inter=shared_inter=%d, group=%d", kH, kI, kGroup);
    MOE_REQUIRE(d.top_k >= 1 && d.top_k <= kMaxK && d.top_k <= d.num_experts, "num_active_experts (%d) must be in 1..%d",
                d.top_k, kMaxK);
    // the fixed scratch array holds the logits of at most kMaxE experts
    MOE_REQUIRE(d.num_experts >= 1 && d.num_experts <= kMaxE,
                "num_experts (%d) exceeds the static scratch of the no-alloc entry point (at most %d experts)",
                d.num_experts, kMaxE);
    MOE_REQUIRE(lp->experts && lp->post_norm && lp->shared && lp->sgate_w && lp->sgate_s && lp->sgate_b &&
                    (lp->router_bf16 || (lp->router_w && lp->router_s && lp->router_b)),
                "no-alloc decode: a tensor pointer is missing");
    MOE_REQUIRE(device >= 0 && device < kNaMaxDevices, "device %d out of range", device);
    MOE_REQUIRE((((uintptr_t)h_in_dev) & 15) == 0 && (((uintptr_t)h_out_dev) & 15) == 0, "h must be 16-byte aligned");
    int prev = 0;
    MOE_CUDA(cudaGetDevice(&prev));
    MOE_CUDA(cudaSetDevice(device));
    int rc = MOE_OK;
    cudaStream_t st = (cudaStream_t)cuda_stream;
    do {
        if (!g_noalloc_dev_ptr[device]) {
            // one-time set-up on this device (with the device current): device address of the array
            unsigned char* ptr = nullptr;
            cudaError_t ce = cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch);
            if (ce != cudaSuccess || !ptr) { rc = cuda_fail(ce, "cudaGetSymbolAddress(g_noalloc_scratch)", __FILE__, __LINE__); break; }
            ce = cudaFuncSetAttribute(decode_stack_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(DecodeSmem));
            int sms = 0;
            if (ce == cudaSuccess) ce = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
            if (ce != cudaSuccess) { rc = cuda_fail(ce, "no-alloc decode set-up", __FILE__, __LINE__); break; }
            g_noalloc_grid[device] = sms;
            g_noalloc_dev_ptr[device] = ptr;
        }
        unsigned char* base = g_noalloc_dev_ptr[device];
        const int G = g_noalloc_grid[device];
        auto cdiv = [](int a, int b) { return (a + b - 1) / b; };
        if (!(cdiv(d.num_experts, G) <= kMaxRouterRows && cdiv(kI, G) <= kMaxSharedRows &&
              cdiv(d.top_k * kI, G) <= kMaxBItems && cdiv(kH, G) <= kMaxCRows)) {
            set_error("decode kernel needs at least 147 SMs for these dimensions (device has %d)", G);
            rc = MOE_ERR_INVALID;
            break;
        }
        LayerDev ld{};
        ld.experts = (const uint8_t*)lp->experts;
        ld.post_norm = (const uint16_t*)lp->post_norm;
        ld.router_bf16 = (const uint16_t*)lp->router_bf16;
        ld.router_q4.w = (const uint32_t*)lp->router_w;
        ld.router_q4.s = (const uint16_t*)lp->router_s;
        ld.router_q4.b = (const uint16_t*)lp->router_b;
        ld.shared = (const uint8_t*)lp->shared;
        ld.sgate.w = (const uint32_t*)lp->sgate_w;
        ld.sgate.s = (const uint16_t*)lp->sgate_s;
        ld.sgate.b = (const uint16_t*)lp->sgate_b;
        // the array keeps whatever the previous call left: the barrier and error words must start at zero
        cudaError_t ce = cudaMemsetAsync(base + kNaSync, 0, 64, st);
        if (ce == cudaSuccess) ce = cudaMemcpyAsync(base + kNaLayer, &ld, sizeof(ld), cudaMemcpyHostToDevice, st);
        if (ce != cudaSuccess) { rc = cuda_fail(ce, "no-alloc decode: scratch set-up", __FILE__, __LINE__); break; }
        DecodeParams p{};
        p.layers = reinterpret_cast<const LayerDev*>(base + kNaLayer);
        p.l0 = 0; p.l1 = 1;
        p.h_in = h_in_dev; p.h_out = h_out_dev;
        p.h_buf0 = reinterpret_cast<float*>(base + kNaH0);
        p.h_buf1 = reinterpret_cast<float*>(base + kNaH1);
        p.logits = reinterpret_cast<float*>(base + kNaLogits);
        p.act = reinterpret_cast<float*>(base + kNaAct);
        p.misc = reinterpret_cast<float*>(base + kNaMisc);
        p.logit_bias = nullptr; p.forced_idx = nullptr;
        p.out_idx = out_idx_dev; p.out_w = out_w_dev;
        p.sync = reinterpret_cast<unsigned int*>(base + kNaSync);
        p.prof = nullptr;
        p.E = d.num_experts; p.K = d.top_k;
        if (moe_expert_layout(d.hidden, d.inter, d.group, &p.lay) != MOE_OK) { rc = MOE_ERR_INVALID; break; }
        void* args[] = {&p};
        ce = cudaLaunchCooperativeKernel((const void*)decode_stack_kernel, dim3(G), dim3(kDecThreads), args,
                                         sizeof(DecodeSmem), st);
        if (ce != cudaSuccess) { rc = cuda_fail(ce, "no-alloc decode launch", __FILE__, __LINE__); break; }
        if (wait) {
            unsigned int flag = 0;
            ce = cudaMemcpyAsync(&flag, base + kNaSync + 8, sizeof(flag), cudaMemcpyDeviceToHost, st);
            if (ce == cudaSuccess) ce = cudaStreamSynchronize(st);
            if (ce != cudaSuccess) { rc = cuda_fail(ce, "no-alloc decode wait", __FILE__, __LINE__); break; }
            if (flag) {
                set_error("a bounded device-side wait gave up (code %u); the result of this call is invalid", flag);
                rc = MOE_ERR_DEVICE_WAIT;
            }
        }
    } while (0);
    cudaSetDevice(prev);
    return rc;
}
